"""Checkpoint I/O in GhostFlow's own formats, through the native reader/writer (``csrc/formats.cpp``).

* ``save_state_dict`` / ``load_state_dict``: GHOSTFLW (ghostflow-core/src/serialize.rs:11-200) or safetensors
  (serialize.rs:223-456), chosen by ``fmt`` / detected by magic on load.
* ``Checkpoint`` + ``save_checkpoint`` / ``load_checkpoint``: GFCP (ghostflow-nn/src/serialization.rs:12-284):
  parameters, optional flat optimizer state, epoch, loss and free-form ``extra`` strings.
* ``save_sharded`` / ``load_sharded`` / ``consolidate`` / ``load_consolidated``: one GFCP per rank for
  ZeRO-partitioned state (``extra`` records rank, world, step and the flat layout of every unit, so the shards can
  be cut again for another world size) and a merge into one file, optionally with the optimizer moments.
* ``training_state_extra`` / ``restore_training_state``: scheduler, loss scaler, data position and generator
  state in the ``extra`` section.

Payloads are always float32 on disk, exactly like the reference; the dtype code of GHOSTFLW records the
tensor's original type so that ``load_state_dict(..., restore_dtype=True)`` can cast back.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field

import torch

from ..dtype import DType
from ..ops import _lib

_BOUND = False


def _lib_io():
    global _BOUND
    lib = _lib.host_lib()
    if not _BOUND:
        c = ctypes
        lib.gfio_open.restype = c.c_void_p
        lib.gfio_open.argtypes = [c.c_char_p]
        lib.gfio_close.argtypes = [c.c_void_p]
        lib.gfio_kind.argtypes = [c.c_void_p]
        lib.gfio_count.argtypes = [c.c_void_p, c.c_int]
        for name, res in (("gfio_name", c.c_char_p), ("gfio_dtype", c.c_int), ("gfio_ndim", c.c_int),
                          ("gfio_numel", c.c_uint64), ("gfio_data", c.POINTER(c.c_float))):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = [c.c_void_p, c.c_int, c.c_int]
        lib.gfio_dims.argtypes = [c.c_void_p, c.c_int, c.c_int, c.POINTER(c.c_uint64)]
        lib.gfio_meta.restype = c.c_char_p
        lib.gfio_meta.argtypes = [c.c_void_p, c.c_int]
        lib.gfio_epoch.restype = c.c_uint64
        lib.gfio_epoch.argtypes = [c.c_void_p]
        lib.gfio_loss.restype = c.c_float
        lib.gfio_loss.argtypes = [c.c_void_p]
        lib.gfio_extra_count.argtypes = [c.c_void_p]
        lib.gfio_extra_key.restype = c.c_char_p
        lib.gfio_extra_key.argtypes = [c.c_void_p, c.c_int]
        lib.gfio_extra_value.restype = c.c_char_p
        lib.gfio_extra_value.argtypes = [c.c_void_p, c.c_int]
        lib.gfio_last_error.restype = c.c_char_p
        _BOUND = True
    return lib


def _as_f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", torch.float32).contiguous()


def _pack(named: dict):
    names = list(named.keys())
    tensors = [_as_f32(named[k]) for k in names]
    n = len(names)
    c_names = (ctypes.c_char_p * n)(*[k.encode() for k in names])
    ndims = (ctypes.c_int * n)(*[t.dim() for t in tensors])
    flat_dims = [d for t in tensors for d in t.shape]
    dims = (ctypes.c_uint64 * max(1, len(flat_dims)))(*flat_dims)
    data = (ctypes.POINTER(ctypes.c_float) * n)(*[ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_float))
                                                 for t in tensors])
    return n, c_names, ndims, dims, data, tensors


def _read_section(lib, h, section):
    out, dtypes = {}, {}
    for i in range(lib.gfio_count(h, section)):
        name = lib.gfio_name(h, section, i).decode()
        nd = lib.gfio_ndim(h, section, i)
        dims = (ctypes.c_uint64 * max(1, nd))()
        lib.gfio_dims(h, section, i, dims)
        ne = lib.gfio_numel(h, section, i)
        ptr = lib.gfio_data(h, section, i)
        if ne:
            buf = (ctypes.c_float * ne).from_address(ctypes.addressof(ptr.contents))
            t = torch.frombuffer(buf, dtype=torch.float32).clone()
        else:
            t = torch.empty(0)
        out[name] = t.reshape([int(dims[k]) for k in range(nd)]) if nd else t.reshape(())
        dtypes[name] = lib.gfio_dtype(h, section, i)
    return out, dtypes


def _open(path):
    lib = _lib_io()
    h = lib.gfio_open(os.fspath(path).encode())
    if not h:
        raise IOError(f"cannot read {path}: {lib.gfio_last_error().decode()}")
    return lib, h


# ------------------------------------------------------------------------------------------- state dicts
def save_state_dict(state: dict, path, fmt: str = "ghostflw") -> None:
    lib = _lib_io()
    state = {k: (v.data if hasattr(v, "data") and not isinstance(v, torch.Tensor) else v) for k, v in state.items()}
    n, names, ndims, dims, data, keep = _pack(state)
    p = os.fspath(path).encode()
    if fmt == "ghostflw":
        codes = (ctypes.c_uint8 * max(1, n))(*[int(DType.from_torch(v.dtype)) if v.dtype in _KNOWN else 2
                                                for v in state.values()])
        rc = lib.gfio_write_ghostflw(p, n, names, codes, ndims, dims, data)
    elif fmt == "safetensors":
        rc = lib.gfio_write_safetensors(p, n, names, ndims, dims, data)
    else:
        raise ValueError(f"unknown format {fmt!r}")
    if rc != 0:
        raise IOError(f"cannot write {path}: {lib.gfio_last_error().decode()}")


_KNOWN = {torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int8, torch.int16, torch.int32,
          torch.int64, torch.uint8, torch.bool}


def load_state_dict(path, restore_dtype: bool = False) -> dict:
    lib, h = _open(path)
    try:
        out, dtypes = _read_section(lib, h, 0)
    finally:
        lib.gfio_close(h)
    if restore_dtype:
        out = {k: v.to(DType(dtypes[k]).to_torch()) for k, v in out.items()}
    return out


# ------------------------------------------------------------------------------------------- GFCP
@dataclass
class Checkpoint:
    parameters: dict
    optimizer_state: dict | None = None
    epoch: int = 0
    loss: float = 0.0
    model_name: str = "model"
    version: str = "1.0.0"
    framework_version: str = "0.4.0"
    extra: dict = field(default_factory=dict)


@dataclass
class ModelMetadata:
    """Metadata block of a checkpoint (ghostflow-nn/src/serialization.rs:27-50)."""
    name: str = "model"
    version: str = "1.0.0"
    framework_version: str = "0.4.0"
    epoch: int = 0
    loss: float = 0.0
    extra: dict = field(default_factory=dict)


@dataclass
class ModelCheckpoint:
    """The reference's checkpoint object (ghostflow-nn/src/serialization.rs:12-25): parameters, metadata and an
    optional optimizer state, with ``save`` / ``load`` on the GFCP format. :class:`Checkpoint` is the flat record the
    rest of this package passes around; the two convert into each other."""
    parameters: dict
    metadata: ModelMetadata = field(default_factory=ModelMetadata)
    optimizer_state: dict | None = None

    def with_optimizer_state(self, state: dict) -> "ModelCheckpoint":
        self.optimizer_state = dict(state)
        return self

    def to_checkpoint(self) -> "Checkpoint":
        m = self.metadata
        return Checkpoint(self.parameters, self.optimizer_state, m.epoch, m.loss, m.name, m.version,
                          m.framework_version, dict(m.extra))

    @classmethod
    def from_checkpoint(cls, ck: "Checkpoint") -> "ModelCheckpoint":
        return cls(ck.parameters, ModelMetadata(ck.model_name, ck.version, ck.framework_version, ck.epoch, ck.loss,
                                                dict(ck.extra)), ck.optimizer_state)

    def save(self, path) -> None:
        save_checkpoint(self.to_checkpoint(), path)

    @classmethod
    def load(cls, path) -> "ModelCheckpoint":
        return cls.from_checkpoint(load_checkpoint(path))


def save_checkpoint(ckpt: Checkpoint, path) -> None:
    lib = _lib_io()
    n, names, ndims, dims, data, keep = _pack(ckpt.parameters)
    ek = list(ckpt.extra.keys())
    c_ek = (ctypes.c_char_p * max(1, len(ek)))(*[k.encode() for k in ek])
    c_ev = (ctypes.c_char_p * max(1, len(ek)))(*[str(ckpt.extra[k]).encode() for k in ek])
    if ckpt.optimizer_state is not None:
        on = list(ckpt.optimizer_state.keys())
        ot = [_as_f32(torch.as_tensor(ckpt.optimizer_state[k])).reshape(-1) for k in on]
        c_on = (ctypes.c_char_p * max(1, len(on)))(*[k.encode() for k in on])
        c_ol = (ctypes.c_uint64 * max(1, len(on)))(*[t.numel() for t in ot])
        c_od = (ctypes.POINTER(ctypes.c_float) * max(1, len(on)))(
            *[ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_float)) for t in ot])
        n_opt = len(on)
    else:
        c_on = c_ol = c_od = None
        n_opt = -1
    rc = lib.gfio_write_gfcp(os.fspath(path).encode(), ckpt.model_name.encode(), ckpt.version.encode(),
                             ckpt.framework_version.encode(), ctypes.c_uint64(int(ckpt.epoch)),
                             ctypes.c_float(float(ckpt.loss)), len(ek), c_ek, c_ev, n, names, ndims, dims, data,
                             n_opt, c_on, c_ol, c_od)
    if rc != 0:
        raise IOError(f"cannot write {path}: {lib.gfio_last_error().decode()}")


def load_checkpoint(path) -> Checkpoint:
    lib, h = _open(path)
    try:
        if lib.gfio_kind(h) != 2:
            raise IOError(f"{path} is not a GFCP checkpoint")
        params, _ = _read_section(lib, h, 0)
        opt, _ = _read_section(lib, h, 1)
        extra = {lib.gfio_extra_key(h, i).decode(): lib.gfio_extra_value(h, i).decode()
                 for i in range(lib.gfio_extra_count(h))}
        ck = Checkpoint(params, opt if lib.gfio_count(h, 1) else None, int(lib.gfio_epoch(h)),
                        float(lib.gfio_loss(h)), lib.gfio_meta(h, 0).decode(), lib.gfio_meta(h, 1).decode(),
                        lib.gfio_meta(h, 2).decode(), extra)
    finally:
        lib.gfio_close(h)
    return ck


# ------------------------------------------------------------------------------------------- resume state
def capture_rng_state(device=None) -> str:
    """Generator states of the CPU and (when ``device`` is a CUDA device) that device, as one hex string for the
    ``extra`` section of a GFCP checkpoint. The reference saves no generator state (its RNG is ``thread_rng()``
    everywhere: ghostflow-core/src/tensor.rs:94,105), so a resumed run could not repeat an uninterrupted one."""
    parts = [torch.get_rng_state().numpy().tobytes().hex()]
    if device is not None and torch.device(device).type == "cuda":
        parts.append(torch.cuda.get_rng_state(torch.device(device)).cpu().numpy().tobytes().hex())
    return "|".join(parts)


def restore_rng_state(state: str, device=None) -> None:
    import numpy as np

    parts = state.split("|")
    torch.set_rng_state(torch.from_numpy(np.frombuffer(bytes.fromhex(parts[0]), dtype=np.uint8).copy()))
    if len(parts) > 1 and device is not None and torch.device(device).type == "cuda":
        torch.cuda.set_rng_state(torch.from_numpy(np.frombuffer(bytes.fromhex(parts[1]), dtype=np.uint8).copy()),
                                 torch.device(device))


def training_state_extra(scheduler=None, scaler=None, data_position: int | None = None, rng: bool = True,
                         device=None) -> dict:
    """Everything a run needs beyond weights and moments, as the string map that GFCP's ``extra`` section holds
    (ghostflow-nn/src/serialization.rs:12-37 has the section but nothing writes resume state into it): learning-rate
    scheduler, loss scaler, position in the data stream, generator states."""
    import json

    ex = {}
    if scheduler is not None:
        ex["lr_scheduler"] = json.dumps(scheduler.state_dict())
    if scaler is not None:
        ex["grad_scaler"] = json.dumps(scaler.state_dict())
    if data_position is not None:
        ex["data_position"] = str(int(data_position))
    if rng:
        ex["rng_state"] = capture_rng_state(device)
    return ex


def restore_training_state(extra: dict, scheduler=None, scaler=None, device=None) -> dict:
    """Inverse of :func:`training_state_extra`; returns ``{"data_position": int}`` when one was saved."""
    import json

    out = {}
    if scheduler is not None and "lr_scheduler" in extra:
        scheduler.load_state_dict(json.loads(extra["lr_scheduler"]))
    if scaler is not None and "grad_scaler" in extra:
        scaler.load_state_dict(json.loads(extra["grad_scaler"]))
    if "data_position" in extra:
        out["data_position"] = int(extra["data_position"])
    if "rng_state" in extra:
        restore_rng_state(extra["rng_state"], device)
    return out


# ------------------------------------------------------------------------------------------- sharded (ZeRO)
def _shard_path(directory, rank: int, world: int) -> str:
    return os.path.join(directory, f"shard_{rank:05d}_of_{world:05d}.gfcp")


def save_sharded(engine, directory, epoch: int = 0, loss: float = 0.0, extra: dict | None = None) -> str:
    """One GFCP file per rank with that rank's fp32 master shards and Adam moments. ``extra`` records rank,
    world, step, ZeRO stage and, per unit, the flat layout (``flat.<unit>`` = ``numel:padded:shard_numel:lo``),
    which is what :func:`load_sharded` needs to cut the state again for another world size. Pass
    :func:`training_state_extra` as ``extra`` to carry scheduler / scaler / data position / generator state."""
    os.makedirs(directory, exist_ok=True)
    st = engine.shard_state()
    params = {k: v for k, v in st.items() if k.endswith(".master")}
    opt = {k: v for k, v in st.items() if k.endswith(".exp_avg") or k.endswith(".exp_avg_sq")}
    ex = {"rank": engine.rank, "world": engine.world, "step": st["step"], "stage": 3}
    for name, lay in engine.flat_layout().items():
        ex[f"flat.{name}"] = f"{lay['numel']}:{lay['padded']}:{lay['shard_numel']}:{lay['lo']}"
    ex.update(extra or {})
    path = _shard_path(directory, engine.rank, engine.world)
    save_checkpoint(Checkpoint(params, opt, epoch, loss, "zero3-shard", extra=ex), path)
    return path


def _find_source_world(directory) -> int:
    import re

    worlds = {int(m.group(1)) for f in os.listdir(directory)
              if (m := re.match(r"shard_\d{5}_of_(\d{5})\.gfcp$", f))}
    if len(worlds) != 1:
        raise IOError(f"{directory}: expected the shards of exactly one world size, found {sorted(worlds)}")
    return worlds.pop()


def _recut(engine, directory, src_world: int) -> tuple[dict, Checkpoint]:
    """Builds this rank's shards from the files of another world size. Every unit is one flat buffer whose
    logical prefix ``[0, numel)`` does not depend on the world size (only the zero padding behind it does), so a
    new shard ``[lo, lo + shard_numel)`` is the concatenation of the overlapping pieces of the old shards."""
    layout = engine.flat_layout()
    keys = ("master", "exp_avg", "exp_avg_sq")
    out = {f"{u}.{k}": torch.zeros(lay["shard_numel"], dtype=torch.float32) for u, lay in layout.items() for k in keys}
    first = None
    for r in range(src_world):
        ck = load_checkpoint(_shard_path(directory, r, src_world))
        first = first or ck
        for u, lay in layout.items():
            numel, _, s_shard, s_lo = (int(x) for x in ck.extra[f"flat.{u}"].split(":"))
            if numel != lay["numel"]:
                raise ValueError(f"unit {u}: checkpoint has {numel} elements, engine has {lay['numel']}")
            lo = max(lay["lo"], s_lo)
            hi = min(lay["lo"] + lay["shard_numel"], s_lo + s_shard, numel)
            if hi <= lo:
                continue
            for k in keys:
                src = ck.parameters[f"{u}.master"] if k == "master" else ck.optimizer_state[f"{u}.{k}"]
                out[f"{u}.{k}"][lo - lay["lo"]:hi - lay["lo"]] = src.reshape(-1)[lo - s_lo:hi - s_lo]
    return out, first


def load_sharded(engine, directory) -> Checkpoint:
    """Restores the engine from :func:`save_sharded` files. With the same world size every rank reads its own
    file; with a different one (a job restarted on fewer or more GPUs) every rank re-cuts its shards from the
    files of the old world. Returns rank-local checkpoint metadata (``extra`` holds the saved resume state)."""
    src_world = _find_source_world(directory)
    if src_world == engine.world:
        ck = load_checkpoint(_shard_path(directory, engine.rank, engine.world))
        st = {"step": int(ck.extra["step"])}
        st.update({k: v.to(engine.device) for k, v in ck.parameters.items()})
        st.update({k: v.to(engine.device) for k, v in (ck.optimizer_state or {}).items()})
    else:
        tensors, ck = _recut(engine, directory, src_world)
        st = {"step": int(ck.extra["step"])}
        st.update({k: v.to(engine.device) for k, v in tensors.items()})
    engine.load_shard_state(st)
    return ck


def consolidate(engine, path, fmt: str = "ghostflw", with_optimizer: bool = False) -> None:
    """Gathers the full fp32 weights on every rank and lets rank 0 write one file: a GHOSTFLW / safetensors
    state dict, or with ``with_optimizer`` a GFCP checkpoint that also carries the gathered Adam moments
    (``exp_avg.<name>``, ``exp_avg_sq.<name>``) and the step, from which :func:`load_consolidated` restores
    an engine of any world size."""
    sd = engine.state_dict(master=True)
    if not with_optimizer:
        if engine.rank == 0:
            save_state_dict(sd, path, fmt=fmt)
        return
    opt = {}
    for prefix, which in (("exp_avg", "m"), ("exp_avg_sq", "v")):
        for k, v in engine.state_dict(which=which).items():
            opt[f"{prefix}.{k}"] = v
    if engine.rank == 0:
        save_checkpoint(Checkpoint(sd, opt, 0, 0.0, "zero3-consolidated", extra={"step": engine.step_count}), path)


def load_consolidated(engine, path) -> Checkpoint:
    """Restores weights, moments and step of a ZeRO engine (any world size) from :func:`consolidate`
    ``(with_optimizer=True)`` output; every rank reads the file and keeps its own slices."""
    ck = load_checkpoint(path)
    engine.load_full_state(ck.parameters, {k[len("exp_avg."):]: v for k, v in ck.optimizer_state.items()
                                           if k.startswith("exp_avg.")},
                           {k[len("exp_avg_sq."):]: v for k, v in ck.optimizer_state.items()
                            if k.startswith("exp_avg_sq.")}, int(ck.extra.get("step", 0)))
    return ck
