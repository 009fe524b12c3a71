"""Checkpoint I/O in GhostFlow's own formats, through the native reader/writer (``csrc/formats.cpp``).

* ``save_state_dict`` / ``load_state_dict``: GHOSTFLW (ghostflow-core/src/serialize.rs:11-200) or safetensors
  (serialize.rs:223-456), chosen by ``fmt`` / detected by magic on load.
* ``Checkpoint`` + ``save_checkpoint`` / ``load_checkpoint``: GFCP (ghostflow-nn/src/serialization.rs:12-284):
  parameters, optional flat optimizer state, epoch, loss and free-form ``extra`` strings.
* ``save_sharded`` / ``load_sharded`` / ``consolidate``: one GFCP per rank for ZeRO-partitioned state
  (``extra`` records rank, world, step) and a merge into one GHOSTFLW file.

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


# ------------------------------------------------------------------------------------------- sharded (ZeRO)
def save_sharded(engine, directory, epoch: int = 0, loss: float = 0.0, extra: dict | None = None) -> str:
    """One GFCP file per rank with that rank's fp32 master shards and Adam moments."""
    os.makedirs(directory, exist_ok=True)
    st = engine.shard_state()
    params = {k: v for k, v in st.items() if k.endswith(".master")}
    opt = {k: v for k, v in st.items() if k.endswith(".exp_avg") or k.endswith(".exp_avg_sq")}
    ex = {"rank": engine.rank, "world": engine.world, "step": st["step"], "stage": 3, **(extra or {})}
    path = os.path.join(directory, f"shard_{engine.rank:05d}_of_{engine.world:05d}.gfcp")
    save_checkpoint(Checkpoint(params, opt, epoch, loss, "zero3-shard", extra=ex), path)
    return path


def load_sharded(engine, directory) -> Checkpoint:
    path = os.path.join(directory, f"shard_{engine.rank:05d}_of_{engine.world:05d}.gfcp")
    ck = load_checkpoint(path)
    if int(ck.extra["world"]) != engine.world:
        raise ValueError(f"checkpoint was written with world size {ck.extra['world']}, engine has {engine.world}; "
                         "use consolidate() and engine.load_unit() to re-shard")
    st = {"step": int(ck.extra["step"])}
    st.update({k: v.to(engine.device) for k, v in ck.parameters.items()})
    st.update({k: v.to(engine.device) for k, v in (ck.optimizer_state or {}).items()})
    engine.load_shard_state(st)
    return ck


def consolidate(engine, path, fmt: str = "ghostflw") -> None:
    """Gathers the full fp32 weights on every rank and lets rank 0 write one state-dict file."""
    sd = engine.state_dict(master=True)
    if engine.rank == 0:
        save_state_dict(sd, path, fmt=fmt)
