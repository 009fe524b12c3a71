"""REST serving with the reference's seven routes and real model execution.

Reference: ghostflow-serve/src/main.rs:45-52 (routes), models.rs:48-62 (``load_model`` never opens the file and
hard-codes 784 -> 10), :81-105 (``predict`` echoes its input). Here ``POST /models/load`` reads the checkpoint
(GHOSTFLW, GFCP or safetensors through the native reader), infers an architecture from the tensor names, and
``predict`` runs it on the GPU when one is present (CPU otherwise).

    GET  /                      service banner
    GET  /health                {status, version, timestamp}
    GET  /models                list of loaded models
    GET  /models/{id}           one model's description
    POST /models/load           {name, path[, kind]} -> {id, status}
    POST /models/{id}/predict   {inputs: [[f32]], shape} -> {outputs, shape, inference_time_ms}
                                (a LLaMA checkpoint: inputs = token ids, optional max_new_tokens -> generated ids;
                                 concurrent requests are batched by ``GenerationBatcher``)
    POST /models/{id}/unload    -> {id, status}

The control plane is the standard library's threading HTTP server; ``ModelRegistry`` can be used without HTTP.
"""
from __future__ import annotations

import json
import os
import re
import threading
import time
import uuid
from dataclasses import dataclass
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import torch

VERSION = "1.1.1"


class ModelNotFound(KeyError):
    pass


def _build_from_state(state: dict, kind: str | None):
    """Returns (callable, description). Recognised layouts: a stack of ``<i>.weight`` / ``<i>.bias`` linear layers
    (an MLP, ReLU between layers), a single ``weight``/``bias`` pair, or ``kind='llama'``-style decoder weights
    handled by :class:`ghost_flow_b200.models.llama.LLaMAForCausalLM` when a ``config`` entry accompanies them."""
    names = sorted(state)
    lin = sorted({int(m.group(1)) for n in names if (m := re.match(r"^(?:layers\.|fc|net\.)?(\d+)\.weight$", n))})
    if kind in (None, "mlp") and lin:
        prefix = next(n[: n.index(f"{lin[0]}.weight")] for n in names if n.endswith(f"{lin[0]}.weight"))
        layers = []
        for i in lin:
            w = state[f"{prefix}{i}.weight"].float()
            b = state.get(f"{prefix}{i}.bias")
            layers.append((w, b.float() if b is not None else None))

        def to(dev):
            return [(w.to(dev), b.to(dev) if b is not None else None) for w, b in layers]

        def run(x, params):
            from ..ops.gemm import linear as gf_linear
            for j, (w, b) in enumerate(params):
                if x.is_cuda and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
                    x = gf_linear(x.to(torch.bfloat16), w.to(torch.bfloat16), b.to(torch.bfloat16) if b is not None else None).float()
                else:
                    x = torch.nn.functional.linear(x, w, b)
                if j < len(params) - 1:
                    x = torch.relu(x)
            return x

        desc = {"architecture": "mlp", "layers": [list(w.shape) for w, _ in layers], "input_shape": [layers[0][0].shape[1]],
                "output_shape": [layers[-1][0].shape[0]]}
        return run, to, desc
    if "weight" in state:
        return _build_from_state({"0.weight": state["weight"], **({"0.bias": state["bias"]} if "bias" in state else {})}, "mlp")
    raise ValueError(f"cannot infer an architecture from tensors {names[:6]}...; pass kind=")


def _llama_config_from_state(state: dict, extra: dict | None = None):
    """LLaMA hyper-parameters from tensor shapes (``extra`` may override: ``num_attention_heads``,
    ``num_key_value_heads``, ``rope_theta``...; the head count cannot be read from shapes, head_dim 128 is assumed
    for hidden sizes that allow it, else 64)."""
    from ..models.configs import LLaMAConfig

    emb = state["model.embed_tokens.weight"]
    vocab, hidden = emb.shape
    n_layers = 1 + max(int(m.group(1)) for n in state if (m := re.match(r"^model\.layers\.(\d+)\.", n)))
    qkv_out = state["model.layers.0.attn.wqkv.weight"].shape[0]
    inter = state["model.layers.0.mlp.w_gate_up.weight"].shape[0] // 2 if "model.layers.0.mlp.w_gate_up.weight" in state \
        else state["model.layers.0.mlp.gate_up.weight"].shape[0] // 2
    ex = dict(extra or {})
    heads = int(ex.pop("num_attention_heads", hidden // (128 if hidden % 128 == 0 and hidden >= 512 else 64)))
    hd = hidden // heads
    kv = int(ex.pop("num_key_value_heads", (qkv_out // hd - heads) // 2))
    return LLaMAConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=n_layers,
                       num_attention_heads=heads, num_key_value_heads=kv, **ex)


class GenerationBatcher:
    """Batching queue in front of a causal LM: requests wait up to ``max_wait_ms`` for company, compatible ones
    (same prompt length and number of new tokens) are stacked with :class:`~ghost_flow_b200.nn.inference.BatchInference`
    and run as ONE ``generate`` call; each request gets its own row back. The reference has the batching helper
    (ghostflow-nn/src/inference.rs:151-215) but its server never executes a model (ghostflow-serve/src/models.rs:81-105)."""

    def __init__(self, model, device, batch_size: int = 16, max_wait_ms: float = 4.0):
        from ..nn.inference import BatchInference

        self.model, self.device = model, device
        self.batch_size, self.max_wait_ms = batch_size, max_wait_ms
        self._mk = lambda: BatchInference(batch_size, max_wait_ms)
        self._queues: dict = {}            # (prompt_len, new_tokens) -> (BatchInference, [waiters])
        self._cv = threading.Condition()
        self._stop = False
        self.batches_run = 0
        self.requests_run = 0
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def submit(self, ids: torch.Tensor, max_new_tokens: int):
        """ids: 1-D int64 prompt. Blocks until the continuation is there; returns the full token row."""
        slot = {"done": threading.Event(), "out": None, "err": None}
        key = (int(ids.numel()), int(max_new_tokens))
        with self._cv:
            q = self._queues.get(key)
            if q is None:
                q = self._queues[key] = (self._mk(), [])
            q[0].add(ids)
            q[1].append(slot)
            self._cv.notify()
        slot["done"].wait()
        if slot["err"] is not None:
            raise slot["err"]
        return slot["out"]

    def _loop(self):
        while True:
            with self._cv:
                while not self._stop and not any(b.is_ready() for b, _ in self._queues.values()):
                    self._cv.wait(timeout=self.max_wait_ms / 1e3 if self._queues else None)
                if self._stop:
                    return
                key = next(k for k, (b, _) in self._queues.items() if b.is_ready())
                b, waiters = self._queues[key]
                batch = b.get_batch()
                mine, rest = waiters[:batch.shape[0]], waiters[batch.shape[0]:]
                if rest:
                    self._queues[key] = (b, rest)
                else:
                    del self._queues[key]
            try:
                with torch.no_grad():
                    out = self.model.generate(batch.to(self.device), key[1]).cpu()
                for i, w in enumerate(mine):
                    w["out"] = out[i]
            except Exception as e:       # hand the failure to every request of the batch
                for w in mine:
                    w["err"] = e
            self.batches_run += 1
            self.requests_run += len(mine)
            for w in mine:
                w["done"].set()

    def close(self):
        with self._cv:
            self._stop = True
            self._cv.notify_all()


def _build_llama(state: dict, device, extra: dict | None = None):
    from ..models.llama import LLaMAForCausalLM

    cfg = _llama_config_from_state(state, extra)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model = LLaMAForCausalLM(cfg, device=device, dtype=dtype)
    own = model.state_dict()
    missing = [k for k in own if k not in state]
    if missing:
        raise ValueError(f"LLaMA checkpoint lacks {missing[:4]}")
    with torch.no_grad():
        for k, v in own.items():
            v.copy_(state[k].to(device=device, dtype=dtype))
    model.eval()
    desc = {"architecture": "llama", "layers": cfg.num_hidden_layers, "hidden_size": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "vocab_size": cfg.vocab_size,
            "input_shape": ["prompt_len"], "output_shape": ["prompt_len + max_new_tokens"]}
    return model, desc


@dataclass
class ModelInfo:
    """What the registry reports about a loaded model (ghostflow-serve/src/models.rs:8-17)."""
    id: str
    name: str
    version: str
    input_shape: list
    output_shape: list
    loaded_at: str


@dataclass
class PredictionRequest:
    """Body of ``POST /models/{id}/predict`` (ghostflow-serve/src/models.rs:19-24)."""
    inputs: list
    shape: list | None = None

    @classmethod
    def from_json(cls, body: dict) -> "PredictionRequest":
        if "inputs" not in body:
            raise ValueError("missing 'inputs'")
        return cls(body["inputs"], body.get("shape"))


@dataclass
class PredictionResponse:
    """Answer of the predict route (ghostflow-serve/src/models.rs:26-32)."""
    outputs: list
    shape: list
    inference_time_ms: float

    def to_json(self) -> dict:
        return {"outputs": self.outputs, "shape": self.shape, "inference_time_ms": self.inference_time_ms}


class LoadedLlama:
    """A LLaMA checkpoint behind the generation batcher. ``predict`` takes token ids (one prompt per row) and
    ``max_new_tokens`` and returns the greedy continuation."""

    def __init__(self, mid, name, path, model, desc, device, batch_size=16, max_wait_ms=4.0):
        self.id, self.name, self.path, self.desc, self.device = mid, name, path, desc, device
        self.model = model
        self.batcher = GenerationBatcher(model, device, batch_size, max_wait_ms)
        self.loaded_at = time.time()
        self.requests = 0

    def describe(self):
        return {"id": self.id, "name": self.name, "path": self.path, "device": str(self.device),
                "requests": self.requests, "loaded_at": self.loaded_at, "batches_run": self.batcher.batches_run,
                **self.desc}

    def predict(self, inputs, shape=None, max_new_tokens: int = 16):
        ids = torch.tensor(inputs, dtype=torch.int64)
        if shape:
            ids = ids.reshape(shape)
        if ids.ndim == 1:
            ids = ids[None]
        if int(ids.min()) < 0 or int(ids.max()) >= self.desc["vocab_size"]:
            raise ValueError("token id out of range")
        t0 = time.perf_counter()
        rows = [None] * ids.shape[0]
        threads = [threading.Thread(target=lambda i=i: rows.__setitem__(i, self.batcher.submit(ids[i], max_new_tokens)))
                   for i in range(ids.shape[0])]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        self.requests += 1
        out = torch.stack(rows)
        return {"outputs": out.tolist(), "shape": list(out.shape), "inference_time_ms": (time.perf_counter() - t0) * 1e3}

    def close(self):
        self.batcher.close()


class LoadedModel:
    def __init__(self, mid, name, path, run, to_dev, desc, device):
        self.id, self.name, self.path, self.desc, self.device = mid, name, path, desc, device
        self._run, self._params = run, to_dev(device)
        self.loaded_at = time.time()
        self.requests = 0
        self.lock = threading.Lock()

    def describe(self):
        return {"id": self.id, "name": self.name, "path": self.path, "device": str(self.device), "requests": self.requests,
                "loaded_at": self.loaded_at, **self.desc}

    @torch.no_grad()
    def predict(self, inputs, shape=None):
        x = torch.tensor(inputs, dtype=torch.float32)
        if shape:
            x = x.reshape(shape)
        if x.ndim == 1:
            x = x[None]
        t0 = time.perf_counter()
        with self.lock:
            y = self._run(x.to(self.device), self._params)
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.requests += 1
        ms = (time.perf_counter() - t0) * 1e3
        y = y.float().cpu()
        return {"outputs": y.tolist(), "shape": list(y.shape), "inference_time_ms": ms}


class ModelRegistry:
    def __init__(self, device=None):
        self.device = torch.device(device) if device is not None else torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
        self.models: dict[str, LoadedModel] = {}
        self._lock = threading.Lock()

    def load_model(self, name: str, path: str, kind: str | None = None) -> str:
        from .. import io as gf_io
        state = gf_io.load_state_dict(path)
        mid = uuid.uuid4().hex[:12]
        if kind == "llama" or (kind is None and "model.embed_tokens.weight" in state):
            # decoder checkpoints (the names of models.llama.LLaMAForCausalLM.state_dict()) run behind the
            # generation batcher; an optional JSON file beside the checkpoint carries what shapes cannot tell
            extra = None
            if os.path.exists(os.fspath(path) + ".json"):
                with open(os.fspath(path) + ".json") as f:
                    extra = json.load(f)
            model, desc = _build_llama(state, self.device, extra)
            with self._lock:
                self.models[mid] = LoadedLlama(mid, name, path, model, desc, self.device)
            return mid
        run, to_dev, desc = _build_from_state(state, kind)
        with self._lock:
            self.models[mid] = LoadedModel(mid, name, path, run, to_dev, desc, self.device)
        return mid

    def register(self, name: str, fn, input_shape, output_shape) -> str:
        """Registers an in-process callable (any torch function of a float tensor)."""
        mid = uuid.uuid4().hex[:12]
        desc = {"architecture": "callable", "input_shape": list(input_shape), "output_shape": list(output_shape)}
        with self._lock:
            self.models[mid] = LoadedModel(mid, name, "", lambda x, _p: fn(x), lambda d: None, desc, self.device)
        return mid

    def get(self, mid) -> LoadedModel:
        try:
            return self.models[mid]
        except KeyError:
            raise ModelNotFound(mid) from None

    def info(self, mid) -> ModelInfo:
        m = self.get(mid)
        return ModelInfo(m.id, m.name, str(m.desc.get("version", "1.0.0")), list(m.desc.get("input_shape", [])),
                         list(m.desc.get("output_shape", [])),
                         time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime(m.loaded_at)))

    def handle(self, mid, request: PredictionRequest) -> PredictionResponse:
        """Typed form of :meth:`predict`."""
        r = self.predict(mid, request.inputs, request.shape)
        return PredictionResponse(r["outputs"], r["shape"], r["inference_time_ms"])

    def predict(self, mid, inputs, shape=None):
        """Runs model ``mid`` on ``inputs`` (the reference's ``ModelRegistry::predict``, ghostflow-serve/src/models.rs:81-105,
        echoes its input; this one executes the model)."""
        return self.get(mid).predict(inputs, shape)

    def unload(self, mid):
        with self._lock:
            m = self.models.pop(mid, None)
            if m is None:
                raise ModelNotFound(mid)
        if hasattr(m, "close"):
            m.close()

    def list(self):
        return [m.describe() for m in self.models.values()]


def make_handler(registry: ModelRegistry):
    class Handler(BaseHTTPRequestHandler):
        server_version = "ghostflow-serve/" + VERSION

        def log_message(self, fmt, *args):
            pass

        def _send(self, code, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.send_header("Access-Control-Allow-Origin", "*")
            self.end_headers()
            self.wfile.write(body)

        def _body(self):
            n = int(self.headers.get("Content-Length") or 0)
            return json.loads(self.rfile.read(n) or b"{}")

        def do_OPTIONS(self):
            self.send_response(204)
            self.send_header("Access-Control-Allow-Origin", "*")
            self.send_header("Access-Control-Allow-Methods", "GET, POST, OPTIONS")
            self.send_header("Access-Control-Allow-Headers", "*")
            self.end_headers()

        def do_GET(self):
            try:
                if self.path == "/":
                    return self._send(200, {"service": "ghostflow-serve", "version": VERSION})
                if self.path == "/health":
                    return self._send(200, {"status": "healthy", "version": VERSION, "timestamp": time.time()})
                if self.path == "/models":
                    return self._send(200, {"models": registry.list()})
                m = re.match(r"^/models/([^/]+)$", self.path)
                if m:
                    return self._send(200, registry.get(m.group(1)).describe())
                self._send(404, {"error": "not found"})
            except ModelNotFound as e:
                self._send(404, {"error": f"model {e.args[0]} not found"})

        def do_POST(self):
            try:
                if self.path == "/models/load":
                    b = self._body()
                    mid = registry.load_model(b["name"], b["path"], b.get("kind"))
                    return self._send(200, {"id": mid, "status": "loaded"})
                m = re.match(r"^/models/([^/]+)/(predict|unload)$", self.path)
                if not m:
                    return self._send(404, {"error": "not found"})
                if m.group(2) == "unload":
                    registry.unload(m.group(1))
                    return self._send(200, {"id": m.group(1), "status": "unloaded"})
                b = self._body()
                model = registry.get(m.group(1))
                if isinstance(model, LoadedLlama):
                    return self._send(200, model.predict(b["inputs"], b.get("shape"), int(b.get("max_new_tokens", 16))))
                self._send(200, model.predict(b["inputs"], b.get("shape")))
            except ModelNotFound as e:
                self._send(404, {"error": f"model {e.args[0]} not found"})
            except (KeyError, ValueError, RuntimeError, OSError) as e:
                self._send(400, {"error": str(e)})

    return Handler


class Server:
    """``Server(port=8080).start()`` serves in a background thread; ``serve_forever()`` blocks."""

    def __init__(self, host="0.0.0.0", port=8080, registry: ModelRegistry | None = None):
        self.registry = registry or ModelRegistry()
        self.httpd = ThreadingHTTPServer((host, port), make_handler(self.registry))
        self.port = self.httpd.server_address[1]
        self._thread = None

    def start(self):
        self._thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self._thread.start()
        return self

    def serve_forever(self):
        self.httpd.serve_forever()

    def stop(self):
        self.httpd.shutdown()
        self.httpd.server_close()


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="ghostflow-serve")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8080)
    a = ap.parse_args(argv)
    Server(a.host, a.port).serve_forever()


if __name__ == "__main__":
    main()
