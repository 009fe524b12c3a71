"""The seven REST routes against a real checkpoint and a real forward pass."""
import json
import urllib.error
import urllib.request

import torch

from ghost_flow_b200 import io as gf_io
from ghost_flow_b200.serve import Server


def _call(url, payload=None):
    req = urllib.request.Request(url, data=json.dumps(payload).encode() if payload is not None else None,
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req) as r:
        return json.loads(r.read())


def test_routes_load_predict_unload(tmp_path):
    torch.manual_seed(0)
    state = {"0.weight": torch.randn(32, 16), "0.bias": torch.randn(32), "1.weight": torch.randn(8, 32), "1.bias": torch.randn(8)}
    path = str(tmp_path / "mlp.gf")
    gf_io.save_state_dict(state, path)
    srv = Server("127.0.0.1", 0).start()
    try:
        base = f"http://127.0.0.1:{srv.port}"
        assert _call(base + "/")["service"] == "ghostflow-serve"
        assert _call(base + "/health")["status"] == "healthy"
        assert _call(base + "/models")["models"] == []
        mid = _call(base + "/models/load", {"name": "mlp", "path": path})["id"]
        info = _call(base + f"/models/{mid}")
        assert info["input_shape"] == [16] and info["output_shape"] == [8]
        x = torch.randn(3, 16)
        out = _call(base + f"/models/{mid}/predict", {"inputs": x.flatten().tolist(), "shape": [3, 16]})
        ref = torch.relu(x @ state["0.weight"].t() + state["0.bias"]) @ state["1.weight"].t() + state["1.bias"]
        tol = 1e-4 if not torch.cuda.is_available() else 0.5
        assert out["shape"] == [3, 8] and (torch.tensor(out["outputs"]) - ref).abs().max() < tol
        assert out["inference_time_ms"] > 0
        assert len(_call(base + "/models")["models"]) == 1
        assert _call(base + f"/models/{mid}/unload", {})["status"] == "unloaded"
        try:
            _call(base + f"/models/{mid}")
            raise AssertionError("expected 404")
        except urllib.error.HTTPError as e:
            assert e.code == 404
    finally:
        srv.stop()
