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


def test_llama_checkpoint_is_served_behind_the_batching_queue(tmp_path):
    """POST /models/load on a LLaMA state dict builds the decoder; /predict takes token ids and returns the greedy
    continuation; concurrent requests of the same shape share one generate() call."""
    import threading

    from ghost_flow_b200.models import LLaMAConfig, LLaMAForCausalLM

    torch.manual_seed(0)
    cfg = LLaMAConfig(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    model = LLaMAForCausalLM(cfg)
    path = str(tmp_path / "llama.gf")
    gf_io.save_state_dict(model.state_dict(), path)
    with open(path + ".json", "w") as f:
        json.dump({"num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 64}, f)
    srv = Server("127.0.0.1", 0).start()
    try:
        base = f"http://127.0.0.1:{srv.port}"
        mid = _call(base + "/models/load", {"name": "tiny-llama", "path": path})["id"]
        info = _call(base + f"/models/{mid}")
        assert info["architecture"] == "llama" and info["layers"] == 2 and info["kv_heads"] == 2
        prompts = torch.randint(0, 200, (4, 9))
        ref = model.generate(prompts, 5) if srv.registry.device.type == "cpu" else None
        results = [None] * 4

        def ask(i):
            results[i] = _call(base + f"/models/{mid}/predict",
                               {"inputs": prompts[i].tolist(), "shape": [1, 9], "max_new_tokens": 5})

        ts = [threading.Thread(target=ask, args=(i,)) for i in range(4)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        for i, r in enumerate(results):
            assert r["shape"] == [1, 14] and r["outputs"][0][:9] == prompts[i].tolist()
            if ref is not None:
                assert r["outputs"][0] == ref[i].tolist()
        after = _call(base + f"/models/{mid}")
        assert after["requests"] == 4 and 1 <= after["batches_run"] <= 4
        assert _call(base + f"/models/{mid}/unload", {})["status"] == "unloaded"
    finally:
        srv.stop()
