"""Walks the serving API end to end: writes a small MLP checkpoint, starts the server in this process, loads the
model over HTTP, runs a prediction and unloads it (the flow of the reference's ghostflow-serve/examples/client.py)."""
import json
import os
import sys
import tempfile
import urllib.request

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import io as gf_io  # noqa: E402
from ghost_flow_b200.serve import Server  # noqa: E402


def call(url, payload=None):
    req = urllib.request.Request(url, data=json.dumps(payload).encode() if payload is not None else None,
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req) as r:
        return json.loads(r.read())


def main():
    torch.manual_seed(0)
    state = {"0.weight": torch.randn(32, 16), "0.bias": torch.randn(32), "1.weight": torch.randn(8, 32), "1.bias": torch.randn(8)}
    path = os.path.join(tempfile.mkdtemp(), "mlp.gf")
    gf_io.save_state_dict(state, path)
    srv = Server("127.0.0.1", 0).start()
    base = f"http://127.0.0.1:{srv.port}"
    print(call(base + "/health"))
    mid = call(base + "/models/load", {"name": "mlp", "path": path})["id"]
    print(call(base + f"/models/{mid}"))
    x = torch.randn(2, 16)
    out = call(base + f"/models/{mid}/predict", {"inputs": x.tolist(), "shape": [2, 16]})
    ref = torch.relu(x @ state["0.weight"].t() + state["0.bias"]) @ state["1.weight"].t() + state["1.bias"]
    print("max abs error vs local reference:", (torch.tensor(out["outputs"]) - ref).abs().max().item(),
          "time ms:", round(out["inference_time_ms"], 3))
    print(call(base + f"/models/{mid}/unload", {}))
    srv.stop()


if __name__ == "__main__":
    main()
