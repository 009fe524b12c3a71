"""Train a small ResNet for a few steps, fold its batch norms, and serve it from the channels-last bf16 program.

    python examples/vision_inference.py            # CPU works too (the serving program then uses plain matmuls)

Shows: ``models.resnet18``, ``optim.SGD`` / ``optim.RMSprop``, ``nn.fuse_conv_bn_relu`` (Conv+BN+ReLU folded into
one layer; on a B200 each folded convolution is a gather kernel + one tcgen05 GEMM with bias and ReLU in the
epilogue), ``model.compile_inference(cuda_graph=True)`` (whole network replayed from one CUDA graph) and
``nn.InferenceSession`` with request batching.
"""
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import models, nn, optim  # noqa: E402


def main():
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    torch.manual_seed(0)
    model = models.resnet18(num_classes=10, small_input=True, width=32).to(dev)
    opt = optim.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=5e-4)
    x, y = torch.randn(64, 3, 32, 32, device=dev), torch.randint(0, 10, (64,), device=dev)
    for step in range(10):
        opt.zero_grad()
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        if step % 3 == 0:
            print(f"step {step}: loss {float(loss):.4f}")

    model.eval()
    with torch.no_grad():
        reference = model(x)
        engine = model.compile_inference(cuda_graph=(dev == "cuda"))
        served = engine(x)
        print("serving program vs model, max abs difference:", float((served - reference).abs().max()))
        fused = nn.fuse_conv_bn_relu(model)
        print(f"folded {fused} Conv+BN(+ReLU) groups; max abs difference:", float((model(x) - reference).abs().max()))

    session = nn.InferenceSession(model, nn.InferenceConfig(batch_size=16, use_cuda_graph=(dev == "cuda")))
    outs = session.run_batch([x[i] for i in range(40)])
    print("served", len(outs), "requests; first prediction:", int(outs[0].argmax()))
    print("accuracy on the training batch:", float((reference.argmax(1) == y).float().mean()))


if __name__ == "__main__":
    main()
