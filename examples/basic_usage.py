"""Tensors, operators, layers: the surface of the reference's only Python example
(ghost-flow-py/examples/basic_usage.py), plus what its documentation advertises (autograd, optimizers, losses)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ghost_flow as gf  # noqa: E402  (alias of ghost_flow_b200)


def main():
    x = gf.Tensor.randn(4, 8)
    y = gf.Tensor.rand(8, 3)
    z = x @ y
    print("matmul", z.shape, "relu mean", z.relu().mean().item())
    print("scalar ops", (x + 1000).mean().item() > 900, "transpose", x.transpose(0, 1).shape, "reshape", x.reshape([2, 16]).shape)
    print("softmax rows sum to", z.softmax(1).sum().item() / 4)

    model = gf.nn.Sequential([gf.nn.Linear(8, 16), gf.nn.ReLU(), gf.nn.Linear(16, 1)])
    opt = gf.optim.Adam(model.parameters(), lr=1e-2)
    target = gf.Tensor.zeros(4, 1)
    for step in range(50):
        opt.zero_grad()
        loss = gf.nn.mse_loss(model(x), target)
        loss.backward()
        opt.step()
    print("trained loss", round(loss.item(), 5))


if __name__ == "__main__":
    main()
