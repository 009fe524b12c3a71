"""Conv1d / Conv3d / TransposeConv2d, GroupNorm / InstanceNorm, newer activations and losses
(the reference's examples/new_layers_demo.rs)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ghost_flow_b200 import nn  # noqa: E402


def main():
    print("Conv1d", tuple(nn.Conv1d(4, 8, 3, 1, 1)(torch.randn(2, 4, 20)).shape))
    print("Conv3d", tuple(nn.Conv3d(2, 4, (3, 3, 3), (1, 1, 1), (1, 1, 1))(torch.randn(1, 2, 6, 8, 8)).shape))
    print("TransposeConv2d", tuple(nn.TransposeConv2d(4, 2, (4, 4), (2, 2), (1, 1), (0, 0))(torch.randn(1, 4, 8, 8)).shape))
    x = torch.randn(2, 8, 6, 6)
    print("GroupNorm", tuple(nn.GroupNorm(4, 8)(x).shape), "InstanceNorm", tuple(nn.InstanceNorm2d(8)(x).shape))
    for act in (nn.Mish(), nn.Swish(), nn.SELU(), nn.ELU(), nn.Softplus()):
        print(type(act).__name__, round(float(act(torch.tensor([1.0]))[0]), 4))
    logits, target = torch.randn(6, 5), torch.randint(0, 5, (6,))
    print("focal", round(float(nn.focal_loss(logits, target)), 4), "huber", round(float(nn.huber_loss(torch.randn(6), torch.randn(6))), 4))


if __name__ == "__main__":
    main()
