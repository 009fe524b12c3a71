"""Convolutions and pooling with the reference's constructors.

``Conv2d(cin, cout, k, stride, padding)`` / ``with_params``; ``Conv1d``, ``Conv3d``, ``TransposeConv2d``
(ghostflow-nn/src/conv.rs:20-47,187-301,329-357,489-520: kaiming-uniform weights, uniform bias) and
``MaxPool2d, AvgPool2d, GlobalAvgPool2d, GlobalMaxPool2d, AdaptiveAvgPool2d`` (ghostflow-nn/src/pooling.rs:7-258).
Inference-time Conv+BN+ReLU folding lives in :mod:`ghost_flow_b200.nn.fused_conv`.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import init
from .module import Module, Parameter


def _tup(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


class _ConvNd(Module):
    nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True):
        super().__init__()
        n = self.nd
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = _tup(kernel_size, n), _tup(stride, n)
        self.padding, self.dilation, self.groups = _tup(padding, n), _tup(dilation, n), groups
        self.weight = Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size))
        self.bias = Parameter(torch.empty(out_channels)) if bias else None
        init.kaiming_uniform(self.weight.data)
        if bias:
            fan_in = (in_channels // groups) * math.prod(self.kernel_size)
            b = 1.0 / math.sqrt(fan_in)
            self.bias.data.uniform_(-b, b)

    @classmethod
    def with_params(cls, in_channels, out_channels, kernel_size, stride, padding, bias=True):
        return cls(in_channels, out_channels, kernel_size, stride, padding, bias=bias)


class Conv1d(_ConvNd):
    nd = 1

    def forward(self, x):
        return F.conv1d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class Conv2d(_ConvNd):
    nd = 2

    def forward(self, x):
        return F.conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class Conv3d(_ConvNd):
    nd = 3

    def forward(self, x):
        return F.conv3d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class TransposeConv2d(Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, bias=True):
        super().__init__()
        self.stride, self.padding, self.output_padding = _tup(stride, 2), _tup(padding, 2), _tup(output_padding, 2)
        self.weight = Parameter(torch.empty(in_channels, out_channels, *_tup(kernel_size, 2)))
        self.bias = Parameter(torch.empty(out_channels)) if bias else None
        init.kaiming_uniform(self.weight.data)
        if bias:
            b = 1.0 / math.sqrt(in_channels * math.prod(_tup(kernel_size, 2)))
            self.bias.data.uniform_(-b, b)

    def forward(self, x):
        return F.conv_transpose2d(x, self.weight, self.bias, self.stride, self.padding, self.output_padding)


ConvTranspose2d = TransposeConv2d


class MaxPool2d(Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.k, self.s, self.p = kernel_size, stride or kernel_size, padding

    def forward(self, x):
        return F.max_pool2d(x, self.k, self.s, self.p)


class AvgPool2d(Module):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.k, self.s, self.p = kernel_size, stride or kernel_size, padding

    def forward(self, x):
        return F.avg_pool2d(x, self.k, self.s, self.p)


class GlobalAvgPool2d(Module):
    def forward(self, x):
        return x.mean(dim=(-2, -1))


class GlobalMaxPool2d(Module):
    def forward(self, x):
        return x.amax(dim=(-2, -1))


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_size):
        super().__init__()
        self.output_size = output_size

    def forward(self, x):
        return F.adaptive_avg_pool2d(x, self.output_size)


class Flatten(Module):
    def __init__(self, start_dim=1):
        super().__init__()
        self.start_dim = start_dim

    def forward(self, x):
        return x.flatten(self.start_dim)
