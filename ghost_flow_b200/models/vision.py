"""Convolutional image classifiers: ResNet-18/34/50/101/152, VGG-11/13/16/19 (with batch norm) and MobileNetV2.

The reference quotes ResNet-18 epoch time, a "ResNet-50 layer" convolution and a fused Conv+BN+ReLU
(ghost-flow-py/PERFORMANCE.md:46-51, DOCS/PERFORMANCE_SUMMARY.md:43-46) and lists these families in its disabled
``deep/architectures`` catalogue (ghostflow-ml/src/lib.rs:133-134) without a working implementation. Training uses
the regular layers of :mod:`ghost_flow_b200.nn`. For serving, :class:`ChannelsLastEngine` compiles a trained ResNet
into a channels-last bf16 program: every batch norm folded into its convolution, every convolution one tcgen05 GEMM
(plus a 16-byte-wide gather for windows larger than 1 x 1), and bias, shortcut addition and ReLU done in that
GEMM's epilogue, so a bottleneck block is three kernels and no separate normalisation or activation pass.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..nn.conv import AdaptiveAvgPool2d, Conv2d, MaxPool2d
from ..nn.fused_conv import fold_batch_norm
from ..nn.layers import BatchNorm2d, Dropout, Linear, ReLU
from ..nn.module import Module, Sequential


def _absorbed(bn) -> bool:
    return bool(getattr(bn, "absorbs_relu", False))


class BasicBlock(Module):
    """Two 3 x 3 convolutions with an identity (or 1 x 1 projection) shortcut."""

    expansion = 1
    _fusable = (("conv1", "bn1", True), ("conv2", "bn2", False))

    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        self.conv1 = Conv2d(in_planes, planes, 3, stride, 1, bias=False)
        self.bn1 = BatchNorm2d(planes)
        self.conv2 = Conv2d(planes, planes, 3, 1, 1, bias=False)
        self.bn2 = BatchNorm2d(planes)
        self.downsample = None
        if stride != 1 or in_planes != planes * self.expansion:
            self.downsample = Sequential(Conv2d(in_planes, planes * self.expansion, 1, stride, 0, bias=False),
                                         BatchNorm2d(planes * self.expansion))

    def forward(self, x):
        out = self.bn1(self.conv1(x))
        if not _absorbed(self.bn1):
            out = torch.relu(out)
        out = self.bn2(self.conv2(out))
        return torch.relu(out + (x if self.downsample is None else self.downsample(x)))


class Bottleneck(Module):
    """1 x 1 reduce, 3 x 3, 1 x 1 expand (x 4) with a shortcut; the stride sits on the 3 x 3 convolution."""

    expansion = 4
    _fusable = (("conv1", "bn1", True), ("conv2", "bn2", True), ("conv3", "bn3", False))

    def __init__(self, in_planes: int, planes: int, stride: int = 1):
        super().__init__()
        self.conv1 = Conv2d(in_planes, planes, 1, 1, 0, bias=False)
        self.bn1 = BatchNorm2d(planes)
        self.conv2 = Conv2d(planes, planes, 3, stride, 1, bias=False)
        self.bn2 = BatchNorm2d(planes)
        self.conv3 = Conv2d(planes, planes * 4, 1, 1, 0, bias=False)
        self.bn3 = BatchNorm2d(planes * 4)
        self.downsample = None
        if stride != 1 or in_planes != planes * 4:
            self.downsample = Sequential(Conv2d(in_planes, planes * 4, 1, stride, 0, bias=False),
                                         BatchNorm2d(planes * 4))

    def forward(self, x):
        out = self.bn1(self.conv1(x))
        if not _absorbed(self.bn1):
            out = torch.relu(out)
        out = self.bn2(self.conv2(out))
        if not _absorbed(self.bn2):
            out = torch.relu(out)
        out = self.bn3(self.conv3(out))
        return torch.relu(out + (x if self.downsample is None else self.downsample(x)))


class ResNet(Module):
    """``ResNet(block, [n1, n2, n3, n4], num_classes)``. ``small_input=True`` swaps the 7 x 7 / stride-2 stem and
    the max pool for a single 3 x 3 convolution (the usual variant for 32 x 32 images)."""

    _fusable = (("conv1", "bn1", True),)

    def __init__(self, block, layers, num_classes: int = 1000, in_channels: int = 3, small_input: bool = False,
                 width: int = 64):
        super().__init__()
        self.block, self.layers_cfg, self.small_input = block, tuple(layers), small_input
        self.in_planes = width
        if small_input:
            self.conv1 = Conv2d(in_channels, width, 3, 1, 1, bias=False)
        else:
            self.conv1 = Conv2d(in_channels, width, 7, 2, 3, bias=False)
        self.bn1 = BatchNorm2d(width)
        self.maxpool = None if small_input else MaxPool2d(3, 2, 1)
        self.layer1 = self._make_layer(block, width, layers[0], 1)
        self.layer2 = self._make_layer(block, width * 2, layers[1], 2)
        self.layer3 = self._make_layer(block, width * 4, layers[2], 2)
        self.layer4 = self._make_layer(block, width * 8, layers[3], 2)
        self.avgpool = AdaptiveAvgPool2d(1)
        self.fc = Linear(width * 8 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, Conv2d):
                torch.nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def _make_layer(self, block, planes, n, stride):
        blocks = []
        for s in [stride] + [1] * (n - 1):
            blocks.append(block(self.in_planes, planes, s))
            self.in_planes = planes * block.expansion
        return Sequential(blocks)

    def features(self, x):
        x = self.bn1(self.conv1(x))
        if not _absorbed(self.bn1):
            x = torch.relu(x)
        if self.maxpool is not None:
            x = self.maxpool(x)
        return self.layer4(self.layer3(self.layer2(self.layer1(x))))

    def forward(self, x):
        return self.fc(self.avgpool(self.features(x)).flatten(1))

    def compile_inference(self, cuda_graph: bool = False) -> "ChannelsLastEngine":
        return ChannelsLastEngine(self, cuda_graph=cuda_graph)


def resnet18(num_classes=1000, **kw): return ResNet(BasicBlock, [2, 2, 2, 2], num_classes, **kw)
def resnet34(num_classes=1000, **kw): return ResNet(BasicBlock, [3, 4, 6, 3], num_classes, **kw)
def resnet50(num_classes=1000, **kw): return ResNet(Bottleneck, [3, 4, 6, 3], num_classes, **kw)
def resnet101(num_classes=1000, **kw): return ResNet(Bottleneck, [3, 4, 23, 3], num_classes, **kw)
def resnet152(num_classes=1000, **kw): return ResNet(Bottleneck, [3, 8, 36, 3], num_classes, **kw)


# ------------------------------------------------------------------ channels-last bf16 serving program
class _PackedConv:
    """One folded convolution of the serving program: bf16 ``[Cout, KH * KW * Cin_padded]`` weights and bias."""

    def __init__(self, conv: Conv2d, bn: BatchNorm2d | None, device):
        from ..ops.render import pack_conv_weight_nhwc

        assert conv.groups == 1 and tuple(conv.dilation) == (1, 1), "grouped/dilated convolutions are not packed"
        if bn is not None:
            w, b = fold_batch_norm(conv.weight, conv.bias, bn.weight, bn.bias, bn.running_mean, bn.running_var, bn.eps)
        else:
            w = conv.weight.detach().float()
            b = conv.bias.detach().float() if conv.bias is not None else torch.zeros(conv.out_channels)
        self.weight, self.bias = pack_conv_weight_nhwc(w.to(device), b.to(device))
        self.kernel_size = tuple(conv.kernel_size)
        self.stride, self.padding = conv.stride[0], conv.padding[0]
        self.cin_padded = self.weight.shape[1] // (self.kernel_size[0] * self.kernel_size[1])

    def __call__(self, x, relu: bool, residual=None):
        from ..ops.render import conv2d_nhwc

        return conv2d_nhwc(x, self.weight, self.bias, self.kernel_size, self.stride, self.padding, relu, residual)


class ChannelsLastEngine:
    """Inference program of a trained :class:`ResNet`: bf16, ``[N, H, W, C]`` activations, folded batch norms.

    ``engine(x)`` takes the same NCHW float input as the model and returns fp32 logits. Weights are snapshotted
    when the engine is built; rebuild it after further training.
    """

    def __init__(self, model: ResNet, device=None, cuda_graph: bool = False):
        """``cuda_graph=True`` replays the whole program from a CUDA graph (one per input shape): for small images
        the program is bound by launch latency, not by the GPU."""
        device = torch.device(device) if device is not None else next(model.parameters()).device
        self.device = device
        self._runner = None
        if cuda_graph and device.type == "cuda":
            from ..nn.inference import CudaGraphRunner

            self._runner = CudaGraphRunner(self._forward)
        self.stem = _PackedConv(model.conv1, model.bn1, device)
        self.pool = model.maxpool is not None
        self.blocks = []
        for stage in (model.layer1, model.layer2, model.layer3, model.layer4):
            for blk in stage:
                convs = [_PackedConv(getattr(blk, c), getattr(blk, b), device) for c, b, _ in blk._fusable]
                down = _PackedConv(blk.downsample[0], blk.downsample[1], device) if blk.downsample is not None else None
                self.blocks.append((convs, down))
        self.fc_w = model.fc.weight.detach().to(device, torch.bfloat16).contiguous()
        self.fc_b = model.fc.bias.detach().to(device, torch.float32) if model.fc.bias is not None else None

    def _to_nhwc(self, x):
        n, c, h, w = x.shape
        cp = self.stem.cin_padded
        out = torch.zeros(n, h, w, cp, device=self.device, dtype=torch.bfloat16)
        out[..., :c] = x.to(self.device).permute(0, 2, 3, 1)
        return out

    def __call__(self, x):
        if self._runner is not None and torch.is_tensor(x) and x.is_cuda:
            return self._runner(x)
        return self._forward(x)

    @torch.no_grad()
    def _forward(self, x):
        x = self.stem(self._to_nhwc(x), relu=True)
        if self.pool:
            x = F.max_pool2d(x.permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1).contiguous()
        for convs, down in self.blocks:
            identity = x if down is None else down(x, relu=False)
            y = x
            for conv in convs[:-1]:
                y = conv(y, relu=True)
            x = convs[-1](y, relu=True, residual=identity)  # bias + shortcut + ReLU in the GEMM epilogue
        pooled = x.float().mean(dim=(1, 2))
        if pooled.is_cuda and pooled.shape[0] >= 64 and self.fc_w.shape[0] >= 128 and self.fc_w.shape[0] % 8 == 0:
            from ..ops.gemm import matmul_nt

            logits = matmul_nt(pooled.to(torch.bfloat16), self.fc_w).float()
        else:  # a handful of rows: not worth a tensor-core launch
            logits = pooled @ self.fc_w.float().t()
        return logits + self.fc_b if self.fc_b is not None else logits


# ------------------------------------------------------------------ VGG
_VGG_CFG = {
    11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    13: [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
    19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"],
}


class VGG(Module):
    """VGG with batch norm; ``Conv2d -> BatchNorm2d -> ReLU`` runs sit in one ``Sequential`` so that
    :func:`ghost_flow_b200.nn.fused_conv.fuse_conv_bn_relu` folds them for inference."""

    def __init__(self, depth: int = 16, num_classes: int = 1000, in_channels: int = 3, hidden: int = 4096,
                 pool_size: int = 7, dropout: float = 0.5):
        super().__init__()
        layers, c = [], in_channels
        for v in _VGG_CFG[depth]:
            if v == "M":
                layers.append(MaxPool2d(2, 2))
            else:
                layers += [Conv2d(c, v, 3, 1, 1), BatchNorm2d(v), ReLU()]
                c = v
        self.features = Sequential(layers)
        self.avgpool = AdaptiveAvgPool2d(pool_size)
        self.classifier = Sequential(Linear(c * pool_size * pool_size, hidden), ReLU(), Dropout(dropout),
                                     Linear(hidden, hidden), ReLU(), Dropout(dropout), Linear(hidden, num_classes))

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)).flatten(1))


def vgg11(num_classes=1000, **kw): return VGG(11, num_classes, **kw)
def vgg16(num_classes=1000, **kw): return VGG(16, num_classes, **kw)
def vgg19(num_classes=1000, **kw): return VGG(19, num_classes, **kw)


# ------------------------------------------------------------------ MobileNetV2
class InvertedResidual(Module):
    def __init__(self, cin: int, cout: int, stride: int, expand: int):
        super().__init__()
        hid = cin * expand
        self.use_res = stride == 1 and cin == cout
        layers = []
        if expand != 1:
            layers += [Conv2d(cin, hid, 1, 1, 0, bias=False), BatchNorm2d(hid), _ReLU6()]
        layers += [Conv2d(hid, hid, 3, stride, 1, groups=hid, bias=False), BatchNorm2d(hid), _ReLU6(),
                   Conv2d(hid, cout, 1, 1, 0, bias=False), BatchNorm2d(cout)]
        self.conv = torch.nn.Sequential(*layers)

    def forward(self, x):
        return x + self.conv(x) if self.use_res else self.conv(x)


class _ReLU6(Module):
    def forward(self, x):
        return torch.clamp(x, 0.0, 6.0)


class MobileNetV2(Module):
    _CFG = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, num_classes: int = 1000, width_mult: float = 1.0, in_channels: int = 3):
        super().__init__()
        c = int(32 * width_mult)
        layers = [Conv2d(in_channels, c, 3, 2, 1, bias=False), BatchNorm2d(c), _ReLU6()]
        for t, ch, n, s in self._CFG:
            out = int(ch * width_mult)
            for i in range(n):
                layers.append(InvertedResidual(c, out, s if i == 0 else 1, t))
                c = out
        last = int(1280 * max(1.0, width_mult))
        layers += [Conv2d(c, last, 1, 1, 0, bias=False), BatchNorm2d(last), _ReLU6()]
        self.features = torch.nn.Sequential(*layers)
        self.classifier = Sequential(Dropout(0.2), Linear(last, num_classes))

    def forward(self, x):
        return self.classifier(self.features(x).mean(dim=(2, 3)))
