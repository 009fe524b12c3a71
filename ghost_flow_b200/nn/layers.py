"""Core layers: Linear, embeddings, dropout, activations, norms.

bf16 CUDA inputs run the hand-written kernels (tcgen05 GEMM with fused bias, LayerNorm / RMSNorm, GELU /
SiLU ...); CPU and other dtypes use PyTorch ops with the same formulas.

Reference: ghostflow-nn/src/linear.rs:23-69 (init U(+-sqrt(6/fan_in)), bias U(+-1/sqrt(fan_in))),
embedding.rs:16-185, dropout.rs:26-115, activation.rs:7-315, norm.rs:39-442, llama.rs:154-185 (RMSNorm).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .. import ops
from . import init
from .module import Module, Parameter


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype or torch.float32))
        self.bias = Parameter(torch.empty(out_features, device=device, dtype=dtype or torch.float32)) if bias else None
        self.reset_parameters()

    @classmethod
    def with_bias(cls, in_features, out_features, bias: bool):
        return cls(in_features, out_features, bias)

    def reset_parameters(self):
        init.kaiming_uniform(self.weight.data)
        if self.bias is not None:
            b = 1.0 / math.sqrt(self.in_features)
            self.bias.data.uniform_(-b, b)

    def forward(self, x, residual=None):
        return ops.linear(x, self.weight, self.bias, residual)

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class Embedding(Module):
    """Lookup table, N(0,1) init; ids may be integer or float tensors (the reference stores ids as f32),
    out-of-range ids give zero rows (ghostflow-nn/src/embedding.rs:85-127)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None, device=None,
                 dtype=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = Parameter(torch.randn(num_embeddings, embedding_dim, device=device, dtype=dtype or torch.float32))
        if padding_idx is not None:
            with torch.no_grad():
                self.weight[padding_idx].zero_()

    @classmethod
    def with_padding(cls, n, d, padding_idx):
        return cls(n, d, padding_idx)

    @classmethod
    def from_pretrained(cls, weight, freeze: bool = True):
        w = weight.data if hasattr(weight, "data") and not isinstance(weight, torch.Tensor) else weight
        m = cls(w.shape[0], w.shape[1])
        m.weight = Parameter(w.clone(), requires_grad=not freeze)
        return m

    def forward(self, ids):
        idx = ids.long() if ids.is_floating_point() else ids
        oob = (idx < 0) | (idx >= self.num_embeddings)
        out = F.embedding(idx.clamp(0, self.num_embeddings - 1), self.weight, self.padding_idx)
        # applied unconditionally: asking the device whether any id is out of range would stall the host on every
        # call and cannot be captured in a CUDA graph
        return out.masked_fill_(oob.unsqueeze(-1), 0.0)

    forward_indices = forward


class TokenPositionEmbedding(Module):
    """Token embedding + learned positional embedding (+ dropout) (ghostflow-nn/src/embedding.rs:130-185)."""

    def __init__(self, vocab_size, max_len, dim, dropout: float = 0.0):
        super().__init__()
        self.tok = Embedding(vocab_size, dim)
        self.pos = Embedding(max_len, dim)
        self.drop = Dropout(dropout)

    def forward(self, ids, start_pos: int = 0):
        S = ids.shape[-1]
        pos = torch.arange(start_pos, start_pos + S, device=ids.device)
        return self.drop(self.tok(ids) + self.pos(pos))


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return F.dropout(x, self.p, self.training)


class Dropout2d(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return F.dropout2d(x, self.p, self.training)


# ----------------------------------------------------------------------------- activations
class _Act(Module):
    name = "relu"

    def forward(self, x):
        return ops.unary(x, self.name)


class ReLU(_Act):
    name = "relu"


class GELU(_Act):
    """tanh-form GELU (ghostflow-core/src/ops/activation.rs:101-112)."""
    name = "gelu"


class Sigmoid(_Act):
    name = "sigmoid"


class Tanh(_Act):
    name = "tanh"


class SiLU(_Act):
    name = "silu"


class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.negative_slope = negative_slope

    def forward(self, x):
        return F.leaky_relu(x, self.negative_slope)


class Softmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return torch.softmax(x, self.dim)


class LogSoftmax(Module):
    def __init__(self, dim: int = -1):
        super().__init__()
        self.dim = dim

    def forward(self, x):
        return torch.log_softmax(x, self.dim)


class Swish(Module):
    def __init__(self, beta: float = 1.0):
        super().__init__()
        self.beta = beta

    def forward(self, x):
        return x * torch.sigmoid(self.beta * x)


class Mish(Module):
    def forward(self, x):
        return F.mish(x)


class ELU(Module):
    def __init__(self, alpha: float = 1.0):
        super().__init__()
        self.alpha = alpha

    def forward(self, x):
        return F.elu(x, self.alpha)


class SELU(Module):
    def forward(self, x):
        return torch.selu(x)


class Softplus(Module):
    def __init__(self, beta: float = 1.0, threshold: float = 20.0):
        super().__init__()
        self.beta, self.threshold = beta, threshold

    def forward(self, x):
        return F.softplus(x, self.beta, self.threshold)


# ----------------------------------------------------------------------------- norms
class LayerNorm(Module):
    """Biased variance, eps 1e-5 (ghostflow-nn/src/norm.rs:222-270)."""

    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True, bias: bool = True,
                 device=None, dtype=None):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        kw = dict(device=device, dtype=dtype or torch.float32)
        self.weight = Parameter(torch.ones(self.normalized_shape, **kw)) if elementwise_affine else None
        self.bias = Parameter(torch.zeros(self.normalized_shape, **kw)) if elementwise_affine and bias else None

    @classmethod
    def with_eps(cls, shape, eps):
        return cls(shape, eps)

    def forward(self, x):
        if len(self.normalized_shape) == 1 and self.weight is not None:
            return ops.layer_norm(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)


class RMSNorm(Module):
    """``x / sqrt(mean(x^2) + eps) * w`` (ghostflow-nn/src/llama.rs:154-185)."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(torch.ones(dim, device=device, dtype=dtype or torch.float32))

    def forward(self, x, residual=None):
        return ops.rms_norm(x, self.weight, self.eps, residual)


class _BatchNorm(Module):
    """Batch norm that updates its running statistics in training (the reference never does:
    ghostflow-nn/src/norm.rs:50-79) and uses them in eval."""
    _dims = (2, 3)

    def __init__(self, num_features, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.weight = Parameter(torch.ones(num_features)) if affine else None
        self.bias = Parameter(torch.zeros(num_features)) if affine else None
        self.register_buffer("running_mean", torch.zeros(num_features))
        self.register_buffer("running_var", torch.ones(num_features))
        self.register_buffer("num_batches_tracked", torch.tensor(0, dtype=torch.long))

    def forward(self, x):
        if self.training:
            self.num_batches_tracked += 1
        return F.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training,
                            self.momentum, self.eps)


class BatchNorm1d(_BatchNorm):
    pass


class BatchNorm2d(_BatchNorm):
    pass


class _SyncBNFn(torch.autograd.Function):
    """Batch norm whose statistics are taken over the batches of every rank: one all-reduce of
    ``[sum, sum of squares, count]`` in forward and one of ``[sum dy, sum dy * xhat]`` in backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, eps, momentum, group):
        import torch.distributed as dist

        C = x.shape[1]
        dims = [0] + list(range(2, x.dim()))
        xf = x.float()
        stats = torch.cat([xf.sum(dims), (xf * xf).sum(dims), torch.full((1,), float(x.numel() // C), device=x.device)])
        dist.all_reduce(stats, group=group)
        n = stats[-1]
        mean = stats[:C] / n
        var = (stats[C:2 * C] / n - mean * mean).clamp_min_(0.0)
        rstd = torch.rsqrt(var + eps)
        shape = [1, C] + [1] * (x.dim() - 2)
        xhat = (xf - mean.view(shape)) * rstd.view(shape)
        if running_mean is not None:
            with torch.no_grad():
                running_mean.mul_(1 - momentum).add_(mean, alpha=momentum)
                running_var.mul_(1 - momentum).add_(var * (n / (n - 1).clamp_min(1.0)), alpha=momentum)
        y = xhat * weight.float().view(shape) + bias.float().view(shape) if weight is not None else xhat
        ctx.save_for_backward(xhat, weight, rstd)
        ctx.group, ctx.n, ctx.dims, ctx.shape = group, n, dims, shape
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        import torch.distributed as dist

        xhat, weight, rstd = ctx.saved_tensors
        dyf = dy.float()
        C = xhat.shape[1]
        dw = (dyf * xhat).sum(ctx.dims)
        db = dyf.sum(ctx.dims)
        red = torch.cat([db, dw])
        dist.all_reduce(red, group=ctx.group)
        g = dyf * weight.float().view(ctx.shape) if weight is not None else dyf
        sum_g, sum_gx = red[:C], red[C:]
        if weight is not None:
            sum_g, sum_gx = sum_g * weight.float(), sum_gx * weight.float()
        dx = (g - sum_g.view(ctx.shape) / ctx.n - xhat * sum_gx.view(ctx.shape) / ctx.n) * rstd.view(ctx.shape)
        return (dx.to(dy.dtype), dw.to(weight.dtype) if weight is not None else None,
                db.to(weight.dtype) if weight is not None else None, None, None, None, None, None)


class SyncBatchNorm(_BatchNorm):
    """Batch norm over the global batch of a data-parallel group (the reference's BatchNorm neither synchronises
    nor updates running statistics: ghostflow-nn/src/norm.rs:50-79). Without an initialised process group, or in
    eval mode, it is the plain layer. ``SyncBatchNorm.convert(model)`` swaps every BatchNorm1d/2d of a model."""

    def __init__(self, num_features, eps: float = 1e-5, momentum: float = 0.1, affine: bool = True, group=None):
        super().__init__(num_features, eps, momentum, affine)
        self.group = group

    def forward(self, x):
        import torch.distributed as dist

        if not (self.training and dist.is_available() and dist.is_initialized()
                and dist.get_world_size(self.group) > 1):
            return super().forward(x)
        self.num_batches_tracked += 1
        return _SyncBNFn.apply(x, self.weight, self.bias, self.running_mean, self.running_var, self.eps,
                               self.momentum, self.group)

    @classmethod
    def convert(cls, module: torch.nn.Module, group=None) -> torch.nn.Module:
        for name, child in list(module.named_children()):
            if isinstance(child, _BatchNorm) and not isinstance(child, cls):
                new = cls(child.num_features, child.eps, child.momentum, child.weight is not None, group)
                new.load_state_dict(child.state_dict())
                new.to(child.running_mean.device)
                if isinstance(module, (torch.nn.ModuleList, torch.nn.Sequential)) and name.isdigit():
                    module[int(name)] = new
                else:
                    setattr(module, name, new)
            else:
                cls.convert(child, group)
        return module


class GroupNorm(Module):
    def __init__(self, num_groups, num_channels, eps: float = 1e-5, affine: bool = True):
        super().__init__()
        self.num_groups, self.num_channels, self.eps = num_groups, num_channels, eps
        self.weight = Parameter(torch.ones(num_channels)) if affine else None
        self.bias = Parameter(torch.zeros(num_channels)) if affine else None

    def forward(self, x):
        return F.group_norm(x, self.num_groups, self.weight, self.bias, self.eps)


class InstanceNorm(Module):
    def __init__(self, num_features, eps: float = 1e-5, affine: bool = False):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(torch.ones(num_features)) if affine else None
        self.bias = Parameter(torch.zeros(num_features)) if affine else None

    def forward(self, x):
        return F.instance_norm(x, weight=self.weight, bias=self.bias, eps=self.eps)


InstanceNorm2d = InstanceNorm


class SwiGLU(Module):
    """``down(silu(gate(x)) * up(x))`` with gate and up fused into one projection
    (ghostflow-nn/src/llama.rs:266-286)."""

    def __init__(self, dim: int, hidden: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.gate_up = Linear(dim, 2 * hidden, bias, device, dtype)
        self.down = Linear(hidden, dim, bias, device, dtype)

    def forward(self, x, residual=None):
        return self.down(ops.swiglu(self.gate_up(x)), residual)
