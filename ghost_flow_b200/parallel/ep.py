"""Expert-parallel mixture of experts: router, all-to-all dispatch/combine over peer memory, grouped expert GEMMs.

The reference routes token by token on the CPU and runs every expert in one process
(ghostflow-nn/src/mixture_of_experts.rs:152-177 router, :212-274 dispatch loop, :289-323 load-balance loss).
Here ``num_experts`` SwiGLU experts are sharded over the ranks of one NVSwitch box. One forward is

    logits = x Wg^T -> route (softmax, top-k, renormalise) -> publish histogram -> plan segments
    -> dispatch token rows into the owner ranks' buffers (peer stores) -> grouped GEMM W13 (waits per tile for the
    source ranks it reads) -> SwiGLU -> grouped GEMM W2 whose epilogue stores every output row straight into the
    token's home rank -> weighted sum per token

and the backward runs the same machinery in reverse (the gradient of the combine is a dispatch, the gradient of
the dispatch is a combine) plus grouped weight-gradient GEMMs that contract over each expert's row segment.
With ``world == 1`` the same kernels run on plain local buffers. ``forward``/``backward`` are explicit (no autograd
graph), ``ExpertParallelMoE.apply`` wraps them in a ``torch.autograd.Function`` for use inside torch models.
On CPU tensors a dense PyTorch restatement is used (the test oracle).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _lib, raw

_BOUND = False


def _bind():
    global _BOUND
    lib = _lib.cuda_lib()
    if not _BOUND:
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.gf_moe_route.argtypes = [P, I, I, I, I, I, P, P, P, P, P]
        lib.gf_moe_publish.argtypes = [P, P, P, I, I, I, I, I, P]
        lib.gf_moe_plan.argtypes = [P, P, I, I, I, I, I, I, P, P, P, P, P, P]
        lib.gf_moe_dispatch.argtypes = [P, L, P, P, I, I, I, I, I, I, I, P, P, P, I, P, P, P, I, I, P, P]
        lib.gf_moe_zero_pad.argtypes = [P, I, P, P, P, I, I, I, P]
        lib.gf_moe_combine.argtypes = [P, P, P, P, I, I, I, P, I, I, I, P, P, P, P]
        lib.gf_gemm_bf16_grouped.argtypes = [P, P, P, I, I, I, I, I, L, I, L, L, I, I, F, P, P, I,
                                             P, P, I, I, P, P, P, L, I, I, P, P]
        for n in ("gf_moe_route", "gf_moe_publish", "gf_moe_plan", "gf_moe_dispatch", "gf_moe_zero_pad",
                  "gf_moe_combine", "gf_gemm_bf16_grouped"):
            getattr(lib, n).restype = I
        _BOUND = True
    return lib


def _u64(vals):
    return (ctypes.c_ulonglong * len(vals))(*[int(v) for v in vals])


def _ptr(t):
    return t.data_ptr() if t is not None else None


FLAG_COUNTS, FLAG_DISPATCH, FLAG_COMBINE = 0, 1, 2


def grouped_gemm(a, b, out, mode, offsets, experts, *, rows_cap, M=0, N, K, b_mn=False, out_fp32=False,
                 accumulate=False, wait=None, scatter=None):
    """Thin wrapper over ``gf_gemm_bf16_grouped`` (see the comment above that function for the two modes).

    ``wait = (src_start, arrived, world, epoch)`` makes every tile wait for the source ranks of its rows;
    ``scatter = (ret, dst_ptrs, flag_ptrs, ld, rank, world, epoch, counter)`` sends the output rows home."""
    lib = _bind()
    dev = a.device
    ws = wait or (None, None, 1, 0)
    world = ws[2]
    sc = scatter
    rc = lib.gf_gemm_bf16_grouped(
        a.data_ptr(), b.data_ptr(), _ptr(out), mode, rows_cap, M, N, K, a.stride(0),
        1 if b_mn else 0, b.stride(-2), out.stride(-2) if out is not None else 0, 1 if out_fp32 else 0,
        1 if accumulate else 0, 1.0, _lib.status_word(dev).data_ptr(), offsets.data_ptr(), experts,
        _ptr(ws[0]), _ptr(ws[1]), sc[5] if sc else world, ws[3],
        _ptr(sc[0]) if sc else None, sc[1] if sc else None, sc[2] if sc else None, sc[3] if sc else 0,
        sc[4] if sc else 0, sc[6] if sc else 0, _ptr(sc[7]) if sc else None, _lib.stream_ptr())
    _lib.check_rc(rc, "gf_gemm_bf16_grouped")
    return out


@dataclass
class MoEContext:
    """What one forward leaves behind for its backward."""
    x: torch.Tensor
    idx: torch.Tensor
    w: torch.Tensor
    probs: torch.Tensor
    dest_row: torch.Tensor
    seg_offsets: torch.Tensor
    src_start: torch.Tensor
    h: torch.Tensor
    a: torch.Tensor
    # copies of the workspaces the backward pass reads, taken when the layer object is shared between layers:
    comb: torch.Tensor = None     # per-slot expert outputs [T * k, d]
    xs: torch.Tensor = None       # the rows this rank's experts received [rows_cap, d]
    ret: torch.Tensor = None      # their return addresses (source rank, slot) [rows_cap, 2]


class ExpertParallelMoE:
    """SwiGLU experts sharded over ``group`` (``num_experts % world == 0``), top-``k`` softmax routing with
    renormalised weights (the Mixtral recipe).

    Parameters (bf16): ``gate [E, d]``, ``w13 [E_local, 2 * d_ff, d]`` (gate rows then up rows), ``w2 [E_local, d, d_ff]``.
    ``tokens`` is the number of tokens per rank and call; ``capacity_factor`` bounds the rows a rank accepts:
    ``rows_cap = capacity_factor * tokens * k`` (+ padding); the default ``world`` is the drop-free worst case. If more rows
    arrive than fit the owner's kernel records status 8 and :func:`ghost_flow_b200.ops._lib.check_status` raises.
    """

    def __init__(self, d_model, d_ff, num_experts, k, tokens, device, group=None, capacity_factor=None, seed=0,
                 init_weights: bool = True):
        self.group = group
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        assert num_experts % self.world == 0 and d_model % 8 == 0 and d_ff % 8 == 0
        self.d, self.f, self.E, self.k, self.T = d_model, d_ff, num_experts, k, tokens
        self.el = num_experts // self.world
        self.device = torch.device(device)
        cf = float(capacity_factor if capacity_factor is not None else self.world)
        self.rows_cap = (int(cf * tokens * k) + self.el * 128 + 127) // 128 * 128
        g = torch.Generator(device="cpu").manual_seed(seed)
        bf = torch.bfloat16

        def init(*shape, std):
            return (torch.randn(*shape, generator=g) * std).to(bf).to(self.device)

        # the router weight is stored padded to a multiple of 128 rows (zeros) so that the router GEMMs have
        # tile-sized extents; ``gate`` and its gradient are views of the first ``num_experts`` rows
        ep_rows = (num_experts + 127) // 128 * 128
        self.gate_pad = torch.zeros(ep_rows, d_model, dtype=bf, device=self.device)
        self.gate = self.gate_pad[:num_experts]
        self.gate_grad_pad = torch.zeros_like(self.gate_pad)
        if init_weights:
            self.gate_pad[:num_experts] = init(num_experts, d_model, std=0.02)
            all13 = init(num_experts, 2 * d_ff, d_model, std=0.02)
            all2 = init(num_experts, d_model, d_ff, std=0.02)
            lo, hi = self.rank * self.el, (self.rank + 1) * self.el
            self.w13, self.w2 = all13[lo:hi].contiguous(), all2[lo:hi].contiguous()
            self.grads = {"gate": self.gate_grad_pad[:num_experts], "w13": torch.zeros_like(self.w13),
                          "w2": torch.zeros_like(self.w2)}
        else:
            # a workspace without parameters of its own: the owner points it at a layer with set_weights
            self.w13 = self.w2 = None
            self.grads = {}
        self.epoch = 0
        self.last_counts = None
        # One instance can serve every MoE layer of a model (its buffers are workspaces; the weights are swapped
        # with set_weights): then the per-slot outputs, which the backward pass needs, must be copied out of the
        # workspace into the layer's context.
        self.keep_slot_outputs = False
        self.aux_coef = 0.0
        # backward adds into ``grads`` (several micro-batches per step) unless this is False: then it overwrites them,
        # which saves zeroing and re-reading 1.4 GB of expert gradients per Mixtral-sized layer
        self.accumulate_grads = True
        if self.device.type == "cuda":
            self._alloc()

    def set_weights(self, gate_pad, w13, w2, gate_grad_pad, g13, g2):
        """Points the layer at another set of parameters and gradient buffers (same shapes)."""
        self.gate_pad, self.gate = gate_pad, gate_pad[:self.E]
        self.w13, self.w2 = w13, w2
        self.gate_grad_pad = gate_grad_pad
        self.grads = {"gate": gate_grad_pad[:self.E], "w13": g13, "w2": g2}

    # ------------------------------------------------------------------ buffers
    def _alloc(self):
        R, d, T, k, E, W = self.rows_cap, self.d, self.T, self.k, self.E, self.world
        sizes = {"xs": R * d * 2, "dys": R * d * 2, "ret": R * 8, "comb": T * k * d * 2, "dcomb": T * k * d * 2,
                 "table": W * E * 4, "flags": 4 * 8 * 4}
        total = sum((v + 255) // 256 * 256 for v in sizes.values()) + 4096
        if W > 1:
            from .tp import SymmetricWorkspace
            self.ws = SymmetricWorkspace(total, self.device, self.group or dist.group.WORLD)
            alloc, peers = self.ws.alloc, self.ws.peer_ptrs
        else:
            from .canary import SLACK_BYTES, CanaryLedger

            buf = torch.zeros(total + SLACK_BYTES, dtype=torch.uint8, device=self.device)
            self._buf = buf
            self.canaries = CanaryLedger(buf, "expert-parallel workspace")
            off = [self.canaries.plant(0, "start of the workspace")]

            def alloc(numel, dtype):
                esz = torch.empty((), dtype=dtype).element_size()
                t = buf[off[0]:off[0] + numel * esz].view(dtype)
                off[0] = self.canaries.plant(off[0] + (numel * esz + 255) // 256 * 256,
                                             f"carve-out {len(self.canaries.blocks)}")
                return t

            def peers(t):
                return [t.data_ptr()]
        bf, i32 = torch.bfloat16, torch.int32
        self.xs = alloc(R * d, bf).view(R, d)
        self.dys = alloc(R * d, bf).view(R, d)
        self.ret = alloc(R * 2, i32).view(R, 2)
        self.comb = alloc(T * k * d, bf).view(T * k, d)
        self.dcomb = alloc(T * k * d, bf).view(T * k, d)
        self.table = alloc(W * E, i32).view(W, E)
        self.flags = alloc(32, i32)
        self.p = {n: _u64(peers(getattr(self, n))) for n in ("xs", "dys", "ret", "comb", "dcomb", "table", "flags")}
        dev = self.device
        self.counts = torch.zeros(E, dtype=i32, device=dev)
        self.send_base = torch.zeros(E, dtype=i32, device=dev)
        self.cursor = torch.zeros(E, dtype=i32, device=dev)
        self.done = torch.zeros(4, dtype=i32, device=dev)

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, residual=None):
        """x [T, d] bf16 -> (y [T, d], ctx)."""
        if x.device.type != "cuda":
            return self._forward_ref(x, residual)
        lib, st = _bind(), _lib.stream_ptr
        T, k, d, f, E, W, R = self.T, self.k, self.d, self.f, self.E, self.world, self.rows_cap
        assert x.shape == (T, d) and x.dtype == torch.bfloat16 and x.is_contiguous()
        dev, status = self.device, _lib.status_word(self.device).data_ptr()
        logits = raw.gemm(x, False, self.gate_pad, True, out_dtype=torch.float32)[:, :E].contiguous()
        idx = torch.empty(T, k, dtype=torch.int32, device=dev)
        w = torch.empty(T, k, dtype=torch.float32, device=dev)
        probs = torch.empty(T, E, dtype=torch.float32, device=dev)
        self.counts.zero_()
        _lib.check_rc(lib.gf_moe_route(logits.data_ptr(), 1, T, E, k, 1, idx.data_ptr(), w.data_ptr(), probs.data_ptr(),
                                       self.counts.data_ptr(), st()), "gf_moe_route")
        self.epoch += 1
        ep = self.epoch
        _lib.check_rc(lib.gf_moe_publish(self.p["table"], self.p["flags"], self.counts.data_ptr(), E, W, self.rank,
                                         FLAG_COUNTS, ep, st()), "gf_moe_publish")
        seg = torch.empty(self.el + 1, dtype=torch.int32, device=dev)
        src_start = torch.empty(self.el, W + 1, dtype=torch.int32, device=dev)
        _lib.check_rc(lib.gf_moe_plan(self.table.data_ptr(), self.flags.data_ptr(), FLAG_COUNTS, ep, E, W, self.rank, R,
                                      seg.data_ptr(), src_start.data_ptr(), self.send_base.data_ptr(),
                                      self.cursor.data_ptr(), status, st()), "gf_moe_plan")
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        _lib.check_rc(lib.gf_moe_dispatch(x.data_ptr(), x.stride(0), idx.data_ptr(), None, T, k, d, E, W, self.rank, R,
                                          self.send_base.data_ptr(), self.cursor.data_ptr(), dest_row.data_ptr(), 0,
                                          self.p["xs"], self.p["ret"], self.p["flags"], FLAG_DISPATCH, ep,
                                          self.done.data_ptr(), st()), "gf_moe_dispatch")
        _lib.check_rc(lib.gf_moe_zero_pad(self.xs.data_ptr(), d, self.ret.data_ptr(), seg.data_ptr(),
                                          src_start.data_ptr(), self.el, W, R, st()), "gf_moe_zero_pad")
        h = torch.empty(R, 2 * f, dtype=torch.bfloat16, device=dev)
        grouped_gemm(self.xs, self.w13, h, 1, seg, self.el, rows_cap=R, N=2 * f, K=d,
                     wait=(src_start, self.flags[FLAG_DISPATCH * 8:], W, ep))
        # Copies for a backward pass that runs after other layers reused the workspace. They are taken here, before
        # the second GEMM: a peer starts its next dispatch into xs / ret only after its combine, which waits for this
        # rank's second GEMM, so everything submitted before that GEMM reads the rows of this call.
        keep_in = (self.xs.clone(), self.ret.clone()) if self.keep_slot_outputs else (None, None)
        a = raw.swiglu_fwd(h)
        grouped_gemm(a, self.w2, self.comb, 1, seg, self.el, rows_cap=R, N=d, K=f,
                     scatter=(self.ret, self.p["comb"], self._flag_ptrs(FLAG_COMBINE), d, self.rank, W, ep,
                              self.done[1:]))
        y = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
        _lib.check_rc(lib.gf_moe_combine(self.comb.data_ptr(), w.data_ptr(), _ptr(residual), y.data_ptr(), T, k, d,
                                         self.flags.data_ptr(), FLAG_COMBINE, ep, W, None, None, status, st()),
                      "gf_moe_combine")
        self.last_counts = self.counts.clone()
        # comb is written by the peers' second GEMM of a call, which needs this rank's dispatch of that call: later
        keep_out = self.comb.clone() if self.keep_slot_outputs else None
        return y, MoEContext(x, idx, w, probs, dest_row, seg, src_start, h, a, keep_out, *keep_in)

    def _flag_ptrs(self, row):
        """Every rank's flag row ``row`` (the kernels index it by source rank)."""
        return _u64([int(v) + row * 8 * 4 for v in self.p["flags"]])

    # ------------------------------------------------------------------ backward
    def backward(self, ctx: MoEContext, dy: torch.Tensor):
        """Accumulates into ``self.grads`` and returns dx [T, d] (without the residual branch)."""
        if dy.device.type != "cuda":
            return self._backward_ref(ctx, dy)
        lib, st = _bind(), _lib.stream_ptr
        T, k, d, f, E, W, R = self.T, self.k, self.d, self.f, self.E, self.world, self.rows_cap
        dev, status = self.device, _lib.status_word(self.device).data_ptr()
        seg, src_start = ctx.seg_offsets, ctx.src_start
        dy = dy.contiguous()
        # d(weights): <dy[t], expert output of slot s>; the per-slot outputs are still in comb
        dots = torch.empty(T, k, dtype=torch.float32, device=dev)
        comb = ctx.comb if ctx.comb is not None else self.comb
        xs = ctx.xs if ctx.xs is not None else self.xs
        ret = ctx.ret if ctx.ret is not None else self.ret
        _lib.check_rc(lib.gf_moe_combine(comb.data_ptr(), None, None, None, T, k, d, None, 0, 0, W, dy.data_ptr(),
                                         dots.data_ptr(), status, st()), "gf_moe_combine(dots)")
        # gradient of the combine = dispatch of w * dy to the forward rows
        self.epoch += 1
        ep = self.epoch
        _lib.check_rc(lib.gf_moe_dispatch(dy.data_ptr(), dy.stride(0), ctx.idx.data_ptr(), ctx.w.data_ptr(), T, k, d, E, W,
                                          self.rank, R, self.send_base.data_ptr(), self.cursor.data_ptr(),
                                          ctx.dest_row.data_ptr(), 1, self.p["dys"], self.p["ret"], self.p["flags"],
                                          FLAG_DISPATCH, ep, self.done.data_ptr(), st()), "gf_moe_dispatch(bwd)")
        _lib.check_rc(lib.gf_moe_zero_pad(self.dys.data_ptr(), d, None, seg.data_ptr(), src_start.data_ptr(), self.el, W,
                                          R, st()), "gf_moe_zero_pad")
        wait = (src_start, self.flags[FLAG_DISPATCH * 8:], W, ep)
        da = torch.empty(R, f, dtype=torch.bfloat16, device=dev)
        grouped_gemm(self.dys, self.w2, da, 1, seg, self.el, rows_cap=R, N=f, K=d, b_mn=True, wait=wait)
        acc = self.accumulate_grads
        grouped_gemm(self.dys, ctx.a, self.grads["w2"], 2, seg, self.el, rows_cap=R, M=d, N=f, K=R, accumulate=acc)
        dh = raw.swiglu_bwd(ctx.h, da)
        # padding rows of h are zero, so dh is zero there as well and the weight gradient ignores them
        grouped_gemm(dh, xs, self.grads["w13"], 2, seg, self.el, rows_cap=R, M=2 * f, N=d, K=R, accumulate=acc)
        grouped_gemm(dh, self.w13, self.dcomb, 1, seg, self.el, rows_cap=R, N=d, K=2 * f, b_mn=True,
                     scatter=(ret, self.p["dcomb"], self._flag_ptrs(FLAG_COMBINE), d, self.rank, W, ep,
                              self.done[1:]))
        dx = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
        _lib.check_rc(lib.gf_moe_combine(self.dcomb.data_ptr(), None, None, dx.data_ptr(), T, k, d,
                                         self.flags.data_ptr(), FLAG_COMBINE, ep, W, None, None, status, st()),
                      "gf_moe_combine(dx)")
        # router: weights -> probabilities -> logits (small [T, E] tensors)
        dlogits = self._router_backward(ctx, dots, self.aux_coef, self.E)
        dl = torch.zeros(T, self.gate_pad.shape[0], dtype=torch.bfloat16, device=dev)
        dl[:, :E] = dlogits
        raw.gemm(dl, False, self.gate_pad, False, out=dx, accumulate=True)
        raw.gemm(dl, True, ctx.x, False, out=self.gate_grad_pad, accumulate=acc)
        return dx

    @staticmethod
    def _router_backward(ctx: MoEContext, dw: torch.Tensor, aux_coef: float = 0.0, E: int = 0) -> torch.Tensor:
        """Gradient of the routing weights (and, with ``aux_coef``, of ``aux_coef * aux_loss``) w.r.t. the router
        logits. The load-balance loss ``E * sum_e f_e * P_e`` is differentiated through the mean probabilities
        ``P_e`` only; the token fractions ``f_e`` are counts."""
        p = ctx.probs
        idx = ctx.idx.long()
        psel = p.gather(1, idx)
        s = psel.sum(1, keepdim=True)
        wn = psel / s
        dpsel = (dw - (dw * wn).sum(1, keepdim=True)) / s
        dp = torch.zeros_like(p).scatter_(1, idx, dpsel)
        if aux_coef:
            frac = torch.bincount(idx.flatten(), minlength=E).float() / idx.numel()
            dp = dp + (aux_coef * E / p.shape[0]) * frac[None, :]
        return p * (dp - (dp * p).sum(1, keepdim=True))

    # ------------------------------------------------------------------ statistics / auxiliary loss
    def expert_counts(self) -> torch.Tensor:
        """Tokens routed to every expert by this rank in the last forward."""
        return self.last_counts

    def aux_loss(self, ctx: MoEContext) -> torch.Tensor:
        """Switch-style load-balance loss ``E * sum_e f_e * P_e``."""
        frac = torch.bincount(ctx.idx.flatten().long(), minlength=self.E).float() / ctx.idx.numel()
        return self.E * (frac * ctx.probs.mean(0)).sum()

    # ------------------------------------------------------------------ CPU / oracle path
    def full_weights(self):
        """All experts' weights on every rank (for the dense oracle); all-gathers when sharded."""
        if self.world == 1:
            return self.w13, self.w2
        w13 = torch.empty(self.E, 2 * self.f, self.d, dtype=self.w13.dtype, device=self.w13.device)
        w2 = torch.empty(self.E, self.d, self.f, dtype=self.w2.dtype, device=self.w2.device)
        dist.all_gather_into_tensor(w13, self.w13, group=self.group)
        dist.all_gather_into_tensor(w2, self.w2, group=self.group)
        return w13, w2

    def dense_reference(self, x, w13=None, w2=None, residual=None, gate=None):
        """fp32 PyTorch restatement: every token through its top-k experts, differentiable."""
        w13 = self.w13 if w13 is None else w13
        w2 = self.w2 if w2 is None else w2
        gate = self.gate if gate is None else gate
        xf = x.float()
        probs = torch.softmax(xf @ gate.float().t(), -1)
        top, idx = probs.topk(self.k, -1)
        wts = top / top.sum(-1, keepdim=True)
        y = torch.zeros_like(xf)
        for e in range(w13.shape[0]):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            hh = xf[tok] @ w13[e].float().t()
            g, u = hh.chunk(2, -1)
            out = (torch.nn.functional.silu(g) * u) @ w2[e].float().t()
            y.index_add_(0, tok, out * wts[tok, slot, None])
        if residual is not None:
            y = y + residual.float()
        return y

    def _forward_ref(self, x, residual):
        """CPU path. One rank: the dense oracle under autograd. Several ranks (gloo): tokens are all-gathered, every
        rank runs ITS experts over the tokens of all ranks that were routed to them, and the partial outputs are
        summed back to the tokens' owners: the same mathematics as the dispatch / combine kernels, written with
        collectives."""
        xr = x.detach().clone().requires_grad_(True)
        # leaves that share storage with the current weights; the context keeps them, so the backward pass still
        # differentiates this call's weights after set_weights pointed the layer somewhere else
        gate, w13, w2 = (t.detach().requires_grad_(True) for t in (self.gate, self.w13, self.w2))
        if self.world == 1:
            y = self.dense_reference(xr, w13, w2, residual=residual, gate=gate)
            x_all, lo = xr, 0
        else:
            T = x.shape[0]
            gathered = torch.empty(self.world * T, x.shape[1], dtype=x.dtype)
            dist.all_gather_into_tensor(gathered, x.detach().contiguous(), group=self.group)
            x_all = gathered.requires_grad_(True)
            lo = self.rank * T
            y = self._local_experts(x_all, gate, w13, w2)            # [W * T, d]: this rank's experts only
        probs = torch.softmax(x_all[lo:lo + x.shape[0]].float() @ gate.float().t(), -1)
        idx = probs.topk(self.k, -1).indices
        frac = torch.bincount(idx.flatten(), minlength=self.E).float() / idx.numel()
        aux = self.E * (frac * probs.mean(0)).sum()
        if self.world == 1:
            out = y
        else:
            part = y.detach().clone()
            dist.all_reduce(part, group=self.group)
            out = part[lo:lo + x.shape[0]]
            if residual is not None:
                out = out + residual.float()
        return out.to(x.dtype).detach(), (x_all, y, aux, (gate, w13, w2), lo, x.shape[0])

    def _local_experts(self, x_all, gate, w13, w2):
        """Sum over this rank's experts of (routing weight x expert output) for every token of ``x_all``."""
        xf = x_all.float()
        probs = torch.softmax(xf @ gate.float().t(), -1)
        top, idx = probs.topk(self.k, -1)
        wts = top / top.sum(-1, keepdim=True)
        y = torch.zeros_like(xf)
        for j in range(self.el):
            e = self.rank * self.el + j
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            g, u = (xf[tok] @ w13[j].float().t()).chunk(2, -1)
            y = y.index_add(0, tok, ((torch.nn.functional.silu(g) * u) @ w2[j].float().t()) * wts[tok, slot, None])
        return y

    def _backward_ref(self, ctx, dy):
        x_all, y, aux, leaves, lo, T = ctx
        if self.world == 1:
            dy_all = dy.float()
        else:
            dy_all = torch.empty(self.world * T, dy.shape[1], dtype=torch.float32)
            dist.all_gather_into_tensor(dy_all, dy.float().contiguous(), group=self.group)
        total = (y * dy_all).sum() + self.aux_coef * aux
        gx, gg, g13, g2 = torch.autograd.grad(total, [x_all, *leaves], allow_unused=True)
        if self.world > 1:
            gx = gx.contiguous()
            dist.all_reduce(gx, group=self.group)          # every rank's experts contributed to my tokens' gradient
            gx = gx[lo:lo + T]
        for name, g in (("gate", gg), ("w13", g13), ("w2", g2)):
            g = torch.zeros_like(self.grads[name]) if g is None else g
            if self.accumulate_grads:
                self.grads[name] += g.to(self.grads[name].dtype)
            else:
                self.grads[name].copy_(g.to(self.grads[name].dtype))
        return gx.to(dy.dtype)

    # ------------------------------------------------------------------ autograd wrapper
    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """Differentiable call for use inside a torch model (weight gradients land in ``self.grads``)."""
        return _MoEFn.apply(x, self)


class _MoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        y, c = layer.forward(x)
        ctx.layer, ctx.c = layer, c
        return y

    @staticmethod
    def backward(ctx, dy):
        return ctx.layer.backward(ctx.c, dy), None
