"""CUDA-graph capture of a whole training step.

A small model on a B200 is bound by the host: a GPT-2-small step is some 600 kernel launches of 10 to 30 microseconds
of GPU time each, while Python, autograd and the launch path need several times that per launch. Recording the step
once and replaying it removes the host from the loop. The reference has no counterpart (its training loop is a host
loop over CPU tensors, ghostflow-nn/src/zero_optimizer.rs:262-309); the nearest thing it names is the JIT / fusion
engine's promise to cut per-op overhead (ghostflow-core/src/fusion.rs).

What a step must satisfy to be recorded: no host read of device memory (``.item()``, ``float(loss)``, status polls),
no allocation outside torch's caching allocator, and no launch argument that changes from step to step. The
optimizers of this package have a ``capturable`` mode for the last point: the step number lives in a device counter.
"""
from __future__ import annotations

import torch


class GraphedStep:
    """``fn(*inputs) -> tensor or tuple of tensors`` recorded in a CUDA graph.

    ``fn`` must contain the whole step (``zero_grad``, forward, backward, ``optimizer.step()``). It is run ``warmup``
    times for real before the capture (those are ordinary optimizer steps: lazily created buffers, workspaces and
    kernel attributes must exist before recording), then recorded once; the recording itself does not execute.
    Calling the object copies the new inputs into the recorded input buffers and replays. The returned tensors
    are the recorded outputs: they are overwritten by the next call. On several ranks every rank must record and
    replay the same number of times.
    """

    def __init__(self, fn, example_inputs, warmup: int = 3):
        self.fn = fn
        self.static_inputs = [t.clone() for t in example_inputs]
        self.warmup_outputs = []
        self.replays = 0
        self.graph = None
        if not (torch.cuda.is_available() and all(t.is_cuda for t in self.static_inputs)):
            # no GPU: the same object runs the step eagerly, so a script written for graphs runs anywhere
            for _ in range(warmup):
                out = fn(*self.static_inputs)
                self.warmup_outputs.append(out.detach().clone() if torch.is_tensor(out) else out)
            self.static_output = None
            return
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                out = fn(*self.static_inputs)
                self.warmup_outputs.append(out.detach().clone() if torch.is_tensor(out) else out)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        # thread_local: other threads (the NCCL watchdog polls events) may keep calling the runtime during the recording
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.static_output = fn(*self.static_inputs)
        self.replays = 0

    def __call__(self, *inputs):
        if self.graph is None:
            self.replays += 1
            self.static_output = self.fn(*inputs)
            return self.static_output
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_output

    def release(self):
        """Drops the recording (and the memory pool it holds). Call it before tearing a process group down: a live
        graph that contains collectives keeps the communicator's watchdog from finishing."""
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph.reset()
        self.static_output = None
