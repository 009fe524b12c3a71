"""Host model of the device-side signalling protocols, with threads as ranks.

The peer-memory kernels of this package order themselves with int32 flags that one rank stores into another rank's
signal pad (release) and the owner polls (acquire): ``READY`` / ``CONSUMED`` / ``VERSION`` in the ZeRO-3 engine
(``parallel/symm.py``, ``csrc/comm_kernels.cu``) and the per-source ``DISPATCH`` / ``COMBINE`` epochs of the
expert-parallel layer (``parallel/ep.py``, ``csrc/moe_kernels.cu``). No race detector runs on those kernels, so
the rules are restated here in plain Python and executed by one thread per rank under randomised delays. Every
shared buffer carries a tag (what it holds) and a reader count; a step that would read a buffer before its
producer finished, overwrite one that a peer may still read, or take a weight version other than the one the
schedule promises raises :class:`ProtocolViolation`. Each rule of the protocol can be switched off
(``Rules(...)``): the tests check that the model then reports the hazard the rule exists to prevent, i.e. that it
would notice if a kernel dropped the rule.

The reference has no such protocol (its collectives are single-process stubs, ghostflow-nn/src/distributed.rs:147-207).
"""
from __future__ import annotations

import queue
import random
import threading
import time
from dataclasses import dataclass


class ProtocolViolation(AssertionError):
    pass


@dataclass
class Rules:
    """Every field is one ordering rule of the protocols; False removes it."""
    wait_ready: bool = True          # the reducer waits for READY of every rank before it reads their gradients
    wait_consumed: bool = True       # a rank waits for CONSUMED of every rank before it rewrites a gradient slot
    wait_version: bool = True        # a gather waits for the VERSION it expects before it reads a peer's shard
    wait_dispatch: bool = True       # the expert GEMM waits for the DISPATCH epoch of every source rank
    wait_combine: bool = True        # the combine waits for the COMBINE epoch of every owner rank


class _Buffer:
    """A piece of memory of one rank that other ranks read or write: a tag plus bookkeeping to detect hazards."""

    def __init__(self, name):
        self.name = name
        self.tag = None
        self.writing = 0
        self.readers = 0
        self.lock = threading.Lock()

    def begin_write(self, who):
        with self.lock:
            if self.readers:
                raise ProtocolViolation(f"{who} overwrites {self.name} while {self.readers} reader(s) are active")
            if self.writing:
                raise ProtocolViolation(f"{who} overwrites {self.name} while another write is in flight")
            self.writing += 1
            self.tag = None

    def end_write(self, tag):
        with self.lock:
            self.writing -= 1
            self.tag = tag

    def begin_read(self, who, expect):
        with self.lock:
            if self.writing or self.tag != expect:
                raise ProtocolViolation(f"{who} reads {self.name}: holds {self.tag!r}"
                                        f"{' (write in flight)' if self.writing else ''}, expected {expect!r}")
            self.readers += 1

    def end_read(self):
        with self.lock:
            self.readers -= 1


class _Pads:
    """``world`` signal pads of ``n`` ints; ``store`` is the release store into a peer's pad, ``wait_ge`` the bounded
    acquire poll of the owner (the kernels give up after a limit and set a status word; here that is an exception)."""

    def __init__(self, world, n):
        self.v = [[0] * n for _ in range(world)]

    def store(self, dst_rank, idx, value):
        self.v[dst_rank][idx] = value

    def wait_ge(self, rank, idx, value, what, limit_s=5.0):
        t0 = time.monotonic()
        while self.v[rank][idx] < value:
            if time.monotonic() - t0 > limit_s:
                raise ProtocolViolation(f"rank {rank} gave up waiting for {what} >= {value} (has {self.v[rank][idx]})")
            time.sleep(0)


def _run_ranks(world, body):
    errors = []

    def guarded(r):
        try:
            body(r)
        except BaseException as e:     # noqa: BLE001 - a failing rank must not leave the others spinning silently
            errors.append(e)

    threads = [threading.Thread(target=guarded, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        first = next((e for e in errors if isinstance(e, ProtocolViolation)), errors[0])
        raise first


# ------------------------------------------------------------------------------------------------- ZeRO-3 step
def run_zero3(world=4, units=5, steps=3, rules: Rules | None = None, seed=0, jitter=2e-4, regather=True):
    """``steps`` training steps of the ZeRO-3 schedule over ``units`` flat units.

    Per step and rank: forward gathers every unit (pull all-gather: wait for the peer's VERSION, read its shard);
    backward walks the units in reverse, writes the unit's gradient into one of two slots (after every rank has
    CONSUMED the slot's previous use) and signals READY; the rank's reducer, a second thread that stands for the
    communication stream, reads its slice of all ranks' slot, updates its shard and publishes CONSUMED and the new
    VERSION while the first thread is already in the backward pass of the next unit. ``regather``: weights are gathered
    again in backward (rotating buffers) instead of being kept from the forward pass.
    Returns the number of flag waits that were executed."""
    rules = rules or Rules()
    READY, CONSUMED, VERSION = 0, 2 * world, 4 * world          # [slot][src], [slot][src], [unit][src]
    pads = _Pads(world, VERSION + units * world)
    shard = [[_Buffer(f"shard[{r}][{u}]") for u in range(units)] for r in range(world)]
    grads = [[_Buffer(f"grad[{r}][slot {s}]") for s in range(2)] for r in range(world)]
    for r in range(world):
        for u in range(units):
            shard[r][u].tag = ("w", u, 0)
    waits = [0] * world

    def nap(rng):
        if jitter:
            time.sleep(rng.random() * jitter)

    def gather(r, u, version, rng):
        for o in range(1, world + 1):
            src = (r + o) % world
            if src != r and rules.wait_version:
                pads.wait_ge(r, VERSION + u * world + src, version, f"VERSION[{u}][{src}]")
                waits[r] += 1
            shard[src][u].begin_read(f"rank {r} gather", ("w", u, version))
            nap(rng)
            shard[src][u].end_read()

    def reducer(r, q, errors):
        """The rank's communication stream: reduce tasks in submission order."""
        rng = random.Random(seed * 1000 + 500 + r)
        while True:
            task = q.get()
            if task is None:
                return
            if errors:
                task[-1].set()
                continue
            slot, u, t, use, done = task
            try:
                if rules.wait_ready:
                    for src in range(world):
                        pads.wait_ge(r, READY + slot * world + src, use, f"READY[{slot}][{src}]")
                        waits[r] += 1
                for src in range(world):
                    grads[src][slot].begin_read(f"rank {r} reducer", ("g", u, t))
                nap(rng)
                for src in range(world):
                    grads[src][slot].end_read()
                shard[r][u].begin_write(f"rank {r} update of unit {u}")
                nap(rng)
                shard[r][u].end_write(("w", u, t))
                for dst in range(world):
                    pads.store(dst, CONSUMED + slot * world + r, use)
                    pads.store(dst, VERSION + u * world + r, t)
            except BaseException as e:     # noqa: BLE001
                errors.append(e)
            finally:
                done.set()

    def body(r):
        rng = random.Random(seed * 1000 + r)
        uses = [0, 0]
        q, errors = queue.Queue(), []
        comm = threading.Thread(target=reducer, args=(r, q, errors))
        comm.start()
        try:
            for t in range(1, steps + 1):
                for u in range(units):
                    gather(r, u, t - 1, rng)
                    nap(rng)
                slot = 0
                pending = []
                for u in reversed(range(units)):
                    if regather:
                        gather(r, u, t - 1, rng)
                    # the slot's previous use must have been read by every rank (this rank's own reducer included)
                    if rules.wait_consumed and uses[slot]:
                        for src in range(world):
                            pads.wait_ge(r, CONSUMED + slot * world + src, uses[slot], f"CONSUMED[{slot}][{src}]")
                            waits[r] += 1
                    grads[r][slot].begin_write(f"rank {r} backward of unit {u}")
                    nap(rng)
                    uses[slot] += 1
                    grads[r][slot].end_write(("g", u, t))
                    for dst in range(world):
                        pads.store(dst, READY + slot * world + r, uses[slot])
                    # the fused reducer goes to the communication stream; backward of the next unit carries on
                    done = threading.Event()
                    q.put((slot, u, t, uses[slot], done))
                    pending.append(done)
                    slot = 1 - slot
                    if errors:
                        raise errors[0]
                for d in pending:                      # end of step: the compute stream joins the reducers
                    d.wait()
                if errors:
                    raise errors[0]
        finally:
            q.put(None)
            comm.join()
    _run_ranks(world, body)
    return sum(waits)


# ------------------------------------------------------------------------------------------------- MoE layer
def run_moe(world=4, calls=6, rules: Rules | None = None, seed=0, jitter=2e-4):
    """``calls`` consecutive uses of one expert-parallel workspace (forward or backward, the flags do not differ).

    Per call ``e`` and rank: dispatch writes this rank's rows into every owner's ``xs`` and stores DISPATCH[src] = e
    in the owner's pad; the owner's first GEMM waits for all sources and reads ``xs``; its second GEMM writes the
    results into every source's ``comb`` and stores COMBINE[owner] = e there; the source's combine waits for all
    owners and reads ``comb``. Nothing else orders call e + 1 against call e."""
    rules = rules or Rules()
    DISPATCH, COMBINE = 0, world
    pads = _Pads(world, 2 * world)
    xs = [[_Buffer(f"xs[{o}] rows of source {s}") for s in range(world)] for o in range(world)]
    comb = [[_Buffer(f"comb[{s}] slots of owner {o}") for o in range(world)] for s in range(world)]
    waits = [0] * world

    def body(r):
        rng = random.Random(seed * 1000 + r)

        def nap():
            if jitter:
                time.sleep(rng.random() * jitter)

        for e in range(1, calls + 1):
            for owner in range(world):                       # dispatch
                xs[owner][r].begin_write(f"rank {r} dispatch of call {e}")
                nap()
                xs[owner][r].end_write(("x", e))
                pads.store(owner, DISPATCH + r, e)
            if rules.wait_dispatch:                          # first grouped GEMM of this rank's experts
                for src in range(world):
                    pads.wait_ge(r, DISPATCH + src, e, f"DISPATCH[{src}]")
                    waits[r] += 1
            for src in range(world):
                xs[r][src].begin_read(f"rank {r} expert GEMM of call {e}", ("x", e))
            nap()
            for src in range(world):
                xs[r][src].end_read()
            for src in range(world):                         # second GEMM scatters the results home
                comb[src][r].begin_write(f"rank {r} scatter of call {e}")
                nap()
                comb[src][r].end_write(("y", e))
                pads.store(src, COMBINE + r, e)
            if rules.wait_combine:                           # combine of this rank's tokens
                for owner in range(world):
                    pads.wait_ge(r, COMBINE + owner, e, f"COMBINE[{owner}]")
                    waits[r] += 1
            for owner in range(world):
                comb[r][owner].begin_read(f"rank {r} combine of call {e}", ("y", e))
            nap()
            for owner in range(world):
                comb[r][owner].end_read()
    _run_ranks(world, body)
    return sum(waits)
