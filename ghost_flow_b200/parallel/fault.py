"""Failure detection on the host: heartbeats, a step watchdog, peer checks before a launch, host-side fault
injection, and the bounded device wait.

The reference has no failure handling at all. The rules followed here: a failure is always made and observed on the
host (an exception, a rank that stops beating or never joins, a dropped message); device code never traps or spins
without bound: every wait in the kernels has an iteration limit and reports through a status word that the host
reads, so the CUDA context stays usable. A rank leaves only between steps, and the others learn of it from the store
before their next launch or from a short process-group timeout.
"""
from __future__ import annotations

import threading
import time

import torch
import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, ranks, detail=""):
        super().__init__(f"ranks {sorted(ranks)} stopped responding{': ' + detail if detail else ''}")
        self.ranks = sorted(ranks)


class Heartbeat:
    """Every rank writes a counter to the store every ``interval`` seconds from a daemon thread.
    ``dead_ranks(timeout)`` lists the ranks whose counter has not moved for ``timeout`` seconds."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.2, prefix: str = "hb"):
        self.store, self.rank, self.world, self.interval, self.prefix = store, rank, world, interval, prefix
        self._stop = threading.Event()
        self._seen: dict[int, tuple[int, float]] = {}
        self._thread = None

    def start(self):
        self.store.set(f"{self.prefix}/{self.rank}", "0")
        self._thread = threading.Thread(target=self._beat, daemon=True)
        self._thread.start()
        return self

    def _beat(self):
        n = 0
        while not self._stop.wait(self.interval):
            n += 1
            try:
                self.store.set(f"{self.prefix}/{self.rank}", str(n))
            except Exception:
                return

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def dead_ranks(self, timeout: float) -> list[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.get(f"{self.prefix}/{r}"))
            except Exception:
                val = -1
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > timeout:
                dead.append(r)
        return dead


class StepGuard:
    """Call ``check()`` before every step: raises :class:`PeerFailure` if a peer has stopped beating or has
    published a failure, so that no kernel or collective is launched towards a rank that is gone."""

    def __init__(self, heartbeat: Heartbeat, timeout: float = 2.0):
        self.hb, self.timeout = heartbeat, timeout

    def report_failure(self, detail: str = ""):
        self.hb.store.set(f"fail/{self.hb.rank}", detail or "failed")

    def check(self):
        failed = []
        for r in range(self.hb.world):
            if r != self.hb.rank and self.hb.store.check([f"fail/{r}"]):
                failed.append(r)
        if failed:
            raise PeerFailure(failed, "reported a failure")
        dead = self.hb.dead_ranks(self.timeout)
        if dead:
            raise PeerFailure(dead, f"no heartbeat for {self.timeout}s")

    def wait_healthy(self, seconds: float, poll: float = 0.1):
        """Polls ``check`` for ``seconds``; returns normally if nobody failed in that time."""
        end = time.monotonic() + seconds
        while time.monotonic() < end:
            self.check()
            time.sleep(poll)


class Watchdog:
    """``with Watchdog(5.0, on_timeout=...)`` around a step: if the block runs longer than the limit the callback
    fires from a timer thread (default: record the event). The block itself is not interrupted."""

    def __init__(self, timeout_s: float, on_timeout=None):
        self.timeout_s = timeout_s
        self.on_timeout = on_timeout
        self.fired = False
        self.events: list[float] = []
        self._timer = None

    def _fire(self):
        self.fired = True
        self.events.append(time.monotonic())
        if self.on_timeout:
            self.on_timeout()

    def __enter__(self):
        self.fired = False
        self._timer = threading.Timer(self.timeout_s, self._fire)
        self._timer.daemon = True
        self._timer.start()
        return self

    def __exit__(self, *a):
        self._timer.cancel()
        return False


class FaultInjector:
    """Host-side faults for tests: raise at a given step, go silent (stop the heartbeat), or drop a message."""

    def __init__(self, raise_at: int | None = None, silent_at: int | None = None, drop_messages: set | None = None):
        self.raise_at, self.silent_at = raise_at, silent_at
        self.drop_messages = drop_messages or set()
        self.step = 0

    def before_step(self, heartbeat: Heartbeat | None = None):
        self.step += 1
        if self.raise_at is not None and self.step == self.raise_at:
            raise RuntimeError(f"injected failure at step {self.step}")
        if self.silent_at is not None and self.step == self.silent_at and heartbeat is not None:
            heartbeat.stop()

    def should_drop(self, message_id) -> bool:
        return message_id in self.drop_messages


def bounded_device_wait(pad: torch.Tensor, index: int, world: int, value: int, limit: int = 1 << 18) -> int:
    """Runs the flag-wait kernel on ``pad[index : index + world]`` with an iteration limit and returns the status
    word afterwards (0 = the flags arrived, 5 = the wait ran out). The context stays usable either way."""
    from ..ops import _lib
    import ctypes

    lib = _lib.cuda_lib()
    lib.gf_wait_flags.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_longlong,
                                  ctypes.c_void_p, ctypes.c_void_p]
    lib.gf_wait_flags.restype = ctypes.c_int
    status = _lib.status_word(pad.device)
    _lib.check_rc(lib.gf_wait_flags(pad.data_ptr(), index, world, value, limit, status.data_ptr(), _lib.stream_ptr()),
                  "gf_wait_flags")
    torch.cuda.synchronize(pad.device)
    code = int(status[0].item())
    status.zero_()
    return code


# ------------------------------------------------------------------ elastic restart
RESTART_MARKER = "RESTART.json"
EXIT_RESTART = 75   # EX_TEMPFAIL: the job may be started again (from the marker's checkpoint, at its world size)


def write_restart_marker(directory, checkpoint_dir, failed_ranks, world: int, step: int, detail: str = "") -> str:
    """Called by a surviving rank after :class:`PeerFailure` (between steps, nothing in flight): records where
    to resume from and with how many ranks. The launcher (or the operator) reads it with
    :func:`read_restart_marker`, starts ``new_world`` ranks, and every rank calls ``io.load_sharded``, which
    re-cuts the shards of the old world size."""
    import json
    import os

    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, RESTART_MARKER)
    tmp = path + f".tmp{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump({"checkpoint_dir": os.fspath(checkpoint_dir), "failed_ranks": sorted(int(r) for r in failed_ranks),
                   "old_world": int(world), "new_world": int(world) - len(set(failed_ranks)), "step": int(step),
                   "detail": detail}, f)
    os.replace(tmp, path)   # atomic: several survivors may write the same content
    return path


def read_restart_marker(directory):
    import json
    import os

    path = os.path.join(directory, RESTART_MARKER)
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)
