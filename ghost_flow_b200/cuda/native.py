"""ctypes binding of the native device layer (``csrc/runtime.cu``): device properties, streams, events, a timer and
the pooled device allocator, all C++ over the CUDA runtime. The pure-Python classes of :mod:`ghost_flow_b200.cuda`
ride on PyTorch's runtime; these are the standalone native equivalents of ghostflow-cuda/src/{device,stream,memory,
error}.rs and can be used without torch tensors (raw device pointers)."""
from __future__ import annotations

import ctypes

from ..ops import _lib


class NativeCudaError(RuntimeError):
    def __init__(self, code: int):
        super().__init__(_lib.cuda_lib().gfrt_error_string(code).decode())
        self.code = code


class _Props(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 256), ("major", ctypes.c_int), ("minor", ctypes.c_int),
                ("multiprocessors", ctypes.c_int), ("warp_size", ctypes.c_int), ("max_threads_per_block", ctypes.c_int),
                ("clock_khz", ctypes.c_int), ("memory_clock_khz", ctypes.c_int), ("l2_bytes", ctypes.c_int),
                ("max_shared_per_block_optin", ctypes.c_int), ("total_memory", ctypes.c_ulonglong)]


_BOUND = False


def _lib_():
    global _BOUND
    lib = _lib.cuda_lib()
    if not _BOUND:
        lib.gfrt_error_string.restype = ctypes.c_char_p
        lib.gfrt_error_string.argtypes = [ctypes.c_int]
        P = ctypes.c_void_p
        PP = ctypes.POINTER(ctypes.c_void_p)
        sig = {"gfrt_device_count": [ctypes.POINTER(ctypes.c_int)], "gfrt_device_props": [ctypes.c_int, ctypes.POINTER(_Props)],
               "gfrt_memory_info": [ctypes.c_int, ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong)],
               "gfrt_synchronize": [ctypes.c_int], "gfrt_stream_create": [ctypes.c_int, ctypes.c_int, PP],
               "gfrt_stream_destroy": [P], "gfrt_stream_synchronize": [P], "gfrt_stream_query": [P],
               "gfrt_stream_wait_event": [P, P], "gfrt_event_create": [ctypes.c_int, PP], "gfrt_event_destroy": [P],
               "gfrt_event_record": [P, P], "gfrt_event_synchronize": [P], "gfrt_event_query": [P],
               "gfrt_event_elapsed_ms": [P, P, ctypes.POINTER(ctypes.c_float)], "gfrt_pool_create": [ctypes.c_int, PP],
               "gfrt_pool_alloc": [P, ctypes.c_ulonglong, PP], "gfrt_pool_free": [P, P], "gfrt_pool_trim": [P],
               "gfrt_pool_stats": [P, ctypes.POINTER(ctypes.c_ulonglong)], "gfrt_pool_destroy": [P]}
        for n, a in sig.items():
            getattr(lib, n).argtypes = a
            getattr(lib, n).restype = ctypes.c_int
        _BOUND = True
    return lib


def _ck(code):
    if code != 0:
        raise NativeCudaError(code)


def device_count() -> int:
    n = ctypes.c_int(0)
    _lib_().gfrt_device_count(ctypes.byref(n))
    return n.value


def device_properties(device: int = 0) -> dict:
    p = _Props()
    _ck(_lib_().gfrt_device_props(device, ctypes.byref(p)))
    return {f: (getattr(p, f).decode() if f == "name" else getattr(p, f)) for f, _ in _Props._fields_}


def memory_info(device: int = 0):
    f, t = ctypes.c_ulonglong(), ctypes.c_ulonglong()
    _ck(_lib_().gfrt_memory_info(device, ctypes.byref(f), ctypes.byref(t)))
    return f.value, t.value


class Event:
    def __init__(self, timing=True):
        self.h = ctypes.c_void_p()
        _ck(_lib_().gfrt_event_create(1 if timing else 0, ctypes.byref(self.h)))

    def record(self, stream=None):
        _ck(_lib_().gfrt_event_record(self.h, stream.h if stream else None))

    def synchronize(self):
        _ck(_lib_().gfrt_event_synchronize(self.h))

    def query(self) -> bool:
        return _lib_().gfrt_event_query(self.h) == 0

    def elapsed_ms(self, end: "Event") -> float:
        ms = ctypes.c_float()
        _ck(_lib_().gfrt_event_elapsed_ms(self.h, end.h, ctypes.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            _lib_().gfrt_event_destroy(self.h)
        except Exception:
            pass


class Stream:
    def __init__(self, device=0, high_priority=False):
        self.h = ctypes.c_void_p()
        _ck(_lib_().gfrt_stream_create(device, 1 if high_priority else 0, ctypes.byref(self.h)))

    def synchronize(self):
        _ck(_lib_().gfrt_stream_synchronize(self.h))

    def query(self) -> bool:
        return _lib_().gfrt_stream_query(self.h) == 0

    def wait_event(self, ev: Event):
        _ck(_lib_().gfrt_stream_wait_event(self.h, ev.h))

    def __del__(self):
        try:
            _lib_().gfrt_stream_destroy(self.h)
        except Exception:
            pass


class Timer:
    def __init__(self):
        self.a, self.b = Event(), Event()

    def start(self, stream=None):
        self.a.record(stream)

    def stop(self, stream=None):
        self.b.record(stream)

    def elapsed_ms(self):
        self.b.synchronize()
        return self.a.elapsed_ms(self.b)


class MemoryPool:
    """Power-of-two size classes with cached free lists; ``allocate`` returns a raw device pointer (int)."""

    def __init__(self, device=0):
        self.h = ctypes.c_void_p()
        _ck(_lib_().gfrt_pool_create(device, ctypes.byref(self.h)))

    def allocate(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        _ck(_lib_().gfrt_pool_alloc(self.h, nbytes, ctypes.byref(p)))
        return p.value

    def free(self, ptr: int):
        _ck(_lib_().gfrt_pool_free(self.h, ctypes.c_void_p(ptr)))

    def trim(self):
        _ck(_lib_().gfrt_pool_trim(self.h))

    def stats(self) -> dict:
        s = (ctypes.c_ulonglong * 6)()
        _ck(_lib_().gfrt_pool_stats(self.h, s))
        return dict(zip(("current_usage", "peak_usage", "cached", "hits", "misses", "live_blocks"), [int(v) for v in s]))

    def current_usage(self):
        return self.stats()["current_usage"]

    def peak_usage(self):
        return self.stats()["peak_usage"]

    def close(self):
        if self.h:
            _lib_().gfrt_pool_destroy(self.h)
            self.h = None
