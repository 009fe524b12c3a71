"""Python face of the library's own symmetric-memory allocator (``csrc/symm_alloc.cpp``).

Every rank of a node allocates ``nbytes`` of device memory; all allocations are mapped into every process at
``base + rank * bytes_per_rank``, so a kernel reaches a peer's buffer with plain loads and stores. The driver calls
are the CUDA virtual-memory-management ones (create, export as a file descriptor, import, reserve, map, set access);
the descriptors travel over unix-domain sockets. ``host=True`` runs the same flow on memfd-backed host memory, which is
how it is tested without a GPU. The package uses ``torch.distributed._symmetric_memory`` by default; this allocator is
selected with ``GF_SYMM_ALLOC=own`` (not run on a GPU so far).
"""
from __future__ import annotations

import ctypes
import os
import tempfile

import torch

from ..ops import _lib


def _bind():
    lib = _lib.host_lib()
    if getattr(lib, "_gf_symm_bound", False):
        return lib
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.gf_symm_create.argtypes = [I, ctypes.c_size_t, I, I, ctypes.c_char_p, ctypes.c_char_p, I, ctypes.POINTER(P)]
    lib.gf_symm_create.restype = I
    lib.gf_symm_ptr.argtypes = [P, I]
    lib.gf_symm_ptr.restype = ctypes.c_ulonglong
    lib.gf_symm_bytes_per_rank.argtypes = [P]
    lib.gf_symm_bytes_per_rank.restype = ctypes.c_ulonglong
    lib.gf_symm_destroy.argtypes = [P]
    lib.gf_symm_destroy.restype = I
    lib.gf_symm_use_host_driver.argtypes = [I]
    lib.gf_symm_last_error.restype = ctypes.c_char_p
    lib._gf_symm_bound = True
    return lib


class _Span:
    """Exposes a raw address range through the array interfaces so that torch / numpy can wrap it without a copy."""

    def __init__(self, ptr: int, nbytes: int, cuda: bool, owner):
        self._owner = owner                                  # keeps the allocation alive
        iface = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}
        if cuda:
            self.__cuda_array_interface__ = iface
        else:
            self.__array_interface__ = iface


class SymmetricAllocation:
    """Collective over the ``world`` processes of one node (every rank passes the same ``nbytes`` and ``job``)."""

    def __init__(self, nbytes: int, rank: int, world: int, device: int = 0, job: str = "job", sock_dir: str | None = None,
                 host: bool = False, timeout_s: int = 60):
        self.lib = _bind()
        self.rank, self.world, self.host, self.device = rank, world, host, device
        self.lib.gf_symm_use_host_driver(1 if host else 0)
        if not host:
            torch.cuda.init()
            torch.empty(1, device=torch.device("cuda", device))          # the device's primary context exists
        handle = ctypes.c_void_p()
        sock_dir = sock_dir or tempfile.gettempdir()
        rc = self.lib.gf_symm_create(device, nbytes, rank, world, os.fspath(sock_dir).encode(), job.encode(), timeout_s,
                                     ctypes.byref(handle))
        if rc != 0:
            raise RuntimeError(f"symmetric allocation failed ({rc}): {self.lib.gf_symm_last_error().decode()}")
        self.handle = handle
        self.bytes_per_rank = int(self.lib.gf_symm_bytes_per_rank(handle))
        self.ptrs = [int(self.lib.gf_symm_ptr(handle, r)) for r in range(world)]

    def tensor(self, rank: int | None = None, dtype=torch.uint8) -> torch.Tensor:
        """Rank ``rank``'s slot (default: this rank's) as a tensor over the mapped memory."""
        r = self.rank if rank is None else rank
        span = _Span(self.ptrs[r], self.bytes_per_rank, not self.host, self)
        if self.host:
            import numpy as np

            t = torch.from_numpy(np.asarray(span))
        else:
            t = torch.as_tensor(span, device=torch.device("cuda", self.device))
        return t.view(dtype)

    def close(self):
        if self.handle is not None:
            self.lib.gf_symm_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
