"""The library's own symmetric-memory allocator, driven through its host stand-in: the virtual-memory-management flow
(create, export a file descriptor, pass it between processes over a unix socket, import, reserve, map every rank's
allocation at base + rank * size, set access) runs for real on memfd-backed memory, so what one process stores into
a peer's slot is read by the peer."""
import os
import subprocess
import sys
import tempfile
import uuid

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_every_rank_sees_every_slot(tmp_path, world):
    job = uuid.uuid4().hex[:8]
    with tempfile.TemporaryDirectory(dir="/tmp") as sock_dir:          # socket paths are limited to 107 characters
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "_symm_alloc_worker.py"), str(r), str(world), job,
                                   sock_dir, str(tmp_path / f"r{r}.txt")], stderr=subprocess.PIPE, text=True)
                 for r in range(world)]
        errs = [p.communicate(timeout=120)[1] for p in procs]
    for r, p in enumerate(procs):
        assert p.returncode == 0, errs[r][-2000:]
        assert (tmp_path / f"r{r}.txt").read_text() == "ok"


def test_bad_arguments_are_refused():
    from ghost_flow_b200.parallel.symm_alloc import SymmetricAllocation

    with pytest.raises(RuntimeError, match="bad argument"):
        SymmetricAllocation(0, 0, 1, host=True)
    with pytest.raises(RuntimeError):
        SymmetricAllocation(4096, 0, 2, host=True, job="alone", timeout_s=1)      # the peer never shows up
