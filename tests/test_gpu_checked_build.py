"""The range-checked kernel library (``GF_CHECKED=1``): a data-dependent index that is out of range is skipped and
reported with kernel site, block, thread, index and limit through the status buffer."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_checked_library_reports_a_corrupted_expert_id_and_skips_the_access():
    from ghost_flow_b200.ops import _lib

    if not (_lib._PKG / "lib" / "libgfb200_checked.so").exists():
        pytest.skip("checked library not built")
    env = dict(os.environ, GF_CHECKED="1")
    r = subprocess.run([sys.executable, os.path.join(HERE, "_checked_build_worker.py")], env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-3000:])
    assert "REPORT:" in r.stdout and "block" in r.stdout and r.stdout.strip().endswith("OK")
