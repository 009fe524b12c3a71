"""Guard blocks behind workspace carve-outs: an overrun is reported with the carve-out's name and the byte offset."""
import pytest
import torch

from ghost_flow_b200.parallel import canary


def test_overrun_is_reported_with_name_and_offset():
    buf = torch.zeros(8192, dtype=torch.uint8)
    led = canary.CanaryLedger(buf, "test workspace")
    off = led.plant(0, "start")
    a = buf[off:off + 1000].view(torch.int16)
    off = led.plant(off + 1024, "a (500 x int16)")
    b = buf[off:off + 512]
    off = led.plant(off + 512, "b")
    a.fill_(7)
    b.fill_(9)
    assert canary.check_all() >= 3                      # in-bounds writes leave the guards alone
    buf[256 + 1024 + 3] = 0                             # 4th byte behind a's 1024-byte slot
    with pytest.raises(canary.CanaryError) as e:
        led.check()
    msg = str(e.value)
    assert "a (500 x int16)" in msg and "arena byte 1283" in msg and "1 of 256" in msg
    buf[256 + 1024 + 3] = canary.PATTERN
    led.check()
    buf[0:4] = 1                                        # a write in front of the first carve-out
    with pytest.raises(canary.CanaryError, match="start"):
        canary.check_all()
    buf[0:4] = canary.PATTERN


def test_expert_workspace_on_cpu_has_no_ledger_but_cuda_constructors_reserve_slack():
    # the constructors add SLACK_BYTES on top of what their callers computed, enough for 255 guard blocks
    assert canary.SLACK_BYTES >= 255 * canary.CANARY_BYTES
