"""The guard-band helper itself (CPU)."""

import pytest
import torch

from systems_for_llms_b200.ops.canary import FILL_BYTE, guarded


def test_guard_bands_detect_writes_on_either_side():
    g = guarded((5, 7), torch.float32, "cpu", guard_bytes=256)
    assert g.tensor.shape == (5, 7) and g.intact()
    assert g.untouched() == 5 * 7 * 4
    g.tensor.zero_()
    assert g.intact() and g.untouched() == 0
    g.raw[g.guard - 1] = 0                     # one byte before the tensor
    assert not g.intact()
    g.raw[g.guard - 1] = 0xA5
    g.raw[g.guard + g.nbytes] = 1              # first byte after it (alignment slack counts)
    assert not g.intact()


def test_partial_writes_leave_fill_bytes():
    g = guarded((4, 8), torch.bfloat16, "cpu", guard_bytes=256)
    g.tensor[:3].fill_(1.0)
    assert g.untouched() == 8 * 2
    assert bytes([FILL_BYTE]) * 2 == g.raw[g.guard + 3 * 16:g.guard + 3 * 16 + 2].numpy().tobytes()


def test_bad_guard_size():
    with pytest.raises(ValueError):
        guarded((1,), torch.float32, "cpu", guard_bytes=100)
