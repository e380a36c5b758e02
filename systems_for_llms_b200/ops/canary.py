"""Guard bands around kernel outputs, checked on the host.

``compute-sanitizer`` is not available on every machine these kernels run on, so the
tests catch out-of-bounds stores another way: an output tensor is carved out of a larger
allocation whose bytes before and after it hold a fixed pattern; after the kernel ran,
``intact()`` says whether both bands still hold it.  The interior can be pre-filled with
a second pattern so that ``untouched()`` reports elements a kernel was supposed to write
and did not.  A band only detects writes that land inside it; 4 KiB on either side covers
the usual off-by-one-tile and wrong-pitch mistakes of row-major kernels.
"""

from __future__ import annotations

import math

import torch

GUARD_BYTE = 0xA5
FILL_BYTE = 0x5A


class Guarded:
    """``tensor`` is the usable view; the object keeps the surrounding allocation."""

    def __init__(self, shape, dtype: torch.dtype, device, *, guard_bytes: int = 4096,
                 fill: bool = True):
        if guard_bytes <= 0 or guard_bytes % 256:
            raise ValueError("guard_bytes must be a positive multiple of 256")
        element = torch.empty((), dtype=dtype).element_size()
        self.nbytes = math.prod(shape) * element
        self.guard = guard_bytes
        padded = -(-self.nbytes // 256) * 256          # keeps the rear band 256-byte aligned
        self.raw = torch.full((guard_bytes + padded + guard_bytes,), GUARD_BYTE,
                              dtype=torch.uint8, device=device)
        inner = self.raw[guard_bytes:guard_bytes + self.nbytes]
        if fill:
            inner.fill_(FILL_BYTE)
        self.tensor = inner.view(dtype).view(*shape)

    def intact(self) -> bool:
        """True when no byte of either guard band (or of the alignment slack) changed."""
        front = self.raw[:self.guard]
        rear = self.raw[self.guard + self.nbytes:]
        return bool((front == GUARD_BYTE).all().item() and (rear == GUARD_BYTE).all().item())

    def untouched(self) -> int:
        """Number of interior bytes that still hold the fill pattern (an output that a kernel
        wrote completely has close to none: a genuine value can contain the byte by chance)."""
        inner = self.raw[self.guard:self.guard + self.nbytes]
        return int((inner == FILL_BYTE).sum().item())


def guarded(shape, dtype: torch.dtype, device, **options) -> Guarded:
    return Guarded(tuple(shape), dtype, device, **options)
