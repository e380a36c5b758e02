"""Mask language and its compiler to block-sparse schedules.

``MaskSpec`` is a conjunction of constraints on (query position q, key position
k): causal (k <= q), a left window (k >= q - window_left), a right window
(k <= q + window_right) and same-document (label[q] == label[k]).  ``compile_mask``
turns a spec into a CSR over query tiles with an exact empty / partial / full
classification of every tile, never materialising an N x N mask; ``allows`` is
the scalar oracle.  Semantics and data layout follow the reference
(attention_lab/masks.py:22-191).

Additions that the reference does not have:

* ``strided_schedule`` - a block-level "local + strided" pattern (the
  sparse-transformer layout) expressed as a schedule over a causal spec.
* ``KernelSchedule`` / ``to_kernel_schedule`` - regroups a schedule of any block
  size from {16, 32, 64, 128} into the 128 x 128 tiles the sm_100a kernels walk,
  keeping a 64-bit presence bitmap of 16 x 16 sub-blocks per tile so dropped
  blocks stay dropped, and builds the key-major transpose the backward pass needs.
"""

from __future__ import annotations

from bisect import bisect_left
from collections.abc import Sequence
from dataclasses import dataclass, field

BLOCK_SIZES = (16, 32, 64, 128)
KERNEL_TILE = 128
SUB = 16


def _require_int(name: str, value: object, minimum: int) -> None:
    if isinstance(value, bool) or not isinstance(value, int):
        raise TypeError(f"{name} must be an integer")
    if value < minimum:
        raise ValueError(f"{name} must be at least {minimum}")


@dataclass(frozen=True)
class MaskSpec:
    """Conjunctive constraints; a window of ``None`` is unbounded."""

    causal: bool = False
    window_left: int | None = None
    window_right: int | None = None
    same_document: bool = False

    def __post_init__(self) -> None:
        for name in ("causal", "same_document"):
            if not isinstance(getattr(self, name), bool):
                raise TypeError(f"{name} must be a bool")
        for name in ("window_left", "window_right"):
            value = getattr(self, name)
            if value is not None:
                _require_int(name, value, 0)

    @property
    def effective_right(self) -> int | None:
        """Causality caps the right window at zero."""
        return 0 if self.causal else self.window_right


@dataclass
class BlockSchedule:
    """CSR over query tiles.  ``full_blocks[i]`` describes ``col_idx[i]``."""

    length: int
    block_q: int
    block_k: int
    row_ptr: list[int]
    col_idx: list[int]
    full_blocks: list[bool]


def _labels(document_ids, *, length: int | None, required: bool) -> tuple[int, ...] | None:
    if document_ids is None:
        if required:
            raise ValueError("same_document requires document_ids")
        return None
    if isinstance(document_ids, (str, bytes)) or not isinstance(document_ids, Sequence):
        raise TypeError("document_ids must be a sequence of integer labels")
    labels = tuple(document_ids)
    if length is not None and len(labels) != length:
        raise ValueError("document_ids must have exactly length elements")
    for label in labels:
        if isinstance(label, bool) or not isinstance(label, int):
            raise TypeError("document_ids must contain integer labels")
    return labels


def _check_spec(spec: object) -> None:
    if not isinstance(spec, MaskSpec):
        raise TypeError("spec must be a MaskSpec")


def allows(q: int, k: int, spec: MaskSpec, document_ids: Sequence[int] | None = None) -> bool:
    """Scalar semantics of a spec for in-range positions."""
    _check_spec(spec)
    _require_int("q", q, 0)
    _require_int("k", k, 0)
    labels = _labels(document_ids, length=None, required=spec.same_document)
    if labels is not None and max(q, k) >= len(labels):
        raise ValueError("q and k must be within document_ids")
    distance = k - q
    if spec.causal and distance > 0:
        return False
    if spec.window_left is not None and -distance > spec.window_left:
        return False
    if spec.window_right is not None and distance > spec.window_right:
        return False
    if spec.same_document and labels[q] != labels[k]:
        return False
    return True


def compile_mask(length: int, spec: MaskSpec, block_q: int = 64, block_k: int = 64,
                 document_ids: Sequence[int] | None = None) -> BlockSchedule:
    """Exact tile classification in O(query_tiles + stored_tiles) for window masks.

    For each query tile the union of its rows' key intervals is one interval
    (every row sees itself), which gives the candidate key tiles; a candidate is
    geometrically full when its extreme corners satisfy both window bounds.
    Document masks additionally intersect per-tile label sets and, only for
    geometrically partial tiles with mixed labels, look for one permitted pair
    by binary search in a per-label position index.
    """
    _check_spec(spec)
    _require_int("length", length, 1)
    _require_int("block_q", block_q, 1)
    _require_int("block_k", block_k, 1)
    labels = _labels(document_ids, length=length, required=spec.same_document)
    left, right = spec.window_left, spec.effective_right

    where: dict[int, list[int]] = {}
    q_sets: list[frozenset[int]] = []
    k_sets: list[frozenset[int]] = []
    if spec.same_document:
        for position, label in enumerate(labels):
            where.setdefault(label, []).append(position)
        q_sets = [frozenset(labels[s:s + block_q]) for s in range(0, length, block_q)]
        k_sets = [frozenset(labels[s:s + block_k]) for s in range(0, length, block_k)]

    def any_pair(q_lo: int, q_hi: int, k_lo: int, k_hi: int) -> bool:
        for q in range(q_lo, q_hi + 1):
            lo = k_lo if left is None else max(k_lo, q - left)
            hi = k_hi if right is None else min(k_hi, q + right)
            if lo > hi:
                continue
            same = where[labels[q]]
            at = bisect_left(same, lo)
            if at < len(same) and same[at] <= hi:
                return True
        return False

    row_ptr, col_idx, full_blocks = [0], [], []
    for row, q_lo in enumerate(range(0, length, block_q)):
        q_hi = min(q_lo + block_q, length) - 1
        k_first = 0 if left is None else max(0, q_lo - left)
        k_last = length - 1 if right is None else min(length - 1, q_hi + right)
        for col in range(k_first // block_k, k_last // block_k + 1):
            k_lo = col * block_k
            k_hi = min(k_lo + block_k, length) - 1
            full = ((left is None or k_lo >= q_hi - left)
                    and (right is None or k_hi <= q_lo + right))
            if spec.same_document:
                shared = q_sets[row] & k_sets[col]
                if not shared:
                    continue
                uniform = len(q_sets[row]) == 1 and len(k_sets[col]) == 1
                if not uniform and not full and not any_pair(q_lo, q_hi, k_lo, k_hi):
                    continue
                full = full and uniform
            col_idx.append(col)
            full_blocks.append(full)
        row_ptr.append(len(col_idx))
    return BlockSchedule(length, block_q, block_k, row_ptr, col_idx, full_blocks)


def strided_schedule(length: int, block: int = 128, stride: int = 4,
                     local_blocks: int = 1) -> tuple[BlockSchedule, MaskSpec]:
    """Causal "local + strided" block pattern: query block i keeps key block j <= i
    when ``i - j < local_blocks`` or ``(i - j) % stride == 0``.  Returns the
    schedule together with the causal spec that masks the diagonal blocks."""
    _require_int("length", length, 1)
    _require_int("stride", stride, 1)
    _require_int("local_blocks", local_blocks, 1)
    if block not in BLOCK_SIZES:
        raise ValueError("block must be one of 16, 32, 64, 128")
    blocks = -(-length // block)
    row_ptr, col_idx, full_blocks = [0], [], []
    for i in range(blocks):
        for j in range(i + 1):
            if i - j < local_blocks or (i - j) % stride == 0:
                col_idx.append(j)
                full_blocks.append(j < i)
        row_ptr.append(len(col_idx))
    return (BlockSchedule(length, block, block, row_ptr, col_idx, full_blocks),
            MaskSpec(causal=True))


def validate_schedule(schedule: BlockSchedule) -> tuple[int, int]:
    """Structural checks (types, ranges, sorted unique columns); returns tile counts."""
    limit = (1 << 31) - 1

    def integer(name, value, minimum=0):
        if isinstance(value, bool) or not isinstance(value, int):
            raise TypeError(f"{name} must be an integer (bool is not accepted)")
        if not minimum <= value <= limit:
            raise ValueError(f"{name} must be in [{minimum}, {limit}]")

    integer("schedule.length", schedule.length, 1)
    integer("schedule.block_q", schedule.block_q, 1)
    integer("schedule.block_k", schedule.block_k, 1)
    if schedule.block_q not in BLOCK_SIZES or schedule.block_k not in BLOCK_SIZES:
        raise ValueError("block_q and block_k must each be one of 16, 32, 64, 128")
    for value in schedule.row_ptr:
        integer("row_ptr entry", value)
    for value in schedule.col_idx:
        integer("col_idx entry", value)
    if any(not isinstance(flag, bool) for flag in schedule.full_blocks):
        raise TypeError("full_blocks entries must be bool values")
    q_tiles = -(-schedule.length // schedule.block_q)
    k_tiles = -(-schedule.length // schedule.block_k)
    row_ptr, col_idx = list(schedule.row_ptr), list(schedule.col_idx)
    consistent = (len(row_ptr) == q_tiles + 1 and row_ptr[0] == 0 and row_ptr[-1] == len(col_idx)
                  and len(schedule.full_blocks) == len(col_idx)
                  and all(a <= b for a, b in zip(row_ptr, row_ptr[1:]))
                  and all(c < k_tiles for c in col_idx))
    if not consistent:
        raise ValueError("invalid CSR block schedule")
    for begin, end in zip(row_ptr, row_ptr[1:]):
        columns = col_idx[begin:end]
        if any(a >= b for a, b in zip(columns, columns[1:])):
            raise ValueError("CSR columns must be sorted and unique in each row")
    return q_tiles, k_tiles


@dataclass
class KernelSchedule:
    """A schedule regrouped to 128 x 128 tiles, with its key-major transpose.

    ``bitmap[e]`` has bit ``qs * 8 + ks`` set when the 16 x 16 sub-block (qs, ks)
    of stored tile ``e`` is retained; ``None`` when every stored tile is complete.
    """

    length: int
    row_ptr: list[int]
    col_idx: list[int]
    full: list[bool]
    bitmap: list[int] | None
    t_row_ptr: list[int] = field(default_factory=list)
    t_col_idx: list[int] = field(default_factory=list)
    t_full: list[bool] = field(default_factory=list)
    t_bitmap: list[int] | None = None

    @property
    def stored_tiles(self) -> int:
        return len(self.col_idx)


def to_kernel_schedule(schedule: BlockSchedule) -> KernelSchedule:
    q_tiles, _ = validate_schedule(schedule)
    length, bq, bk = schedule.length, schedule.block_q, schedule.block_k
    tiles = -(-length // KERNEL_TILE)
    per_q, per_k = KERNEL_TILE // bq, KERNEL_TILE // bk
    sub_q, sub_k = bq // SUB, bk // SUB
    subs_total = -(-length // SUB)
    entries: list[dict[int, list]] = [dict() for _ in range(tiles)]
    for row in range(q_tiles):
        tile_row, in_row = divmod(row, per_q)
        for e in range(schedule.row_ptr[row], schedule.row_ptr[row + 1]):
            col = schedule.col_idx[e]
            tile_col, in_col = divmod(col, per_k)
            slot = entries[tile_row].setdefault(tile_col, [0, True, 0])
            bits = 0
            for qs in range(in_row * sub_q, (in_row + 1) * sub_q):
                for ks in range(in_col * sub_k, (in_col + 1) * sub_k):
                    bits |= 1 << (qs * 8 + ks)
            slot[0] |= bits
            slot[1] = slot[1] and schedule.full_blocks[e]
            slot[2] += 1
    row_ptr, col_idx, full, bitmap = [0], [], [], []
    partial_presence = False
    for tile_row in range(tiles):
        for tile_col in sorted(entries[tile_row]):
            bits, all_full, _ = entries[tile_row][tile_col]
            # Sub-blocks beyond the sequence end count as present (they are masked
            # by the length check anyway) so complete edge tiles stay bitmap-free.
            needed = 0
            for qs in range(8):
                for ks in range(8):
                    if (tile_row * 8 + qs) < subs_total and (tile_col * 8 + ks) < subs_total:
                        needed |= 1 << (qs * 8 + ks)
            complete = (bits & needed) == needed
            if complete:
                bits = (1 << 64) - 1
            else:
                partial_presence = True
            col_idx.append(tile_col)
            full.append(bool(all_full and complete))
            bitmap.append(bits)
        row_ptr.append(len(col_idx))
    result = KernelSchedule(length, row_ptr, col_idx, full, bitmap if partial_presence else None)
    # key-major transpose; bitmaps keep their (query, key) orientation
    columns: list[list[tuple[int, int]]] = [[] for _ in range(tiles)]
    for tile_row in range(tiles):
        for e in range(row_ptr[tile_row], row_ptr[tile_row + 1]):
            columns[col_idx[e]].append((tile_row, e))
    result.t_row_ptr = [0]
    t_bitmap = []
    for tile_col in range(tiles):
        for tile_row, e in columns[tile_col]:
            result.t_col_idx.append(tile_row)
            result.t_full.append(full[e])
            t_bitmap.append(bitmap[e])
        result.t_row_ptr.append(len(result.t_col_idx))
    result.t_bitmap = t_bitmap if partial_presence else None
    return result


def transpose_schedule(schedule: BlockSchedule) -> BlockSchedule:
    """Key-tile-major view of a schedule (rows become key tiles)."""
    q_tiles, k_tiles = validate_schedule(schedule)
    buckets: list[list[tuple[int, bool]]] = [[] for _ in range(k_tiles)]
    for row in range(q_tiles):
        for e in range(schedule.row_ptr[row], schedule.row_ptr[row + 1]):
            buckets[schedule.col_idx[e]].append((row, schedule.full_blocks[e]))
    row_ptr, col_idx, full = [0], [], []
    for bucket in buckets:
        for row, flag in bucket:
            col_idx.append(row)
            full.append(flag)
        row_ptr.append(len(col_idx))
    return BlockSchedule(schedule.length, schedule.block_k, schedule.block_q, row_ptr, col_idx, full)
