"""Mask compiler against an independent dense oracle (CPU)."""

import random

import pytest

from systems_for_llms_b200.attention.flash import interval_regions
from systems_for_llms_b200.attention.masks import (BlockSchedule, MaskSpec, allows, compile_mask,
                                                   strided_schedule, to_kernel_schedule,
                                                   transpose_schedule, validate_schedule)


def dense(length, spec, docs=None):
    def ok(q, k):
        if spec.causal and k > q:
            return False
        if spec.window_left is not None and k < q - spec.window_left:
            return False
        if spec.window_right is not None and k > q + spec.window_right:
            return False
        return not spec.same_document or docs[q] == docs[k]
    return [[ok(q, k) for k in range(length)] for q in range(length)]


def classify(mask, length, bq, bk, row, col):
    cells = [mask[q][k] for q in range(row * bq, min(length, (row + 1) * bq))
             for k in range(col * bk, min(length, (col + 1) * bk))]
    return any(cells), all(cells)


SPECS = [MaskSpec(), MaskSpec(causal=True), MaskSpec(causal=True, window_left=5),
         MaskSpec(window_left=3, window_right=2), MaskSpec(window_right=0), MaskSpec(window_left=0),
         MaskSpec(causal=True, window_left=0), MaskSpec(causal=True, window_right=7)]


@pytest.mark.parametrize("spec", SPECS)
@pytest.mark.parametrize("length", [1, 7, 16, 33])
@pytest.mark.parametrize("bq,bk", [(4, 4), (8, 4), (4, 16), (16, 16)])
def test_schedule_matches_dense_oracle(spec, length, bq, bk):
    mask = dense(length, spec)
    schedule = compile_mask(length, spec, bq, bk)
    rows = -(-length // bq)
    cols = -(-length // bk)
    assert len(schedule.row_ptr) == rows + 1
    for row in range(rows):
        stored = dict(zip(schedule.col_idx[schedule.row_ptr[row]:schedule.row_ptr[row + 1]],
                          schedule.full_blocks[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]))
        assert list(stored) == sorted(stored)
        for col in range(cols):
            nonempty, full = classify(mask, length, bq, bk, row, col)
            assert (col in stored) == nonempty
            if nonempty:
                assert stored[col] == full


@pytest.mark.parametrize("seed", range(6))
def test_random_documents(seed):
    rng = random.Random(seed)
    length = rng.choice([17, 32, 45])
    docs = [rng.randrange(3) for _ in range(length)]
    if seed % 2:
        docs = sorted(docs)
    spec = MaskSpec(causal=bool(seed % 3), window_left=rng.choice([None, 4, 9]),
                    same_document=True)
    mask = dense(length, spec, docs)
    bq, bk = rng.choice([(4, 8), (8, 8), (16, 4)])
    schedule = compile_mask(length, spec, bq, bk, docs)
    for row in range(-(-length // bq)):
        stored = dict(zip(schedule.col_idx[schedule.row_ptr[row]:schedule.row_ptr[row + 1]],
                          schedule.full_blocks[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]))
        for col in range(-(-length // bk)):
            nonempty, full = classify(mask, length, bq, bk, row, col)
            assert (col in stored) == nonempty
            if nonempty:
                assert stored[col] == full
    for q in range(length):
        for k in range(length):
            assert allows(q, k, spec, docs) == mask[q][k]


def test_long_window_without_dense_mask():
    schedule = compile_mask(100_000, MaskSpec(causal=True, window_left=127), 64, 64)
    assert len(schedule.col_idx) < 3 * len(schedule.row_ptr)


@pytest.mark.parametrize("spec", [s for s in SPECS])
@pytest.mark.parametrize("length,bq,bk", [(50, 8, 8), (64, 16, 8), (37, 4, 16)])
def test_interval_regions_equal_csr(spec, length, bq, bk):
    schedule = compile_mask(length, spec, bq, bk)
    for row in range(-(-length // bq)):
        begin, full_begin, full_end, end = interval_regions(length, spec, bq, bk, row)
        cols = schedule.col_idx[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]
        flags = schedule.full_blocks[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]
        assert cols == list(range(begin, end))
        for col, flag in zip(cols, flags):
            if full_begin <= col < full_end:
                assert flag
            # tiles outside the full range may still be full only at ragged edges
            if not flag:
                assert not (full_begin <= col < full_end)


def test_interval_rejects_documents_and_bad_arguments():
    with pytest.raises(ValueError):
        interval_regions(16, MaskSpec(same_document=True), 4, 4, 0)
    with pytest.raises(ValueError):
        interval_regions(16, MaskSpec(), 4, 4, 4)
    with pytest.raises(ValueError):
        interval_regions(0, MaskSpec(), 4, 4, 0)


def test_argument_validation():
    with pytest.raises(TypeError):
        MaskSpec(causal=1)
    with pytest.raises(ValueError):
        MaskSpec(window_left=-1)
    with pytest.raises(TypeError):
        MaskSpec(window_right=True)
    with pytest.raises(ValueError):
        compile_mask(8, MaskSpec(same_document=True))
    with pytest.raises(ValueError):
        compile_mask(8, MaskSpec(same_document=True), document_ids=[0] * 7)
    with pytest.raises(TypeError):
        compile_mask(8, MaskSpec(same_document=True), document_ids=[0.5] * 8)
    with pytest.raises(TypeError):
        compile_mask(8, "causal")


def test_validate_schedule_rejects_malformed():
    good = compile_mask(64, MaskSpec(causal=True), 16, 16)
    validate_schedule(good)
    bad = BlockSchedule(64, 16, 16, good.row_ptr, list(reversed(good.col_idx)), good.full_blocks)
    with pytest.raises(ValueError):
        validate_schedule(bad)
    with pytest.raises(ValueError):
        validate_schedule(BlockSchedule(64, 24, 16, good.row_ptr, good.col_idx, good.full_blocks))
    with pytest.raises(TypeError):
        validate_schedule(BlockSchedule(64, 16, 16, good.row_ptr, good.col_idx,
                                        [1] * len(good.col_idx)))


def expand(ks, length):
    """Dense presence/full maps at 16x16 granularity from a kernel schedule."""
    subs = -(-length // 16)
    present = [[False] * subs for _ in range(subs)]
    for row in range(len(ks.row_ptr) - 1):
        for e in range(ks.row_ptr[row], ks.row_ptr[row + 1]):
            bits = ks.bitmap[e] if ks.bitmap is not None else (1 << 64) - 1
            for qs in range(8):
                for kk in range(8):
                    q, k = row * 8 + qs, ks.col_idx[e] * 8 + kk
                    if q < subs and k < subs and (bits >> (qs * 8 + kk)) & 1:
                        present[q][k] = True
    return present


@pytest.mark.parametrize("bq,bk", [(16, 16), (32, 64), (64, 32), (128, 128), (16, 128)])
def test_kernel_schedule_preserves_presence(bq, bk):
    length = 300
    spec = MaskSpec(causal=True, window_left=100)
    schedule = compile_mask(length, spec, bq, bk)
    ks = to_kernel_schedule(schedule)
    present = expand(ks, length)
    subs = -(-length // 16)
    for q in range(subs):
        for k in range(subs):
            row, col = (q * 16) // bq, (k * 16) // bk
            cols = schedule.col_idx[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]
            assert present[q][k] == (col in cols)
    # transpose lists the same tiles
    pairs = {(r, ks.col_idx[e]) for r in range(len(ks.row_ptr) - 1)
             for e in range(ks.row_ptr[r], ks.row_ptr[r + 1])}
    t_pairs = {(ks.t_col_idx[e], c) for c in range(len(ks.t_row_ptr) - 1)
               for e in range(ks.t_row_ptr[c], ks.t_row_ptr[c + 1])}
    assert pairs == t_pairs


def test_strided_schedule_and_transpose():
    schedule, spec = strided_schedule(1024, 64, stride=4, local_blocks=2)
    assert spec.causal
    validate_schedule(schedule)
    row = 9
    cols = schedule.col_idx[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]
    assert cols == [1, 5, 8, 9]
    back = transpose_schedule(transpose_schedule(schedule))
    assert back.row_ptr == schedule.row_ptr and back.col_idx == schedule.col_idx
