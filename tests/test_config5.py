"""Host-side logic of the block-sparse attention table (no GPU: workers injected)."""

import pytest

from systems_for_llms_b200.attention import config5, decode_study


def fake_check(name, length, dim):
    density = {"causal": 0.5, "window": 0.25, "strided": 0.2}[name]
    return {"mask": name, "length": length, "density": density, "errors": {}, "correct": True}


def fake_ours(name, length, *, batch, heads, dim):
    return {"mask": name, "length": length, "forward_ms": 1.0, "backward_ms": 3.0}


def fake_sdpa(length, *, batch, heads, dim):
    return {"length": length, "forward_ms": 2.0, "forward_backward_ms": 6.0}


def test_run_orders_checks_before_timing_and_tabulates():
    order = []

    def check(name, length, dim):
        order.append(("check", name, length))
        return fake_check(name, length, dim)

    def ours(name, length, **kw):
        order.append(("time", name, length))
        return fake_ours(name, length, **kw)

    records = config5.run(lengths=(1024, 4096), masks=("causal", "strided"), check=check,
                          time_ours=ours, time_baseline=fake_sdpa)
    first_timing = next(i for i, item in enumerate(order) if item[0] == "time")
    assert all(item[0] == "check" for item in order[:first_timing])
    assert len(records["cases"]) == 4 and len(records["sdpa"]) == 2
    rows = records["table"].splitlines()
    assert len(rows) == 2 + 4
    # causal, N = 1024: 4*8*16*1024^2*64*0.5 FLOP in 1 ms forward, 3.5x in 4 ms both ways
    cells = [c.strip() for c in rows[2].strip("|").split("|")]
    work = config5.flops(8, 16, 1024, 64, 0.5)
    assert cells[:3] == ["1024", "causal", "0.500"]
    assert float(cells[5]) == pytest.approx(work / 1e9, abs=0.5)
    assert float(cells[6]) == pytest.approx(3.5 * work / 4.0 / 1e9, abs=0.5)
    assert cells[-1] == "2.00, 1.50"


def test_failed_check_stops_before_any_timing():
    def bad(name, length, dim):
        return {**fake_check(name, length, dim), "correct": False}

    def never(*a, **k):
        raise AssertionError("timed a kernel that failed its check")

    with pytest.raises(RuntimeError, match="correctness"):
        config5.run(lengths=(1024,), masks=("causal",), check=bad, time_ours=never,
                    time_baseline=never)


def test_input_sets_exceed_twice_the_l2():
    small = 8 * 16 * 1024 * 64 * 2 * 9
    sets = config5.input_sets(small)
    assert sets * small >= 2 * config5.L2_BYTES
    assert config5.input_sets(10 * config5.L2_BYTES) == 1
    assert decode_study.cold_copies(33_554_432) * 33_554_432 >= 2 * decode_study.L2_BYTES
    assert decode_study.cold_copies(1 << 30) == 1


def test_named_masks():
    spec, schedule, implementation = config5.mask_for("window", 512, window=1023)
    assert spec.causal and spec.window_left == 511 and schedule is None
    spec, schedule, implementation = config5.mask_for("strided", 1024)
    assert implementation == "csr" and schedule.length == 1024
    with pytest.raises(ValueError):
        config5.mask_for("banded", 1024)
