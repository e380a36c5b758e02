"""Host-side pieces of the measurement tools: roofline denominators, cold-cache planning of
the decode study, the three-variant decode summary, and the microbench command line."""

import json

import pytest

from systems_for_llms_b200.attention import decode_study
from systems_for_llms_b200.ops import microbench


def test_roofline_denominators_come_from_the_measured_file_or_the_fallback(tmp_path, monkeypatch):
    values, label = microbench.peaks()
    assert label in ("of measured", "of fallback")
    assert set(values) == set(microbench.FALLBACK_PEAKS) and all(v > 0 for v in values.values())
    # a file without the three keys is ignored
    fake = tmp_path / "pkg" / "ops" / "microbench.py"
    fake.parent.mkdir(parents=True)
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 1.0}))
    monkeypatch.setattr(microbench, "__file__", str(fake))
    assert microbench.peaks() == (microbench.FALLBACK_PEAKS, "of fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"hbm_gbs": 6000, "bf16_tflops": 1600, "bf16_tflops_sustained": 1300, "note": "x"}))
    assert microbench.peaks() == ({"hbm_gbs": 6000.0, "bf16_tflops": 1600.0,
                                   "bf16_tflops_sustained": 1300.0}, "of measured")


def test_cold_copies_cover_twice_the_l2_and_are_bounded():
    l2 = decode_study.L2_BYTES
    assert decode_study.cold_copies(4 * l2) == 1          # one copy already exceeds the cache
    assert decode_study.cold_copies(l2) == 2
    assert decode_study.cold_copies(l2 // 8) == 16
    assert decode_study.cold_copies(1) == 64              # tiny caches: capped
    assert decode_study.cold_copies(0) == 64


def test_decode_summary_ranks_all_three_variants():
    timings = {}
    for variant, base in (("token", 4.0), ("tile", 2.0), ("mma", 1.0)):
        for splits in decode_study.STUDY_SPLITS:
            timings[f"cuda_{variant}_split_{splits}"] = {"median_ms": base / min(splits, 4) + 0.02 * splits}
    timings["sdpa_flash"] = {"median_ms": 0.4}
    record = {"timings": timings, "cache_bytes": 1 << 26}
    decode_study.summarise_case(record)
    assert record["best_observed"] == "cuda_mma_split_4"
    assert record["best_observed_by_variant"] == {"token": "cuda_token_split_4",
                                                  "tile": "cuda_tile_split_4",
                                                  "mma": "cuda_mma_split_4"}
    assert record["speedups"]["sdpa_flash"] == pytest.approx(0.4 / (0.25 + 0.08))
    assert record["best_tile_over_best_token"] == pytest.approx((1.0 + 0.08) / (0.5 + 0.08))
    assert decode_study.VARIANTS == decode_study.REFERENCE_VARIANTS + ("mma",)


def test_microbench_command_line(monkeypatch, capsys):
    monkeypatch.setattr("sys.argv", ["microbench", "no-such-suite"])
    with pytest.raises(SystemExit):
        microbench.main()
    assert "invalid choice" in capsys.readouterr().err
    for name in ("gemm", "attention", "elementwise", "decode"):
        assert name in microbench.SUITES
