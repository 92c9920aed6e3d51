"""Tracing helpers: no-op NVTX ranges without a device, section timers, roofline arithmetic."""

import json
import time

import pytest
import torch

from ohara_b200.utils import profiling
from ohara_b200.utils.profiling import DeviceTimer, Peaks, load_peaks, nvtx_annotate, nvtx_range, roofline


def test_nvtx_ranges_are_shared_no_ops_when_disabled():
    profiling.enable_nvtx(False)
    assert nvtx_range("a") is nvtx_range("b")
    with nvtx_range("phase"):
        pass

    @nvtx_annotate("fn")
    def double(x):
        """doc"""
        return 2 * x

    assert double(4) == 8 and double.__doc__ == "doc"
    profiling.enable_nvtx(True)  # still a no-op without a CUDA device
    try:
        if not torch.cuda.is_available():
            assert nvtx_range("a") is nvtx_range("b")
        assert double(5) == 10
    finally:
        profiling.enable_nvtx(False)


def test_device_timer_accumulates_sections_on_the_host():
    timer = DeviceTimer("cpu")
    for _ in range(3):
        with timer.section("work"):
            time.sleep(0.01)
    with timer.section("other"):
        pass
    summary = timer.summary()
    assert summary["work"]["calls"] == 3 and summary["work"]["ms"] >= 25.0
    assert summary["other"]["calls"] == 1 and summary["other"]["ms"] < summary["work"]["ms"]
    timer.reset()
    assert timer.summary() == {}


def test_section_is_closed_when_the_body_raises():
    timer = DeviceTimer("cpu")
    with pytest.raises(RuntimeError):
        with timer.section("boom"):
            raise RuntimeError("x")
    assert timer.summary()["boom"]["calls"] == 1


def test_peaks_are_read_from_the_file_or_fall_back(tmp_path, monkeypatch):
    path = tmp_path / "peaks.json"
    path.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1200.0}))
    peaks = load_peaks(path)
    assert (peaks.hbm_gbs, peaks.bf16_tflops, peaks.bf16_tflops_sustained, peaks.source) == (
        6000.0, 1500.0, 1200.0, "measured")
    monkeypatch.setenv("OHARA_MEASURED_PEAKS", str(tmp_path / "missing.json"))
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    assert load_peaks(bad).source in ("measured", "fallback")  # falls through to the next candidate


def test_roofline_picks_the_binding_resource():
    peaks = Peaks(hbm_gbs=5000.0, bf16_tflops=1000.0, bf16_tflops_sustained=800.0, nvlink_gbs=500.0,
                  source="measured")
    # 1e12 FLOPs = 1 ms of compute, 1e9 bytes = 0.2 ms of HBM, 1e9 bytes over NVLink = 2 ms
    report = roofline(4.0, flops=1e12, hbm_bytes=1e9, nvlink_bytes=1e9, peaks=peaks)
    assert report["bound"] == "nvlink" and report["bound_ms"] == pytest.approx(2.0)
    assert report["fraction"] == pytest.approx(0.5) and report["peaks"] == "of measured"
    assert report["achieved_tflops"] == pytest.approx(250.0)
    report = roofline(2.0, flops=1e12, hbm_bytes=1e9, sustained=True, peaks=peaks)
    assert report["bound"] == "compute" and report["compute_ms"] == pytest.approx(1.25)
    report = roofline(1.0, hbm_bytes=2.5e9, peaks=peaks)
    assert report["bound"] == "hbm" and report["fraction"] == pytest.approx(0.5)
    with pytest.raises(ValueError):
        roofline(0.0, flops=1.0, peaks=peaks)
