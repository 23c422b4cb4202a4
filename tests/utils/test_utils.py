"""GPU monitor parsing / throttle rules, MFU arithmetic, environment capture."""

import json

import pytest

from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.utils import gpumon, mfu
from nanonemo_b200.utils.env import capture_env, gpu_slug


def test_parse_line():
    s = gpumon.parse_line("1965, 3996, 41, 702.31, 100, 0x0000000000000004, 1965")
    assert s == {"sm_mhz": 1965, "mem_mhz": 3996, "temp_c": 41, "power_w": 702.31, "util_pct": 100, "reasons": 4, "sm_max_mhz": 1965}
    assert gpumon.parse_line("1965, 3996, 41, [N/A], 100, 0x0, 1965") is None
    assert gpumon.parse_line("garbage") is None


def samples(mhz, reasons=0, n=10):
    return [{"sm_mhz": mhz, "mem_mhz": 3996, "temp_c": 50, "power_w": 900.0, "util_pct": 100, "reasons": reasons,
             "sm_max_mhz": 1965, "t": float(i)} for i in range(n)]


def test_summarize_and_clocks_record():
    s = gpumon.summarize(samples(1500, 0x4) + samples(1300, 0x4))
    assert s["sm_mhz"] == {"median": 1400.0, "min": 1300, "max": 1500} and s["slowdown_reasons"] == [] and s["noted_reasons"] == ["sw_power_cap"]
    rec = gpumon.clocks_record(samples(1300, 0x4 | 0x40))
    assert rec["sm_mhz"] == 1300 and rec["sm_max_mhz"] == 1965 and set(rec["reasons"]) == {"hw_thermal_slowdown", "sw_power_cap"}
    assert gpumon.summarize([]) == {"n_samples": 0} and gpumon.clocks_record([])["n_samples"] == 0


def test_throttle_flags(monkeypatch):
    ok = [gpumon.summarize(samples(1500)) for _ in range(3)]
    assert gpumon.throttle_flags(ok) == []
    assert any("median SM clock" in f for f in gpumon.throttle_flags(ok[:2] + [gpumon.summarize(samples(1100))]))
    assert any("hw_slowdown" in f for f in gpumon.throttle_flags(ok[:2] + [gpumon.summarize(samples(1500, 0x8))]))
    assert gpumon.throttle_flags([{"n_samples": 0}]) == ["no GPU samples"]
    assert any("floor" in f for f in gpumon.throttle_flags(ok, min_mhz=1600))
    monkeypatch.setenv("NANONEMO_LOCKED_SM_MHZ", "1140")
    assert gpumon.locked_sm_mhz() == 1140 and gpumon.clock_floor(1140, "anything") == 1117
    monkeypatch.delenv("NANONEMO_LOCKED_SM_MHZ")
    assert gpumon.locked_sm_mhz() is None and gpumon.clock_floor(None, "NVIDIA GeForce RTX 2070 SUPER") == 1380


def test_monitor_without_nvidia_smi_records_nothing(monkeypatch):
    monkeypatch.setenv("PATH", "/nonexistent")
    with gpumon.GpuMonitor(50) as mon:
        pass
    assert mon.samples == []


def test_flops_and_mfu():
    cfg = ModelConfig()
    assert mfu.flops_per_token(cfg, 1024) == 798_031_872
    from nanonemo_b200.models.model import NanoNemo

    small = ModelConfig(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, d_ff=128, vocab_size=512, max_seq_len=32)
    model = NanoNemo(small)
    assert mfu.matmul_params(small) == sum(p.numel() for p in model.parameters() if p.dim() == 2)
    assert mfu.mfu(1000.0, 10**9, 2.0) == pytest.approx(0.5)
    assert mfu.peak_tflops("NVIDIA B200")["bf16_tc"] == 2250.0 and mfu.peak_tflops("Tesla T4")["fp16_tc"] == 65.0
    assert mfu.peak_tflops("NVIDIA H100") is None and mfu.peak_gbps("Tesla T4") == 320.0
    assert mfu.peak_tflops("NVIDIA GeForce RTX 2070 SUPER Laptop GPU")["fp32"] == 7.07


def test_env_is_json_serialisable():
    env = capture_env()
    json.dumps(env)
    assert {"timestamp", "torch", "git", "devices"} <= set(env) and isinstance(gpu_slug(), str)
