"""scripts/make_figures.py builds its tables from results/ JSON only (nothing is measured); works without matplotlib."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


def test_tables_from_results_only(tmp_path):
    ladder = tmp_path / "results" / "ladder" / "b200"
    ladder.mkdir(parents=True)
    for i, name in enumerate(("s0_fp32", "s1_fp16")):
        (ladder / f"{name}.json").write_text(json.dumps({"tokens_per_s": {"median": 1000.0 * (i + 1)}, "step_ms": {"median": 16.0 / (i + 1)}}))
    dist = tmp_path / "results" / "dist" / "b200-x2"
    dist.mkdir(parents=True)
    (dist / "ddp.json").write_text(json.dumps({"tokens_per_s": {"median": 5000.0}, "bench": {"world": 2}}))
    kern = tmp_path / "results" / "kernels"
    kern.mkdir(parents=True)
    (kern / "gemm.json").write_text(json.dumps({"device": "B200", "rows": [{"shape": "qkv", "ours_ms": 0.1}]}))
    out = tmp_path / "figures"
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "make_figures.py"), "--results", str(tmp_path / "results"), "--out", str(out)],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    text = (out / "tables.md").read_text()
    assert "| b200 | s0_fp32 | 1,000 | 16.00 |" in text and "| b200-x2 | ddp | 5,000 | 2 |" in text and "| qkv | 0.1 |" in text
    # figures are plain SVG files: one bar per ladder stage, one per multi-GPU row
    bars = (out / "ladder_tokens_per_s.svg").read_text()
    assert bars.startswith("<svg") and bars.count("<rect") == 1 + 2 and "s1_fp16" in bars and (out / "dist_tokens_per_s.svg").exists()
    # the README block between the markers is regenerated from the same tables, text around it is kept
    readme = tmp_path / "README.md"
    readme.write_text("intro\n<!-- results:begin -->\nstale number 123\n<!-- results:end -->\noutro\n")
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / "make_figures.py"), "--results", str(tmp_path / "results"), "--out", str(out),
                        "--readme", str(readme)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    new = readme.read_text()
    assert new.startswith("intro\n") and new.endswith("outro\n") and "stale number" not in new and "| b200 | s1_fp16 | 2,000 | 8.00 |" in new


def test_loss_curve_and_tick_values(tmp_path):
    import importlib.util

    spec = importlib.util.spec_from_file_location("make_figures", ROOT / "scripts" / "make_figures.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.nice_ticks(0.0, 950_000.0) == [0.0, 200000.0, 400000.0, 600000.0, 800000.0, 1000000.0]
    assert mod.nice_ticks(3.2, 10.9)[0] <= 3.2 and mod.nice_ticks(3.2, 10.9)[-1] >= 10.9
    assert mod.human(1_500_000.0) == "1.5M" and mod.human(12.0) == "12"
    metrics = tmp_path / "metrics.jsonl"
    recs = [{"step": i, "tokens": (i + 1) * 1000, "loss": 10.0 - 0.1 * i} for i in range(20)] + [{"step": 9, "val_loss": 9.3}]
    metrics.write_text("\n".join(json.dumps(r) for r in recs) + "\n")
    (tmp_path / "results").mkdir()
    mod.main(["--results", str(tmp_path / "results"), "--out", str(tmp_path / "fig"), "--metrics", str(metrics)])
    svg = (tmp_path / "fig" / "loss.svg").read_text()
    assert svg.count("<path") == 2 and ">train<" in svg and ">val<" in svg


def test_nvtx_spans_are_noops_without_cuda(monkeypatch):
    from nanonemo_b200.utils import nvtx

    monkeypatch.setattr(nvtx, "_ON", None)
    monkeypatch.setenv("NANONEMO_NVTX", "1")
    with nvtx.span("forward"):
        x = 1 + 1
    assert x == 2


def test_step_breakdown_groups_kernel_names():
    import importlib.util

    spec = importlib.util.spec_from_file_location("step_breakdown", ROOT / "scripts" / "step_breakdown.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.group_of("(anonymous namespace)::gemm2_tcgen05_kernel(CUtensorMap_st)") == "tcgen05 GEMM (CTA pair)"
    assert mod.group_of("void (anonymous namespace)::gemm_tcgen05_kernel<256, false>(...)") == "tcgen05 GEMM (single CTA)"
    assert mod.group_of("(anonymous namespace)::flash_delta_kernel(...)") == "flash attention backward"
    assert mod.group_of("void add_rmsnorm_bwd_kernel<float, __nv_bfloat16, __nv_bfloat16, 3>") == "add + RMSNorm"
    assert mod.group_of("ncclDevKernel_AllReduce_Sum_f32_RING_LL") == "collectives"
    assert mod.group_of("something_else") == "other"


def test_timeline_report_finds_gaps_and_exposed_collective_time():
    import importlib.util

    spec = importlib.util.spec_from_file_location("step_breakdown", ROOT / "scripts" / "step_breakdown.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    k = lambda name, ts, dur, stream: {"ph": "X", "cat": "kernel", "name": name, "ts": ts, "dur": dur, "args": {"stream": stream}}
    # compute stream 7: busy 0-100, idle 100-150, busy 150-250; an all-reduce on stream 9 runs 80-140 (40 us of it in the gap)
    events = [k("gemm2_tcgen05_kernel<0>", 0, 100, 7), k("adamw_flat_kernel", 150, 100, 7), k("allreduce_f32_kernel<2, 4>", 80, 60, 9),
              {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 5}]
    lines = mod.timeline_report(events, steps=1)
    assert "wall 0.25 ms / step" in lines[0] and "compute stream busy 0.20" in lines[0] and "compute stream idle 0.05" in lines[0]
    assert "collective kernels 0.06 of which exposed (compute stream idle) 0.04" in lines[0]
    assert "50.0" in lines[2] and "allreduce_f32_kernel" in lines[2]
