"""Background GPU sampler: SM clock, temperature, power and clock-event reasons over time.

An ``nvidia-smi --loop-ms`` child process streams CSV samples; a reader thread stamps each with
``time.monotonic()`` so a benchmark can cut out the samples of one timed window
(cf. nanonemo/utils/gpumon.py:1-143). Nothing here changes a GPU setting: it only reads.

Reason bits (NVML ``nvmlClocksEventReasons``): 0x4 sw_power_cap (normal for a 1 kW part under a
dense GEMM: kept, reported), 0x8 hw_slowdown, 0x20 sw_thermal, 0x40 hw_thermal, 0x80 hw_power_brake.
"""

import os
import subprocess
import threading
import time
from statistics import median

FIELDS = ["clocks.sm", "clocks.mem", "temperature.gpu", "power.draw", "utilization.gpu",
          "clocks_event_reasons.active", "clocks.max.sm"]
SLOWDOWN_REASONS = {0x08: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                    0x80: "hw_power_brake"}
NOTED_REASONS = {0x04: "sw_power_cap"}


def parse_line(line: str) -> dict | None:
    """One ``--format=csv,noheader,nounits`` line -> sample dict, or None if it does not parse."""
    cells = [c.strip() for c in line.split(",")]
    if len(cells) not in (len(FIELDS) - 1, len(FIELDS)):
        return None
    try:
        sample = {"sm_mhz": int(cells[0]), "mem_mhz": int(cells[1]), "temp_c": int(cells[2]),
                  "power_w": float(cells[3]), "util_pct": int(cells[4]), "reasons": int(cells[5], 16)}
        if len(cells) == len(FIELDS):
            sample["sm_max_mhz"] = int(cells[6])
        return sample
    except ValueError:
        return None


class GpuMonitor:
    """``with GpuMonitor(200) as mon: ...; mon.window(t0, t1)``. Records nothing without nvidia-smi."""

    def __init__(self, interval_ms: int = 200, gpu_index: int = 0):
        self.cmd = ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={','.join(FIELDS)}",
                    "--format=csv,noheader,nounits", f"--loop-ms={interval_ms}"]
        self.samples: list[dict] = []
        self._proc = None
        self._thread = None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        self._thread = threading.Thread(target=self._pump, daemon=True)
        self._thread.start()
        return self

    def _pump(self):
        for line in self._proc.stdout:
            s = parse_line(line)
            if s is not None:
                s["t"] = time.monotonic()
                self.samples.append(s)

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()  # the exact child this object started
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            self._thread.join(timeout=2)

    def window(self, t0: float, t1: float) -> list[dict]:
        return [s for s in self.samples if t0 <= s["t"] <= t1]


def summarize(samples: list[dict]) -> dict:
    if not samples:
        return {"n_samples": 0}
    sm = [s["sm_mhz"] for s in samples]
    mask = 0
    for s in samples:
        mask |= s["reasons"]
    out = {
        "n_samples": len(samples),
        "sm_mhz": {"median": median(sm), "min": min(sm), "max": max(sm)},
        "mem_mhz_median": median(s["mem_mhz"] for s in samples),
        "temp_c": {"median": median(s["temp_c"] for s in samples), "max": max(s["temp_c"] for s in samples)},
        "power_w_median": median(s["power_w"] for s in samples),
        "util_pct_median": median(s["util_pct"] for s in samples),
        "slowdown_reasons": [n for bit, n in SLOWDOWN_REASONS.items() if mask & bit],
        "noted_reasons": [n for bit, n in NOTED_REASONS.items() if mask & bit],
        "reasons_mask": hex(mask),
    }
    mx = [s["sm_max_mhz"] for s in samples if "sm_max_mhz" in s]
    if mx:
        out["sm_max_mhz"] = max(mx)
    return out


def clocks_record(samples: list[dict]) -> dict:
    """The compact ``clocks`` entry of a benchmark line: median SM MHz under load, max, active reasons."""
    s = summarize(samples)
    if not s["n_samples"]:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "n_samples": 0}
    return {"sm_mhz": s["sm_mhz"]["median"], "sm_max_mhz": s.get("sm_max_mhz"),
            "reasons": s["slowdown_reasons"] + s["noted_reasons"], "n_samples": s["n_samples"],
            "power_w": s["power_w_median"]}


def locked_sm_mhz() -> int | None:
    """SM clock the operator declares the GPU was locked to (NANONEMO_LOCKED_SM_MHZ); None = floating.
    Only read here: this framework never sets or resets clocks."""
    v = os.environ.get("NANONEMO_LOCKED_SM_MHZ")
    return int(v) if v else None


def clock_floor(locked: int | None, device_name: str) -> int | None:
    from nanonemo_b200.utils.mfu import rated_boost_mhz

    return int(locked * 0.98) if locked else rated_boost_mhz(device_name)


def throttle_flags(trials: list[dict], tol: float = 0.10, min_mhz: int | None = None) -> list[str]:
    """Reasons to distrust a set of trial summaries; [] means clean. Flags: a trial whose median SM
    clock is > tol below the median over trials, a median below `min_mhz`, any slowdown reason."""
    live = [t for t in trials if t.get("n_samples")]
    if not live:
        return ["no GPU samples"]
    ref = median(t["sm_mhz"]["median"] for t in live)
    flags = []
    for i, t in enumerate(trials):
        if not t.get("n_samples"):
            flags.append(f"trial {i}: no GPU samples")
            continue
        med = t["sm_mhz"]["median"]
        if med < (1 - tol) * ref:
            flags.append(f"trial {i}: median SM clock {med:.0f} MHz (median of trials {ref:.0f})")
        if min_mhz and med < min_mhz:
            flags.append(f"trial {i}: median SM clock {med:.0f} MHz is below the floor {min_mhz}")
        if t["slowdown_reasons"]:
            flags.append(f"trial {i}: {', '.join(t['slowdown_reasons'])}")
    return flags
