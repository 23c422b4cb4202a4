"""Clock / power / temperature trace of one GPU while a benchmark runs, and the rules that decide whether
the numbers measured under that trace can be trusted.

A child ``nvidia-smi --loop-ms`` process prints one CSV row per interval; a reader thread turns each row into
a sample and stamps it with ``time.monotonic()``, the clock the benchmark uses for its timed windows, so
``window(t0, t1)`` returns exactly the samples taken while the timed steps ran. Everything here READS the
GPU's state; nothing sets or resets a clock, a power limit or any other setting.

Columns and the verdict rules are tables (``COLUMNS``, ``REASON_BITS``): the row parser, the summary and the
flag messages are all driven by them. Reason bits are NVML's ``nvmlClocksEventReasons``: ``sw_power_cap``
(0x4) is the normal state of a 1 kW part under dense GEMMs and is only noted; ``hw_slowdown`` (0x8),
``sw_thermal_slowdown`` (0x20), ``hw_thermal_slowdown`` (0x40) and ``hw_power_brake`` (0x80) invalidate a
measurement. Same role as the reference's monitor (nanonemo/utils/gpumon.py:1-143).
"""

import bisect
import os
import subprocess
import threading
import time
from statistics import median

# (nvidia-smi query field, key in a sample, text -> value); the last column is optional in a row
COLUMNS = (
    ("clocks.sm", "sm_mhz", int),
    ("clocks.mem", "mem_mhz", int),
    ("temperature.gpu", "temp_c", int),
    ("power.draw", "power_w", float),
    ("utilization.gpu", "util_pct", int),
    ("clocks_event_reasons.active", "reasons", lambda text: int(text, 16)),
    ("clocks.max.sm", "sm_max_mhz", int),
)
FIELDS = [c[0] for c in COLUMNS]
# bit -> (name, invalidates the measurement)
REASON_BITS = {0x04: ("sw_power_cap", False), 0x08: ("hw_slowdown", True), 0x20: ("sw_thermal_slowdown", True),
               0x40: ("hw_thermal_slowdown", True), 0x80: ("hw_power_brake", True)}
SLOWDOWN_REASONS = {bit: name for bit, (name, bad) in REASON_BITS.items() if bad}
NOTED_REASONS = {bit: name for bit, (name, bad) in REASON_BITS.items() if not bad}


def parse_line(line: str) -> dict | None:
    """One ``--format=csv,noheader,nounits`` row -> sample; None for anything that is not a complete row
    (a header, ``[N/A]`` cells, a truncated line)."""
    cells = [cell.strip() for cell in line.split(",")]
    if not len(COLUMNS) - 1 <= len(cells) <= len(COLUMNS):
        return None
    sample = {}
    for (_, key, convert), cell in zip(COLUMNS, cells):
        try:
            sample[key] = convert(cell)
        except ValueError:
            return None
    return sample


class GpuMonitor:
    """``with GpuMonitor(200, gpu_index=0) as mon: ...`` then ``mon.window(t0, t1)`` (``time.monotonic()`` bounds).
    Without nvidia-smi on the PATH the trace simply stays empty."""

    def __init__(self, interval_ms: int = 200, gpu_index: int = 0):
        self.cmd = ["nvidia-smi", f"--id={gpu_index}", "--query-gpu=" + ",".join(FIELDS), "--format=csv,noheader,nounits",
                    f"--loop-ms={interval_ms}"]
        self.samples: list[dict] = []
        self._stamps: list[float] = []   # parallel to samples, ascending: window() bisects it
        self._lock = threading.Lock()
        self._child = None
        self._reader = None

    def start(self) -> "GpuMonitor":
        try:
            self._child = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._child = None
            return self
        self._reader = threading.Thread(target=self._drain, args=(self._child.stdout,), daemon=True)
        self._reader.start()
        return self

    def stop(self) -> None:
        child, self._child = self._child, None
        if child is None:
            return
        child.terminate()  # exactly the process this object started
        try:
            child.wait(timeout=5)
        except subprocess.TimeoutExpired:
            child.kill()
        if self._reader is not None:
            self._reader.join(timeout=2)

    def _drain(self, stream) -> None:
        for row in stream:
            sample = parse_line(row)
            if sample is None:
                continue
            now = time.monotonic()
            sample["t"] = now
            with self._lock:
                self.samples.append(sample)
                self._stamps.append(now)

    def window(self, t0: float, t1: float) -> list[dict]:
        with self._lock:
            lo, hi = bisect.bisect_left(self._stamps, t0), bisect.bisect_right(self._stamps, t1)
            return self.samples[lo:hi]

    def __enter__(self) -> "GpuMonitor":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()


def _column(samples: list[dict], key: str) -> list:
    return [s[key] for s in samples if key in s]


def summarize(samples: list[dict]) -> dict:
    """Condense a window: SM clock median / min / max, the other medians, and which reason bits were ever active."""
    if not samples:
        return {"n_samples": 0}
    seen = 0
    for s in samples:
        seen |= s["reasons"]
    sm, temp = _column(samples, "sm_mhz"), _column(samples, "temp_c")
    summary = {
        "n_samples": len(samples),
        "sm_mhz": {"median": median(sm), "min": min(sm), "max": max(sm)},
        "mem_mhz_median": median(_column(samples, "mem_mhz")),
        "temp_c": {"median": median(temp), "max": max(temp)},
        "power_w_median": median(_column(samples, "power_w")),
        "util_pct_median": median(_column(samples, "util_pct")),
        "slowdown_reasons": [name for bit, name in SLOWDOWN_REASONS.items() if seen & bit],
        "noted_reasons": [name for bit, name in NOTED_REASONS.items() if seen & bit],
        "reasons_mask": hex(seen),
    }
    ceilings = _column(samples, "sm_max_mhz")
    if ceilings:
        summary["sm_max_mhz"] = max(ceilings)
    return summary


def clocks_record(samples: list[dict]) -> dict:
    """The ``clocks`` entry of a benchmark's JSON line: median SM MHz while the timed steps ran, the GPU's maximum,
    and every reason that was active (invalidating ones first)."""
    s = summarize(samples)
    if s["n_samples"] == 0:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "n_samples": 0}
    return {"sm_mhz": s["sm_mhz"]["median"], "sm_max_mhz": s.get("sm_max_mhz"), "reasons": s["slowdown_reasons"] + s["noted_reasons"],
            "n_samples": s["n_samples"], "power_w": s["power_w_median"]}


def locked_sm_mhz() -> int | None:
    """The SM clock an operator says the GPU was locked to (``NANONEMO_LOCKED_SM_MHZ``), or None when it floats.
    It is only a declaration that this module reads; the framework never locks a clock."""
    declared = os.environ.get("NANONEMO_LOCKED_SM_MHZ", "").strip()
    return int(declared) if declared else None


def clock_floor(locked: int | None, device_name: str) -> int | None:
    """Lowest median SM clock a clean run may show: 2 % under a declared lock, else the device's rated boost clock."""
    if locked:
        return int(locked * 0.98)
    from nanonemo_b200.utils.mfu import rated_boost_mhz

    return rated_boost_mhz(device_name)


def _trial_findings(summary: dict, across_trials: float, tol: float, min_mhz: int | None) -> list[str]:
    if not summary.get("n_samples"):
        return ["no GPU samples"]
    found = []
    here = summary["sm_mhz"]["median"]
    if here < across_trials * (1.0 - tol):
        found.append(f"median SM clock {here:.0f} MHz (median of trials {across_trials:.0f})")
    if min_mhz and here < min_mhz:
        found.append(f"median SM clock {here:.0f} MHz is below the floor {min_mhz}")
    if summary["slowdown_reasons"]:
        found.append(", ".join(summary["slowdown_reasons"]))
    return found


def throttle_flags(trials: list[dict], tol: float = 0.10, min_mhz: int | None = None) -> list[str]:
    """Why a set of per-trial summaries should not be trusted; an empty list means clean. A trial is flagged when its
    median SM clock sits more than `tol` under the median over all trials, when it is under `min_mhz`, when a slowdown
    reason was active, or when the sampler delivered nothing."""
    medians = [t["sm_mhz"]["median"] for t in trials if t.get("n_samples")]
    if not medians:
        return ["no GPU samples"]
    across = median(medians)
    return [f"trial {i}: {finding}" for i, t in enumerate(trials) for finding in _trial_findings(t, across, tol, min_mhz)]
