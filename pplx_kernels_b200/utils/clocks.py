"""Samples GPU clocks and throttle reasons with nvidia-smi while a benchmark runs.

Only reads settings; never changes clocks, power limits or modes.
"""

from __future__ import annotations

import csv
import io
import shutil
import statistics
import subprocess
import tempfile

_FIELDS = [
    "index",
    "clocks.sm",
    "clocks.max.sm",
    "power.draw",
    "clocks_event_reasons.active",
    "clocks_event_reasons.hw_slowdown",
    "clocks_event_reasons.hw_thermal_slowdown",
    "clocks_event_reasons.sw_thermal_slowdown",
    "clocks_event_reasons.sw_power_cap",
]


class ClockSampler:
    """``with ClockSampler(device_index) as s: ...`` then ``s.summary()``."""

    def __init__(self, device_index: int = 0, period_ms: int = 100) -> None:
        self.device_index = device_index
        self.period_ms = period_ms
        self._proc: subprocess.Popen | None = None
        self._out = None

    def __enter__(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self._out = tempfile.TemporaryFile(mode="w+")
        self._proc = subprocess.Popen(
            [exe, f"--query-gpu={','.join(_FIELDS)}", "--format=csv,noheader,nounits",
             "-i", str(self.device_index), "-lms", str(self.period_ms)],
            stdout=self._out, stderr=subprocess.DEVNULL)
        return self

    def __exit__(self, *exc) -> None:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

    def summary(self) -> dict:
        if self._out is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self._out.seek(0)
        rows = list(csv.reader(io.StringIO(self._out.read())))
        sm, sm_max, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in rows:
            row = [c.strip() for c in row]
            if len(row) != len(_FIELDS):
                continue
            try:
                sm.append(float(row[1]))
                sm_max.append(float(row[2]))
                power.append(float(row[3]))
            except ValueError:
                continue
            for name, val in zip(names, row[5:9], strict=True):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {
            "sm_mhz": statistics.median(sm),
            "sm_max_mhz": max(sm_max),
            "power_w_max": max(power),
            "reasons": sorted(reasons),
            "samples": len(sm),
        }
