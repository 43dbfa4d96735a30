"""Sample GPU clocks and throttle reasons while a timed region runs.

A benchmark number is only trusted together with the clocks it was taken at, so
``ClockSampler`` polls ``nvidia-smi`` (read-only queries) in a child process for
the duration of the timed region and summarises what it saw.  Nothing here
changes a GPU setting.
"""
from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile
import time
from typing import Dict, List, Optional

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.path: Optional[str] = None

    def start(self) -> None:
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        fd, self.path = tempfile.mkstemp(prefix="gx_clocks_", suffix=".csv")
        os.close(fd)
        out = open(self.path, "w")
        try:
            self.proc = subprocess.Popen(
                [exe, "--query-gpu=" + _FIELDS, "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        finally:
            out.close()

    def stop(self) -> Dict[str, object]:
        if self.proc is not None:
            time.sleep(self.period_ms / 1000.0)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        rows: List[List[str]] = []
        if self.path and os.path.exists(self.path):
            with open(self.path) as fh:
                for line in fh:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) >= 9:
                        rows.append(parts)
            os.unlink(self.path)
        return summarise(rows)


def summarise(rows: List[List[str]]) -> Dict[str, object]:
    sm, sm_max, power = [], [], []
    reasons = set()
    names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    for r in rows:
        try:
            sm.append(float(r[1]))
            sm_max.append(float(r[2]))
            power.append(float(r[3]))
        except ValueError:
            continue
        for name, val in zip(names, r[5:9]):
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
