"""Profiling and timing helpers: a torch.profiler wrapper driven by start/stop requests
(Chrome traces ``*.trace.json.gz`` like the reference's scheduler writes,
smcsd/engine.py:376-413, scripts/smc_profile_engine.py:283-303), device-side phase timers
built on CUDA events, and an ``nvidia-smi`` clock sampler for benchmark runs.
"""
from __future__ import annotations

import os
import subprocess
import threading
import time
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch


class SchedulerProfiler:
    """torch.profiler capture driven by the scheduler.  With ``profile_by_stage`` the capture is cut at every change
    between prefill and decode iterations and each piece is exported with its stage in the file name
    (``smc-<time>-rank<r>-<stage>.trace.json.gz``); ``profile_stages`` keeps only the named stages."""

    def __init__(self, req, rank: int = 0):
        self.req = req
        self.rank = rank
        self.prof = None
        self.stage: Optional[str] = None
        self.paths: List[str] = []
        self.out_dir = req.output_dir or os.environ.get("SMC_PROFILE_DIR", "/tmp/smcsd_b200_profile")
        self.by_stage = bool(getattr(req, "profile_by_stage", False))
        st = getattr(req, "profile_stages", None)
        self.stages = {x.lower() for x in st} if st else None

    def _begin(self) -> None:
        acts = []
        wanted = [a.upper() for a in (self.req.activities or ["CPU", "GPU"])]
        if "CPU" in wanted:
            acts.append(torch.profiler.ProfilerActivity.CPU)
        if "GPU" in wanted and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        env = os.environ.get                 # the reference's profiler switches are honoured as defaults
        stack = self.req.with_stack or env("SMC_PROFILE_WITH_STACK", env("SGLANG_PROFILE_WITH_STACK", "0")) == "1"
        shapes = self.req.record_shapes or \
            env("SMC_PROFILE_RECORD_SHAPES", env("SGLANG_PROFILE_RECORD_SHAPES", "0")) == "1"
        self.prof = torch.profiler.profile(activities=acts, with_stack=stack, record_shapes=shapes)
        self.prof.start()

    def _end(self) -> Optional[str]:
        if self.prof is None:
            return None
        self.prof.stop()
        os.makedirs(self.out_dir, exist_ok=True)
        tag = f"-{self.stage}" if (self.by_stage and self.stage) else ""
        path = os.path.join(self.out_dir, f"smc-{time.time_ns() // 1000000}-rank{self.rank}{tag}.trace.json.gz")
        self.prof.export_chrome_trace(path)
        self.prof = None
        self.paths.append(path)
        return path

    def start(self) -> None:
        if not self.by_stage:
            self._begin()

    def enter_stage(self, stage: str) -> None:
        """Called by the scheduler before a prefill or decode iteration (by-stage captures only)."""
        if not self.by_stage or stage == self.stage:
            return
        self._end()
        self.stage = stage
        if self.stages is None or stage in self.stages:
            self._begin()

    def stop(self) -> Optional[str]:
        self._end()
        return self.paths[-1] if self.paths else None


@contextmanager
def span(name: str):
    """Named range visible in torch.profiler traces (graph replays bypass module hooks)."""
    with torch.profiler.record_function(name):
        yield


class PhaseTimers:
    """CUDA-event timers per named phase; ``summary`` synchronises and reports milliseconds."""

    def __init__(self):
        self.records: Dict[str, List] = {}

    @contextmanager
    def phase(self, name: str):
        if not torch.cuda.is_available():
            t0 = time.perf_counter()
            yield
            self.records.setdefault(name, []).append(("cpu", (time.perf_counter() - t0) * 1e3))
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self.records.setdefault(name, []).append((a, b))

    def summary(self) -> Dict[str, float]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = {}
        for k, v in self.records.items():
            ms = [x[1] if x[0] == "cpu" else x[0].elapsed_time(x[1]) for x in v]
            out[k] = sum(ms) / max(len(ms), 1)
        return out


_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons with ``nvidia-smi`` while a timed region runs.
    Read-only: it never changes a GPU setting."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc = None
        self.lines: List[str] = []
        self._t = None

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except (FileNotFoundError, OSError):
            self.proc = None
            return self

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self._t = threading.Thread(target=pump, daemon=True)
        self._t.start()
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}
