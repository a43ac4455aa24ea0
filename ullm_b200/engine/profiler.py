"""Step and kernel-group timing behind `--profile` / `LLM.profile("start" | "stop")`.

The reference starts and stops a torch profiler on its engine and its workers
and writes traces to `profile_dir` (ullm/core/engine.py:54-70, :210-238).  Here
the same two switches give:

  * per step: its kind (prompt portions only, decode tokens only, mixed), how
    many requests and tokens it held, the device time between two CUDA events
    recorded around its launch, and the host time from scheduling to the read
    of its tokens;
  * per kernel group, for steps that run eagerly (every step with prompt
    portions; decode steps too under `enforce_eager`): CUDA-event time, calls,
    and the bytes the group had to read where the wrapper knows them (weights of
    a matrix product), which gives achieved GB/s.  A decode step replayed from a
    CUDA graph is one launch and is timed as a whole.

`stop` prints a table per (kind, requests) and writes everything as JSON to
`profile_dir/ullm_b200_engine_<pid>.json`.
"""

from __future__ import annotations

import json
import os
import time
from collections import defaultdict

import torch


class KernelGroupTimer:
    """Collects (group, start event, end event, bytes) from the kernel wrappers
    while it is installed as `kernels().timer`.  Only outermost calls count: a
    wrapper that calls other wrappers is one group."""

    def __init__(self):
        self.records: list[tuple[str, torch.cuda.Event, torch.cuda.Event, int]] = []
        self.depth = 0

    def begin(self):
        self.depth += 1
        if self.depth > 1 or torch.cuda.is_current_stream_capturing():
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def end(self, group: str, start, nbytes: int = 0) -> None:
        self.depth -= 1
        if start is None:
            return
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.records.append((group, start, e, int(nbytes)))

    def totals(self) -> dict[str, dict]:
        """Per group: calls, microseconds, bytes (synchronizes)."""
        if self.records:
            self.records[-1][2].synchronize()
        out: dict[str, dict] = defaultdict(lambda: {"calls": 0, "us": 0.0, "bytes": 0})
        for group, e0, e1, nbytes in self.records:
            t = out[group]
            t["calls"] += 1
            t["us"] += e0.elapsed_time(e1) * 1e3
            t["bytes"] += nbytes
        for t in out.values():
            t["us"] = round(t["us"], 1)
            if t["bytes"] and t["us"] > 0:
                t["gb_per_s"] = round(t["bytes"] / t["us"] / 1e3, 3)
        return dict(out)


class StepProfiler:
    def __init__(self, profile_dir: str, cuda: bool):
        self.profile_dir = profile_dir
        self.cuda = cuda
        self.started = False
        self.steps: list[dict] = []
        self._open: list[tuple[dict, object, object]] = []  # steps whose end event has not been read yet
        self.timer: KernelGroupTimer | None = None

    # -- switches ---------------------------------------------------------------------
    def start(self) -> None:
        if self.started:
            return
        self.started = True
        self.steps, self._open = [], []
        if self.cuda:
            from ..csrc import kernels

            self.timer = KernelGroupTimer()
            kernels().timer = self.timer

    def stop(self) -> dict | None:
        """Ends the collection, prints the tables, writes the JSON file; returns what was written."""
        if not self.started:
            return None
        self.started = False
        groups = {}
        if self.cuda:
            from ..csrc import kernels

            kernels().timer = None
            torch.cuda.synchronize()
            groups = self.timer.totals() if self.timer is not None else {}
        self._close_open()
        for rec in self.steps:
            rec.pop("t0", None)
            rec.pop("_e0", None)
        report = {"steps": self.steps, "by_kind": self.summary(), "kernel_groups": groups}
        os.makedirs(self.profile_dir, exist_ok=True)
        path = os.path.join(self.profile_dir, f"ullm_b200_engine_{os.getpid()}.json")
        with open(path, "w") as f:
            json.dump(report, f)
        report["path"] = path
        print(self.format(report), flush=True)
        return report

    # -- one step ------------------------------------------------------------------------
    def step_begin(self, scheduled) -> dict:
        n_prompt = sum(1 for s in scheduled if s.num_tokens > 1 or not s.samples)
        kind = "decode" if n_prompt == 0 else ("prefill" if n_prompt == len(scheduled) else "mixed")
        rec = {"kind": kind, "requests": len(scheduled), "tokens": sum(s.num_tokens for s in scheduled),
               "t0": time.perf_counter()}
        e0 = None
        if self.cuda:
            e0 = torch.cuda.Event(enable_timing=True)
            e0.record()
        rec["_e0"] = e0
        return rec

    def step_launched(self, rec: dict) -> None:
        e1 = None
        if self.cuda:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
        self._open.append((rec, rec.pop("_e0"), e1))

    def step_read(self, rec: dict) -> None:
        t0 = rec.pop("t0", None)
        if t0 is not None:
            rec["host_ms"] = round((time.perf_counter() - t0) * 1e3, 4)
        self._close_open()

    def _close_open(self) -> None:
        still = []
        for rec, e0, e1 in self._open:
            if e1 is not None and not e1.query():
                still.append((rec, e0, e1))
                continue
            if e1 is not None:
                rec["device_ms"] = round(e0.elapsed_time(e1), 4)
            self.steps.append(rec)  # (its host time is filled in when its tokens are read)
        self._open = still
        if not self.started:  # stopping: wait for the rest
            for rec, e0, e1 in self._open:
                if e1 is not None:
                    e1.synchronize()
                    rec["device_ms"] = round(e0.elapsed_time(e1), 4)
                rec.pop("t0", None)
                self.steps.append(rec)
            self._open = []

    # -- reports ---------------------------------------------------------------------------
    def summary(self) -> list[dict]:
        rows: dict[tuple, list[dict]] = defaultdict(list)
        for s in self.steps:
            rows[(s["kind"], s["requests"])].append(s)
        out = []
        for (kind, reqs), ss in sorted(rows.items()):
            n = len(ss)
            dev = [s["device_ms"] for s in ss if "device_ms" in s]
            host = [s["host_ms"] for s in ss if "host_ms" in s]
            toks = sum(s["tokens"] for s in ss)
            mean_dev = sum(dev) / len(dev) if dev else None
            mean_host = sum(host) / len(host) if host else None
            per = mean_dev if mean_dev else mean_host
            out.append({"kind": kind, "requests": reqs, "steps": n, "tokens": toks,
                        "mean_device_ms": None if mean_dev is None else round(mean_dev, 4),
                        "mean_host_ms": None if mean_host is None else round(mean_host, 4),
                        "tokens_per_s": None if not per else round(toks / n / (per / 1e3), 1)})
        return out

    @staticmethod
    def format(report: dict) -> str:
        lines = ["profile: steps by kind and number of requests",
                 f"  {'kind':8s} {'requests':>8s} {'steps':>7s} {'tokens':>9s} {'device ms':>10s} {'host ms':>9s} {'tok/s':>10s}"]
        for r in report["by_kind"]:
            f = lambda v, w, p: (f"{v:{w}.{p}f}" if v is not None else " " * (w - 1) + "-")
            lines.append(f"  {r['kind']:8s} {r['requests']:8d} {r['steps']:7d} {r['tokens']:9d} "
                         f"{f(r['mean_device_ms'], 10, 3)} {f(r['mean_host_ms'], 9, 3)} {f(r['tokens_per_s'], 10, 1)}")
        if report["kernel_groups"]:
            lines.append("profile: kernel groups of the steps that ran eagerly (CUDA events)")
            lines.append(f"  {'group':24s} {'calls':>8s} {'us':>12s} {'us/call':>9s} {'GB/s':>8s}")
            for g, t in sorted(report["kernel_groups"].items(), key=lambda kv: -kv[1]["us"]):
                gb = f"{t['gb_per_s']:8.1f}" if "gb_per_s" in t else "       -"
                lines.append(f"  {g:24s} {t['calls']:8d} {t['us']:12.1f} {t['us'] / max(t['calls'], 1):9.2f} {gb}")
        if "path" in report:
            lines.append(f"profile: written to {report['path']}")
        return "\n".join(lines)
