"""Per-scope device timers behind print_debug_timers / reset_debug_timers.

The reference keeps per-thread CPU timers per named scope (RECORD_SCOPE; printed by src/csrc/init.cpp:81-153 with a
count, total milliseconds and GFLOP / TFLOP/s per scope). Here a scope is a pair of CUDA events recorded on the current
stream around an op of the path (the scope names are the reference's: qkv_gemm, o_gemm, i_gemm, o_mlp, ac_gemm, rope,
pln_gemm, ...); the table adds GB/s of the bytes the op has to move, the number that matters on an HBM-bound path.
Timers are off by default: events between launches forbid the launch overlap the decode path relies on, so a timed run
is slower than an untimed one. Enable with TPP_DEBUG_TIMERS=1 in the environment or enable(True)."""
import os

import torch

_enabled = os.environ.get("TPP_DEBUG_TIMERS", "0") == "1"
_records = {}  # scope -> {"events": [(start, end)], "flops": f, "bytes": b}


def enabled():
    return _enabled


def enable(flag=True):
    global _enabled
    _enabled = bool(flag)


class scope:
    """with scope("qkv_gemm", flops=..., nbytes=...): launches"""

    __slots__ = ("name", "flops", "nbytes", "ev")

    def __init__(self, name, flops=0, nbytes=0):
        self.name, self.flops, self.nbytes = name, flops, nbytes
        self.ev = None

    def __enter__(self):
        if _enabled and not torch.cuda.is_current_stream_capturing():
            self.ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self.ev[0].record()
        return self

    def __exit__(self, *exc):
        if self.ev is not None:
            self.ev[1].record()
            r = _records.setdefault(self.name, {"events": [], "flops": 0, "bytes": 0})
            r["events"].append(self.ev)
            r["flops"] += self.flops
            r["bytes"] += self.nbytes
        return False


def reset_debug_timers():
    _records.clear()


def summary():
    """scope -> (count, total ms, GFLOP, TFLOP/s, GB/s); waits for the device."""
    if _records:
        torch.cuda.synchronize()
    out = {}
    for name, r in _records.items():
        ms = sum(a.elapsed_time(b) for a, b in r["events"])
        s = max(ms * 1e-3, 1e-12)
        out[name] = (len(r["events"]), ms, r["flops"] * 1e-9, r["flops"] * 1e-12 / s, r["bytes"] * 1e-9 / s)
    return out


def print_debug_timers(tid=0, detailed=True):
    rank = int(os.environ.get("RANK", "0"))
    want = int(os.environ.get("TPP_DEBUG_TIMER_RANK", "0"))
    if want != -1 and rank != want:
        return
    if not _enabled:
        print("### tpp debug timers are off (set TPP_DEBUG_TIMERS=1)")
        return
    print("### ##: %-11s:  %9s  %6s  %10s  %8s  %8s" % ("#KEY#", "Total(ms)", "Count", "TotalGF", "TF/s", "GB/s"))
    for name, (cnt, ms, gf, tfs, gbs) in summary().items():
        print("GPU %2d: %-11s:  %9.3f  %6d  %10.3f  %8.3f  %8.1f" % (rank, name, ms, cnt, gf, tfs, gbs))
