"""Timing and comparison helpers with the method of the reference's deep_gemm/testing
(bench.py:7-33: CUDA events around repeated calls with an L2 flush before each; numeric.py:5-21)."""
from __future__ import annotations

import torch


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y> / (|x|^2 + |y|^2) in float64."""
    x, y = x.double(), y.double()
    denom = (x * x + y * y).sum()
    if denom == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / denom)


def count_bytes(*tensors) -> int:
    total = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.numel() * t.element_size()
    return total


def assert_bitwise_equal(x: torch.Tensor, y: torch.Tensor, label: str = "") -> None:
    assert x.shape == y.shape and x.dtype == y.dtype, label
    xb, yb = x.contiguous().view(torch.uint8), y.contiguous().view(torch.uint8)
    if not torch.equal(xb, yb):
        bad = (xb != yb).flatten().nonzero()
        raise AssertionError(f"bitwise mismatch ({label}): {bad.numel()} bytes differ, first at byte {int(bad[0])}")


def bench(fn, num_warmups: int = 5, num_tests: int = 20, flush_l2_bytes: int = 256 << 20) -> float:
    """Mean device seconds of fn(), each call preceded by a write of `flush_l2_bytes` (larger than the
    126 MB L2) that is excluded from the timing."""
    flush = torch.empty(flush_l2_bytes // 4, dtype=torch.int, device="cuda") if flush_l2_bytes else None
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    for i in range(num_tests):
        if flush is not None:
            flush.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / num_tests / 1e3


def bench_kineto(fn, kernel_names, num_tests: int = 20, flush_l2_bytes: int = 256 << 20, span: bool = False) -> float:
    """Mean device seconds per call of fn(), counting only kernels whose name contains one of `kernel_names`
    (a string or a tuple), from the torch profiler's kernel records, with an L2 flush before every call: the method
    of the reference's deep_gemm/testing/bench.py:79-146.  Unlike event timing it excludes launch gaps, which
    matter for kernels of a few microseconds.  With `span`, a call that launches several matching kernels counts
    from the start of its first to the end of its last (kernels launched with programmatic dependent launch overlap,
    so their durations must not be added)."""
    names = (kernel_names,) if isinstance(kernel_names, str) else tuple(kernel_names)
    flush = torch.empty(flush_l2_bytes // 4, dtype=torch.int, device="cuda") if flush_l2_bytes else None
    fn()
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            if flush is not None:
                flush.zero_()
            fn()
        torch.cuda.synchronize()
    matched = [evt for evt in prof.events()
               if evt.device_type == torch.autograd.DeviceType.CUDA and any(n in evt.name for n in names)]
    assert matched, f"no kernel matching {names} was recorded"
    if span:
        matched.sort(key=lambda e: e.time_range.start)
        per_call, rem = divmod(len(matched), num_tests)
        assert rem == 0, f"{len(matched)} matching kernels over {num_tests} calls"
        total_us = 0.0
        for i in range(num_tests):
            group = matched[i * per_call:(i + 1) * per_call]
            total_us += max(e.time_range.end for e in group) - min(e.time_range.start for e in group)
        return total_us / num_tests / 1e6
    total_us = sum(evt.device_time_total if hasattr(evt, "device_time_total") else evt.cuda_time_total for evt in matched)
    return total_us / num_tests / 1e6


class empty_suppress:
    """Context manager that suppresses nothing (deep_gemm/testing/bench.py: the counterpart of suppress_stdout_stderr)."""

    def __enter__(self):
        return self

    def __exit__(self, *_):
        return False


class suppress_stdout_stderr:
    """Redirects the process's file descriptors 1 and 2 to the null device for the duration of the block, so that output
    written by native code (a profiler's banner) disappears too; restores them afterwards."""

    def __enter__(self):
        import os
        import sys
        sys.stdout.flush(); sys.stderr.flush()
        self._null = os.open(os.devnull, os.O_WRONLY)
        self._saved = (os.dup(1), os.dup(2))
        os.dup2(self._null, 1); os.dup2(self._null, 2)
        return self

    def __exit__(self, *_):
        import os
        import sys
        sys.stdout.flush(); sys.stderr.flush()
        os.dup2(self._saved[0], 1); os.dup2(self._saved[1], 2)
        for fd in (*self._saved, self._null):
            os.close(fd)
        return False
