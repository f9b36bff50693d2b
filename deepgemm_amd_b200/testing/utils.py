"""Decorators and probes of the reference's test scripts (deep_gemm/testing/utils.py)."""
from __future__ import annotations

import functools
import os
from typing import Callable

import torch


def get_arch_major() -> int:
    """Major compute capability of the current device (10 on the GPUs this library is written for)."""
    return torch.cuda.get_device_capability()[0]


def test_filter(condition: Callable):
    """Run the decorated test only while condition() holds; otherwise print that it was filtered."""
    def decorate(fn):
        @functools.wraps(fn)
        def run(*args, **kwargs):
            if not condition():
                print(f"{fn.__name__}:\n > Filtered by {condition}\n")
                return None
            return fn(*args, **kwargs)
        return run
    return decorate


test_filter.__test__ = False        # not a test itself, whatever its name


def ignore_env(name: str, condition: Callable):
    """Run the decorated function with the environment variable `name` removed while condition() holds."""
    def decorate(fn):
        @functools.wraps(fn)
        def run(*args, **kwargs):
            if not condition():
                return fn(*args, **kwargs)
            saved = os.environ.pop(name, None)
            try:
                return fn(*args, **kwargs)
            finally:
                if saved is not None:
                    os.environ[name] = saved
        return run
    return decorate
