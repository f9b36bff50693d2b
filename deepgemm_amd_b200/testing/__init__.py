from .bench import (  # noqa: F401
    bench, bench_kineto, calc_diff, count_bytes, assert_bitwise_equal, suppress_stdout_stderr, empty_suppress,
)
from .utils import get_arch_major, test_filter, ignore_env  # noqa: F401
