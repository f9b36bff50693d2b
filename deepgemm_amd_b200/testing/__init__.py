from .bench import bench, bench_kineto, calc_diff, count_bytes, assert_bitwise_equal  # noqa: F401
