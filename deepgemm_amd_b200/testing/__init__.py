from .bench import bench, calc_diff, count_bytes, assert_bitwise_equal  # noqa: F401
