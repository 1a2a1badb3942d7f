from .numeric import calc_diff, count_bytes, max_rel_err  # noqa: F401
