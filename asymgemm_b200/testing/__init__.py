from .numeric import calc_diff, count_bytes, max_rel_err  # noqa: F401
from . import moe_reference  # noqa: F401
