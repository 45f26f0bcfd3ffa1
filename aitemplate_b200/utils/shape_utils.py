"""shape helpers (python/aitemplate/utils/shape_utils.py:42-51)."""
from ..testing.test_utils import gen_int_var, gen_int_var_min_max  # noqa: F401
