from .mem_eff_attention import mem_eff_attention  # noqa: F401
from .flash_attention import flash_attention  # noqa: F401
