from .mem_eff_attention import mem_eff_attention  # noqa: F401
