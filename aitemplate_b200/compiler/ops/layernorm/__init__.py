from .layernorm import layernorm  # noqa: F401
