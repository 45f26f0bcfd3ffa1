from .softmax import softmax  # noqa: F401
