from .tensor_ops import concatenate, permute, permute021, permute0213, permute102, permute210, split  # noqa: F401
