from .dtypes import hccl_dtype, data_ptr, numel, is_device  # noqa: F401
