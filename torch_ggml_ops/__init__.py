"""Import alias so that code written against the reference package name keeps working:
``import torch_ggml_ops; torch_ggml_ops.mmq(...)`` resolves to the B200-native implementation."""
from torch_ggml_ops_b200 import grouped_mmq, grouped_mmq_pair, mmq  # noqa: F401

__all__ = ["grouped_mmq", "grouped_mmq_pair", "mmq"]
