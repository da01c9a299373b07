"""B200-native quantized-weight matmul (MMQ) operators.

Drop-in for the reference package's public surface (torch_ggml_ops/__init__.py:1-7): importing
this package registers the six ``torch.ops.torch_ggml_ops.*`` operators (native, sm_100a) with
their fake kernels and autograd formulas, and exports ``mmq``, ``grouped_mmq`` and
``grouped_mmq_pair``.  Beyond that surface it exports the steps either side of it (``mmq_multi``,
``swiglu``, ``moe_mlp``, ``lm_head_loss``; ``extras.py``) under the package's own operator namespace.  There is no CPU or eager fallback: if the native module has not been built
the import fails.
"""
import torch  # noqa: F401  (libtorch and the CUDA runtime must be loaded before the native module)

try:
    from . import _C  # noqa: F401  registers torch_ggml_ops::* (static registrars run on import)
except ImportError as exc:  # pragma: no cover - build problem, not a runtime path
    raise ImportError(
        "torch_ggml_ops_b200: the native module is missing or failed to load "
        f"({exc}). Build it with `python torch_ggml_ops_b200/_build.py`; there is no fallback path."
    ) from exc

from . import native  # noqa: E402,F401  ctypes view of the same C ABI (tests, benchmarks)
from .grouped_mmq import grouped_mmq, grouped_mmq_pair  # noqa: E402
from .mmq import mmq  # noqa: E402
from .extras import lm_head_loss, mmq_multi, moe_mlp, swiglu  # noqa: E402
from .quant_types import GGML_TYPE_IDS, block_bytes  # noqa: E402

__all__ = ["GGML_TYPE_IDS", "block_bytes", "grouped_mmq", "grouped_mmq_pair", "lm_head_loss", "mmq", "mmq_multi",
           "moe_mlp", "native", "swiglu"]
