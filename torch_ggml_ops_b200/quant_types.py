"""GGML type ids and block sizes of the supported formats
(reference: csrc/vendor/llama_cpp/common.cuh:43-50, csrc/mmq_hip.cu:38-48)."""

GGML_TYPE_IDS = {"Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14, "IQ2_S": 22}
_BLOCK_BYTES = {11: 110, 12: 144, 13: 176, 14: 210, 22: 82}
QK_K = 256


def block_bytes(quant_type: int) -> int:
    """Bytes of one 256-weight super-block."""
    try:
        return _BLOCK_BYTES[int(quant_type)]
    except KeyError:
        raise ValueError(f"unsupported quant_type: {quant_type}") from None


def row_bytes(quant_type: int, in_features: int) -> int:
    if in_features <= 0 or in_features % QK_K:
        raise ValueError(f"in_features must be a positive multiple of 256; got {in_features}")
    return (in_features // QK_K) * block_bytes(quant_type)
