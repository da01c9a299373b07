"""Regenerates tests/golden/gguf_golden.npz.

Run in a container that has gguf-py (``python tests/golden/make_golden.py``).  For every
supported block type it stores a few seeded random valid super-blocks plus hand-built extreme
blocks, and their fp32 dequantisation computed by gguf-py 0.19.0 (``gguf.quants.dequantize``),
which is an implementation independent of both the CPU oracle in ``oracle/`` and the CUDA
decoders.  A tiny dense matmul case (fp32 ``x @ W.T`` and ``dy @ W`` by numpy float64, rounded
to fp32) is stored per type as a known-answer vector for the forward and input-gradient ops.
The reference repository ships no golden vectors of its own (its tests read a GGUF checkpoint
that is not distributed with it), so these fixtures are the committed known answers.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from gguf import GGMLQuantizationType as T  # noqa: E402
from gguf import quants  # noqa: E402

from oracle import blocks, ref  # noqa: E402

GG = {ref.Q3_K: T.Q3_K, ref.Q4_K: T.Q4_K, ref.Q5_K: T.Q5_K, ref.Q6_K: T.Q6_K, ref.IQ2_S: T.IQ2_S}


def main() -> None:
    out = {}
    for name, qt in ref.QTYPES.items():
        blk = np.concatenate([blocks.random_blocks(qt, 8, 1234 + qt), blocks.extreme_blocks(qt)])
        deq = quants.dequantize(blk, GG[qt]).astype(np.float32).reshape(-1)
        out[f"{name}_blocks"] = blk
        out[f"{name}_fp32"] = deq
        # known-answer matmul: N=16 rows of one block each (K=256), M=8 tokens
        w = blocks.random_blocks(qt, 16, 99 + qt)
        W = quants.dequantize(w, GG[qt]).astype(np.float64).reshape(16, 256)
        rng = np.random.Generator(np.random.PCG64(7 + qt))
        x = rng.standard_normal((8, 256)).astype(np.float32)
        dy = rng.standard_normal((8, 16)).astype(np.float32)
        # inputs are stored already rounded to bf16-representable values
        x = ref.bf16_bits_to_f32(ref.round_bf16_bits(x))
        dy = ref.bf16_bits_to_f32(ref.round_bf16_bits(dy))
        out[f"{name}_mm_w"] = w
        out[f"{name}_mm_x"] = x
        out[f"{name}_mm_dy"] = dy
        out[f"{name}_mm_y"] = (x.astype(np.float64) @ W.T).astype(np.float32)
        out[f"{name}_mm_dx"] = (dy.astype(np.float64) @ W).astype(np.float32)
    path = Path(__file__).resolve().parent / "gguf_golden.npz"
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size)


if __name__ == "__main__":
    main()
