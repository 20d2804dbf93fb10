"""Generate ``gguf_blocks.npz``: GGML blocks with their dequantized values from gguf-py.

gguf-py (package ``gguf``, 0.19.0) is an implementation of the GGML block
formats that is independent of both the reference and this repository; it
serves as a second opinion on the bit patterns of the dequantized weights.
Inputs are random block bytes (every bit field exercised) with finite f16
scale fields, plus blocks produced by this project's encoders from N(0, 0.02)
weights. Run from the repository root: ``python tests/golden/make_golden.py``.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gguf import GGMLQuantizationType as T  # noqa: E402
from gguf import quants  # noqa: E402

from oxydllm_b200 import formats as F  # noqa: E402

TYPES = {F.GGML_Q4_0: T.Q4_0, F.GGML_Q8_0: T.Q8_0, F.GGML_Q4_K: T.Q4_K, F.GGML_Q6_K: T.Q6_K,
         F.GGML_Q4_1: T.Q4_1, F.GGML_Q5_0: T.Q5_0, F.GGML_Q5_1: T.Q5_1, F.GGML_Q5_K: T.Q5_K,
         F.GGML_Q2_K: T.Q2_K, F.GGML_Q3_K: T.Q3_K}
F16_FIELDS = {F.GGML_Q4_0: [0], F.GGML_Q8_0: [0], F.GGML_Q4_K: [0, 2], F.GGML_Q6_K: [208],
              F.GGML_Q4_1: [0, 2], F.GGML_Q5_0: [0], F.GGML_Q5_1: [0, 2], F.GGML_Q5_K: [0, 2],
              F.GGML_Q2_K: [80, 82], F.GGML_Q3_K: [108]}


def main():
    rng = np.random.default_rng(1234)
    out = {}
    for t, gt in TYPES.items():
        bel, bby = F.GGML_BLOCK[t]
        rows, nb = 6, 512 // bel if bel == 256 else 4
        raw = rng.integers(0, 256, size=(rows, nb, bby), dtype=np.uint8)
        for off in F16_FIELDS[t]:
            v = (rng.standard_normal((rows, nb)) * 0.01).astype(np.float16)
            raw[:, :, off:off + 2] = v.view(np.uint8).reshape(rows, nb, 2)
        w = (rng.standard_normal((rows, nb * bel)) * 0.02).astype(np.float32)
        enc = F.GGML_QUANTIZE[t](w).reshape(rows, nb, bby)
        blocks = np.concatenate([raw, enc], axis=0)
        deq = quants.dequantize(blocks.reshape(2 * rows, nb * bby), gt).astype(np.float32)
        out[f"blocks_{t}"] = blocks.reshape(-1)
        out[f"shape_{t}"] = np.array([2 * rows, nb * bel], np.int64)
        out[f"deq_{t}"] = deq
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "gguf_blocks.npz"), **out)


if __name__ == "__main__":
    main()
