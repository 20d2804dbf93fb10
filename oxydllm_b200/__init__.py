"""oxydllm_b200: B200 (sm_100a) kernels behind oxydLLM's quantized-linear operator surface.

``liboxq.so`` (hand-written CUDA behind a C ABI, ``include/oxq.h``) does the
work; this package is the thin host-side mirror of the reference's operator
types. Importing the operator modules requires the compiled library.
"""
from . import formats  # noqa: F401  (pure numpy: usable without a GPU)

__all__ = ["formats", "linear", "synth"]
