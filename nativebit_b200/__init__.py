"""nativebit_b200 — B200-native (sm_100a) packed-inference hot path of NativeBit.

Host-side Python mirrors the reference's packed-linear and decode interfaces
(inference/triton_kernel.py, inference/cuda_kernel.py, nativebit/pack.py, nativebit/inference.py,
inference/generate_torch.py) and calls hand-written CUDA through the C ABI declared in
include/nativebit_b200.h.  There is no CPU or multi-backend fallback.
"""
from . import ops  # noqa: F401
from .packed_linear import (BS, NE, TILE_N, PackedLinear, dequant_matvec, dequant_matvec_3bit,  # noqa: F401
                            dequant_matvec_3bit_cuda, pack_indices_to_3bit)

from .stream import MatvecGroup  # noqa: F401,E402

__version__ = "0.1.0"
