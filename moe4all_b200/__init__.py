"""B200-native (sm_100a) quantized MoE FFN path of MoE4All behind the reference's backend seam.

The product is the C-ABI library declared in include/infr_cuda.h (built from csrc/ into
_lib/libinfr_cuda.so).  This package is the host-side mirror of the reference's operator
interface for that path: `CudaBackend` follows `infr_core::backend::Backend`
(crates/infr-core/src/backend.rs:630-1088) and `MoeFfn` follows `Op::MoeFfn`
(crates/infr-core/src/graph.rs:1259-1352).  There is no CPU fallback: without the CUDA library
every call raises.
"""
from .backend import (  # noqa: F401
    Activation, BackendError, Buffer, Config, CudaBackend, DType, MoeFfn, MoeGating, Unsupported, load_library,
)
