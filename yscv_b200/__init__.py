"""B200 (sm_100a) replacement for the quantized-matmul hot path of yscv.

The product is ``libyscv_cuda.so`` (hand-written CUDA behind a C ABI, declared
in ``include/yscv_cuda.h``). This package is the thin ctypes binding that the
tests and the benchmark use to call that ABI; it contains no compute of its
own and no CPU fallback.
"""
from .lib import (  # noqa: F401
    Context,
    I8B,
    Requant,
    Int4Weight,
    YscvCudaError,
    DecodePlan,
    Registry,
    TpComm,
    int4_container_read,
    int4_container_write,
    int4_from_matmulnbits,
    int4_to_matmulnbits,
    quant_stats,
    quant_stats_reset,
    load_library,
    library_path,
)
