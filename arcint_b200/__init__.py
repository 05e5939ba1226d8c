"""arcint_b200 -- B200 (sm_100a) quantized weight mat-mul behind ggml's operator contract.

The product is the C-ABI shared library `lib/libb200q.so` (declared in include/b200q.h);
this package is a thin ctypes binding over it for tests and benchmarks. There is no CPU
fallback: importing `binding` fails loudly when the library is missing.
"""
from .binding import (  # noqa: F401
    B200QError, Context, Tensor, lib, lib_path,
    F32, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS, I32, OP_MUL_MAT, OP_MUL_MAT_ID,
    OK, UNSUPPORTED, INVALID, block_size, block_bytes, row_bytes, tp_unique_id, tp_shard,
)
