"""kronos-2t B200 backend: ctypes access to libkronos_cuda.so (the C ABI of include/kronos_cuda_ffi.h).

The library holds sm_100a code only and there is no CPU fallback: loading fails loudly when the
shared object has not been built, and context creation fails when no B200 is visible.
"""
from .ffi import (  # noqa: F401
    Context,
    Engine,
    KronosCudaError,
    Matrix,
    MatrixDesc,
    bipolar_desc,
    k2tb_load,
    moe_load,
    k2tb_save,
    matrix_image,
    nf_desc,
    lib_path,
    load_library,
)
from .build import build  # noqa: F401
