"""B200 execution runtime for Luminal-style compiled decoder graphs.

The product is the C-ABI shared library built from ``csrc/`` (declared in ``include/lum_b200.h``).
This package is the thin Python host over it: ctypes bindings whose method names follow the
reference's runtime interface (``luminal::op::Runtime``, src/op.rs:10-30, and the inherent
``set_data`` / ``get_f32`` of crates/luminal_cuda/src/runtime.rs:133-236).

There is no CPU path: importing works anywhere, but creating a runtime without the built
library or without a CUDA device raises.
"""
from . import llir, serving, tp  # noqa: F401
from .runtime import (  # noqa: F401
    B200Runtime,
    LumError,
    ModelDesc,
    Config,
    CONFIGS,
    DTYPE,
    SLOT,
    load_library,
    library_path,
    decode_bytes_per_token,
    describe_llir,
    describe_llir_chunk,
    mbu,
    Stats,
    Sampling,
    safetensors_read,
    safetensors_write,
)
