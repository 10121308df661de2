"""quintrit_b200: B200 (sm_100a) device for quintrit's ternary decode path.

The product is ``libquintrit_b200.so`` (C ABI in ``include/quintrit_b200.h``); this package is the Python host side
over that ABI. It mirrors the reference's GPU launcher interface (``rust/crates/quintrit-cuda/src/gemv.rs``: ``Gemv``,
``pack.rs``: ``pack_planar``, ``row_bytes``) so that tests read like the reference's. There is no CPU fallback: every
compute call goes to the CUDA library and raises ``QuintritError`` if it is missing or the device is unusable.
"""
from .api import (  # noqa: F401
    ARCH_BITNET,
    ARCH_LLAMA,
    ARCH_QWEN,
    Batch,
    Decoder,
    DeviceInfo,
    Matrix,
    Moe,
    Plan,
    QuintritError,
    SRC_I2_S,
    SRC_PLANAR,
    SRC_Q2_0,
    SRC_TQ1_0,
    SRC_TQ2_0,
    device_count,
    device_info,
    gguf_describe,
    last_selftest_released,
    launch_count,
    library_path,
    load_library,
    pack_planar,
    quantize_q8_0,
    row_bytes,
    sample_logits,
    selftest_barrier,
    version,
)
