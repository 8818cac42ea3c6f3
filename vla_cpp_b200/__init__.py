"""vla_cpp_b200 -- host-side mirror of the vla.cpp denoise-step interfaces over libvla_b200.so.

The library is hand-written sm_100a CUDA behind a C ABI (include/vla_b200.h).  This
package only loads it and marshals device pointers; there is no CPU or PyTorch fallback:
importing works anywhere (so the exported symbols can be checked), but every compute
call needs the built library and a B200.
"""
from .api import (  # noqa: F401
    LIB_PATH,
    MASK_CAUSAL,
    MASK_LAST_PRIVATE,
    MASK_NONE,
    MASK_PI0,
    BitvlaLM,
    DenoiseAttn,
    Gguf,
    KvStore,
    PolicyEngine,
    Prefill,
    VisionTower,
    VlaB200Error,
    VlaModel,
    act_quant,
    attention,
    bitvla_norm_quant,
    device_status,
    fold_norm_weight,
    lib,
    node_bin,
    node_mul_mat,
    node_norm,
    node_scale,
    node_unary,
    qkv_rope_append,
    rope_table,
    selftest_bounded_wait,
    set_gemm_tiling,
    ternarize_pack,
    ternary_linear,
)
