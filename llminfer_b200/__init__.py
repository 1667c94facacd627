"""B200-native decode-phase grouped-query attention behind the LLMInfer operator boundary.

The product is the CUDA library ``lib/libgqa_b200.so`` (C ABI in ``include/gqa_b200.h``) and
the C++ shim in ``shim/`` that keeps the reference's operator interface. This Python package
is the thin binding used by the tests and the benchmark; it has no CPU fallback.
"""
from .binding import (  # noqa: F401
    FusedFront,
    SPLIT_EVEN,
    GqaError,
    KvLayout,
    KvPool,
    Session,
    ShardComm,
    decode,
    decode_partial,
    decode_plan,
    decode_seqpar,
    decode_sharded,
    decode_static_scratch,
    layout_pool,
    layout_reference,
    lib,
    merge_partials,
    oproj_residual,
    oproj_workspace,
    qk_norm_rope_append,
    qkv_gemv,
    qkv_workspace,
    shard_plan,
    sin_cos_cache,
    status_string,
)
