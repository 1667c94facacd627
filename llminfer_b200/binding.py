"""ctypes binding of ``libgqa_b200.so`` (the C ABI in ``include/gqa_b200.h``).

Tensors are ``torch`` tensors used only as owners of device memory: every call passes raw
``data_ptr()`` values and sizes across the C ABI. There is no fallback path: if the library
has not been built, importing it raises; if a call fails, ``GqaError`` carries the status.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

import torch

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libgqa_b200.so"

DTYPE_F32 = 1
DTYPE_BF16 = 2
CHUNK_KEYS = 32
COMM_ID_BYTES = 128


class GqaError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status} ({status_string(status)})")


class _Layout(C.Structure):
    _fields_ = [
        ("block_tokens", C.c_int32),
        ("num_blocks", C.c_int32),
        ("stride_block", C.c_int64),
        ("stride_token", C.c_int64),
        ("stride_head", C.c_int64),
    ]


class _DecodeParams(C.Structure):
    _fields_ = [
        ("dtype", C.c_int32),
        ("batch", C.c_int32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("blocks_per_seq", C.c_int32),
        ("fixed_block", C.c_int32),
        ("split_keys", C.c_int32),
        ("max_ctas", C.c_int32),
        ("plan_len_hint", C.c_int32),
        ("early_prefetch", C.c_int32),
        ("q_tokens", C.c_int32),
        ("layout", _Layout),
        ("q", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("out", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("seq_lens_host", C.POINTER(C.c_int32)),
        ("seq_lens_dev", C.c_void_p),
        ("block_table_dev", C.c_void_p),
        ("status_dev", C.c_void_p),
        ("stream", C.c_void_p),
    ]


SPLIT_EVEN = -1  # split_keys value: cut all units evenly over the CTAs (GQA_SPLIT_EVEN)


class _PlanInfo(C.Structure):
    _fields_ = [
        ("split_chunks", C.c_int32),
        ("max_splits", C.c_int32),
        ("num_items", C.c_int32),
        ("num_ctas", C.c_int32),
        ("needs_combine", C.c_int32),
        ("cluster_size", C.c_int32),
        ("workspace_bytes", C.c_size_t),
        ("even_cut", C.c_int32),
        ("reserved", C.c_int32),
    ]


class _FrontParams(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("blocks_per_seq", C.c_int32),
        ("fixed_block", C.c_int32),
        ("table_len", C.c_int32),
        ("eps", C.c_float),
        ("layout", _Layout),
        ("q", C.c_void_p),
        ("q_out", C.c_void_p),
        ("k_new", C.c_void_p),
        ("v_new", C.c_void_p),
        ("qk_weight", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("sin_cache", C.c_void_p),
        ("cos_cache", C.c_void_p),
        ("positions_host", C.POINTER(C.c_int32)),
        ("positions_dev", C.c_void_p),
        ("block_table_dev", C.c_void_p),
        ("stream", C.c_void_p),
        ("status_dev", C.c_void_p),
        ("q_tokens", C.c_int32),
        ("reserved", C.c_int32),
    ]


class _FusedFront(C.Structure):
    _fields_ = [
        ("k_new", C.c_void_p),
        ("v_new", C.c_void_p),
        ("qk_weight", C.c_void_p),
        ("q_out", C.c_void_p),
        ("sin_cache", C.c_void_p),
        ("cos_cache", C.c_void_p),
        ("table_len", C.c_int32),
        ("eps", C.c_float),
    ]


# Every symbol include/gqa_b200.h declares, with its ctypes signature.
class _OprojParams(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("hidden", C.c_int32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("reserved", C.c_int32),
        ("weight_ld", C.c_int64),
        ("attn_out", C.c_void_p),
        ("weight", C.c_void_p),
        ("residual", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status_dev", C.c_void_p),
        ("stream", C.c_void_p),
    ]


class _QkvParams(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("hidden", C.c_int32),
        ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("reserved", C.c_int32),
        ("weight_ld", C.c_int64),
        ("x", C.c_void_p),
        ("weight", C.c_void_p),
        ("q_out", C.c_void_p),
        ("k_out", C.c_void_p),
        ("v_out", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status_dev", C.c_void_p),
        ("stream", C.c_void_p),
    ]


_SIGNATURES = {
    "gqa_status_string": (C.c_char_p, [C.c_int]),
    "gqa_abi_version": (C.c_int, []),
    "gqa_layout_reference": (C.c_int, [C.c_int32] * 4 + [C.POINTER(_Layout)]),
    "gqa_layout_pool": (C.c_int, [C.c_int32] * 4 + [C.POINTER(_Layout)]),
    "gqa_decode_plan": (C.c_int, [C.POINTER(_DecodeParams), C.c_int32, C.POINTER(_PlanInfo)]),
    "gqa_decode": (C.c_int, [C.POINTER(_DecodeParams)]),
    "gqa_cluster_capacity": (C.c_int32, [C.c_int32]),
    "gqa_decode_static_scratch": (C.c_int, [C.POINTER(_DecodeParams)]),
    "gqa_decode_fused": (C.c_int, [C.POINTER(_DecodeParams), C.POINTER(_FusedFront)]),
    "gqa_decode_partial": (C.c_int, [C.POINTER(_DecodeParams), C.c_void_p]),
    "gqa_merge_partials": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                     C.c_void_p, C.c_void_p]),
    "gqa_qk_norm_rope_append": (C.c_int, [C.POINTER(_FrontParams)]),
    "gqa_sin_cos_cache": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "gqa_session_create": (C.c_int, [C.c_int32] * 6 + [C.POINTER(C.c_void_p)]),
    "gqa_session_destroy": (None, [C.c_void_p]),
    "gqa_session_step": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(_Layout),
                                   C.POINTER(C.c_int32), C.c_void_p, C.c_int32, C.c_int32,
                                   C.c_void_p]),
    "gqa_session_step_sharded": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.POINTER(_Layout), C.POINTER(C.c_int32),
                                           C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "gqa_session_last_timing": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64)]),
    "gqa_comm_peer_gather_fits": (C.c_int, [C.c_void_p, C.c_size_t]),
    "gqa_kv_pool_bytes": (C.c_size_t, [C.c_int32] * 5),
    "gqa_kv_pool_create": (C.c_int, [C.c_int32] * 7 + [C.POINTER(C.c_void_p)]),
    "gqa_kv_pool_destroy": (None, [C.c_void_p]),
    "gqa_kv_pool_layout": (C.c_int, [C.c_void_p, C.POINTER(_Layout)]),
    "gqa_kv_pool_reserve": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    "gqa_kv_pool_release": (C.c_int, [C.c_void_p, C.c_int32]),
    "gqa_kv_pool_free_blocks": (C.c_int32, [C.c_void_p]),
    "gqa_kv_pool_seq_blocks": (C.c_int32, [C.c_void_p, C.c_int32]),
    "gqa_kv_pool_block_table": (C.POINTER(C.c_int32), [C.c_void_p]),
    "gqa_shard_plan": (C.c_int, [C.c_int32] * 4 + [C.POINTER(C.c_int32)] * 4),
    "gqa_comm_nranks": (C.c_int32, [C.c_void_p]),
    "gqa_comm_all_gather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "gqa_comm_enable_peer_gather": (C.c_int, [C.c_void_p, C.c_size_t]),
    "gqa_comm_disable_peer_gather": (None, [C.c_void_p]),
    "gqa_comm_peer_gather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                       C.c_void_p, C.c_void_p]),
    "gqa_comm_unique_id": (C.c_int, [C.c_void_p]),
    "gqa_comm_init": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "gqa_comm_destroy": (None, [C.c_void_p]),
    "gqa_decode_sharded": (C.c_int, [C.POINTER(_DecodeParams), C.c_void_p, C.c_void_p]),
    "gqa_decode_sharded_fused": (C.c_int, [C.POINTER(_DecodeParams), C.POINTER(_FusedFront),
                                           C.c_void_p, C.c_void_p]),
    "gqa_decode_seqpar": (C.c_int, [C.POINTER(_DecodeParams), C.c_void_p]),
    "gqa_oproj_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "gqa_qkv_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "gqa_qkv_gemv": (C.c_int, [C.POINTER(_QkvParams)]),
    "gqa_oproj_residual": (C.c_int, [C.POINTER(_OprojParams)]),
    "gqa_oproj_residual_sharded": (C.c_int, [C.POINTER(_OprojParams), C.c_void_p]),
}

_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it was not built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python -m llminfer_b200.build`; "
                "there is no CPU or PyTorch fallback for this path")
        handle = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def exported_symbols() -> Sequence[str]:
    return tuple(_SIGNATURES)


def status_string(status: int) -> str:
    return lib().gqa_status_string(status).decode()


def _check(status: int, where: str) -> None:
    if status != 0:
        raise GqaError(status, where)


@dataclass(frozen=True)
class KvLayout:
    block_tokens: int
    num_blocks: int
    stride_block: int
    stride_token: int
    stride_head: int

    def c(self) -> _Layout:
        return _Layout(self.block_tokens, self.num_blocks, self.stride_block, self.stride_token,
                       self.stride_head)

    @staticmethod
    def from_c(l: _Layout) -> "KvLayout":
        return KvLayout(l.block_tokens, l.num_blocks, l.stride_block, l.stride_token,
                        l.stride_head)


def layout_reference(layer_num: int, max_seq_len: int, num_kv_heads: int,
                     head_dim: int = 128) -> KvLayout:
    out = _Layout()
    _check(lib().gqa_layout_reference(layer_num, max_seq_len, num_kv_heads, head_dim,
                                      C.byref(out)), "gqa_layout_reference")
    return KvLayout.from_c(out)


def layout_pool(num_blocks: int, block_tokens: int, num_kv_heads: int,
                head_dim: int = 128) -> KvLayout:
    out = _Layout()
    _check(lib().gqa_layout_pool(num_blocks, block_tokens, num_kv_heads, head_dim, C.byref(out)),
           "gqa_layout_pool")
    return KvLayout.from_c(out)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    if t.dtype == torch.float32:
        return DTYPE_F32
    raise TypeError(f"unsupported dtype {t.dtype}")


def _int_array(values: Optional[Sequence[int]]):
    if values is None:
        return None
    return (C.c_int32 * len(values))(*[int(v) for v in values])


def _decode_params(q, k_cache, v_cache, out, layout, seq_lens_host, seq_lens_dev, block_table,
                   fixed_block, workspace, split_keys, max_ctas, plan_len_hint, status, stream,
                   keep, early_prefetch=False):
    if q.dim() == 4:  # [batch, q_tokens, heads, head_dim]
        batch, tokens, hq, d = q.shape
    else:
        (batch, hq, d), tokens = q.shape, 1
    p = _DecodeParams()
    p.dtype = _dtype_code(q)
    p.batch, p.num_q_heads, p.head_dim = batch, hq, d
    p.q_tokens = tokens
    p.num_kv_heads = keep["num_kv_heads"]
    p.blocks_per_seq = 0 if block_table is None else block_table.shape[1]
    p.fixed_block = fixed_block
    p.split_keys = split_keys
    p.max_ctas = max_ctas
    p.plan_len_hint = plan_len_hint
    p.early_prefetch = 1 if early_prefetch else 0
    p.layout = layout.c()
    p.q, p.k_cache, p.v_cache, p.out = _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out)
    p.workspace = _ptr(workspace)
    p.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    lens = _int_array(seq_lens_host)
    keep["lens"] = lens
    p.seq_lens_host = lens
    p.seq_lens_dev = _ptr(seq_lens_dev)
    p.block_table_dev = _ptr(block_table)
    p.status_dev = _ptr(status)
    p.stream = stream
    return p


def decode_plan(*, dtype: int, batch: int, num_q_heads: int, num_kv_heads: int, layout: KvLayout,
                seq_lens: Optional[Sequence[int]], blocks_per_seq: int = 0, fixed_block: int = 0,
                split_keys: int = 0, max_ctas: int = 0, plan_len_hint: int = 0,
                workspace_bytes: int = 0, sm_count: int = 148, paged: bool = False,
                device_lens: bool = False, head_dim: int = 128, q_tokens: int = 0) -> dict:
    """Host-only split planning (no device memory is touched; pointers are placeholders)."""
    p = _DecodeParams()
    p.dtype, p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim = (
        dtype, batch, num_q_heads, num_kv_heads, head_dim)
    p.blocks_per_seq, p.fixed_block = blocks_per_seq, fixed_block
    p.split_keys, p.max_ctas, p.plan_len_hint = split_keys, max_ctas, plan_len_hint
    p.q_tokens = q_tokens
    p.layout = layout.c()
    fake = 0x1000  # validation only looks at nullness and alignment
    p.q = p.k_cache = p.v_cache = p.out = fake
    p.workspace = fake if workspace_bytes else None
    p.workspace_bytes = workspace_bytes
    lens = _int_array(seq_lens)
    p.seq_lens_host = lens
    p.seq_lens_dev = fake if device_lens else None
    p.block_table_dev = fake if paged else None
    info = _PlanInfo()
    _check(lib().gqa_decode_plan(C.byref(p), sm_count, C.byref(info)), "gqa_decode_plan")
    return {f: getattr(info, f) for f, _ in _PlanInfo._fields_}


def decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor, *,
           num_kv_heads: int, layout: KvLayout, seq_lens: Optional[Sequence[int]] = None,
           seq_lens_dev: Optional[torch.Tensor] = None,
           block_table: Optional[torch.Tensor] = None, fixed_block: int = 0,
           workspace: Optional[torch.Tensor] = None, split_keys: int = 0, max_ctas: int = 0,
           plan_len_hint: int = 0, status: Optional[torch.Tensor] = None,
           stream: Optional[int] = None, early_prefetch: bool = False,
           front: Optional["FusedFront"] = None) -> None:
    """Decode attention for q [batch, num_q_heads, 128] (or [batch, q_tokens, num_q_heads, 128])
    on the current stream (or `stream`). With `front`, q holds the raw query rows and the
    kernel runs QK-Norm + RoPE + KV append itself (gqa_decode_fused)."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    keep = {"num_kv_heads": num_kv_heads}
    p = _decode_params(q, k_cache, v_cache, out, layout, seq_lens, seq_lens_dev, block_table,
                       fixed_block, workspace, split_keys, max_ctas, plan_len_hint, status,
                       stream, keep, early_prefetch)
    if front is None:
        _check(lib().gqa_decode(C.byref(p)), "gqa_decode")
    else:
        f = front.c()
        _check(lib().gqa_decode_fused(C.byref(p), C.byref(f)), "gqa_decode_fused")


@dataclass
class FusedFront:
    """Inputs of the front stage when it runs inside the attention kernel (gqa_fused_front)."""
    k_new: torch.Tensor
    v_new: torch.Tensor
    qk_weight: torch.Tensor
    q_out: Optional[torch.Tensor] = None
    sin_cache: Optional[torch.Tensor] = None
    cos_cache: Optional[torch.Tensor] = None
    eps: float = 1e-6

    def c(self) -> _FusedFront:
        f = _FusedFront()
        f.k_new, f.v_new, f.qk_weight = _ptr(self.k_new), _ptr(self.v_new), _ptr(self.qk_weight)
        f.q_out = _ptr(self.q_out)
        f.sin_cache, f.cos_cache = _ptr(self.sin_cache), _ptr(self.cos_cache)
        f.table_len = 0 if self.sin_cache is None else self.sin_cache.shape[0]
        f.eps = self.eps
        return f


def decode_partial(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   records: torch.Tensor, *, num_kv_heads: int, layout: KvLayout,
                   seq_lens: Optional[Sequence[int]] = None,
                   seq_lens_dev: Optional[torch.Tensor] = None,
                   block_table: Optional[torch.Tensor] = None, fixed_block: int = 0,
                   workspace: Optional[torch.Tensor] = None, split_keys: int = 0,
                   status: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """Attention over a slice of the keys; leaves records [batch * heads, 130] FP32."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    keep = {"num_kv_heads": num_kv_heads}
    p = _decode_params(q, k_cache, v_cache, q, layout, seq_lens, seq_lens_dev, block_table,
                       fixed_block, workspace, split_keys, 0, 0, status, stream, keep)
    _check(lib().gqa_decode_partial(C.byref(p), _ptr(records)), "gqa_decode_partial")


def merge_partials(records: torch.Tensor, out: torch.Tensor, stream: Optional[int] = None) -> None:
    """records [nparts, rows, 130] FP32 -> out [rows..., 128] (BF16 or FP32)."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    nparts, rows, _ = records.shape
    _check(lib().gqa_merge_partials(_ptr(records), nparts, rows, out.shape[-1], _dtype_code(out),
                                    _ptr(out), stream), "gqa_merge_partials")


STATIC_SCRATCH_BYTES = 8 << 20


def decode_static_scratch(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          out: torch.Tensor, *, num_kv_heads: int, layout: KvLayout,
                          seq_lens: Optional[Sequence[int]] = None,
                          seq_lens_dev: Optional[torch.Tensor] = None,
                          block_table: Optional[torch.Tensor] = None, fixed_block: int = 0,
                          split_keys: int = 0, max_ctas: int = 0, plan_len_hint: int = 0,
                          status: Optional[torch.Tensor] = None, stream: Optional[int] = None,
                          early_prefetch: bool = False) -> None:
    """decode() without a workspace argument: the split scratch is the library's own static
    device array (for callers that may not allocate device memory); see the header for limits."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    keep = {"num_kv_heads": num_kv_heads}
    p = _decode_params(q, k_cache, v_cache, out, layout, seq_lens, seq_lens_dev, block_table,
                       fixed_block, None, split_keys, max_ctas, plan_len_hint, status, stream,
                       keep, early_prefetch)
    _check(lib().gqa_decode_static_scratch(C.byref(p)), "gqa_decode_static_scratch")


def workspace_for(batch: int, num_q_heads: int, num_kv_heads: int, device,
                  sm_count: int = 148) -> torch.Tensor:
    """A scratch tensor large enough for any plan the library may pick for this shape."""
    group = num_q_heads // num_kv_heads
    records = 16 * sm_count + 2 * batch * num_kv_heads
    return torch.empty(records * group * 130, dtype=torch.float32, device=device)


def qk_norm_rope_append(q: torch.Tensor, k_new: torch.Tensor, v_new: Optional[torch.Tensor],
                        qk_weight: torch.Tensor, k_cache: torch.Tensor,
                        v_cache: Optional[torch.Tensor], *, layout: KvLayout,
                        positions: Optional[Sequence[int]] = None,
                        positions_dev: Optional[torch.Tensor] = None,
                        q_out: Optional[torch.Tensor] = None,
                        sin_cache: Optional[torch.Tensor] = None,
                        cos_cache: Optional[torch.Tensor] = None,
                        block_table: Optional[torch.Tensor] = None, fixed_block: int = 0,
                        eps: float = 1e-6, stream: Optional[int] = None,
                        status: Optional[torch.Tensor] = None) -> None:
    """q is [batch, heads, 128] or, for several new tokens per sequence, [batch, tokens, heads,
    128] (k_new and v_new likewise); positions are those of each sequence's first new token."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    if q.dim() == 4:
        batch, tokens, hq, d = q.shape
    else:
        (batch, hq, d), tokens = q.shape, 1
    f = _FrontParams()
    f.batch, f.num_q_heads, f.num_kv_heads, f.head_dim = batch, hq, k_new.shape[-2], d
    f.q_tokens = tokens
    f.status_dev = _ptr(status)
    f.blocks_per_seq = 0 if block_table is None else block_table.shape[1]
    f.fixed_block = fixed_block
    f.table_len = 0 if sin_cache is None else sin_cache.shape[0]
    f.eps = eps
    f.layout = layout.c()
    f.q = _ptr(q)
    f.q_out = _ptr(q if q_out is None else q_out)
    f.k_new, f.v_new, f.qk_weight = _ptr(k_new), _ptr(v_new), _ptr(qk_weight)
    f.k_cache, f.v_cache = _ptr(k_cache), _ptr(v_cache)
    f.sin_cache, f.cos_cache = _ptr(sin_cache), _ptr(cos_cache)
    pos = _int_array(positions)
    f.positions_host = pos
    f.positions_dev = _ptr(positions_dev)
    f.block_table_dev = _ptr(block_table)
    f.stream = stream
    _check(lib().gqa_qk_norm_rope_append(C.byref(f)), "gqa_qk_norm_rope_append")


def sin_cos_cache(sin_cache: torch.Tensor, cos_cache: torch.Tensor, head_dim: int,
                  stream: Optional[int] = None) -> None:
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    _check(lib().gqa_sin_cos_cache(_ptr(sin_cache), _ptr(cos_cache), head_dim,
                                   sin_cache.shape[0], stream), "gqa_sin_cos_cache")


class Session:
    """Decode steps from host buffers (H2D of the new rows, kernels, D2H of the output)."""

    def __init__(self, max_batch: int, num_q_heads: int, num_kv_heads: int, max_seq_len: int,
                 head_dim: int = 128):
        self._h = C.c_void_p()
        _check(lib().gqa_session_create(DTYPE_BF16, max_batch, num_q_heads, num_kv_heads,
                                        head_dim, max_seq_len, C.byref(self._h)),
               "gqa_session_create")
        self._marshal = {}

    def step(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
             qk_weight: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             layout: KvLayout, positions: Sequence[int], out_host: torch.Tensor,
             block_table: Optional[torch.Tensor] = None, fixed_block: int = 0,
             comm: Optional["ShardComm"] = None) -> None:
        """With `comm`, out_host is the gathered [nranks, batch, local_q_heads, 128] output."""
        # The marshalled layout and positions are kept between steps: a decode loop passes the
        # same layout every step, and the same positions for every layer of a token.
        cache = self._marshal
        if cache.get("layout_key") is not layout:
            cache["layout_key"], cache["layout"] = layout, layout.c()
        key = tuple(positions)
        if cache.get("pos_key") != key:
            cache["pos_key"], cache["pos"] = key, _int_array(positions)
        lay, pos = cache["layout"], cache["pos"]
        bps = 0 if block_table is None else block_table.shape[1]
        table = None if block_table is None else block_table.data_ptr()
        handle = lib()
        if comm is None:
            rc = handle.gqa_session_step(self._h, q_host.shape[0], q_host.data_ptr(),
                                         k_host.data_ptr(), v_host.data_ptr(),
                                         qk_weight.data_ptr(), k_cache.data_ptr(),
                                         v_cache.data_ptr(), C.byref(lay), pos, table, bps,
                                         fixed_block, out_host.data_ptr())
            if rc != 0:
                raise GqaError(rc, "gqa_session_step")
        else:
            rc = handle.gqa_session_step_sharded(
                self._h, comm._h, q_host.shape[0], q_host.data_ptr(), k_host.data_ptr(),
                v_host.data_ptr(), qk_weight.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                C.byref(lay), pos, table, bps, fixed_block, out_host.data_ptr())
            if rc != 0:
                raise GqaError(rc, "gqa_session_step_sharded")

    def last_timing(self) -> dict:
        """Host-side nanoseconds of the last step: staging, launches, wait, copy-out."""
        ns = (C.c_int64 * 4)()
        _check(lib().gqa_session_last_timing(self._h, ns), "gqa_session_last_timing")
        return dict(zip(("stage_ns", "launch_ns", "wait_ns", "copy_out_ns"), ns))

    def close(self) -> None:
        if self._h:
            lib().gqa_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KvPool:
    """Host-side block pool; `table()` returns the [max_seqs, max_blocks_per_seq] block table."""

    def __init__(self, num_blocks: int, block_tokens: int, num_kv_heads: int, max_seqs: int,
                 max_blocks_per_seq: int, dtype: int = DTYPE_BF16, head_dim: int = 128):
        self._h = C.c_void_p()
        self.max_seqs, self.max_blocks_per_seq = max_seqs, max_blocks_per_seq
        self.bytes = lib().gqa_kv_pool_bytes(num_blocks, block_tokens, num_kv_heads, head_dim,
                                             dtype)
        _check(lib().gqa_kv_pool_create(num_blocks, block_tokens, num_kv_heads, head_dim, dtype,
                                        max_seqs, max_blocks_per_seq, C.byref(self._h)),
               "gqa_kv_pool_create")

    def layout(self) -> KvLayout:
        out = _Layout()
        _check(lib().gqa_kv_pool_layout(self._h, C.byref(out)), "gqa_kv_pool_layout")
        return KvLayout.from_c(out)

    def reserve(self, seq: int, num_tokens: int) -> None:
        _check(lib().gqa_kv_pool_reserve(self._h, seq, num_tokens), "gqa_kv_pool_reserve")

    def release(self, seq: int) -> None:
        _check(lib().gqa_kv_pool_release(self._h, seq), "gqa_kv_pool_release")

    def free_blocks(self) -> int:
        return lib().gqa_kv_pool_free_blocks(self._h)

    def seq_blocks(self, seq: int) -> int:
        return lib().gqa_kv_pool_seq_blocks(self._h, seq)

    def table(self) -> torch.Tensor:
        ptr = lib().gqa_kv_pool_block_table(self._h)
        n = self.max_seqs * self.max_blocks_per_seq
        flat = [ptr[i] for i in range(n)]
        return torch.tensor(flat, dtype=torch.int32).view(self.max_seqs, self.max_blocks_per_seq)

    def close(self) -> None:
        if self._h:
            lib().gqa_kv_pool_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_plan(num_q_heads: int, num_kv_heads: int, nranks: int, rank: int) -> dict:
    vals = [C.c_int32() for _ in range(4)]
    _check(lib().gqa_shard_plan(num_q_heads, num_kv_heads, nranks, rank,
                                *[C.byref(v) for v in vals]), "gqa_shard_plan")
    names = ("first_kv_head", "num_local_kv_heads", "first_q_head", "num_local_q_heads")
    return {n: v.value for n, v in zip(names, vals)}


class ShardComm:
    """NCCL communicator owned by the library (one per process / GPU)."""

    def __init__(self, unique_id: bytes, nranks: int, rank: int):
        self._h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, COMM_ID_BYTES)
        _check(lib().gqa_comm_init(buf, nranks, rank, C.byref(self._h)), "gqa_comm_init")
        self.nranks, self.rank = nranks, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(COMM_ID_BYTES)
        _check(lib().gqa_comm_unique_id(buf), "gqa_comm_unique_id")
        return buf.raw

    def enable_peer_gather(self, max_bytes_per_rank: int) -> None:
        """Collective: from now on decode_sharded gathers with peer stores over NVLink."""
        _check(lib().gqa_comm_enable_peer_gather(self._h, max_bytes_per_rank),
               "gqa_comm_enable_peer_gather")

    def disable_peer_gather(self) -> None:
        lib().gqa_comm_disable_peer_gather(self._h)

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor,
                   stream: Optional[int] = None) -> None:
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        _check(lib().gqa_comm_all_gather(self._h, _ptr(send), _ptr(recv),
                                         send.numel() * send.element_size(), stream),
               "gqa_comm_all_gather")

    def peer_gather(self, send: torch.Tensor, recv: torch.Tensor,
                    status: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        _check(lib().gqa_comm_peer_gather(self._h, _ptr(send), _ptr(recv),
                                          send.numel() * send.element_size(), _ptr(status),
                                          stream), "gqa_comm_peer_gather")

    def close(self) -> None:
        if self._h:
            lib().gqa_comm_destroy(self._h)
            self._h = C.c_void_p()


def decode_sharded(comm: ShardComm, gathered: torch.Tensor, q, k_cache, v_cache, out, *,
                   num_kv_heads: int, layout: KvLayout, **kw) -> None:
    """Local decode on this rank's heads followed by the all-gather into `gathered`."""
    stream = kw.pop("stream", None)
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    keep = {"num_kv_heads": num_kv_heads}
    p = _decode_params(q, k_cache, v_cache, out, layout, kw.get("seq_lens"),
                       kw.get("seq_lens_dev"), kw.get("block_table"), kw.get("fixed_block", 0),
                       kw.get("workspace"), kw.get("split_keys", 0), kw.get("max_ctas", 0),
                       kw.get("plan_len_hint", 0), kw.get("status"), stream, keep,
                       kw.get("early_prefetch", False))
    front = kw.get("front")
    if front is None:
        _check(lib().gqa_decode_sharded(C.byref(p), comm._h, _ptr(gathered)), "gqa_decode_sharded")
    else:
        f = front.c()
        _check(lib().gqa_decode_sharded_fused(C.byref(p), C.byref(f), comm._h, _ptr(gathered)),
               "gqa_decode_sharded_fused")


def decode_seqpar(comm: ShardComm, q, k_cache, v_cache, out, *, num_kv_heads: int,
                  layout: KvLayout, **kw) -> None:
    """Sequence-parallel decode: this rank's slice of every sequence, all heads; `out` gets the
    complete output on every rank."""
    stream = kw.pop("stream", None)
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    keep = {"num_kv_heads": num_kv_heads}
    p = _decode_params(q, k_cache, v_cache, out, layout, kw.get("seq_lens"),
                       kw.get("seq_lens_dev"), kw.get("block_table"), kw.get("fixed_block", 0),
                       kw.get("workspace"), kw.get("split_keys", 0), kw.get("max_ctas", 0),
                       kw.get("plan_len_hint", 0), kw.get("status"), stream, keep,
                       kw.get("early_prefetch", False))
    _check(lib().gqa_decode_seqpar(C.byref(p), comm._h), "gqa_decode_seqpar")


def oproj_workspace(hidden: int, num_kv_heads: int, device) -> Optional[torch.Tensor]:
    """Zero-filled workspace for oproj_residual (None when none is needed)."""
    nbytes = lib().gqa_oproj_workspace_bytes(hidden, num_kv_heads)
    if nbytes == 0:
        return None
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def oproj_residual(attn_out: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, *,
                   num_kv_heads: int, workspace: Optional[torch.Tensor] = None,
                   comm: Optional[ShardComm] = None, weight_ld: Optional[int] = None, status: Optional[torch.Tensor] = None,
                   stream: Optional[int] = None) -> None:
    """residual [batch, hidden] += attn_out [batch, heads, 128] . weight[hidden, heads * 128]^T.

    `weight` may be a column slice of a wider matrix: pass the slice's first element as a
    tensor view and the full row length as `weight_ld`. With `comm` the per-KV-head sums are
    exchanged over the peer windows and every rank ends with the complete result.
    `workspace` comes from oproj_workspace() (needed for more than one KV head)."""
    batch, heads, dim = attn_out.shape
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    p = _OprojParams()
    p.batch, p.hidden = batch, residual.shape[-1]
    p.num_q_heads, p.num_kv_heads, p.head_dim = heads, num_kv_heads, dim
    p.weight_ld = weight_ld if weight_ld is not None else weight.stride(0)
    p.attn_out, p.weight, p.residual = _ptr(attn_out), _ptr(weight), _ptr(residual)
    p.status_dev, p.stream = _ptr(status), stream
    if workspace is not None:
        p.workspace, p.workspace_bytes = _ptr(workspace), workspace.numel() * workspace.element_size()
    if comm is None:
        _check(lib().gqa_oproj_residual(C.byref(p)), "gqa_oproj_residual")
    else:
        _check(lib().gqa_oproj_residual_sharded(C.byref(p), comm._h),
               "gqa_oproj_residual_sharded")


def qkv_workspace(hidden: int, num_q_heads: int, num_kv_heads: int, device) -> Optional[torch.Tensor]:
    """Zero-filled workspace for qkv_gemv (None when none is needed)."""
    nbytes = lib().gqa_qkv_workspace_bytes(hidden, num_q_heads, num_kv_heads)
    if nbytes == 0:
        return None
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def qkv_gemv(x: torch.Tensor, weight: torch.Tensor, q_out: torch.Tensor, k_out: torch.Tensor,
             v_out: torch.Tensor, *, workspace: Optional[torch.Tensor] = None,
             status: Optional[torch.Tensor] = None, stream: Optional[int] = None) -> None:
    """Packed QKV projection: x [batch, hidden], weight [(Hq + 2 Hkv) * 128, hidden] ->
    q_out [batch, Hq, 128], k_out and v_out [batch, Hkv, 128]."""
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    p = _QkvParams()
    p.batch, p.hidden = x.shape
    p.num_q_heads, p.num_kv_heads, p.head_dim = q_out.shape[1], k_out.shape[1], q_out.shape[2]
    p.weight_ld = weight.stride(0)
    p.x, p.weight = _ptr(x), _ptr(weight)
    p.q_out, p.k_out, p.v_out = _ptr(q_out), _ptr(k_out), _ptr(v_out)
    if workspace is not None:
        p.workspace, p.workspace_bytes = _ptr(workspace), workspace.numel() * workspace.element_size()
    p.status_dev, p.stream = _ptr(status), stream
    _check(lib().gqa_qkv_gemv(C.byref(p)), "gqa_qkv_gemv")
