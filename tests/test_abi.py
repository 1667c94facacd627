"""Host-side behaviour of the C ABI that needs no GPU: the library loads and exports every
symbol the header declares, argument validation returns the documented codes, the split
planner, the KV block pool and the head-parallel partition."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    return pkg


def test_library_exports_every_declared_symbol(gqa):
    header = (ROOT / "include" / "gqa_b200.h").read_text()
    declared = set(re.findall(r"\b(gqa_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 25
    handle = gqa.lib()
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert declared == set(gqa.binding.exported_symbols())
    assert handle.gqa_abi_version() == 3
    assert gqa.status_string(0) == "ok"
    assert "workspace" in gqa.status_string(-6)


def test_missing_library_fails_loudly(monkeypatch, gqa, tmp_path):
    from llminfer_b200 import binding
    monkeypatch.setattr(binding, "_lib", None)
    monkeypatch.setattr(binding, "_LIB_PATH", tmp_path / "libgqa_b200.so")
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        binding.lib()


def test_layouts(gqa):
    ref = gqa.layout_reference(36, 4096, 8)
    assert (ref.block_tokens, ref.num_blocks) == (4096, 36)
    assert (ref.stride_head, ref.stride_token, ref.stride_block) == (128, 1024, 4096 * 1024)
    pool = gqa.layout_pool(100, 256, 8)
    assert (pool.stride_token, pool.stride_head, pool.stride_block) == (128, 256 * 128, 8 * 256 * 128)
    with pytest.raises(gqa.GqaError) as e:
        gqa.layout_pool(100, 100, 8)  # not a multiple of the 32-key chunk
    assert e.value.status == -3


def plan(gqa, **kw):
    base = dict(dtype=2, batch=1, num_q_heads=32, num_kv_heads=8,
                layout=gqa.layout_reference(1, 131072, 8), seq_lens=[1024])
    base.update(kw)
    return gqa.decode_plan(**base)


def test_validation_codes(gqa):
    codes = {}
    for name, kw in {
        "dtype": dict(dtype=3),
        "head_dim": dict(head_dim=64),
        "group_not_integer": dict(num_q_heads=30),
        "group_too_wide": dict(num_q_heads=128),
        "len_zero": dict(seq_lens=[0]),
        "len_past_cache": dict(seq_lens=[131073]),
        "block_out_of_range": dict(fixed_block=1),
        "batch_needs_table": dict(batch=2, seq_lens=[5, 5]),
        "ragged_needs_device_lens": dict(batch=2, seq_lens=[5, 6], paged=True, blocks_per_seq=1),
        "negative_split": dict(split_keys=-2),
    }.items():
        with pytest.raises(gqa.GqaError) as e:
            plan(gqa, **kw)
        codes[name] = e.value.status
    assert codes == {"dtype": -2, "head_dim": -3, "group_not_integer": -3, "group_too_wide": -8,
                     "len_zero": -5, "len_past_cache": -5, "block_out_of_range": -5,
                     "batch_needs_table": -3, "ragged_needs_device_lens": -8,
                     "negative_split": -5}
    bad = gqa.KvLayout(4096, 1, 4096 * 1024, 1028, 128)  # token stride not 16-byte aligned
    with pytest.raises(gqa.GqaError) as e:
        plan(gqa, layout=bad)
    assert e.value.status == -4


def test_compute_entry_points_reject_bad_arguments_before_touching_the_device(gqa):
    handle = gqa.lib()
    assert handle.gqa_decode(None) == -1
    assert handle.gqa_qk_norm_rope_append(None) == -1
    assert handle.gqa_sin_cos_cache(None, None, 128, 16, None) == -1
    out = C.c_void_p()
    assert handle.gqa_session_create(1, 1, 32, 8, 128, 64, C.byref(out)) == -2  # FP32 session
    assert handle.gqa_session_create(2, 1, 32, 8, 64, 64, C.byref(out)) == -3


def test_binding_structs_match_the_header_layout(gqa, tmp_path):
    """The ctypes mirrors of the parameter structs have the size and field offsets the C
    compiler gives the declarations in include/gqa_b200.h."""
    import subprocess
    from llminfer_b200 import binding as B
    mirrors = {"gqa_kv_layout": B._Layout, "gqa_decode_params": B._DecodeParams,
               "gqa_decode_plan_info": B._PlanInfo, "gqa_front_params": B._FrontParams,
               "gqa_oproj_params": B._OprojParams, "gqa_qkv_params": B._QkvParams,
               "gqa_fused_front": B._FusedFront}
    lines = ["#include <stddef.h>", "#include <stdio.h>", '#include "gqa_b200.h"', "int main(void) {"]
    for name, mirror in mirrors.items():
        lines.append(f'printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in mirror._fields_:
            lines.append(f'printf("{name}.{field} %zu\\n", offsetof({name}, {field}));')
    lines += ["return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    got = dict(line.split() for line in out.strip().splitlines())
    for name, mirror in mirrors.items():
        assert int(got[name]) == C.sizeof(mirror), name
        for field, _ in mirror._fields_:
            assert int(got[f"{name}.{field}"]) == getattr(mirror, field).offset, (name, field)


def test_projection_entry_points_validate_on_the_host(gqa):
    """Workspace sizes are pure functions; bad shapes and missing buffers are refused before
    any CUDA call (device pointers here are fake, non-null and aligned)."""
    from llminfer_b200 import binding as B
    handle = gqa.lib()
    assert handle.gqa_oproj_residual(None) == -1
    assert handle.gqa_qkv_gemv(None) == -1
    assert handle.gqa_oproj_residual_sharded(None, None) == -1
    assert handle.gqa_oproj_workspace_bytes(5120, 1) == 0           # one KV head: nothing to meet
    assert handle.gqa_oproj_workspace_bytes(5120, 8) == 256 + 8 * 8 * 5120 * 8
    assert handle.gqa_oproj_workspace_bytes(0, 8) == 0
    assert handle.gqa_qkv_workspace_bytes(1024, 16, 8) == 0         # 8 column heads: one group
    assert handle.gqa_qkv_workspace_bytes(5120, 64, 8) == 256 + 5 * 8 * (80 * 128) * 8
    assert handle.gqa_qkv_workspace_bytes(1000, 16, 8) == 0         # not whole 128-column heads

    def oproj(**kw):
        p = B._OprojParams()
        p.batch, p.hidden, p.num_q_heads, p.num_kv_heads, p.head_dim = 1, 64, 8, 1, 128
        p.weight_ld = 1024
        p.attn_out = p.weight = p.residual = 0x1000
        for k, v in kw.items():
            setattr(p, k, v)
        return handle.gqa_oproj_residual(C.byref(p))

    assert oproj(residual=None) == -1
    assert oproj(hidden=56) == -3              # rows not a multiple of 16
    assert oproj(head_dim=64) == -3
    assert oproj(num_kv_heads=3) == -3         # heads not divisible
    assert oproj(num_q_heads=34, num_kv_heads=2, weight_ld=34 * 128) == -3  # 17 heads per KV head
    assert oproj(weight_ld=512) == -3          # pitch below the columns
    assert oproj(weight_ld=1028) == -3         # pitch not a multiple of 8
    assert oproj(weight=0x1008) == -4          # not 16-byte aligned
    assert oproj(num_kv_heads=8) == -1         # workspace missing
    assert oproj(num_kv_heads=8, workspace=0x2000, workspace_bytes=64) == -6

    q = B._QkvParams()
    q.batch, q.hidden, q.num_q_heads, q.num_kv_heads, q.head_dim = 1, 192, 1, 1, 128
    q.weight_ld = 192
    q.x = q.weight = q.q_out = q.k_out = q.v_out = 0x1000
    assert handle.gqa_qkv_gemv(C.byref(q)) == -3   # hidden not a multiple of 128
    q.hidden, q.weight_ld, q.v_out = 256, 256, None
    assert handle.gqa_qkv_gemv(C.byref(q)) == -1   # a destination is missing


def test_planner_short_context_needs_no_second_launch(gqa):
    p = plan(gqa, seq_lens=[96])
    assert p["needs_combine"] == 0 and p["workspace_bytes"] == 0
    assert p["num_items"] == 8 and p["num_ctas"] == 8 and p["max_splits"] == 1


def test_planner_fills_the_gpu_at_long_context(gqa):
    for hq, batch, length in ((32, 1, 32768), (64, 4, 131072), (32, 1, 1024)):
        layout = gqa.layout_pool(batch * (length // 256), 256, 8)
        p = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=8, layout=layout,
                            seq_lens=[length] * batch, paged=True, blocks_per_seq=length // 256,
                            device_lens=True)
        chunks = length // 32
        assert p["needs_combine"] == 1
        fair = batch * 8 * chunks / 148
        assert p["even_cut"] == 0  # equal lengths: uniform splits
        assert p["num_ctas"] >= 128 or p["num_items"] < 148
        rounds = -(-p["num_items"] // 148)
        # No CTA works on more than ~6% above its fair share of the chunks.
        per_cta = rounds * p["split_chunks"]
        assert per_cta <= max(1.10 * fair + 4, 8), (length, p)
        assert p["workspace_bytes"] == p["num_items"] * (hq // 8) * 130 * 4
    assert p["cluster_size"] > 0  # 1K: merged inside clusters


def test_planner_cuts_ragged_batches_evenly(gqa):
    """Lengths that differ: uniform splits leave some CTAs with far more keys than others; the
    even cut gives every CTA the same number of stages and needs num_ctas + units records
    whatever the lengths are. An explicit split size, a scratch that cannot hold those records,
    equal lengths and lengths known on the device only keep uniform splits."""
    lens = [7041, 4359, 4800, 4966, 5665, 4013, 2459, 3116, 4044, 6423, 4328, 6447, 630, 7337,
            4651, 4958]
    layout = gqa.layout_pool(16 * 32, 256, 8)
    kw = dict(dtype=2, batch=16, num_q_heads=32, num_kv_heads=8, layout=layout, seq_lens=lens,
              paged=True, blocks_per_seq=32, device_lens=True)
    p = gqa.decode_plan(**kw)
    rec = 4 * 130 * 4
    assert p["even_cut"] == 1 and p["num_ctas"] == 148 and p["needs_combine"] == 1
    assert p["split_chunks"] == 2 and p["num_items"] == 148 + 128 and p["cluster_size"] == 0
    assert p["workspace_bytes"] >= p["num_items"] * rec
    assert gqa.decode_plan(split_keys=2048, **kw)["even_cut"] == 0
    tight = gqa.decode_plan(workspace_bytes=200 * rec, **kw)
    assert tight["even_cut"] == 0 and tight["workspace_bytes"] <= 200 * rec
    assert gqa.decode_plan(**dict(kw, seq_lens=[4096] * 16))["even_cut"] == 0  # equal lengths
    asked = gqa.decode_plan(**dict(kw, seq_lens=[4096] * 16, split_keys=gqa.SPLIT_EVEN))
    assert asked["even_cut"] == 1 and asked["num_items"] == 148 + 128
    with pytest.raises(gqa.GqaError) as e:  # asked for, but the scratch cannot hold the records
        gqa.decode_plan(workspace_bytes=200 * rec, split_keys=gqa.SPLIT_EVEN, **kw)
    assert e.value.status == -6
    with pytest.raises(gqa.GqaError) as e:
        gqa.decode_plan(**dict(kw, dtype=1, split_keys=gqa.SPLIT_EVEN))
    assert e.value.status == -8
    with pytest.raises(gqa.GqaError) as e:
        gqa.decode_plan(**dict(kw, split_keys=-2))
    assert e.value.status == -5
    assert gqa.decode_plan(**dict(kw, seq_lens=None, plan_len_hint=8192))["even_cut"] == 0


def test_planner_respects_overrides_and_workspace(gqa):
    p = plan(gqa, seq_lens=[4096], split_keys=100)
    assert p["split_chunks"] == 4 and p["max_splits"] == 32 and p["num_items"] == 256
    p = plan(gqa, seq_lens=[4096], max_ctas=16)
    assert p["num_ctas"] <= 16
    small = 8 * 4 * 130 * 4 * 3  # room for three splits per unit
    p = plan(gqa, seq_lens=[32768], workspace_bytes=small)
    assert p["workspace_bytes"] <= small and p["max_splits"] <= 3
    with pytest.raises(gqa.GqaError) as e:
        plan(gqa, seq_lens=[32768], workspace_bytes=small, split_keys=64)
    assert e.value.status == -6


def test_planner_device_lengths_size_the_scratch_for_full_sequences(gqa):
    layout = gqa.layout_pool(16 * 32, 256, 8)
    p = gqa.decode_plan(dtype=2, batch=16, num_q_heads=32, num_kv_heads=8, layout=layout,
                        seq_lens=None, paged=True, blocks_per_seq=32, device_lens=True,
                        plan_len_hint=4096)
    full_items = 16 * 8 * -(-(32 * 256 // 32) // p["split_chunks"])
    assert p["num_items"] == full_items
    assert p["workspace_bytes"] == full_items * 4 * 130 * 4


def test_planner_coarsens_a_hinted_split_that_the_scratch_cannot_hold(gqa):
    """Lengths on the device only: the hint asks for a fine split, the records are sized for
    full sequences, and a scratch too small for that split gets a coarser one, not an error."""
    layout = gqa.layout_pool(16 * 32, 256, 8)
    kw = dict(dtype=2, batch=16, num_q_heads=32, num_kv_heads=8, layout=layout, seq_lens=None,
              paged=True, blocks_per_seq=32, device_lens=True, plan_len_hint=512)
    free = gqa.decode_plan(**kw)
    small = free["workspace_bytes"] // 3
    tight = gqa.decode_plan(workspace_bytes=small, **kw)
    assert tight["workspace_bytes"] <= small
    assert tight["split_chunks"] > free["split_chunks"]
    assert tight["num_items"] == 16 * 8 * -(-(32 * 256 // 32) // tight["split_chunks"])
    with pytest.raises(gqa.GqaError) as e:  # an explicit split is never changed
        gqa.decode_plan(workspace_bytes=small, split_keys=free["split_chunks"] * 32, **kw)
    assert e.value.status == -6


def test_planner_offers_cluster_merge_for_short_contexts_only(gqa):
    """One cluster per unit, one CTA per split: offered when every unit has 2..16 splits and the
    grid is one wave (without a GPU to ask, for the portable sizes up to 8 only)."""
    short = plan(gqa, seq_lens=[1024])
    assert short["needs_combine"] == 1 and 2 <= short["cluster_size"] <= 8
    assert short["cluster_size"] == short["max_splits"] and 8 * short["cluster_size"] <= 148
    assert short["workspace_bytes"] > 0  # still reported: gathers and records need it
    long = plan(gqa, seq_lens=[131072])
    assert long["needs_combine"] == 1 and long["cluster_size"] == 0
    assert plan(gqa, seq_lens=[96])["cluster_size"] == 0  # not split at all
    assert plan(gqa, dtype=1, seq_lens=[1024])["cluster_size"] == 0  # FP32 path
    assert gqa.lib().gqa_cluster_capacity(1) == 0 and gqa.lib().gqa_cluster_capacity(17) == 0


def test_kv_pool_bookkeeping(gqa):
    pool = gqa.KvPool(num_blocks=10, block_tokens=256, num_kv_heads=8, max_seqs=4,
                      max_blocks_per_seq=4)
    assert pool.bytes == 10 * 8 * 256 * 128 * 2
    assert pool.layout() == gqa.layout_pool(10, 256, 8)
    pool.reserve(0, 1)
    pool.reserve(1, 600)
    pool.reserve(0, 257)
    table = pool.table()
    assert table[0].tolist() == [0, 4, -1, -1] and table[1].tolist() == [1, 2, 3, -1]
    assert pool.free_blocks() == 5 and pool.seq_blocks(1) == 3
    pool.reserve(1, 100)  # shrinking requests keep what is held
    assert pool.seq_blocks(1) == 3
    with pytest.raises(gqa.GqaError) as e:
        pool.reserve(2, 5 * 256)  # more blocks than a sequence may hold
    assert e.value.status == -5
    pool.reserve(2, 4 * 256)
    with pytest.raises(gqa.GqaError) as e:
        pool.reserve(3, 2 * 256)  # only one block left: nothing is taken
    assert e.value.status == -10 and pool.free_blocks() == 1 and pool.seq_blocks(3) == 0
    pool.release(1)
    assert pool.free_blocks() == 4 and pool.table()[1].tolist() == [-1] * 4
    pool.reserve(3, 2 * 256)
    used = [b for row in pool.table().tolist() for b in row if b >= 0]
    assert len(used) == len(set(used)) == 8
    pool.close()
    assert gqa.lib().gqa_kv_pool_bytes(10, 100, 8, 128, 2) == 0


def test_shard_plan(gqa):
    for n in (1, 2, 4, 8):
        seen = []
        for r in range(n):
            s = gqa.shard_plan(64, 8, n, r)
            assert s["num_local_kv_heads"] == 8 // n and s["num_local_q_heads"] == 64 // n
            assert s["first_q_head"] == s["first_kv_head"] * 8
            seen += list(range(s["first_kv_head"], s["first_kv_head"] + s["num_local_kv_heads"]))
        assert seen == list(range(8))
    with pytest.raises(gqa.GqaError) as e:
        gqa.shard_plan(64, 8, 3, 0)
    assert e.value.status == -3
    with pytest.raises(gqa.GqaError) as e:
        gqa.shard_plan(64, 8, 4, 4)
    assert e.value.status == -5


def test_shim_exports_the_reference_kernel_symbols(built_lib):
    """The shim library carries kernel::mha_kernel_cu & co. under the reference's mangled names."""
    import subprocess
    from llminfer_b200 import build
    lib = build.build_shim()
    names = subprocess.run(["nm", "-D", "--defined-only", "-C", str(lib)], capture_output=True,
                           text=True, check=True).stdout
    for symbol in ("kernel::mha_kernel_cu(tensor::Tensor const&",
                   "kernel::fused_qk_norm_rope_kernel_cu(tensor::Tensor const&",
                   "kernel::sin_cos_cache_precompute_cu(tensor::Tensor const&",
                   "kernel::fused_gemv_add_kernel_cu(tensor::Tensor const&",
                   "kernel::get_fused_gemv_add_kernel(base::DeviceType)",
                   "kernel::fused_qkv_gemv_kernel_cu(tensor::Tensor const&",
                   "kernel::get_fused_qkv_gemv_kernel(base::DeviceType)",
                   "kernel::get_mha_kernel(base::DeviceType)",
                   "kernel::get_fused_qk_norm_rope_kernel(base::DeviceType)",
                   "op::MultiHeadAttention::forward()",
                   "op::QKNormRoPELaryer::forward()"):
        assert symbol in names, symbol


def test_kernel_shim_compiles_against_the_reference_headers():
    """Drop-in check: the entry points build with the reference's own tensor headers."""
    import os
    import subprocess
    ref = Path(os.environ.get("LLMINFER_REFERENCE") or ROOT.parent / "reference")
    if not (ref / "code" / "include" / "tensor" / "tensor.h").exists():
        pytest.skip("reference checkout not mounted")
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-I", str(ROOT / "oracle" / "ref_build"),
           "-I", str(ref / "code" / "include"), "-I", "/usr/local/cuda/include",
           "-I", str(ROOT / "include"), "-I", str(ROOT / "llminfer_b200" / "shim" / "include"),
           str(ROOT / "llminfer_b200" / "shim" / "src" / "kernel_shim.cpp")]
    run = subprocess.run(cmd, capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
