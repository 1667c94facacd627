"""GPU parity of the output projection with residual add (gqa_oproj_residual) against the
golden outputs of the reference's own kernel and against the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

ULP_TOL = 1            # BF16 units in the last place, against the reference kernel's output
ABS_TOL = 2e-5         # ... or this close in value: near zero a unit in the last place is
                       # smaller than the FP32 rounding of a sum of thousands of unit-scale terms
MISMATCH_TOL = 0.02    # share of outputs allowed to sit on the other side of a rounding boundary


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200
    return llminfer_b200


@pytest.fixture(scope="module")
def golden_proj():
    return np.load(Path(__file__).resolve().parent / "golden" / "ref_cuda_proj.npz")


def run(gqa, x_bits, w_bits, r_bits, *, kv_heads, **kw):
    """x [batch, k], w [n, ld], r [batch, n] bits -> new residual bits."""
    batch, k = x_bits.shape
    x = H.bf16_tensor(x_bits).reshape(batch, k // 128, 128)
    w = H.bf16_tensor(w_bits)
    r = H.bf16_tensor(r_bits).clone()
    ws = gqa.oproj_workspace(r.shape[-1], kv_heads, "cuda:0")
    for _ in range(2):  # the second call finds the workspace as the first one left it
        out = r.clone()
        gqa.oproj_residual(x, w, out, num_kv_heads=kv_heads, workspace=ws, **kw)
    torch.cuda.synchronize()
    return H.bits_of(out)


def check(got, want, where):
    bad = H.bf16_mismatches(got, want, ULP_TOL, ABS_TOL)
    assert not bad.any(), (where, int(bad.sum()))
    assert (got != want).mean() <= MISMATCH_TOL, (where, float((got != want).mean()))


@pytest.mark.parametrize("index", range(len(cases.OPROJ_CASES)))
def test_matches_reference_kernel_output(gqa, golden_proj, index):
    name, n, k = cases.OPROJ_CASES[index]
    x, w, r = cases.oproj_inputs(index)
    heads = k // 128
    for kv_heads in [kv for kv in (1, 2, 8) if heads % kv == 0 and heads // kv <= 16]:
        got = run(gqa, x[None], w, r[None], kv_heads=kv_heads)[0]
        check(got, golden_proj[f"oproj/{name}/out"], (name, kv_heads, "reference kernel"))
        check(got, oracle.gemv_add(x, w, r, accum=1), (name, kv_heads, "fp64 oracle"))


@pytest.mark.parametrize("batch", [1, 3, 8, 11])
@pytest.mark.parametrize("heads,kv_heads", [(1, 1), (2, 1), (4, 2), (8, 8), (16, 8), (40, 8),
                                            (3, 1), (12, 1), (32, 2)])
def test_batches_and_head_counts(gqa, batch, heads, kv_heads):
    rng = np.random.default_rng(1000 * batch + heads)
    n, k = 80, heads * 128
    x = cases.to_bf16_bits(rng.standard_normal((batch, k), dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) / np.float32(np.sqrt(k)))
    r = cases.to_bf16_bits(rng.standard_normal((batch, n), dtype=np.float32))
    got = run(gqa, x, w, r, kv_heads=kv_heads)
    check(got, oracle.gemv_add(x, w, r, accum=1), "fp64 oracle")
    # A token's result does not depend on which other tokens share the launch.
    for b in (0, batch - 1):
        alone = run(gqa, x[b:b + 1], w, r[b:b + 1], kv_heads=kv_heads)
        assert np.array_equal(alone[0], got[b])


def test_column_slice_of_a_wider_matrix(gqa):
    """Each rank of a KV-head-parallel node reads its own columns inside the full matrix."""
    rng = np.random.default_rng(5)
    n, heads, total_heads = 64, 8, 32
    k, ld = heads * 128, total_heads * 128
    x = cases.to_bf16_bits(rng.standard_normal((2, k), dtype=np.float32))
    w_full = cases.to_bf16_bits(rng.standard_normal((n, ld), dtype=np.float32) / np.float32(32.0))
    r = cases.to_bf16_bits(rng.standard_normal((2, n), dtype=np.float32))
    first = 16 * 128
    packed = np.ascontiguousarray(w_full[:, first:first + k])
    want = run(gqa, x, packed, r, kv_heads=2)
    w_dev = H.bf16_tensor(w_full)
    res = H.bf16_tensor(r).clone()
    gqa.oproj_residual(H.bf16_tensor(x).reshape(2, heads, 128), w_dev[:, first:], res,
                       num_kv_heads=2, workspace=gqa.oproj_workspace(n, 2, "cuda:0"))
    torch.cuda.synchronize()
    assert np.array_equal(H.bits_of(res), want)
    check(want, oracle.gemv_add(x, packed, r, accum=1), "fp64 oracle")


def test_qwen3_32b_shape_batch4(gqa):
    """The benchmark model's projection: 5120 rows, 64 heads, 4 tokens."""
    rng = np.random.default_rng(32)
    n, heads, batch = 5120, 64, 4
    k = heads * 128
    x = cases.to_bf16_bits(rng.standard_normal((batch, k), dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) / np.float32(np.sqrt(k)))
    r = cases.to_bf16_bits(rng.standard_normal((batch, n), dtype=np.float32))
    got = run(gqa, x, w, r, kv_heads=8)
    check(got, oracle.gemv_add(x, w, r, accum=1), "fp64 oracle")
    # Linearity in the residual: a zero residual gives the bare product, rounded once.
    bare = run(gqa, x, w, np.zeros_like(r), kv_heads=8)
    full = oracle.gemv_add(x, w, np.zeros_like(r), accum=2)
    check(bare, cases.to_bf16_bits(full.astype(np.float32)), "bare product")


def test_rejects_unsupported_shapes(gqa):
    x = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda:0")
    w = torch.zeros(64, 1024, dtype=torch.bfloat16, device="cuda:0")
    r = torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda:0")
    ws = gqa.oproj_workspace(64, 8, "cuda:0")
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(x, w, r[:, :56], num_kv_heads=8, workspace=ws)  # rows % 16 != 0
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(x, w, r, num_kv_heads=3, workspace=ws)       # heads not divisible
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(x, w, r, num_kv_heads=8)                     # workspace missing
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(x, w, r, num_kv_heads=8, workspace=ws[:64])  # workspace too small
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(x, w, r, num_kv_heads=8, workspace=ws, weight_ld=512)  # pitch < columns
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(x, w.view(-1)[4:4 + 64 * 1016].view(64, 1016), r, num_kv_heads=8,
                           workspace=ws)                                # weight not 16-byte aligned
    wide = torch.zeros(1, 34, 128, dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(gqa.GqaError):
        gqa.oproj_residual(wide, torch.zeros(64, 34 * 128, dtype=torch.bfloat16, device="cuda:0"),
                           r, num_kv_heads=2, workspace=ws)             # 17 heads per KV head


# ---- packed QKV projection (same kernel, split destinations) --------------------------------
def run_qkv(gqa, x_bits, w_bits, hq, hkv):
    batch, hidden = x_bits.shape
    x, w = H.bf16_tensor(x_bits), H.bf16_tensor(w_bits)
    ws = gqa.qkv_workspace(hidden, hq, hkv, "cuda:0")
    for _ in range(2):  # the second call finds the workspace as the first one left it
        q = torch.full((batch, hq, 128), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        k = torch.full((batch, hkv, 128), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        v = torch.full((batch, hkv, 128), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        gqa.qkv_gemv(x, w, q, k, v, workspace=ws)
    torch.cuda.synchronize()
    return [H.bits_of(t).reshape(batch, -1) for t in (q, k, v)]


@pytest.mark.parametrize("index", range(len(cases.QKV_CASES)))
def test_qkv_matches_reference_kernel_output(gqa, golden_proj, index):
    name, hidden, hq, hkv = cases.QKV_CASES[index]
    x, w = cases.qkv_inputs(index)
    got = run_qkv(gqa, x[None], w, hq, hkv)
    want64 = oracle.qkv_gemv(x, w, hq * 128, hkv * 128, accum=1)
    for part, bits, w64 in zip("qkv", got, want64):
        check(bits[0], golden_proj[f"qkv/{name}/{part}"], (name, part, "reference kernel"))
        check(bits[0], w64, (name, part, "fp64 oracle"))


@pytest.mark.parametrize("batch", [1, 4, 9])
@pytest.mark.parametrize("hidden,hq,hkv", [(128, 1, 1), (640, 2, 1), (1024, 16, 8), (5120, 8, 1)])
def test_qkv_batches_and_shapes(gqa, batch, hidden, hq, hkv):
    rng = np.random.default_rng(7 * batch + hidden)
    rows = (hq + 2 * hkv) * 128
    x = cases.to_bf16_bits(rng.standard_normal((batch, hidden), dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((rows, hidden), dtype=np.float32)
                           / np.float32(np.sqrt(hidden)))
    got = run_qkv(gqa, x, w, hq, hkv)
    want = oracle.qkv_gemv(x, w, hq * 128, hkv * 128, accum=1)
    for part, bits, w64 in zip("qkv", got, want):
        check(bits, w64, (part, "fp64 oracle"))


def test_qkv_feeds_the_front_stage(gqa):
    """q, k and v of the projection are exactly what the QK-Norm + RoPE + append stage takes."""
    rng = np.random.default_rng(99)
    hidden, hq, hkv, max_seq_len, pos = 1024, 16, 8, 64, 17
    x = cases.to_bf16_bits(rng.standard_normal((1, hidden), dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal(((hq + 2 * hkv) * 128, hidden), dtype=np.float32) / 32)
    norm_w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(256, dtype=np.float32))
    xq = H.bf16_tensor(x)
    q = torch.zeros(1, hq, 128, dtype=torch.bfloat16, device="cuda:0")
    k = torch.zeros(1, hkv, 128, dtype=torch.bfloat16, device="cuda:0")
    v = torch.zeros(1, hkv, 128, dtype=torch.bfloat16, device="cuda:0")
    gqa.qkv_gemv(xq, H.bf16_tensor(w), q, k, v, workspace=gqa.qkv_workspace(hidden, hq, hkv, "cuda:0"))
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    k_cache = torch.zeros(1, max_seq_len, hkv * 128, dtype=torch.bfloat16, device="cuda:0")
    v_cache = torch.zeros_like(k_cache)
    q_rot = torch.zeros_like(q)
    gqa.qk_norm_rope_append(q, k, v, H.bf16_tensor(norm_w), k_cache, v_cache, layout=layout,
                            positions=[pos], q_out=q_rot)
    torch.cuda.synchronize()
    want_q, want_k, want_v = oracle.qkv_gemv(x[0], w, hq * 128, hkv * 128, accum=1)
    # The projection's own rounding may move a value by one unit; the front stage is checked
    # against the oracle on the projection's actual output.
    sin, cos = oracle.sin_cos_cache(128, max_seq_len, form=1)
    rq, rk = oracle.qk_norm_rope(H.bits_of(q)[0], H.bits_of(k)[0], norm_w, sin[pos], cos[pos], accum=1)
    assert H.bf16_ulp_distance(H.bits_of(q_rot)[0], rq).max() <= 1
    assert H.bf16_ulp_distance(H.bits_of(k_cache)[0, pos].reshape(hkv, 128), rk).max() <= 1
    assert np.array_equal(H.bits_of(v_cache)[0, pos], H.bits_of(v)[0].reshape(-1))
    check(H.bits_of(v)[0].reshape(-1), want_v, "v rows")
    check(H.bits_of(q)[0].reshape(-1), want_q, "q rows")
    check(H.bits_of(k)[0].reshape(-1), want_k, "k rows")


def test_qkv_rejects_unsupported_shapes(gqa):
    x = torch.zeros(1, 192, dtype=torch.bfloat16, device="cuda:0")
    w = torch.zeros(3 * 128, 192, dtype=torch.bfloat16, device="cuda:0")
    q = torch.zeros(1, 1, 128, dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(gqa.GqaError):
        gqa.qkv_gemv(x, w, q, q.clone(), q.clone())     # hidden is not a multiple of 128
    x2 = torch.zeros(1, 2048, dtype=torch.bfloat16, device="cuda:0")
    w2 = torch.zeros(3 * 128, 2048, dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(gqa.GqaError):
        gqa.qkv_gemv(x2, w2, q, q.clone(), q.clone())   # two column groups: workspace missing


def test_wide_groups_on_a_large_matrix_stay_resident(gqa):
    """Sixteen heads per KV head need so much shared memory per CTA that fewer CTAs fit an SM
    than the tuned number; with a large output dimension the grid would then exceed what the
    GPU holds at once, and its CTAs, which wait for one another's sums, would time out. The
    launcher sizes the grid from the occupancy the runtime reports."""
    rng = np.random.default_rng(77)
    batch, heads, kv_heads, n = 2, 32, 2, 12288
    k = heads * 128
    x = cases.to_bf16_bits(rng.standard_normal((batch, k), dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) / np.float32(np.sqrt(k)))
    r = cases.to_bf16_bits(rng.standard_normal((batch, n), dtype=np.float32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    got = run(gqa, x, w, r, kv_heads=kv_heads, status=status)
    assert int(status.item()) == 0
    check(got, oracle.gemv_add(x, w, r, accum=1), "fp64 oracle")
