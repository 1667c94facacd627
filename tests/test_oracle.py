"""The CPU oracle against an independent numpy restatement, against itself (FP32 vs FP64, the
reference-signature entry point) and against the golden outputs of the reference's own CUDA
kernels (tests/golden/ref_cuda_bf16.npz)."""
import numpy as np
import pytest
from pathlib import Path

import helpers as H

import cases
from oracle import oracle

D = 128


def numpy_attention(q, k_rows, v_rows, kv_mul):
    """q [hq, d]; k_rows, v_rows [len, hkv, d]; all float64."""
    hq, d = q.shape
    out = np.zeros((hq, d))
    for h in range(hq):
        kh, vh = k_rows[:, h // kv_mul], v_rows[:, h // kv_mul]
        s = kh @ q[h] / np.sqrt(d)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ vh
    return out


@pytest.mark.parametrize("hq,hkv,length", [(4, 2, 1), (8, 2, 33), (16, 8, 200)])
def test_oracle_matches_numpy_fp32_cache(hq, hkv, length):
    rng = np.random.default_rng(length)
    layers, layer_id, max_seq_len = 3, 2, length + 7
    q = rng.standard_normal((hq, D), dtype=np.float32)
    k = rng.standard_normal((layers, max_seq_len, hkv * D), dtype=np.float32)
    v = rng.standard_normal((layers, max_seq_len, hkv * D), dtype=np.float32)
    want = numpy_attention(q.astype(np.float64),
                           k[layer_id, :length].reshape(length, hkv, D).astype(np.float64),
                           v[layer_id, :length].reshape(length, hkv, D).astype(np.float64),
                           hq // hkv)
    for accum, tol in ((1, 1e-6), (0, 2e-5)):
        got = oracle.mha_reference_layout(q, k.reshape(-1), v.reshape(-1), layer_id=layer_id,
                                          pos=length - 1, hkv=hkv, max_seq_len=max_seq_len,
                                          accum=accum)
        assert np.max(np.abs(got - want)) <= tol * max(1.0, np.abs(want).max())
    # The reference's own CPU argument list gives the FP32-order result and leaves the softmax
    # probabilities in its score scratch.
    out, score = oracle.mha_kernel_cpu(q.reshape(-1), k.reshape(-1), v.reshape(-1),
                                       layer_id=layer_id, pos=length - 1, kv_dim=hkv * D,
                                       kv_mul=hq // hkv, head_num=hq, head_dim=D,
                                       max_seq_len=max_seq_len)
    fp32 = oracle.mha_reference_layout(q, k.reshape(-1), v.reshape(-1), layer_id=layer_id,
                                       pos=length - 1, hkv=hkv, max_seq_len=max_seq_len, accum=0)
    assert np.array_equal(out.reshape(hq, D), fp32)
    assert np.allclose(score[:, :length].sum(axis=1), 1.0, atol=1e-5)


def test_oracle_threads_and_paging_do_not_change_values():
    rng = np.random.default_rng(5)
    batch, hq, hkv, block_tokens = 3, 8, 2, 32
    lens = [1, 40, 96]
    blocks_per_seq, num_blocks = 3, 10
    table = rng.permutation(num_blocks)[: batch * blocks_per_seq].reshape(batch, blocks_per_seq)
    table = table.astype(np.int32)
    q = cases.to_bf16_bits(rng.standard_normal((batch, hq, D), dtype=np.float32))
    pool = lambda: cases.to_bf16_bits(
        rng.standard_normal(num_blocks * hkv * block_tokens * D, dtype=np.float32))
    k_pool, v_pool = pool(), pool()
    kw = dict(hkv=hkv, stride_block=hkv * block_tokens * D, stride_token=D,
              stride_head=block_tokens * D, block_tokens=block_tokens, block_table=table)
    one = oracle.gqa_decode(q, k_pool, v_pool, lens, threads=1, **kw)
    many = oracle.gqa_decode(q, k_pool, v_pool, lens, threads=0, **kw)
    assert np.array_equal(one, many)
    kf, vf = cases.bf16_bits_to_f32(k_pool), cases.bf16_bits_to_f32(v_pool)
    for b, length in enumerate(lens):
        rows = lambda flat: np.stack([
            np.stack([flat[((table[b, t // block_tokens] * hkv + hk) * block_tokens
                            + t % block_tokens) * D:][:D] for hk in range(hkv)])
            for t in range(length)]).astype(np.float64)
        want = numpy_attention(cases.bf16_bits_to_f32(q[b]).astype(np.float64), rows(kf), rows(vf),
                               hq // hkv)
        assert np.max(np.abs(one[b] - want)) <= 1e-6


def test_bf16_rounding_helpers_agree():
    rng = np.random.default_rng(9)
    x = np.concatenate([rng.standard_normal(4096, dtype=np.float32) * 10.0,
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38],
                                 dtype=np.float32)])
    assert np.array_equal(oracle.f32_to_bf16(x), cases.to_bf16_bits(x))
    bits = oracle.f32_to_bf16(x)
    assert np.array_equal(oracle.bf16_to_f32(bits), cases.bf16_bits_to_f32(bits))
    # Ties go to the even mantissa.
    assert oracle.f32_to_bf16(np.array([1.00390625], dtype=np.float32))[0] == 0x3F80
    assert oracle.f32_to_bf16(np.array([1.01171875], dtype=np.float32))[0] == 0x3F82


def test_qk_norm_rope_matches_numpy():
    rng = np.random.default_rng(3)
    hq, hkv, pos = 8, 2, 77
    q = cases.to_bf16_bits(rng.standard_normal((hq, D), dtype=np.float32))
    k = cases.to_bf16_bits(rng.standard_normal((hkv, D), dtype=np.float32))
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * D, dtype=np.float32))
    sin, cos = oracle.sin_cos_cache(D, 128, form=1)
    got_q, got_k = oracle.qk_norm_rope(q, k, w, sin[pos], cos[pos], accum=0)

    def one(x_bits, w_bits):
        x = cases.bf16_bits_to_f32(x_bits).astype(np.float64)
        wt = cases.bf16_bits_to_f32(w_bits).astype(np.float64)
        y = x * wt / np.sqrt((x * x).mean(axis=1, keepdims=True) + 1e-6)
        a, b = y[:, :64], y[:, 64:]
        s, c = sin[pos].astype(np.float64), cos[pos].astype(np.float64)
        return np.concatenate([a * c - b * s, a * s + b * c], axis=1)

    for got, want in ((got_q, one(q, w[:D])), (got_k, one(k, w[D:]))):
        assert np.max(np.abs(cases.bf16_bits_to_f32(got) - want)) <= 2e-2
        # One BF16 rounding of an FP32 value: at most one unit in the last place away.
        want_bits = cases.to_bf16_bits(want.astype(np.float32))
        assert np.max(np.abs(got.astype(np.int32) - want_bits.astype(np.int32))) <= 1


def test_sin_cos_forms():
    n = 4096
    s0, c0 = oracle.sin_cos_cache(D, n, form=0)
    s1, c1 = oracle.sin_cos_cache(D, n, form=1)
    inv = 1.0 / (1e6 ** (np.arange(0, D, 2, dtype=np.float64) / D))
    theta = np.arange(n, dtype=np.float64)[:, None] * inv[None, :]
    tol = 2e-6 + 4 * np.spacing(np.maximum(theta, 1.0).astype(np.float32))
    for s, c in ((s0, c0), (s1, c1)):
        assert np.all(np.abs(s - np.sin(theta)) <= tol)
        assert np.all(np.abs(c - np.cos(theta)) <= tol)
    assert np.array_equal(s0[0], np.zeros(D // 2, dtype=np.float32))
    assert np.array_equal(c1[0], np.ones(D // 2, dtype=np.float32))


# ---- pinned against the reference's own CUDA kernels --------------------------------------

@pytest.mark.parametrize("index", range(len(cases.ATTN_CASES)))
def test_oracle_against_reference_cuda_attention(index, golden):
    name, hq, hkv, length, layers, layer_id, max_seq_len = cases.ATTN_CASES[index]
    q, k, v = cases.attention_inputs(index)
    assert cases.checksum(q, k, v) == int(golden[f"attn/{name}/crc"][0]), "input generator drifted"
    ref_bits = golden[f"attn/{name}/out"]
    ref = cases.bf16_bits_to_f32(ref_bits)
    for accum in (0, 1):
        got = oracle.mha_reference_layout(q, k.reshape(-1), v.reshape(-1), layer_id=layer_id,
                                          pos=length - 1, hkv=hkv, max_seq_len=max_seq_len,
                                          accum=accum)
        # The reference rounds its FP32 result once to BF16 and uses fast exponentials: the
        # oracle must sit within the reference's own BF16 tolerance and, tighter, within two
        # BF16 steps of its rounded output.
        assert np.max(np.abs(got - ref)) <= 2e-2
        got_bits = cases.to_bf16_bits(got)
        scale = np.abs(ref).max()
        assert np.max(np.abs(got - ref)) <= 2 * 2.0 ** -8 * scale, name
        close = np.abs(got_bits.astype(np.int32) - ref_bits.astype(np.int32)) <= 1
        assert close.mean() >= 0.98, (name, close.mean())


@pytest.mark.parametrize("index", range(len(cases.FRONT_CASES)))
def test_oracle_against_reference_cuda_front_stage(index, golden):
    name, hq, hkv, pos = cases.FRONT_CASES[index]
    q, k, w = cases.front_inputs(index)
    assert cases.checksum(q, k, w) == int(golden[f"front/{name}/crc"][0]), "input generator drifted"
    got_q, got_k = oracle.qk_norm_rope(q, k, w, golden[f"front/{name}/sin"],
                                       golden[f"front/{name}/cos"], accum=0)
    for got, ref in ((got_q, golden[f"front/{name}/q"]), (got_k, golden[f"front/{name}/k"])):
        step = np.abs(got.astype(np.int32) - ref.astype(np.int32))
        assert step.max() <= 1, name
        assert (step == 0).mean() >= 0.99, (name, (step == 0).mean())


def test_oracle_against_reference_cuda_table(golden):
    s1, c1 = oracle.sin_cos_cache(D, cases.FRONT_TABLE_LEN, form=1)
    rows = np.array(cases.TABLE_ROWS)
    inv = 1.0 / (1e6 ** (np.arange(0, D, 2, dtype=np.float64) / D))
    theta = rows[:, None].astype(np.float64) * inv[None, :]
    tol = 2e-6 + 4 * np.spacing(np.maximum(theta, 1.0).astype(np.float32))
    assert np.all(np.abs(s1[rows] - golden["table/sin_rows"]) <= tol)
    assert np.all(np.abs(c1[rows] - golden["table/cos_rows"]) <= tol)


# ---- projections on either side of attention ------------------------------------------------
@pytest.fixture(scope="module")
def golden_proj():
    return np.load(Path(__file__).resolve().parent / "golden" / "ref_cuda_proj.npz")


@pytest.mark.parametrize("index", range(len(cases.OPROJ_CASES)))
def test_oproj_oracle_is_bit_equal_to_reference_kernel(golden_proj, index):
    """The FP32 restatement follows the reference kernel's summation order exactly, so it
    reproduces the output of kernel::fused_gemv_add_kernel_cu bit for bit."""
    name, n, k = cases.OPROJ_CASES[index]
    x, w, r = cases.oproj_inputs(index)
    assert int(golden_proj[f"oproj/{name}/crc"][0]) == cases.checksum(x, w, r)
    want = golden_proj[f"oproj/{name}/out"]
    assert np.array_equal(oracle.gemv_add(x, w, r, accum=0), want)
    # FP64 accumulation moves a result only across a BF16 rounding boundary.
    got64 = oracle.gemv_add(x, w, r, accum=1)
    assert H.bf16_ulp_distance(got64, want).max() <= 1
    assert (got64 != want).mean() <= 0.01


@pytest.mark.parametrize("index", range(len(cases.QKV_CASES)))
def test_qkv_oracle_is_bit_equal_to_reference_kernel(golden_proj, index):
    name, hidden, hq, hkv = cases.QKV_CASES[index]
    x, w = cases.qkv_inputs(index)
    assert int(golden_proj[f"qkv/{name}/crc"][0]) == cases.checksum(x, w)
    got = oracle.qkv_gemv(x, w, hq * cases.HEAD_DIM, hkv * cases.HEAD_DIM, accum=0)
    for part, bits in zip("qkv", got):
        assert np.array_equal(bits, golden_proj[f"qkv/{name}/{part}"]), part
    got64 = oracle.qkv_gemv(x, w, hq * cases.HEAD_DIM, hkv * cases.HEAD_DIM, accum=1)
    for part, bits in zip("qkv", got64):
        assert H.bf16_ulp_distance(bits, golden_proj[f"qkv/{name}/{part}"]).max() <= 1


def test_gemv_add_batched_pitch_and_linearity():
    """Batch rows are independent, a weight pitch larger than k reads only k columns, and the
    unrounded FP64 result is linear in x."""
    rng = np.random.default_rng(77)
    n, k, ld = 32, 256, 384
    x = cases.to_bf16_bits(rng.standard_normal((3, k), dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((n, ld), dtype=np.float32))
    r = cases.to_bf16_bits(rng.standard_normal((3, n), dtype=np.float32))
    whole = oracle.gemv_add(x, w, r, accum=0, k=k)
    for b in range(3):
        one = oracle.gemv_add(x[b], np.ascontiguousarray(w[:, :k]), r[b], accum=0)
        assert np.array_equal(whole[b], one)
    zero_r = np.zeros_like(r)
    full = oracle.gemv_add(x, w, zero_r, accum=2, k=k)
    xf = cases.bf16_bits_to_f32(x).astype(np.float64)
    wf = cases.bf16_bits_to_f32(w[:, :k]).astype(np.float64)
    assert np.allclose(full, xf @ wf.T, rtol=1e-12, atol=1e-12)
    with pytest.raises(ValueError):
        oracle.gemv_add(x[:, :12], w, r, accum=0)  # k % 8 != 0
