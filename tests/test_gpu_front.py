"""GPU parity of the front stage (QK-Norm + RoPE + KV append), the sin/cos table and the
host-buffer decode step, through the C ABI, against the oracle and the reference's kernels."""
import numpy as np
import pytest
import torch

import cases
import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    assert torch.cuda.is_available(), "these tests need the GPU"
    return pkg


def test_sin_cos_table(gqa, request):
    n = cases.FRONT_TABLE_LEN
    sin = torch.empty(n, 64, dtype=torch.float32, device="cuda:0")
    cos = torch.empty_like(sin)
    gqa.sin_cos_cache(sin, cos, 128)
    torch.cuda.synchronize()
    osin, ocos = oracle.sin_cos_cache(128, n, form=1)
    # Host libm and the device agree to a few ulp of the angle: |d sin| <= |d theta|.
    theta = np.arange(n, dtype=np.float64)[:, None] * 1.0
    tol = 2e-6 + 4 * np.spacing(np.maximum(theta, 1.0).astype(np.float32)).astype(np.float64)
    assert np.all(np.abs(sin.cpu().numpy() - osin) <= tol)
    assert np.all(np.abs(cos.cpu().numpy() - ocos) <= tol)
    try:
        golden = request.getfixturevalue("golden")
    except pytest.skip.Exception:
        return
    rows = torch.tensor(cases.TABLE_ROWS, device="cuda:0")
    # Same formula, same device math library: the reference's table is reproduced exactly.
    assert np.array_equal(sin[rows].cpu().numpy(), golden["table/sin_rows"])
    assert np.array_equal(cos[rows].cpu().numpy(), golden["table/cos_rows"])
    assert sin.double().sum().item() == golden["table/sin_sum"][0]
    assert cos.double().sum().item() == golden["table/cos_sum"][0]


@pytest.mark.parametrize("index", range(len(cases.FRONT_CASES)))
@pytest.mark.parametrize("use_table", [True, False])
def test_front_stage_reference_layout(gqa, index, use_table, request):
    name, hq, hkv, pos = cases.FRONT_CASES[index]
    q, k, w = cases.front_inputs(index)
    rng = np.random.default_rng(31 + index)
    v = H.rand_bits(rng, (hkv, H.D))
    max_seq_len = cases.FRONT_TABLE_LEN
    layers, layer_id = 2, 1
    layout = gqa.layout_reference(layers, max_seq_len, hkv)
    sin = torch.empty(max_seq_len, 64, dtype=torch.float32, device="cuda:0")
    cos = torch.empty_like(sin)
    gqa.sin_cos_cache(sin, cos, 128)
    k_cache = torch.zeros(layers, max_seq_len, hkv * H.D, dtype=torch.bfloat16, device="cuda:0")
    v_cache = torch.zeros_like(k_cache)
    dq = H.bf16_tensor(q).reshape(1, hq, H.D).clone()
    dk = H.bf16_tensor(k).reshape(1, hkv, H.D)
    dv = H.bf16_tensor(v).reshape(1, hkv, H.D)
    gqa.qk_norm_rope_append(dq, dk, dv, H.bf16_tensor(w), k_cache, v_cache, layout=layout,
                            positions=[pos], fixed_block=layer_id,
                            sin_cache=sin if use_table else None,
                            cos_cache=cos if use_table else None)
    torch.cuda.synchronize()
    got_q = H.bits_of(dq)[0]
    got_k = H.bits_of(k_cache[layer_id, pos]).reshape(hkv, H.D)
    got_v = H.bits_of(v_cache[layer_id, pos]).reshape(hkv, H.D)
    assert np.array_equal(got_v, v)
    # Nothing else in the caches was touched.
    assert int((k_cache != 0).sum().item()) <= hkv * H.D
    assert torch.count_nonzero(k_cache[0]).item() == 0
    srow, crow = sin[pos].cpu().numpy(), cos[pos].cpu().numpy()
    want_q, want_k = oracle.qk_norm_rope(q, k, w, srow, crow, accum=1)
    assert H.bf16_ulp_distance(got_q, want_q).max() <= 1
    assert H.bf16_ulp_distance(got_k, want_k).max() <= 1
    try:
        golden = request.getfixturevalue("golden")
    except pytest.skip.Exception:
        return
    # The kernel mirrors the reference's arithmetic step by step.
    assert np.array_equal(srow, golden[f"front/{name}/sin"])
    assert H.bf16_ulp_distance(got_q, golden[f"front/{name}/q"]).max() <= 1
    assert H.bf16_ulp_distance(got_k, golden[f"front/{name}/k"]).max() <= 1
    exact = np.mean(got_q == golden[f"front/{name}/q"])
    assert exact >= 0.999, exact


def test_front_stage_paged_batch(gqa):
    rng = np.random.default_rng(37)
    batch, hq, hkv, block_tokens = 5, 32, 8, 256
    positions = [0, 255, 256, 700, 1023]
    blocks_per_seq, num_blocks = 4, 24
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = rng.permutation(num_blocks)[: batch * blocks_per_seq].reshape(batch, blocks_per_seq)
    q = H.rand_bits(rng, (batch, hq, H.D))
    k = H.rand_bits(rng, (batch, hkv, H.D))
    v = H.rand_bits(rng, (batch, hkv, H.D))
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(256, dtype=np.float32))
    pool_elems = num_blocks * hkv * block_tokens * H.D
    k_pool = torch.zeros(pool_elems, dtype=torch.bfloat16, device="cuda:0")
    v_pool = torch.zeros_like(k_pool)
    dq = H.bf16_tensor(q)
    q_out = torch.zeros_like(dq)
    gqa.qk_norm_rope_append(dq, H.bf16_tensor(k), H.bf16_tensor(v), H.bf16_tensor(w), k_pool,
                            v_pool, layout=layout, positions=positions,
                            positions_dev=torch.tensor(positions, dtype=torch.int32, device="cuda:0"),
                            q_out=q_out,
                            block_table=torch.from_numpy(table.astype(np.int32)).to("cuda:0"))
    torch.cuda.synchronize()
    osin, ocos = oracle.sin_cos_cache(128, 1024, form=1)
    kp, vp = H.bits_of(k_pool), H.bits_of(v_pool)
    for b, pos in enumerate(positions):
        want_q, want_k = oracle.qk_norm_rope(q[b], k[b], w, osin[pos], ocos[pos], accum=1)
        assert H.bf16_ulp_distance(H.bits_of(q_out)[b], want_q).max() <= 1
        blk, tok = table[b, pos // block_tokens], pos % block_tokens
        for hk in range(hkv):
            off = ((blk * hkv + hk) * block_tokens + tok) * H.D
            assert H.bf16_ulp_distance(kp[off:off + H.D], want_k[hk]).max() <= 1
            assert np.array_equal(vp[off:off + H.D], v[b, hk])
    assert np.array_equal(H.bits_of(dq), q)  # q_out given: the input stays as it was


def test_session_step_from_host_buffers(gqa):
    """H2D of the new rows, front stage, attention, D2H: one call with host buffers."""
    rng = np.random.default_rng(41)
    hq, hkv, max_seq_len, pos = 32, 8, 1024, 700
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    k_hist = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v_hist = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    q, k_new, v_new = (H.rand_bits(rng, (1, n, H.D)) for n in (hq, hkv, hkv))
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(256, dtype=np.float32))
    dk, dv = H.bf16_tensor(k_hist), H.bf16_tensor(v_hist)
    session = gqa.Session(1, hq, hkv, max_seq_len)
    as_host = lambda bits: torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).pin_memory()
    out_host = torch.zeros(1, hq, H.D, dtype=torch.bfloat16).pin_memory()
    session.step(as_host(q), as_host(k_new), as_host(v_new), H.bf16_tensor(w), dk, dv, layout,
                 [pos], out_host)
    session.close()
    osin, ocos = oracle.sin_cos_cache(128, max_seq_len, form=1)
    want_q, want_k = oracle.qk_norm_rope(q[0], k_new[0], w, osin[pos], ocos[pos], accum=1)
    k_hist[0, pos] = want_k.reshape(-1)
    v_hist[0, pos] = v_new.reshape(-1)
    want = H.oracle_reference_layout(want_q, k_hist, v_hist, layer_id=0, length=pos + 1, hkv=hkv,
                                     max_seq_len=max_seq_len)
    abs_err, rel_err = H.errors(out_host[0].float().numpy(), want)
    assert abs_err <= 2e-2 and rel_err <= 2e-2, (abs_err, rel_err)
    # Pageable host buffers go through the session's own pinned blocks instead of being used
    # where they lie: same kernels, same bits (the cache row of `pos` is simply written again).
    pageable = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
    out_paged = torch.zeros(1, hq, H.D, dtype=torch.bfloat16)
    session = gqa.Session(1, hq, hkv, max_seq_len)
    for _ in range(2):
        session.step(pageable(q), pageable(k_new), pageable(v_new), H.bf16_tensor(w), dk, dv, layout,
                     [pos], out_paged)
    timing = session.last_timing()
    session.close()
    assert torch.equal(out_paged.view(torch.int16), out_host.view(torch.int16))
    assert all(v >= 0 for v in timing.values()) and timing["wait_ns"] > 0
