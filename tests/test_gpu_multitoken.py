"""Several query tokens per sequence against the same cache (the reference prefills token by
token through its decode kernel, main/main_qwen3.cpp:58-65): token t of T attends positions
0 .. len - T + t. Checked against the FP64 oracle run once per token with that token's length,
at the BF16 tolerances of the decode tests, and bit for bit against T single-token calls where
the split pattern is the same."""
import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

ABS_TOL_BF16 = 2e-2
REL_TOL_BF16 = 1e-2


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    return pkg


def oracle_tokens(q_bits, k_bits, v_bits, lens, tokens, **kw):
    """q_bits [batch, tokens, hq, 128] -> float [batch, tokens, hq, 128], one oracle pass per token."""
    out = []
    for t in range(tokens):
        lens_t = [n - tokens + 1 + t for n in lens]
        out.append(oracle.gqa_decode(np.ascontiguousarray(q_bits[:, t]), k_bits, v_bits, lens_t, **kw))
    return np.stack(out, axis=1)


@pytest.mark.parametrize("hq,hkv,tokens,length,split_keys", [
    (32, 8, 2, 100, 0),     # the causal edge inside a stage
    (32, 8, 2, 65, 0),      # token 0 ends exactly on a stage boundary: the next stage is all hidden
    (32, 8, 4, 130, 64),    # the last split holds keys that tokens 0 and 1 may not see at all
    (32, 8, 4, 1000, 128),  # split units, edge inside the last split
    (64, 8, 2, 777, 0),     # group 8: two N tiles
    (64, 8, 2, 2048, 256),
    (16, 8, 8, 300, 0),     # group 2, eight tokens
    (32, 8, 8, 500, 128),   # 32 columns: two passes over the cache
    (64, 8, 8, 333, 0),     # 64 columns: four passes
    (64, 8, 4, 4000, 0),    # 32 columns, planner's own split
    (32, 8, 3, 3, 0),       # the sequence is nothing but the new tokens
])
def test_multi_token_reference_layout(gqa, hq, hkv, tokens, length, split_keys):
    rng = np.random.default_rng(hq * 7 + tokens * 131 + length)
    max_seq_len = (length + 63) // 64 * 64 + 64
    q = H.rand_bits(rng, (1, tokens, hq, H.D))
    k = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    k[0, length:] = H.NAN_BITS  # rows past the end must never count
    v[0, length:] = H.NAN_BITS
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    out = torch.full((1, tokens, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    ws = torch.empty(16 * 130 * hkv * (max_seq_len // 32 + 1), dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    gqa.decode(H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), out, num_kv_heads=hkv,
               layout=layout, seq_lens=[length], workspace=ws, split_keys=split_keys, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = H.f32_of(out)
    assert np.isfinite(got).all()
    want = oracle_tokens(q, k.reshape(-1), v.reshape(-1), [length], tokens, hkv=hkv,
                         stride_block=max_seq_len * hkv * H.D, stride_token=hkv * H.D,
                         stride_head=H.D, block_tokens=max_seq_len)
    for t in range(tokens):
        abs_err, rel_err = H.errors(got[:, t], want[:, t])
        assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (t, abs_err, rel_err)


def test_multi_token_equals_single_token_steps(gqa):
    """With one split per unit, token t's row is the single-token decode at length len - T + t + 1
    whenever both see the same stages: same values, same order of operations, same bits."""
    rng = np.random.default_rng(5)
    hq, hkv, tokens, length, max_seq_len = 32, 8, 2, 192, 256
    q = H.rand_bits(rng, (1, tokens, hq, H.D))
    k = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    dk, dv = H.bf16_tensor(k), H.bf16_tensor(v)
    out = torch.zeros(1, tokens, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(H.bf16_tensor(q), dk, dv, out, num_kv_heads=hkv, layout=layout, seq_lens=[length],
               split_keys=4096)
    for t in range(tokens):
        one = torch.zeros(1, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
        gqa.decode(H.bf16_tensor(np.ascontiguousarray(q[:, t])), dk, dv, one, num_kv_heads=hkv,
                   layout=layout, seq_lens=[length - tokens + 1 + t], split_keys=4096)
        torch.cuda.synchronize()
        assert torch.equal(out[:, t].view(torch.int16), one.view(torch.int16)), t


@pytest.mark.parametrize("tokens,hq", [(2, 32), (4, 32), (2, 64), (4, 64)])
def test_multi_token_paged_ragged_batch(gqa, tokens, hq):
    """Ragged batch in pool blocks, lengths on the device, front stage appending T rows per
    sequence first (so the new tokens' own rows come from the front-stage kernel)."""
    rng = np.random.default_rng(23 + tokens + hq)
    batch, hkv, block_tokens = 5, 8, 256
    lens = [tokens, 255 + tokens, 256, 1000, 1537]
    blocks_per_seq = 8
    num_blocks = batch * blocks_per_seq
    table = rng.permutation(num_blocks).reshape(batch, blocks_per_seq).astype(np.int32)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    k_pool = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    v_pool = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    q_raw = H.rand_bits(rng, (batch, tokens, hq, H.D))
    k_new = H.rand_bits(rng, (batch, tokens, hkv, H.D))
    v_new = H.rand_bits(rng, (batch, tokens, hkv, H.D))
    import cases
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * H.D, dtype=np.float32))
    positions = [n - tokens for n in lens]
    dq, dk, dv = H.bf16_tensor(q_raw), H.bf16_tensor(k_pool), H.bf16_tensor(v_pool)
    dtab = torch.from_numpy(table).to("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    gqa.qk_norm_rope_append(dq, H.bf16_tensor(k_new), H.bf16_tensor(v_new), H.bf16_tensor(w), dk, dv,
                            layout=layout, positions=positions,
                            positions_dev=torch.tensor(positions, dtype=torch.int32, device="cuda:0"),
                            block_table=dtab, status=status)
    out = torch.full((batch, tokens, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    ws = gqa.binding.workspace_for(batch, hq * tokens, hkv, "cuda:0")
    gqa.decode(dq, dk, dv, out, num_kv_heads=hkv, layout=layout, seq_lens=lens,
               seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
               block_table=dtab, workspace=ws, status=status, early_prefetch=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # Oracle: the front stage per token, then attention per token on the updated cache.
    sin, cos = oracle.sin_cos_cache(H.D, blocks_per_seq * block_tokens, form=1)
    q_rot = np.zeros_like(q_raw)
    for b in range(batch):
        for t in range(tokens):
            pos = positions[b] + t
            want_q, want_k = oracle.qk_norm_rope(q_raw[b, t], k_new[b, t], w, sin[pos], cos[pos], accum=1)
            q_rot[b, t] = want_q
            blk, tok = table[b, pos // block_tokens], pos % block_tokens
            k_pool[blk, :, tok] = want_k
            v_pool[blk, :, tok] = v_new[b, t]
    assert np.array_equal(H.bits_of(dq), q_rot) or \
        (H.bf16_ulp_distance(H.bits_of(dq), q_rot) <= 1).all()
    want = oracle_tokens(H.bits_of(dq), k_pool.reshape(-1), v_pool.reshape(-1), lens, tokens, hkv=hkv,
                         stride_block=layout.stride_block, stride_token=layout.stride_token,
                         stride_head=layout.stride_head, block_tokens=block_tokens, block_table=table)
    got = H.f32_of(out)
    assert np.isfinite(got).all()
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)


def test_multi_token_validation(gqa):
    layout = gqa.layout_reference(1, 256, 8)
    with pytest.raises(gqa.GqaError) as e:  # a sequence shorter than its own new tokens
        gqa.decode_plan(dtype=2, batch=1, num_q_heads=32, num_kv_heads=8, layout=layout,
                        seq_lens=[3], q_tokens=4)
    assert e.value.status == -5
    with pytest.raises(gqa.GqaError) as e:  # FP32 is a single-token parity path
        gqa.decode_plan(dtype=1, batch=1, num_q_heads=16, num_kv_heads=8, layout=layout,
                        seq_lens=[64], q_tokens=2)
    assert e.value.status == -8
