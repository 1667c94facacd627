"""The attention kernel with the front stage inside (gqa_decode_fused): QK-Norm + RoPE of the
raw query, the new key rotated, key and value rows appended to the cache, attention — one
launch. It runs the same operations as gqa_qk_norm_rope_append followed by gqa_decode, so
outputs, rotated queries and cache rows must agree with that pair bit for bit; the pair itself
is checked against the oracle and the reference kernels' golden outputs elsewhere."""
import numpy as np
import pytest
import torch

import cases
import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    return pkg


def norm_weights(rng):
    return cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * H.D, dtype=np.float32))


@pytest.mark.parametrize("hq,hkv,length,split_keys,use_table", [
    (32, 8, 1, 0, True),        # the sequence is the new token alone
    (32, 8, 64, 0, True),       # new row is the last row of a stage
    (32, 8, 65, 0, False),      # new row opens a stage (angles computed in the kernel)
    (32, 8, 1500, 0, True),     # planner's split
    (32, 8, 1500, 128, True),   # explicit split: the appending CTA is the unit's last item
    (64, 8, 4000, 512, True),   # group 8
    (16, 8, 300, 0, False),     # group 2
])
def test_fused_equals_front_then_decode_reference_layout(gqa, hq, hkv, length, split_keys, use_table):
    rng = np.random.default_rng(hq + length + split_keys)
    max_seq_len = (length + 127) // 128 * 128
    pos = length - 1
    layout = gqa.layout_reference(2, max_seq_len, hkv)
    k0 = H.rand_bits(rng, (2, max_seq_len, hkv * H.D))
    v0 = H.rand_bits(rng, (2, max_seq_len, hkv * H.D))
    k0[1, pos:] = H.NAN_BITS  # the new row and everything after it: must come from k_new only
    v0[1, pos:] = H.NAN_BITS
    q_raw = H.rand_bits(rng, (1, hq, H.D))
    k_new, v_new = H.rand_bits(rng, (1, hkv, H.D)), H.rand_bits(rng, (1, hkv, H.D))
    w = H.bf16_tensor(norm_weights(rng))
    sin = cos = None
    if use_table:
        sin = torch.empty(max_seq_len, H.D // 2, dtype=torch.float32, device="cuda:0")
        cos = torch.empty_like(sin)
        gqa.sin_cos_cache(sin, cos, H.D)
    ws = torch.empty(hq * 130 * (max_seq_len // 32 + 1), dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")

    # The pair of launches.
    k_a, v_a = H.bf16_tensor(k0), H.bf16_tensor(v0)
    q_a = H.bf16_tensor(q_raw)
    out_a = torch.zeros(1, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    gqa.qk_norm_rope_append(q_a, H.bf16_tensor(k_new), H.bf16_tensor(v_new), w, k_a, v_a,
                            layout=layout, positions=[pos], fixed_block=1, sin_cache=sin,
                            cos_cache=cos)
    gqa.decode(q_a, k_a, v_a, out_a, num_kv_heads=hkv, layout=layout, seq_lens=[length],
               fixed_block=1, workspace=ws, split_keys=split_keys, status=status)
    # One launch.
    k_b, v_b = H.bf16_tensor(k0), H.bf16_tensor(v0)
    q_rot = torch.zeros(1, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    out_b = torch.full((1, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    front = gqa.FusedFront(H.bf16_tensor(k_new), H.bf16_tensor(v_new), w, q_out=q_rot,
                           sin_cache=sin, cos_cache=cos)
    for early in (False, True):
        gqa.decode(H.bf16_tensor(q_raw), k_b, v_b, out_b, num_kv_heads=hkv, layout=layout,
                   seq_lens=[length], fixed_block=1, workspace=ws, split_keys=split_keys,
                   status=status, front=front, early_prefetch=early)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(out_b.view(torch.int16), out_a.view(torch.int16))
        assert torch.equal(q_rot.view(torch.int16), q_a.view(torch.int16))
        # The appended rows, and nothing but them, changed in the cache.
        assert torch.equal(k_b.view(torch.int16)[1, :length], k_a.view(torch.int16)[1, :length])
        assert torch.equal(v_b.view(torch.int16)[1, :length], v_a.view(torch.int16)[1, :length])
        assert torch.equal(k_b.view(torch.int16)[0], H.bf16_tensor(k0).view(torch.int16)[0])
        assert torch.equal(k_b.view(torch.int16)[1, length:], H.bf16_tensor(k0).view(torch.int16)[1, length:])


@pytest.mark.parametrize("tokens,hq", [(1, 32), (2, 32), (4, 32), (4, 64), (8, 64)])
def test_fused_paged_ragged_batch(gqa, tokens, hq):
    """(4, 64) and (8, 64) have 32 and 64 (token, head) columns per unit: two and four passes
    over the cache, each appending its own tokens' rows before the next one reads them."""
    rng = np.random.default_rng(91 + tokens + hq)
    batch, hkv, block_tokens = 6, 8, 256
    lens = [tokens, 256, 257 + tokens, 1024, 1999, 700]
    blocks_per_seq = 8
    num_blocks = batch * blocks_per_seq
    table = rng.permutation(num_blocks).reshape(batch, blocks_per_seq).astype(np.int32)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    k0 = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    v0 = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    shape_q = (batch, hq, H.D) if tokens == 1 else (batch, tokens, hq, H.D)
    shape_kv = (batch, hkv, H.D) if tokens == 1 else (batch, tokens, hkv, H.D)
    q_raw, k_new, v_new = H.rand_bits(rng, shape_q), H.rand_bits(rng, shape_kv), H.rand_bits(rng, shape_kv)
    w = H.bf16_tensor(norm_weights(rng))
    sin = torch.empty(blocks_per_seq * block_tokens, H.D // 2, dtype=torch.float32, device="cuda:0")
    cos = torch.empty_like(sin)
    gqa.sin_cos_cache(sin, cos, H.D)
    dtab = torch.from_numpy(table).to("cuda:0")
    dlens = torch.tensor(lens, dtype=torch.int32, device="cuda:0")
    positions = [n - tokens for n in lens]
    ws = gqa.binding.workspace_for(batch, hq * tokens, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")

    k_a, v_a, q_a = H.bf16_tensor(k0), H.bf16_tensor(v0), H.bf16_tensor(q_raw)
    out_a = torch.zeros(shape_q, dtype=torch.bfloat16, device="cuda:0")
    gqa.qk_norm_rope_append(q_a, H.bf16_tensor(k_new), H.bf16_tensor(v_new), w, k_a, v_a,
                            layout=layout, positions=positions,
                            positions_dev=torch.tensor(positions, dtype=torch.int32, device="cuda:0"),
                            block_table=dtab, sin_cache=sin, cos_cache=cos, status=status)
    kw = dict(num_kv_heads=hkv, layout=layout, seq_lens=lens, seq_lens_dev=dlens, block_table=dtab,
              workspace=ws, status=status)
    gqa.decode(q_a, k_a, v_a, out_a, **kw)

    k_b, v_b = H.bf16_tensor(k0), H.bf16_tensor(v0)
    out_b = torch.full(shape_q, float("nan"), dtype=torch.bfloat16, device="cuda:0")
    front = gqa.FusedFront(H.bf16_tensor(k_new), H.bf16_tensor(v_new), w, sin_cache=sin, cos_cache=cos)
    gqa.decode(H.bf16_tensor(q_raw), k_b, v_b, out_b, front=front, early_prefetch=True, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(out_b.view(torch.int16), out_a.view(torch.int16))
    assert torch.equal(k_b.view(torch.int16), k_a.view(torch.int16))
    assert torch.equal(v_b.view(torch.int16), v_a.view(torch.int16))


def test_fused_refuses_in_place_rotation(gqa):
    hq, hkv = 32, 8
    layout = gqa.layout_reference(1, 128, hkv)
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device="cuda:0")
    q = z(1, hq, H.D)
    front = gqa.FusedFront(z(1, hkv, H.D), z(1, hkv, H.D), z(2 * H.D), q_out=q)
    with pytest.raises(gqa.GqaError) as e:
        gqa.decode(q, z(1, 128, hkv * H.D), z(1, 128, hkv * H.D), z(1, hq, H.D), num_kv_heads=hkv,
                   layout=layout, seq_lens=[5], front=front)
    assert e.value.status == -8
