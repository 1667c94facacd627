"""Splits merged inside thread-block clusters (one cluster per (sequence, kv head), one CTA per
split, partial results exchanged through distributed shared memory) against the two-launch
path (partial records in the workspace, then the combine kernel). Both perform the same
operations in the same order, so they must agree bit for bit; the two-launch path is selected
here by capping the grid below what the clusters need (max_ctas), with the split given
explicitly so that the cap does not change it."""
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
    return pkg


@pytest.mark.parametrize("hq,hkv,tokens,length,split_keys,fused", [
    (32, 8, 1, 1024, 128, False),  # the 1K decode step as the planner cuts it: 8 units x 8 splits
    (32, 8, 1, 1024, 128, True),
    (32, 8, 1, 300, 64, False),    # 5 splits, the last one short
    (64, 8, 1, 1000, 128, False),  # group 8
    (64, 8, 2, 1000, 256, False),  # two N tiles
    (32, 8, 4, 515, 128, True),    # multi-token with the front stage inside; ragged tail
    (16, 8, 1, 96, 64, False),     # two splits
    (32, 8, 2, 130, 64, False),    # a split that token 0 cannot see at all
])
def test_cluster_merge_equals_combine_launch(gqa, hq, hkv, tokens, length, split_keys, fused):
    rng = np.random.default_rng(hq + tokens * 17 + length)
    max_seq_len = (length + 127) // 128 * 128
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    plan = gqa.decode_plan(dtype=2, batch=1, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=[length], split_keys=split_keys, q_tokens=tokens)
    assert plan["cluster_size"] >= 2, plan
    ctas = hkv * plan["cluster_size"]
    assert gqa.decode_plan(dtype=2, batch=1, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=[length], split_keys=split_keys, q_tokens=tokens,
                           max_ctas=ctas - 1)["cluster_size"] == 0
    shape_q = (1, hq, H.D) if tokens == 1 else (1, tokens, hq, H.D)
    shape_kv = (1, hkv, H.D) if tokens == 1 else (1, tokens, hkv, H.D)
    q_bits = H.rand_bits(rng, shape_q)
    k_bits = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v_bits = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    k_bits[0, length:] = H.NAN_BITS
    v_bits[0, length:] = H.NAN_BITS
    k_new, v_new = H.rand_bits(rng, shape_kv), H.rand_bits(rng, shape_kv)
    w = H.bf16_tensor(cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * H.D, dtype=np.float32)))
    ws = torch.empty(16 * 130 * hkv * (max_seq_len // 32 + 1), dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    outs = []
    for max_ctas, workspace in ((0, None), (ctas - 1, ws)):  # clusters need no workspace
        k, v = H.bf16_tensor(k_bits), H.bf16_tensor(v_bits)
        out = torch.full(shape_q, float("nan"), dtype=torch.bfloat16, device="cuda:0")
        front = gqa.FusedFront(H.bf16_tensor(k_new), H.bf16_tensor(v_new), w) if fused else None
        for _ in range(2):
            gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout,
                       seq_lens=[length], workspace=workspace, split_keys=split_keys,
                       max_ctas=max_ctas, status=status, front=front)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        outs.append((out, k, v))
    assert torch.isfinite(outs[0][0].float()).all()
    assert torch.equal(outs[0][0].view(torch.int16), outs[1][0].view(torch.int16))
    if fused:
        assert torch.equal(outs[0][1].view(torch.int16)[0, :length], outs[1][1].view(torch.int16)[0, :length])
    else:
        want = []
        for t in range(tokens):
            qt = q_bits if tokens == 1 else np.ascontiguousarray(q_bits[:, t])
            want.append(oracle.gqa_decode(qt, k_bits.reshape(-1), v_bits.reshape(-1),
                                          [length - tokens + 1 + t], hkv=hkv,
                                          stride_block=max_seq_len * hkv * H.D,
                                          stride_token=hkv * H.D, stride_head=H.D,
                                          block_tokens=max_seq_len))
        want = want[0] if tokens == 1 else np.stack(want, axis=1)
        abs_err, rel_err = H.errors(H.f32_of(outs[0][0]), want)
        assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)


def test_cluster_merge_paged_ragged_batch_with_device_lengths(gqa):
    """Lengths on the device: the cluster is sized for a full sequence, CTAs past a unit's last
    split idle through the barriers."""
    rng = np.random.default_rng(8)
    batch, hq, hkv, block_tokens, bps = 4, 32, 8, 256, 8
    lens = [2048, 100, 1025, 600]
    num_blocks = batch * bps
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    k_bits = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    v_bits = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    q, k, v = H.bf16_tensor(q_bits), H.bf16_tensor(k_bits), H.bf16_tensor(v_bits)
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=lens, blocks_per_seq=bps, paged=True, device_lens=True,
                           split_keys=512)
    assert plan["cluster_size"] == 4, plan
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    outs = []
    for max_ctas in (0, 100):
        out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        gqa.decode(q, k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=lens,
                   seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
                   block_table=torch.from_numpy(table).to("cuda:0"), workspace=ws, split_keys=512,
                   max_ctas=max_ctas, status=status)
        torch.cuda.synchronize()
        outs.append(out)
    assert int(status.item()) == 0
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    want = oracle.gqa_decode(q_bits, k_bits.reshape(-1), v_bits.reshape(-1), lens, hkv=hkv,
                             stride_block=layout.stride_block, stride_token=layout.stride_token,
                             stride_head=layout.stride_head, block_tokens=block_tokens,
                             block_table=table)
    abs_err, rel_err = H.errors(H.f32_of(outs[0]), want)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)
