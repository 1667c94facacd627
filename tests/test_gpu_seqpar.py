"""Sequence-parallel decode on a single GPU: with one rank the merge across ranks has one
record to merge, so gqa_decode_seqpar must reproduce gqa_decode bit for bit, through the same
kernels a multi-GPU run uses (every unit leaves a partial record, the combine kernel's
cross-rank mode, the peer window), and both must agree with the FP64 oracle. The merge of
several ranks' records (empty ones included) is checked against the oracle on one GPU in
test_gpu_partial_merge.py and across real ranks in multi_gpu_worker.py."""
import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200
    return llminfer_b200


@pytest.fixture(scope="module")
def comm(gqa):
    try:
        c = gqa.ShardComm(gqa.ShardComm.unique_id(), 1, 0)
    except gqa.GqaError:
        pytest.skip("NCCL is not available")
    c.enable_peer_gather(1 << 20)
    yield c
    c.close()


@pytest.mark.parametrize("hq,hkv,lens,split_keys", [
    (32, 8, [700], 0),            # not split: the record comes straight from the streaming kernel
    (32, 8, [700], 128),          # split units
    (64, 8, [257, 3000, 64], 512),  # ragged batch, wide combine grid
    (16, 8, [96], 0),             # shorter than one stage
])
def test_one_rank_reproduces_decode(gqa, comm, hq, hkv, lens, split_keys):
    rng = np.random.default_rng(hq + sum(lens))
    batch, block_tokens, d = len(lens), 256, 128
    blocks_per_seq = max(-(-n // block_tokens) for n in lens)
    num_blocks = batch * blocks_per_seq
    table_np = rng.permutation(num_blocks).reshape(batch, blocks_per_seq).astype(np.int32)
    table = torch.from_numpy(table_np).to("cuda:0")
    q_bits = H.rand_bits(rng, (batch, hq, d))
    k_bits = H.rand_bits(rng, (num_blocks, hkv, block_tokens, d))
    v_bits = H.rand_bits(rng, (num_blocks, hkv, block_tokens, d))
    q, k, v = H.bf16_tensor(q_bits), H.bf16_tensor(k_bits), H.bf16_tensor(v_bits)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    kw = dict(num_kv_heads=hkv, layout=layout, seq_lens=lens,
              seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
              block_table=table, workspace=ws, split_keys=split_keys)
    want = torch.zeros(batch, hq, d, dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(q, k, v, want, **kw)
    for _ in range(3):  # consecutive steps alternate between the halves of the window
        got = torch.full((batch, hq, d), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        gqa.decode_seqpar(comm, q, k, v, got, status=status, **kw)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ref = oracle.gqa_decode(q_bits, k_bits.reshape(-1), v_bits.reshape(-1), lens, hkv=hkv,
                            stride_block=layout.stride_block, stride_token=layout.stride_token,
                            stride_head=layout.stride_head, block_tokens=block_tokens,
                            block_table=table_np)
    abs_err, rel_err = H.errors(H.f32_of(got), ref)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)
