"""Sequence-parallel decode on a single GPU: with one rank the merge across ranks has one
record to merge, so gqa_decode_seqpar must reproduce gqa_decode bit for bit, through the same
kernels a multi-GPU run uses (every unit leaves a partial record, the combine kernel's
cross-rank mode, the peer window)."""
import numpy as np
import pytest
import torch

import helpers as H

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
    table = torch.from_numpy(rng.permutation(num_blocks).reshape(batch, blocks_per_seq)
                             .astype(np.int32)).to("cuda:0")
    q = H.bf16_tensor(H.rand_bits(rng, (batch, hq, d)))
    k = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, d)))
    v = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, d)))
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
