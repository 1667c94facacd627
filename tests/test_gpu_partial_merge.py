"""The arithmetic of the sequence-parallel merge on one GPU: gqa_decode_partial runs attention
over a slice of each sequence's keys and leaves one record per output row, gqa_merge_partials
merges the slices' records with the same device function that gqa_decode_seqpar applies to the
records of the ranks. The slices of several "ranks" are computed one after the other here, so
the cross-record arithmetic (including slices that hold no key of a sequence) is compared with
the oracle without a second GPU."""
import numpy as np
import pytest
import torch

import helpers as H
from llminfer_b200 import sharding
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    return pkg


@pytest.mark.parametrize("nparts,hq,split_keys", [(2, 32, 0), (3, 32, 128), (4, 64, 0), (8, 64, 512)])
def test_slices_merge_to_the_whole_attention(gqa, nparts, hq, split_keys):
    rng = np.random.default_rng(nparts * 100 + hq)
    batch, hkv, block_tokens, bps = 4, 8, 256, 12
    lens = [3000, 257, 64, 2048]  # with 3+ parts some slices hold no key of the short sequences
    num_blocks = batch * bps
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    k_bits = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    v_bits = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    q, k, v = H.bf16_tensor(q_bits), H.bf16_tensor(k_bits), H.bf16_tensor(v_bits)
    rows = batch * hq
    records = torch.full((nparts, rows, H.D + 2), float("nan"), dtype=torch.float32, device="cuda:0")
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    empty_seen = False
    for part in range(nparts):
        local_rows, local_lens = sharding.sequence_slice(lens, table, block_tokens, nparts, part)
        empty_seen = empty_seen or 0 in local_lens
        gqa.decode_partial(q, k, v, records[part], num_kv_heads=hkv, layout=layout,
                           seq_lens=local_lens,
                           seq_lens_dev=torch.tensor(local_lens, dtype=torch.int32, device="cuda:0"),
                           block_table=torch.tensor(local_rows, dtype=torch.int32, device="cuda:0"),
                           workspace=ws, split_keys=split_keys, status=status)
    assert empty_seen  # the 64-key sequence has one block: every part but the first is empty
    out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    gqa.merge_partials(records, out)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rec = records.cpu().numpy()
    assert np.isfinite(rec[..., :H.D]).all() and np.isfinite(rec[..., H.D + 1]).all()
    want = oracle.gqa_decode(q_bits, k_bits.reshape(-1), v_bits.reshape(-1), lens, hkv=hkv,
                             stride_block=layout.stride_block, stride_token=layout.stride_token,
                             stride_head=layout.stride_head, block_tokens=block_tokens,
                             block_table=table)
    got = H.f32_of(out)
    assert np.isfinite(got).all()
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)


def test_hand_made_records_one_empty(gqa):
    """Two records made by hand, one of them empty (0, -inf, 0): the merge returns the other
    one's normalised row; an FP32 merge of two real records follows the log-sum-exp rule."""
    d = H.D
    rec = torch.zeros(3, 2, d + 2, dtype=torch.float32, device="cuda:0")
    o_a = torch.linspace(-1, 1, d, device="cuda:0")
    o_b = torch.linspace(2, -3, d, device="cuda:0")
    # row 0: parts (a, empty, empty); row 1: parts (a, empty, b)
    rec[0, :, :d], rec[0, :, d], rec[0, :, d + 1] = o_a, 1.5, 4.0
    rec[1, :, d], rec[2, 0, d] = float("-inf"), float("-inf")
    rec[2, 1, :d], rec[2, 1, d], rec[2, 1, d + 1] = o_b, 3.0, 2.0
    out = torch.full((2, d), float("nan"), dtype=torch.float32, device="cuda:0")
    gqa.merge_partials(rec, out)
    torch.cuda.synchronize()
    assert torch.allclose(out[0], o_a / 4.0, rtol=1e-6, atol=0)
    w_a, w_b = 2.0 ** (1.5 - 3.0), 1.0
    want = (o_a * w_a + o_b * w_b) / (4.0 * w_a + 2.0 * w_b)
    assert torch.allclose(out[1], want, rtol=1e-6, atol=1e-7)
