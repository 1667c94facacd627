"""Device-side inputs are never trusted: lengths, positions and block ids that the kernels read
from device memory are clamped or skipped and reported through the status word
(GQA_STATUS_BAD_INPUT = 3); partial records that would not fit the caller's scratch are not
written. No case here can touch memory outside the test's own allocations even without the
guards: every out-of-range value points into spare blocks, rows or canary space."""
import numpy as np
import pytest
import torch

import cases
import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

BAD_INPUT = 3


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    return pkg


def paged_setup(gqa, rng, batch, hq, hkv, blocks_per_seq, block_tokens=256, spare_rows=2):
    """A pool with one spare block in front and spare block-table rows behind, so that block id
    -1 and reads past a table row stay inside the allocations."""
    num_blocks = batch * blocks_per_seq + spare_rows * blocks_per_seq
    k_all = H.bf16_tensor(H.rand_bits(rng, (num_blocks + 1, hkv, block_tokens, H.D)))
    v_all = H.bf16_tensor(H.rand_bits(rng, (num_blocks + 1, hkv, block_tokens, H.D)))
    table_all = rng.permutation(num_blocks).reshape(batch + spare_rows, blocks_per_seq).astype(np.int32)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    return layout, k_all, v_all, table_all


def test_lengths_grow_past_the_planned_scratch(gqa):
    """Planned with short host lengths, run with longer device lengths: records that do not fit
    the scratch are skipped and reported; the canary behind the scratch stays intact."""
    rng = np.random.default_rng(1)
    batch, hq, hkv, bps = 3, 32, 8, 16
    layout, k_all, v_all, table_all = paged_setup(gqa, rng, batch, hq, hkv, bps)
    k, v = k_all[1:], v_all[1:]
    table = torch.from_numpy(table_all).to("cuda:0")[:batch]
    q = H.bf16_tensor(H.rand_bits(rng, (batch, hq, H.D)))
    short, grown = [600, 500, 700], [4000, 3900, 4096]
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=short, blocks_per_seq=bps, paged=True, device_lens=True,
                           split_keys=128)
    assert plan["needs_combine"] == 1
    n = plan["workspace_bytes"] // 4
    canary = 1 << 20
    buf = torch.full((n + canary,), 12345.0, dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.zeros(batch, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    kw = dict(num_kv_heads=hkv, layout=layout, seq_lens=short, block_table=table,
              workspace=buf[:n], split_keys=128, status=status)
    gqa.decode(q, k, v, out, seq_lens_dev=torch.tensor(short, dtype=torch.int32, device="cuda:0"), **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    gqa.decode(q, k, v, out, seq_lens_dev=torch.tensor(grown, dtype=torch.int32, device="cuda:0"), **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == BAD_INPUT
    assert bool((buf[n:] == 12345.0).all()), "records were written past the scratch"


def test_lengths_grow_within_the_scratch(gqa):
    """A launch planned with short lengths stays valid as the device lengths grow, as long as
    the scratch holds the records: the combine launch is kept whatever the host lengths say."""
    rng = np.random.default_rng(2)
    batch, hq, hkv, bps, block_tokens = 2, 32, 8, 8, 256
    layout, k_all, v_all, table_all = paged_setup(gqa, rng, batch, hq, hkv, bps)
    k, v = k_all[1:], v_all[1:]
    table = torch.from_numpy(table_all).to("cuda:0")[:batch]
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    planned, grown = [40, 33], [1900, 2048]
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=planned,
               seq_lens_dev=torch.tensor(grown, dtype=torch.int32, device="cuda:0"),
               block_table=table, workspace=ws, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = oracle.gqa_decode(q_bits, H.bits_of(k).reshape(-1), H.bits_of(v).reshape(-1), grown,
                             hkv=hkv, stride_block=layout.stride_block,
                             stride_token=layout.stride_token, stride_head=layout.stride_head,
                             block_tokens=block_tokens, block_table=table_all[:batch])
    abs_err, rel_err = H.errors(H.f32_of(out), want)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_length_past_capacity_is_clamped(gqa, dtype):
    rng = np.random.default_rng(3)
    batch, hq, hkv, bps, block_tokens = 2, 16, 8, 2, 64
    num_blocks = 12
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    mk = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32)).to("cuda:0").to(tdt)
    k, v = mk(num_blocks, hkv, block_tokens, H.D), mk(num_blocks, hkv, block_tokens, H.D)
    q = mk(batch, hq, H.D)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = torch.from_numpy(rng.permutation(num_blocks)[:8].reshape(4, bps).astype(np.int32)).to("cuda:0")
    cap = bps * block_tokens
    ws = torch.empty(1 << 20, dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    outs = []
    for lens in ([cap, cap], [cap + 70, cap + 1]):
        status.zero_()
        out = torch.zeros(batch, hq, H.D, dtype=tdt, device="cuda:0")
        gqa.decode(q, k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=[cap, cap],
                   seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
                   block_table=table[:batch], workspace=ws, status=status)
        torch.cuda.synchronize()
        outs.append((out, int(status.item())))
    assert outs[0][1] == 0 and outs[1][1] == BAD_INPUT
    assert torch.equal(outs[0][0], outs[1][0])  # clamped to the capacity: the same attention


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_unassigned_block_is_reported_not_followed(gqa, dtype):
    rng = np.random.default_rng(4)
    batch, hq, hkv, bps, block_tokens = 1, 16, 8, 4, 64
    num_blocks = 8
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    mk = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32)).to("cuda:0").to(tdt)
    # One spare block in front of the pool: block id -1 points into it.
    k_all, v_all = mk(num_blocks + 1, hkv, block_tokens, H.D), mk(num_blocks + 1, hkv, block_tokens, H.D)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = torch.tensor([[3, -1, 5, 6]], dtype=torch.int32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.zeros(batch, hq, H.D, dtype=tdt, device="cuda:0")
    ws = torch.empty(1 << 18, dtype=torch.float32, device="cuda:0")
    gqa.decode(mk(batch, hq, H.D), k_all[1:], v_all[1:], out, num_kv_heads=hkv, layout=layout,
               seq_lens=[200], seq_lens_dev=torch.tensor([200], dtype=torch.int32, device="cuda:0"),
               block_table=table, workspace=ws, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == BAD_INPUT
    assert torch.isfinite(out.float()).all()


def test_front_stage_skips_rows_with_bad_positions(gqa):
    rng = np.random.default_rng(5)
    batch, hq, hkv, bps, block_tokens = 4, 32, 8, 2, 256
    layout, k_all, v_all, table_all = paged_setup(gqa, rng, batch, hq, hkv, bps)
    k, v = k_all[1:], v_all[1:]
    table_all[2, 1] = -1  # sequence 2 has no second block yet
    table = torch.from_numpy(table_all).to("cuda:0")[:batch]
    cap = bps * block_tokens
    sin = torch.empty(cap, H.D // 2, dtype=torch.float32, device="cuda:0")
    cos = torch.empty_like(sin)
    gqa.sin_cos_cache(sin, cos, H.D)
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    w = H.bf16_tensor(cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * H.D, dtype=np.float32)))
    k_new, v_new = H.bf16_tensor(H.rand_bits(rng, (batch, hkv, H.D))), H.bf16_tensor(H.rand_bits(rng, (batch, hkv, H.D)))
    # Host positions are fine (and only used for planning); the device array is what counts.
    bad = [cap + 3, -1, 300, 17]  # past the cache; negative; unassigned block; the only good one
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    k_before, v_before = k_all.clone(), v_all.clone()
    q = H.bf16_tensor(q_bits)
    q_out = torch.zeros_like(q)
    gqa.qk_norm_rope_append(q, k_new, v_new, w, k, v, layout=layout, positions=[5, 5, 5, 5],
                            positions_dev=torch.tensor(bad, dtype=torch.int32, device="cuda:0"),
                            block_table=table, q_out=q_out, sin_cache=sin, cos_cache=cos,
                            status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == BAD_INPUT
    # Only sequence 3's row was written (block table_all[3, 0], token 17).
    blk = int(table_all[3, 0]) + 1
    changed_k = (k_all.view(torch.int16) != k_before.view(torch.int16)).nonzero()
    changed_v = (v_all.view(torch.int16) != v_before.view(torch.int16)).nonzero()
    for changed in (changed_k, changed_v):
        assert changed.numel() > 0
        assert bool((changed[:, 0] == blk).all()) and bool((changed[:, 2] == 17).all())
    assert bool((q_out[:3] == 0).all()) and bool((q_out[3] != 0).any())
