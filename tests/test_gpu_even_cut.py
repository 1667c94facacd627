"""The even cut: with split_keys = 0 the planner may cut the flat sequence of all units' stages
evenly over the CTAs instead of using uniform splits (gqa_decode_plan_info.even_cut), and
split_keys = GQA_SPLIT_EVEN asks for it whatever the planner would choose (as these tests do).
Every CTA then streams the same number of stages whatever the lengths are, pieces of cut units
leave records at (CTA + unit) and the combine launch merges them. Checked against the FP64 oracle at
the BF16 tolerances of the decode tests, with the lengths the launch was planned for, with much
shorter ones (fewer stages than CTAs) and with longer ones, all through the same scratch."""
import numpy as np
import pytest
import torch

import cases
import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

ABS_TOL_BF16 = 2e-2
REL_TOL_BF16 = 1e-2


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    return pkg


def check(gqa, out, q_bits, k, v, lens, layout, table, hkv, block_tokens):
    want = oracle.gqa_decode(q_bits, H.bits_of(k).reshape(-1), H.bits_of(v).reshape(-1), lens,
                             hkv=hkv, stride_block=layout.stride_block,
                             stride_token=layout.stride_token, stride_head=layout.stride_head,
                             block_tokens=block_tokens, block_table=table)
    got = H.f32_of(out)
    assert np.isfinite(got).all()
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)


@pytest.mark.parametrize("hq", [32, 64])
def test_ragged_batch_follows_the_device_lengths(gqa, hq):
    rng = np.random.default_rng(300 + hq)
    batch, hkv, block_tokens, bps = 12, 8, 256, 32
    num_blocks = batch * bps
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    k = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    v = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    planned = [int(x) for x in rng.integers(1500, 8192, size=batch)]
    planned[3], planned[7] = 8192, 63
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=planned, blocks_per_seq=bps, paged=True, device_lens=True,
                           split_keys=gqa.SPLIT_EVEN)
    assert plan["even_cut"] == 1 and plan["needs_combine"] == 1
    ws = torch.full((plan["workspace_bytes"] // 4,), float("nan"), dtype=torch.float32, device="cuda:0")
    dtab = torch.from_numpy(table).to("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    tiny = [int(x) for x in rng.integers(1, 40, size=batch)]          # fewer stages than CTAs
    grown = [min(8192, n + int(x)) for n, x in zip(planned, rng.integers(0, 3000, size=batch))]
    one_each = [1] * batch
    for lens in (planned, tiny, grown, one_each):
        out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        for early in (False, True):
            gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout,
                       seq_lens=planned, seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
                       block_table=dtab, workspace=ws, status=status, early_prefetch=early,
                       split_keys=gqa.SPLIT_EVEN)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            check(gqa, out, q_bits, k, v, lens, layout, table, hkv, block_tokens)


@pytest.mark.parametrize("hq", [16, 64])
def test_one_long_sequence_among_short_ones(gqa, hq):
    """The long sequence is cut over most of the grid (many records per unit), the short ones
    share CTAs (several whole units per CTA, no record)."""
    rng = np.random.default_rng(hq)
    batch, hkv, block_tokens, bps = 9, 8, 256, 64
    lens = [16384] + [int(x) for x in rng.integers(60, 400, size=batch - 1)]
    num_blocks = 64 + 2 * (batch - 1)
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = np.full((batch, bps), -1, dtype=np.int32)
    order = rng.permutation(num_blocks)
    table[0] = order[:64]
    for b in range(1, batch):
        table[b, :2] = order[64 + 2 * (b - 1):64 + 2 * b]
    k = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    v = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=lens, blocks_per_seq=bps, paged=True, device_lens=True,
                           split_keys=gqa.SPLIT_EVEN)
    assert plan["even_cut"] == 1 and plan["max_splits"] > 8
    ws = torch.full((plan["workspace_bytes"] // 4,), float("nan"), dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=lens,
               seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
               block_table=torch.from_numpy(table).to("cuda:0"), workspace=ws, status=status,
               split_keys=gqa.SPLIT_EVEN)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    check(gqa, out, q_bits, k, v, lens, layout, np.maximum(table, 0), hkv, block_tokens)


def test_equal_lengths_passed_by_value(gqa):
    """No device length array: the cut is computed from the length in the launch arguments."""
    rng = np.random.default_rng(5)
    batch, hq, hkv, block_tokens, length = 3, 64, 8, 256, 9999
    bps = -(-length // block_tokens)
    num_blocks = batch * bps
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    k = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    v = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout,
               seq_lens=[length] * batch, block_table=torch.from_numpy(table).to("cuda:0"),
               workspace=ws, status=status, split_keys=gqa.SPLIT_EVEN)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    check(gqa, out, q_bits, k, v, [length] * batch, layout, table, hkv, block_tokens)


def test_even_cut_refused_where_it_does_not_apply(gqa):
    layout = gqa.layout_reference(1, 512, 8)
    z = lambda *s: torch.zeros(*s, dtype=torch.float32, device="cuda:0")
    with pytest.raises(gqa.GqaError) as e:  # the FP32 path keeps uniform splits
        gqa.decode(z(1, 16, H.D), z(1, 512, 8 * H.D), z(1, 512, 8 * H.D), z(1, 16, H.D), num_kv_heads=8,
                   layout=layout, seq_lens=[512], workspace=z(1 << 16), split_keys=gqa.SPLIT_EVEN)
    assert e.value.status == -8


def test_even_cut_with_fused_front_and_two_tokens(gqa):
    """Two query tokens per sequence and the front stage inside the kernel, on a plan that is
    cut evenly: equal, bit for bit, to the front kernel followed by the attention launch (the
    same plan, so the same cut)."""
    rng = np.random.default_rng(77)
    batch, hq, hkv, block_tokens, bps, tokens = 10, 32, 8, 256, 32, 2
    num_blocks = batch * bps
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    lens = [int(x) for x in rng.integers(1500, 8192, size=batch)]
    lens[0], lens[1] = 8192, 2
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=lens, blocks_per_seq=bps, paged=True, device_lens=True,
                           q_tokens=tokens, split_keys=gqa.SPLIT_EVEN)
    assert plan["even_cut"] == 1
    k0 = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    v0 = H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D))
    q_raw = H.rand_bits(rng, (batch, tokens, hq, H.D))
    k_new, v_new = H.rand_bits(rng, (batch, tokens, hkv, H.D)), H.rand_bits(rng, (batch, tokens, hkv, H.D))
    w = H.bf16_tensor(cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * H.D, dtype=np.float32)))
    sin = torch.empty(bps * block_tokens, H.D // 2, dtype=torch.float32, device="cuda:0")
    cos = torch.empty_like(sin)
    gqa.sin_cos_cache(sin, cos, H.D)
    dtab = torch.from_numpy(table).to("cuda:0")
    dlens = torch.tensor(lens, dtype=torch.int32, device="cuda:0")
    positions = [n - tokens for n in lens]
    ws = torch.empty(plan["workspace_bytes"] // 4, dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    kw = dict(num_kv_heads=hkv, layout=layout, seq_lens=lens, seq_lens_dev=dlens, block_table=dtab,
              workspace=ws, status=status, split_keys=gqa.SPLIT_EVEN)

    k_a, v_a, q_a = H.bf16_tensor(k0), H.bf16_tensor(v0), H.bf16_tensor(q_raw)
    out_a = torch.zeros(batch, tokens, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    gqa.qk_norm_rope_append(q_a, H.bf16_tensor(k_new), H.bf16_tensor(v_new), w, k_a, v_a,
                            layout=layout, positions=positions,
                            positions_dev=torch.tensor(positions, dtype=torch.int32, device="cuda:0"),
                            block_table=dtab, sin_cache=sin, cos_cache=cos, status=status)
    gqa.decode(q_a, k_a, v_a, out_a, **kw)
    k_b, v_b = H.bf16_tensor(k0), H.bf16_tensor(v0)
    out_b = torch.full_like(out_a, float("nan"))
    front = gqa.FusedFront(H.bf16_tensor(k_new), H.bf16_tensor(v_new), w, sin_cache=sin, cos_cache=cos)
    gqa.decode(H.bf16_tensor(q_raw), k_b, v_b, out_b, front=front, early_prefetch=True, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(out_b.view(torch.int16), out_a.view(torch.int16))
    assert torch.equal(k_b.view(torch.int16), k_a.view(torch.int16))
    assert torch.equal(v_b.view(torch.int16), v_a.view(torch.int16))
    # And the pair against the oracle, one pass per token.
    for t in range(tokens):
        lens_t = [n - tokens + 1 + t for n in lens]
        check(gqa, out_a[:, t], np.ascontiguousarray(H.bits_of(q_a)[:, t]), k_a, v_a, lens_t, layout,
              table, hkv, block_tokens)


@pytest.mark.parametrize("seed", range(10))
def test_random_batches(gqa, seed):
    """Random batch sizes, lengths (some below one stage, some zero-padded to the block table's
    capacity), groups, grid limits and query-token counts, through the even cut."""
    rng = np.random.default_rng(1000 + seed)
    hkv, block_tokens = 8, 256
    group = int(rng.choice([1, 2, 4, 8]))
    hq = hkv * group
    tokens = int(rng.choice([1, 1, 2])) if group <= 8 else 1
    if group * tokens > 16:
        tokens = 1
    batch = int(rng.integers(1, 9))
    bps = int(rng.choice([2, 4, 8]))
    cap = bps * block_tokens
    lens = [int(rng.choice([tokens, tokens + 1, 63, 64, 65, int(rng.integers(tokens, cap + 1)), cap]))
            for _ in range(batch)]
    max_ctas = int(rng.choice([0, 0, 1, 7, 40]))
    num_blocks = batch * bps
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    k = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    v = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    shape_q = (batch, hq, H.D) if tokens == 1 else (batch, tokens, hq, H.D)
    q_bits = H.rand_bits(rng, shape_q)
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=lens, blocks_per_seq=bps, paged=True, device_lens=True,
                           q_tokens=tokens, max_ctas=max_ctas, split_keys=gqa.SPLIT_EVEN)
    assert plan["even_cut"] == 1
    ws = torch.full((plan["workspace_bytes"] // 4,), float("nan"), dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.full(shape_q, float("nan"), dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=lens,
               seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
               block_table=torch.from_numpy(table).to("cuda:0"), workspace=ws, status=status,
               max_ctas=max_ctas, split_keys=gqa.SPLIT_EVEN)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, (lens, group, tokens, max_ctas)
    for t in range(tokens):
        lens_t = [n - tokens + 1 + t for n in lens]
        q_t = q_bits if tokens == 1 else np.ascontiguousarray(q_bits[:, t])
        out_t = out if tokens == 1 else out[:, t]
        check(gqa, out_t, q_t, k, v, lens_t, layout, table, hkv, block_tokens)


def test_planner_picks_it_for_the_ragged_benchmark_batch(gqa):
    """BASELINE config 4 at full size (32 q / 8 kv heads, 16 sequences of 256-8192 keys in
    256-token pool blocks), split left to the planner: it chooses the even cut, and every
    sequence agrees with the oracle."""
    import random
    rnd = random.Random(20260614 + 4)
    lens = [rnd.randint(256, 8192) for _ in range(16)]
    rng = np.random.default_rng(44)
    batch, hq, hkv, block_tokens, bps = 16, 32, 8, 256, 32
    num_blocks = batch * bps
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    k = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    v = H.bf16_tensor(H.rand_bits(rng, (num_blocks, hkv, block_tokens, H.D)))
    q_bits = H.rand_bits(rng, (batch, hq, H.D))
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    plan = gqa.decode_plan(dtype=2, batch=batch, num_q_heads=hq, num_kv_heads=hkv, layout=layout,
                           seq_lens=lens, blocks_per_seq=bps, paged=True, device_lens=True,
                           workspace_bytes=ws.numel() * 4)
    assert plan["even_cut"] == 1 and plan["num_ctas"] == 148
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    gqa.decode(H.bf16_tensor(q_bits), k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=lens,
               seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
               block_table=torch.from_numpy(table).to("cuda:0"), workspace=ws, status=status,
               early_prefetch=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    check(gqa, out, q_bits, k, v, lens, layout, table, hkv, block_tokens)
