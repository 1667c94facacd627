"""GPU parity of the decode-attention kernels, called through the C ABI, against the CPU
oracle (FP64 accumulation) and against the outputs of the reference's own CUDA kernels.

Tolerances: BF16 outputs within 2e-2 absolute of the reference and of the oracle (the
reference's own BF16 tolerance, test_kernel/test_qwen3_bf16_ops.py:836-917) and within 1e-2 of
max|out| (so that long contexts, where |out| ~ 1/sqrt(L), are still checked); FP32 within 1e-5
relative (test/test_op/test_op_mha.cpp:62).
"""
import numpy as np
import pytest
import torch

import cases
import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu

ABS_TOL_BF16 = 2e-2
REL_TOL_BF16 = 1e-2
REL_TOL_F32 = 1e-5


@pytest.fixture(scope="module")
def gqa(built_lib):
    import llminfer_b200 as pkg
    assert torch.cuda.is_available(), "these tests need the GPU"
    return pkg


def run_reference_layout(gqa, q_bits, k_bits, v_bits, *, hkv, layer_id, length, split_keys=0,
                         max_ctas=0, early_prefetch=False):
    layers, max_seq_len, _ = k_bits.shape
    hq = q_bits.shape[0]
    layout = gqa.layout_reference(layers, max_seq_len, hkv)
    q = H.bf16_tensor(q_bits).reshape(1, hq, H.D)
    k, v = H.bf16_tensor(k_bits), H.bf16_tensor(v_bits)
    out = torch.full((1, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    # One partial record per 32 keys per query head is the most any split can need.
    ws = torch.empty(hq * 130 * (max_seq_len // 32 + 1), dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    gqa.decode(q, k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=[length],
               fixed_block=layer_id, workspace=ws, split_keys=split_keys, max_ctas=max_ctas,
               status=status, early_prefetch=early_prefetch)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return H.bits_of(out)[0]


@pytest.mark.parametrize("index", range(len(cases.ATTN_CASES)))
def test_bf16_golden_cases(gqa, index, request):
    name, hq, hkv, length, layers, layer_id, max_seq_len = cases.ATTN_CASES[index]
    q, k, v = cases.attention_inputs(index)
    # Rows past the sequence end and other layers must never influence the result.
    k[layer_id, length:] = H.NAN_BITS
    v[layer_id, length:] = H.NAN_BITS
    got_bits = run_reference_layout(gqa, q, k, v, hkv=hkv, layer_id=layer_id, length=length)
    # Requesting old rows before earlier work has finished changes timing, never values.
    early = run_reference_layout(gqa, q, k, v, hkv=hkv, layer_id=layer_id, length=length,
                                 early_prefetch=True)
    assert np.array_equal(got_bits, early)
    got = cases.bf16_bits_to_f32(got_bits)
    want = H.oracle_reference_layout(q, k, v, layer_id=layer_id, length=length, hkv=hkv,
                                     max_seq_len=max_seq_len)
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (name, abs_err, rel_err)
    try:
        golden = request.getfixturevalue("golden")
    except pytest.skip.Exception:
        return
    ref = cases.bf16_bits_to_f32(golden[f"attn/{name}/out"])
    abs_ref, rel_ref = H.errors(got, ref)
    assert abs_ref <= ABS_TOL_BF16 and rel_ref <= 2 * REL_TOL_BF16, (name, abs_ref, rel_ref)


def test_bf16_every_length_to_300(gqa):
    """Every tail size and every short length, rows past the end poisoned with NaN."""
    rng = np.random.default_rng(7)
    hq, hkv, max_seq_len = 32, 8, 320
    q = H.rand_bits(rng, (hq, H.D))
    k_all = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v_all = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    dq = H.bf16_tensor(q).reshape(1, hq, H.D)
    ws = torch.empty(hq * 4 * max_seq_len, dtype=torch.float32, device="cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    worst = 0.0
    for length in range(1, 301):
        k, v = k_all.copy(), v_all.copy()
        k[0, length:] = H.NAN_BITS
        v[0, length:] = H.NAN_BITS
        out = torch.full((1, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        gqa.decode(dq, H.bf16_tensor(k), H.bf16_tensor(v), out, num_kv_heads=hkv, layout=layout,
                   seq_lens=[length], workspace=ws, status=status)
        got = H.f32_of(out)[0]
        want = H.oracle_reference_layout(q, k, v, layer_id=0, length=length, hkv=hkv,
                                         max_seq_len=max_seq_len)
        abs_err, rel_err = H.errors(got, want)
        assert np.isfinite(got).all(), length
        assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (length, abs_err, rel_err)
        worst = max(worst, rel_err)
    assert int(status.item()) == 0


@pytest.mark.parametrize("split_keys", [32, 64, 96, 256, 4096])
def test_bf16_split_override(gqa, split_keys):
    rng = np.random.default_rng(11)
    hq, hkv, length, max_seq_len = 32, 8, 1000, 1024
    q = H.rand_bits(rng, (hq, H.D))
    k = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    got = cases.bf16_bits_to_f32(run_reference_layout(gqa, q, k, v, hkv=hkv, layer_id=0,
                                                      length=length, split_keys=split_keys))
    want = H.oracle_reference_layout(q, k, v, layer_id=0, length=length, hkv=hkv,
                                     max_seq_len=max_seq_len)
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)


def test_bf16_split_is_deterministic_in_grid_size(gqa):
    """With split_keys fixed the result does not depend on how many CTAs share the items."""
    rng = np.random.default_rng(13)
    hq, hkv, length, max_seq_len = 32, 8, 3000, 3072
    q = H.rand_bits(rng, (hq, H.D))
    k = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    a = run_reference_layout(gqa, q, k, v, hkv=hkv, layer_id=0, length=length, split_keys=256)
    b = run_reference_layout(gqa, q, k, v, hkv=hkv, layer_id=0, length=length, split_keys=256,
                             max_ctas=5)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("group", [1, 2, 3, 4, 5, 6, 7, 8])
def test_bf16_group_sizes(gqa, group):
    rng = np.random.default_rng(100 + group)
    hkv, length, max_seq_len = 4, 700, 704
    hq = hkv * group
    q = H.rand_bits(rng, (hq, H.D))
    k = H.rand_bits(rng, (2, max_seq_len, hkv * H.D))
    v = H.rand_bits(rng, (2, max_seq_len, hkv * H.D))
    got = cases.bf16_bits_to_f32(run_reference_layout(gqa, q, k, v, hkv=hkv, layer_id=1,
                                                      length=length))
    want = H.oracle_reference_layout(q, k, v, layer_id=1, length=length, hkv=hkv,
                                     max_seq_len=max_seq_len)
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)


def make_paged_batch(gqa, rng, batch, hq, hkv, lens, block_tokens, spare_blocks=3):
    """Ragged batch in a pool with shuffled physical blocks; returns host and device views."""
    blocks_per_seq = max((l + block_tokens - 1) // block_tokens for l in lens)
    need = sum((l + block_tokens - 1) // block_tokens for l in lens)
    num_blocks = need + spare_blocks
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    pool_elems = num_blocks * hkv * block_tokens * H.D
    k_pool = np.full(pool_elems, H.NAN_BITS, dtype=np.uint16)
    v_pool = np.full(pool_elems, H.NAN_BITS, dtype=np.uint16)
    order = rng.permutation(num_blocks)
    table = np.full((batch, blocks_per_seq), -1, dtype=np.int32)
    nxt = 0
    for b, length in enumerate(lens):
        for lb in range((length + block_tokens - 1) // block_tokens):
            table[b, lb] = order[nxt]
            nxt += 1
            rows = min(block_tokens, length - lb * block_tokens)
            for hk in range(hkv):
                off = (table[b, lb] * hkv + hk) * block_tokens * H.D
                k_pool[off:off + rows * H.D] = H.rand_bits(rng, rows * H.D)
                v_pool[off:off + rows * H.D] = H.rand_bits(rng, rows * H.D)
    q = H.rand_bits(rng, (batch, hq, H.D))
    return layout, q, k_pool, v_pool, table


def test_bf16_paged_ragged_batch(gqa):
    """Ragged batch in 256-token pool blocks in shuffled physical order, lengths on the device."""
    rng = np.random.default_rng(17)
    batch, hq, hkv, block_tokens = 16, 32, 8, 256
    lens = [int(x) for x in rng.integers(256, 2049, size=batch)]
    lens[0], lens[1], lens[2] = 256, 257, 2048
    layout, q, k_pool, v_pool, table = make_paged_batch(gqa, rng, batch, hq, hkv, lens, block_tokens)
    want = oracle.gqa_decode(q, k_pool, v_pool, lens, hkv=hkv, stride_block=layout.stride_block,
                             stride_token=layout.stride_token, stride_head=layout.stride_head,
                             block_tokens=block_tokens, block_table=np.maximum(table, 0))
    dq, dk, dv = H.bf16_tensor(q), H.bf16_tensor(k_pool), H.bf16_tensor(v_pool)
    dtab = torch.from_numpy(table).to("cuda:0")
    dlens = torch.tensor(lens, dtype=torch.int32, device="cuda:0")
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    for host_lens in (lens, None):
        out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        gqa.decode(dq, dk, dv, out, num_kv_heads=hkv, layout=layout, seq_lens=host_lens,
                   seq_lens_dev=dlens, block_table=dtab, workspace=ws, status=status,
                   plan_len_hint=0 if host_lens else 1024)
        got = H.f32_of(out)
        abs_err, rel_err = H.errors(got, want)
        assert np.isfinite(got).all()
        assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)
    assert int(status.item()) == 0


def test_f32_qwen3_06b_shape(gqa):
    """FP32 case of the reference's CPU backend: 16 q / 8 kv heads, 512 cached positions."""
    rng = np.random.default_rng(19)
    hq, hkv, length, max_seq_len = 16, 8, 512, 512
    q = rng.standard_normal((hq, H.D), dtype=np.float32)
    k = rng.standard_normal((1, max_seq_len, hkv * H.D), dtype=np.float32)
    v = rng.standard_normal((1, max_seq_len, hkv * H.D), dtype=np.float32)
    want64 = oracle.mha_reference_layout(q, k.reshape(-1), v.reshape(-1), layer_id=0,
                                         pos=length - 1, hkv=hkv, max_seq_len=max_seq_len, accum=1)
    want32 = oracle.mha_reference_layout(q, k.reshape(-1), v.reshape(-1), layer_id=0,
                                         pos=length - 1, hkv=hkv, max_seq_len=max_seq_len, accum=0)
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    dq = torch.from_numpy(q).to("cuda:0").reshape(1, hq, H.D)
    dk, dv = torch.from_numpy(k).to("cuda:0"), torch.from_numpy(v).to("cuda:0")
    ws = torch.empty(hq * 4 * max_seq_len, dtype=torch.float32, device="cuda:0")
    for split_keys in (0, 64, 512):
        out = torch.full((1, hq, H.D), float("nan"), dtype=torch.float32, device="cuda:0")
        gqa.decode(dq, dk, dv, out, num_kv_heads=hkv, layout=layout, seq_lens=[length],
                   workspace=ws, split_keys=split_keys)
        got = H.f32_of(out)[0]
        for want in (want64, want32):
            _, rel_err = H.errors(got, want)
            assert rel_err <= REL_TOL_F32, (split_keys, rel_err)


@pytest.mark.parametrize("length,group", [(37, 1), (200, 4), (1025, 8)])
def test_f32_lengths_and_groups(gqa, length, group):
    rng = np.random.default_rng(23 + length)
    hkv, max_seq_len = 2, 1056
    hq = hkv * group
    q = rng.standard_normal((hq, H.D), dtype=np.float32)
    k = rng.standard_normal((2, max_seq_len, hkv * H.D), dtype=np.float32)
    v = rng.standard_normal((2, max_seq_len, hkv * H.D), dtype=np.float32)
    k[1, length:] = np.nan
    v[1, length:] = np.nan
    want = oracle.mha_reference_layout(q, k.reshape(-1), v.reshape(-1), layer_id=1,
                                       pos=length - 1, hkv=hkv, max_seq_len=max_seq_len, accum=1)
    layout = gqa.layout_reference(2, max_seq_len, hkv)
    out = torch.full((1, hq, H.D), float("nan"), dtype=torch.float32, device="cuda:0")
    ws = torch.empty(hq * 4 * max_seq_len, dtype=torch.float32, device="cuda:0")
    gqa.decode(torch.from_numpy(q).to("cuda:0").reshape(1, hq, H.D), torch.from_numpy(k).to("cuda:0"),
               torch.from_numpy(v).to("cuda:0"), out, num_kv_heads=hkv, layout=layout,
               seq_lens=[length], fixed_block=1, workspace=ws)
    _, rel_err = H.errors(H.f32_of(out)[0], want)
    assert rel_err <= REL_TOL_F32, rel_err


def test_bf16_decode_steps_with_early_prefetch(gqa):
    """A run of decode steps (front stage appends a row, attention reads the cache) queued
    back to back on one stream with early prefetch: every step must see the row appended just
    before it, and only that one."""
    rng = np.random.default_rng(43)
    hq, hkv, max_seq_len, start, steps = 32, 8, 640, 250, 140
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    k_hist = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    v_hist = H.rand_bits(rng, (1, max_seq_len, hkv * H.D))
    k_hist[0, start:] = H.NAN_BITS
    v_hist[0, start:] = H.NAN_BITS
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(256, dtype=np.float32))
    q_all = H.rand_bits(rng, (steps, 1, hq, H.D))
    k_all = H.rand_bits(rng, (steps, 1, hkv, H.D))
    v_all = H.rand_bits(rng, (steps, 1, hkv, H.D))
    dk, dv, dw = H.bf16_tensor(k_hist), H.bf16_tensor(v_hist), H.bf16_tensor(w)
    dq, dkn, dvn = H.bf16_tensor(q_all), H.bf16_tensor(k_all), H.bf16_tensor(v_all)
    outs = torch.zeros(steps, 1, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    ws = gqa.binding.workspace_for(1, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    for i in range(steps):
        pos = start + i
        gqa.qk_norm_rope_append(dq[i], dkn[i], dvn[i], dw, dk, dv, layout=layout, positions=[pos])
        gqa.decode(dq[i], dk, dv, outs[i], num_kv_heads=hkv, layout=layout, seq_lens=[pos + 1],
                   workspace=ws, status=status, early_prefetch=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    k_final, v_final, q_rot = H.bits_of(dk), H.bits_of(dv), H.bits_of(dq)
    got = H.f32_of(outs)
    for i in (0, 1, 5, 37, 70, 71, 72, steps - 1):
        pos = start + i
        want = H.oracle_reference_layout(q_rot[i, 0], k_final, v_final, layer_id=0, length=pos + 1,
                                         hkv=hkv, max_seq_len=max_seq_len)
        abs_err, rel_err = H.errors(got[i, 0], want)
        assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (i, abs_err, rel_err)


def test_bf16_long_context_properties(gqa):
    """32K keys (the KV-split branch at full size): sampled heads against the oracle, and the
    size-independent property that identical V rows give that row back."""
    torch.manual_seed(29)
    hq, hkv, length = 32, 8, 32768
    layout = gqa.layout_reference(1, length, hkv)
    q = torch.randn(1, hq, H.D, device="cuda:0").to(torch.bfloat16)
    k = torch.randn(1, length, hkv * H.D, device="cuda:0").to(torch.bfloat16)
    v = torch.randn(1, length, hkv * H.D, device="cuda:0").to(torch.bfloat16)
    out = torch.empty(1, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    ws = gqa.binding.workspace_for(1, hq, hkv, "cuda:0")
    gqa.decode(q, k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=[length], workspace=ws)
    want = oracle.mha_reference_layout(H.bits_of(q)[0], H.bits_of(k).reshape(-1),
                                       H.bits_of(v).reshape(-1), layer_id=0, pos=length - 1,
                                       hkv=hkv, max_seq_len=length, accum=1)
    abs_err, rel_err = H.errors(H.f32_of(out)[0], want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)
    # Uniform V: the softmax weights sum to one, so the output is the common row.
    row = torch.randn(hkv * H.D, device="cuda:0").to(torch.bfloat16)
    v[:] = row
    gqa.decode(q, k, v, out, num_kv_heads=hkv, layout=layout, seq_lens=[length], workspace=ws)
    expect = row.view(hkv, 1, H.D).expand(hkv, hq // hkv, H.D).reshape(hq, H.D).float()
    assert torch.allclose(out[0].float(), expect, atol=0, rtol=2 ** -7)


def test_bf16_many_short_sequences_lengths_on_device_only(gqa):
    """64 sequences from 1 to 700 keys, lengths known on the device only (the host plans from a
    hint), 64-token pool blocks."""
    rng = np.random.default_rng(59)
    batch, hq, hkv, block_tokens = 64, 16, 4, 64
    lens = [int(x) for x in rng.integers(1, 701, size=batch)]
    lens[0], lens[1], lens[2], lens[3] = 1, 64, 65, 700
    layout, q, k_pool, v_pool, table = make_paged_batch(gqa, rng, batch, hq, hkv, lens, block_tokens)
    want = oracle.gqa_decode(q, k_pool, v_pool, lens, hkv=hkv, stride_block=layout.stride_block,
                             stride_token=layout.stride_token, stride_head=layout.stride_head,
                             block_tokens=block_tokens, block_table=np.maximum(table, 0))
    out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    ws = gqa.binding.workspace_for(batch, hq, hkv, "cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    gqa.decode(H.bf16_tensor(q), H.bf16_tensor(k_pool), H.bf16_tensor(v_pool), out,
               num_kv_heads=hkv, layout=layout, seq_lens=None,
               seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda:0"),
               block_table=torch.from_numpy(table).to("cuda:0"), workspace=ws, status=status,
               plan_len_hint=256)
    got = H.f32_of(out)
    assert np.isfinite(got).all() and int(status.item()) == 0
    abs_err, rel_err = H.errors(got, want)
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)


def test_bf16_full_size_long_context_batch(gqa):
    """The benchmark's shape at full size (64 q / 8 kv heads, batch 4, 131072 keys, 2 GiB of
    K and V in 256-token pool blocks): size-independent properties, and one (sequence, kv head)
    against the oracle."""
    torch.manual_seed(61)
    dev = "cuda:0"
    batch, hq, hkv, length, block_tokens = 4, 64, 8, 131072, 256
    blocks_per_seq = length // block_tokens
    num_blocks = batch * blocks_per_seq
    layout = gqa.layout_pool(num_blocks, block_tokens, hkv)
    elems = num_blocks * hkv * block_tokens * H.D
    k_pool = torch.empty(elems, dtype=torch.bfloat16, device=dev)
    v_pool = torch.empty(elems, dtype=torch.bfloat16, device=dev)
    for pool in (k_pool, v_pool):
        for start in range(0, elems, 1 << 26):
            n = min(1 << 26, elems - start)
            pool[start:start + n] = torch.randn(n, device=dev).to(torch.bfloat16)
    table = torch.randperm(num_blocks).to(torch.int32).view(batch, blocks_per_seq).to(dev)
    q = torch.randn(batch, hq, H.D, device=dev).to(torch.bfloat16)
    lens = [length] * batch
    lens_dev = torch.tensor(lens, dtype=torch.int32, device=dev)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev).view(torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def run(split_keys=0):
        out = torch.full((batch, hq, H.D), float("nan"), dtype=torch.bfloat16, device=dev)
        gqa.decode(q, k_pool, v_pool, out, num_kv_heads=hkv, layout=layout, seq_lens=lens,
                   seq_lens_dev=lens_dev, block_table=table, workspace=ws, status=status,
                   split_keys=split_keys)
        torch.cuda.synchronize()
        return out

    auto = run()
    assert torch.isfinite(auto.float()).all() and int(status.item()) == 0
    # How the keys are cut must not matter beyond rounding.
    other = run(split_keys=8192)
    scale = auto.float().abs().max().item()
    assert (auto.float() - other.float()).abs().max().item() <= REL_TOL_BF16 * scale
    # One unit against the oracle: sequence 2, kv head 5 (query heads 40..47).
    b, hk, g = 2, 5, hq // hkv
    blocks = table[b].long()
    k_unit = k_pool.view(num_blocks, hkv, block_tokens, H.D)[blocks, hk].reshape(length, H.D)
    v_unit = v_pool.view(num_blocks, hkv, block_tokens, H.D)[blocks, hk].reshape(length, H.D)
    want = oracle.gqa_decode(H.bits_of(q[b:b + 1, hk * g:(hk + 1) * g]), H.bits_of(k_unit).reshape(-1),
                             H.bits_of(v_unit).reshape(-1), [length], hkv=1,
                             stride_block=length * H.D, stride_token=H.D, stride_head=H.D,
                             block_tokens=length)
    abs_err, rel_err = H.errors(H.f32_of(auto[b, hk * g:(hk + 1) * g]), want[0])
    assert abs_err <= ABS_TOL_BF16 and rel_err <= REL_TOL_BF16, (abs_err, rel_err)
    # Identical V rows: the weights sum to one, so every head returns that row.
    row = torch.randn(H.D, device=dev).to(torch.bfloat16)
    v_pool.view(-1, H.D)[:] = row
    same = run()
    assert torch.allclose(same.float(), row.float().expand_as(same), atol=0, rtol=2 ** -7)
