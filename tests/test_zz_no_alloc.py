"""gqa_decode_static_scratch: the decode entry point for callers that may not allocate device
memory (its split scratch is a static device array inside the library).

Called through the C ABI and compared with gqa_decode() on two calls in a row with different
inputs and lengths, so that records left in the shared array by the first call cannot leak into
the second. The file name sorts last on purpose: a run that stops at the first failure has
already run every other test.
"""
import numpy as np
import pytest
import torch

import cases
import helpers as H

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_decode_on_two_calls_in_a_row(built_lib):
    import llminfer_b200 as gqa
    assert torch.cuda.is_available(), "this test needs the GPU"
    rng = np.random.default_rng(47)
    hq, hkv, max_seq_len = 32, 8, 4096
    layout = gqa.layout_reference(1, max_seq_len, hkv)
    k = H.bf16_tensor(H.rand_bits(rng, (1, max_seq_len, hkv * H.D)))
    v = H.bf16_tensor(H.rand_bits(rng, (1, max_seq_len, hkv * H.D)))
    ws = gqa.binding.workspace_for(1, hq, hkv, "cuda:0")
    before = torch.cuda.memory_allocated()
    for length, split_keys in ((4000, 0), (1333, 0), (4000, 256), (777, 64)):
        q = H.bf16_tensor(H.rand_bits(rng, (1, hq, H.D)))
        want = torch.full((1, hq, H.D), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        got = torch.full_like(want, float("nan"))
        gqa.decode(q, k, v, want, num_kv_heads=hkv, layout=layout, seq_lens=[length],
                   workspace=ws, split_keys=split_keys)
        gqa.decode_static_scratch(q, k, v, got, num_kv_heads=hkv, layout=layout,
                                  seq_lens=[length], split_keys=split_keys)
        torch.cuda.synchronize()
        a, b = H.f32_of(got), H.f32_of(want)
        assert np.isfinite(a).all()
        abs_err, rel_err = H.errors(a, b)
        # Same kernels on the same inputs: the tolerance of the parity tests is far from reached,
        # and with an explicit split the two results are bit-equal.
        assert abs_err <= 2e-2 and rel_err <= 1e-2, (length, abs_err, rel_err)
        if split_keys:
            assert np.array_equal(H.bits_of(got), H.bits_of(want)), length
    # The entry point allocated nothing through torch either (only the two output tensors of
    # the last iteration are still alive).
    assert torch.cuda.memory_allocated() - before <= 4 * hq * H.D * 2 + 4096


def test_static_scratch_refuses_plans_beyond_its_array(built_lib):
    import llminfer_b200 as gqa
    hq, hkv, length = 64, 8, 131072
    layout = gqa.layout_reference(1, length, hkv)
    q = torch.zeros(1, hq, H.D, dtype=torch.bfloat16, device="cuda:0")
    k = torch.zeros(1, length, hkv * H.D, dtype=torch.bfloat16, device="cuda:0")
    out = torch.zeros_like(q)
    # 4096 splits x 8 heads x 8 x 130 floats = 136 MB of partials: far beyond the 8 MiB array.
    with pytest.raises(gqa.GqaError) as e:
        gqa.decode_static_scratch(q, k, k, out, num_kv_heads=hkv, layout=layout,
                                  seq_lens=[length], split_keys=32)
    assert e.value.status == -6
    # The automatic plan for the same shape fits and runs.
    gqa.decode_static_scratch(q, k, k, out, num_kv_heads=hkv, layout=layout, seq_lens=[length])
    torch.cuda.synchronize()
