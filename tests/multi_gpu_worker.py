"""One rank of the multi-GPU parity check (launched by test_gpu_multi.py with torchrun):
KV-head-parallel decode through gqa_decode_sharded, gathered over NCCL, compared with the same
attention computed unsharded on this rank's GPU and with the CPU oracle."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests", ROOT / "tests" / "golden"):
    sys.path.insert(0, str(p))

import cases  # noqa: E402
import helpers as H  # noqa: E402
import llminfer_b200 as gqa  # noqa: E402
from llminfer_b200 import sharding  # noqa: E402
from oracle import oracle  # noqa: E402


def missing_peer_case(comm, rank, world, dev) -> None:
    """A rank that does not show up for a gather step: the others' wait runs out after its
    time limit, the status word says so, nothing hangs and the GPU stays usable. The absent
    rank simply skips the call (it is between steps, with nothing in flight)."""
    import time
    comm.enable_peer_gather(4096)
    send = torch.full((1024,), rank + 1, dtype=torch.int32, device=dev)
    recv = torch.zeros(world, 1024, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(2):  # healthy steps first
        comm.peer_gather(send, recv, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and recv[:, 0].tolist() == list(range(1, world + 1))
    dist.barrier()
    if rank != world - 1:  # the last rank stays away from the third step
        t0 = time.perf_counter()
        comm.peer_gather(send, recv, status)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert int(status.item()) == 2, status.item()
        assert 1.5 <= waited <= 10.0, waited
        # The context is intact: ordinary work still runs.
        check = torch.arange(16, device=dev).sum().item()
        assert check == 120
    dist.barrier()


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    ident = [gqa.ShardComm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ident, src=0)
    comm = gqa.ShardComm(ident[0], world, rank)

    if "--timeout-case" in sys.argv:
        missing_peer_case(comm, rank, world, dev)
        comm.close()
        dist.destroy_process_group()
        if rank == 0:
            print("multi_gpu_worker ok")
        return

    hq, hkv, batch, block_tokens, d = 64, 8, 3, 256, 128
    lens = [3000, 257, 1024]
    rng = np.random.default_rng(53)  # identical data on every rank
    blocks_per_seq = 12
    num_blocks = batch * blocks_per_seq
    table = rng.permutation(num_blocks).reshape(batch, blocks_per_seq).astype(np.int32)
    q = H.rand_bits(rng, (batch, hq, d))
    k_pool = H.rand_bits(rng, (num_blocks, hkv, block_tokens, d))
    v_pool = H.rand_bits(rng, (num_blocks, hkv, block_tokens, d))

    def run(q_bits, k_bits, v_bits, heads_q, heads_kv, sharded, split_keys=512):
        layout = gqa.layout_pool(num_blocks, block_tokens, heads_kv)
        dq = H.bf16_tensor(q_bits, dev)
        dk, dv = H.bf16_tensor(k_bits, dev), H.bf16_tensor(v_bits, dev)
        out = torch.zeros(batch, heads_q, d, dtype=torch.bfloat16, device=dev)
        ws = gqa.binding.workspace_for(batch, heads_q, heads_kv, dev)
        kw = dict(num_kv_heads=heads_kv, layout=layout, seq_lens=lens,
                  seq_lens_dev=torch.tensor(lens, dtype=torch.int32, device=dev),
                  block_table=torch.from_numpy(table).to(dev), workspace=ws, split_keys=split_keys)
        if not sharded:
            gqa.decode(dq, dk, dv, out, **kw)
            torch.cuda.synchronize()
            return out
        gathered = torch.zeros(world, batch, heads_q, d, dtype=torch.bfloat16, device=dev)
        gqa.decode_sharded(comm, gathered, dq, dk, dv, out, **kw)
        torch.cuda.synchronize()
        return sharding.unshard_output(gathered)

    full = run(q, k_pool, v_pool, hq, hkv, sharded=False)
    per_q, per_kv = hq // world, hkv // world
    q_l = q[:, rank * per_q:(rank + 1) * per_q]
    k_l = np.ascontiguousarray(k_pool[:, rank * per_kv:(rank + 1) * per_kv])
    v_l = np.ascontiguousarray(v_pool[:, rank * per_kv:(rank + 1) * per_kv])
    whole = run(q_l, k_l, v_l, per_q, per_kv, sharded=True)
    # Same split size per head, so the sharded result is bit-equal to the unsharded one.
    assert torch.equal(whole.view(torch.int16), full.view(torch.int16)), "sharded != unsharded"
    want = oracle.gqa_decode(q, k_pool.reshape(-1), v_pool.reshape(-1), lens, hkv=hkv,
                             stride_block=hkv * block_tokens * d, stride_token=d,
                             stride_head=block_tokens * d, block_tokens=block_tokens,
                             block_table=table)
    abs_err, rel_err = H.errors(whole.float().cpu().numpy(), want)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)

    # The same through the NVLink peer-store gather, step after step (the two window halves
    # alternate) and inside a replayed CUDA graph (the step counter lives on the device).
    comm.enable_peer_gather(max(batch * per_q * d * 2, 4 * per_kv * 3 * 256, batch * hq * (d + 2) * 4))
    for _ in range(5):
        again = run(q_l, k_l, v_l, per_q, per_kv, sharded=True)
        assert torch.equal(again.view(torch.int16), full.view(torch.int16)), "peer gather != unsharded"
    # The even cut of the rank's own units (its summation order differs from the unsharded
    # one, so the comparison is with the oracle), gathered through the same windows.
    even = run(q_l, k_l, v_l, per_q, per_kv, sharded=True, split_keys=gqa.SPLIT_EVEN)
    abs_err, rel_err = H.errors(even.float().cpu().numpy(), want)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, ("even cut, sharded", abs_err, rel_err)
    # The front stage inside the sharded attention kernel (gqa_decode_sharded_fused) against
    # the front kernel followed by gqa_decode_sharded: same gathered bits, same cache rows.
    layout_f = gqa.layout_pool(num_blocks, block_tokens, per_kv)
    kn = H.rand_bits(rng, (batch, hkv, d))[:, rank * per_kv:(rank + 1) * per_kv]
    vn = H.rand_bits(rng, (batch, hkv, d))[:, rank * per_kv:(rank + 1) * per_kv]
    wq = H.bf16_tensor(cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * d, dtype=np.float32)), dev)
    dtab, dlens = torch.from_numpy(table).to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    results = []
    for fused in (False, True):
        dq = H.bf16_tensor(np.ascontiguousarray(q_l), dev)
        dk, dv = H.bf16_tensor(k_l, dev), H.bf16_tensor(v_l, dev)
        dkn, dvn = H.bf16_tensor(np.ascontiguousarray(kn), dev), H.bf16_tensor(np.ascontiguousarray(vn), dev)
        out = torch.zeros(batch, per_q, d, dtype=torch.bfloat16, device=dev)
        gathered = torch.zeros(world, batch, per_q, d, dtype=torch.bfloat16, device=dev)
        kw = dict(num_kv_heads=per_kv, layout=layout_f, seq_lens=lens, seq_lens_dev=dlens,
                  block_table=dtab, workspace=gqa.binding.workspace_for(batch, per_q, per_kv, dev),
                  split_keys=512, status=st)
        if fused:
            kw["front"] = gqa.FusedFront(dkn, dvn, wq)
        else:
            gqa.qk_norm_rope_append(dq, dkn, dvn, wq, dk, dv, layout=layout_f,
                                    positions=[n - 1 for n in lens],
                                    positions_dev=torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=dev),
                                    block_table=dtab)
        gqa.decode_sharded(comm, gathered, dq, dk, dv, out, **kw)
        torch.cuda.synchronize()
        results.append((gathered, dk, dv))
    assert int(st.item()) == 0
    for a_, b_ in zip(results[0], results[1]):
        assert torch.equal(a_.view(torch.int16), b_.view(torch.int16)), "fused sharded front differs"

    send = torch.zeros(1024, dtype=torch.int32, device=dev)
    recv = torch.zeros(world, 1024, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    seen = torch.zeros(6, world, dtype=torch.int32, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        comm.peer_gather(send, recv, status)  # warm-up outside the capture
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(3):
                send.add_(rank + 1)
                comm.peer_gather(send, recv, status)
                seen[i].copy_(recv[:, 7])
        for rep in range(2):
            graph.replay()
            torch.cuda.synchronize()
            base = 3 * rep
            for i in range(3):
                want = [(base + i + 1) * (r + 1) for r in range(world)]
                assert seen[i].tolist() == want, (rep, i, seen[i].tolist(), want)
    torch.cuda.current_stream().wait_stream(side)
    assert int(status.item()) == 0

    # FP32 rows through the same gather: sharded equals unsharded bit for bit.
    hq32, hkv32, len32 = 16, 8, 512
    q32 = torch.from_numpy(rng.standard_normal((1, hq32, d), dtype=np.float32)).to(dev)
    k32 = torch.from_numpy(rng.standard_normal((1, len32, hkv32, d), dtype=np.float32)).to(dev)
    v32 = torch.from_numpy(rng.standard_normal((1, len32, hkv32, d), dtype=np.float32)).to(dev)
    ws32 = torch.empty(hq32 * 4 * len32, dtype=torch.float32, device=dev)
    full32 = torch.zeros(1, hq32, d, dtype=torch.float32, device=dev)
    gqa.decode(q32, k32, v32, full32, num_kv_heads=hkv32, layout=gqa.layout_reference(1, len32, hkv32),
               seq_lens=[len32], workspace=ws32, split_keys=64)
    pq32, pkv32 = hq32 // world, hkv32 // world
    out32 = torch.zeros(1, pq32, d, dtype=torch.float32, device=dev)
    gathered32 = torch.zeros(world, 1, pq32, d, dtype=torch.float32, device=dev)
    gqa.decode_sharded(comm, gathered32, q32[:, rank * pq32:(rank + 1) * pq32].contiguous(),
                       k32[:, :, rank * pkv32:(rank + 1) * pkv32].contiguous(),
                       v32[:, :, rank * pkv32:(rank + 1) * pkv32].contiguous(), out32,
                       num_kv_heads=pkv32, layout=gqa.layout_reference(1, len32, pkv32),
                       seq_lens=[len32], workspace=ws32, split_keys=64)
    torch.cuda.synchronize()
    whole32 = sharding.unshard_output(gathered32)
    assert torch.equal(whole32.view(torch.int32), full32.view(torch.int32)), "fp32 sharded != unsharded"

    # Output projection behind attention: every rank multiplies its own heads' columns and the
    # per-KV-head sums travel through the peer windows. Every rank ends with the complete
    # residual, bit-equal to the unsharded result.
    hidden, tokens = 256, 3
    attn = H.rand_bits(rng, (tokens, hq, d))
    w_o = cases.to_bf16_bits(rng.standard_normal((hidden, hq * d), dtype=np.float32) / np.float32(90.0))
    res0 = H.rand_bits(rng, (tokens, hidden))
    want_res = H.bf16_tensor(res0, dev).clone()
    gqa.oproj_residual(H.bf16_tensor(attn, dev), H.bf16_tensor(w_o, dev), want_res, num_kv_heads=hkv,
                       workspace=gqa.oproj_workspace(hidden, hkv, dev))
    w_dev = H.bf16_tensor(w_o, dev)
    attn_l = H.bf16_tensor(np.ascontiguousarray(attn[:, rank * per_q:(rank + 1) * per_q]), dev)
    ws_l = gqa.oproj_workspace(hidden, per_kv, dev)
    for _ in range(3):  # consecutive steps alternate between the two halves of the windows
        got_res = H.bf16_tensor(res0, dev).clone()
        gqa.oproj_residual(attn_l, w_dev[:, rank * per_q * d:], got_res, num_kv_heads=per_kv,
                           workspace=ws_l, comm=comm, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got_res.view(torch.int16), want_res.view(torch.int16)), "sharded o-proj"
    want_np = oracle.gemv_add(attn.reshape(tokens, -1), w_o, res0, accum=1)
    assert not H.bf16_mismatches(H.bits_of(got_res), want_np).any()

    # Sequence-parallel: every rank holds all heads and every world-th block of each sequence;
    # the combine kernel merges the ranks' records. Every rank gets the same bits, and they
    # agree with the oracle on the whole sequences.
    sp_lens = [3000, 200, 2048]  # rank 1 and up hold no key of the second sequence
    local_rows, local_lens = sharding.sequence_slice(sp_lens, table, block_tokens, world, rank)
    local_tab = np.array(local_rows, dtype=np.int32)
    layout_sp = gqa.layout_pool(num_blocks, block_tokens, hkv)
    dq_sp, dk_sp, dv_sp = H.bf16_tensor(q, dev), H.bf16_tensor(k_pool, dev), H.bf16_tensor(v_pool, dev)
    ws_sp = gqa.binding.workspace_for(batch, hq, hkv, dev)
    for split_keys in (0, 512):
        out_sp = torch.zeros(batch, hq, d, dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            gqa.decode_seqpar(comm, dq_sp, dk_sp, dv_sp, out_sp, num_kv_heads=hkv, layout=layout_sp,
                              seq_lens=local_lens,
                              seq_lens_dev=torch.tensor(local_lens, dtype=torch.int32, device=dev),
                              block_table=torch.from_numpy(local_tab).to(dev), workspace=ws_sp,
                              split_keys=split_keys, status=status)
            torch.cuda.synchronize()
        assert int(status.item()) == 0
        want_sp = oracle.gqa_decode(q, k_pool.reshape(-1), v_pool.reshape(-1), sp_lens, hkv=hkv,
                                    stride_block=hkv * block_tokens * d, stride_token=d,
                                    stride_head=block_tokens * d, block_tokens=block_tokens,
                                    block_table=table)
        abs_err, rel_err = H.errors(out_sp.float().cpu().numpy(), want_sp)
        assert abs_err <= 2e-2 and rel_err <= 1e-2, ("sequence-parallel", split_keys, abs_err, rel_err)
        sp_bits = [None] * world
        dist.all_gather_object(sp_bits, H.bits_of(out_sp).tobytes())
        assert all(x == sp_bits[0] for x in sp_bits), "ranks disagree on the merged output"

    # The same in FP32 on contiguous parts of a reference-layout cache (the narrow combine grid
    # takes the kernel's other width).
    part = len32 // world
    sl = slice(rank * part, (rank + 1) * part)
    out_sp32 = torch.zeros(1, hq32, d, dtype=torch.float32, device=dev)
    gqa.decode_seqpar(comm, q32, k32[:, sl].contiguous(), v32[:, sl].contiguous(), out_sp32,
                      num_kv_heads=hkv32, layout=gqa.layout_reference(1, part, hkv32),
                      seq_lens=[part], workspace=ws32, split_keys=32, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rel32 = ((out_sp32 - full32).abs().max() / full32.abs().max()).item()
    assert rel32 <= 1e-5, rel32
    sp32_bits = [None] * world
    dist.all_gather_object(sp32_bits, out_sp32.cpu().numpy().tobytes())
    assert all(x == sp32_bits[0] for x in sp32_bits), "ranks disagree on the FP32 merged output"

    # The host-buffer step with the gather inside.
    layout_l = gqa.layout_pool(num_blocks, block_tokens, per_kv)
    session = gqa.Session(batch, per_q, per_kv, blocks_per_seq * block_tokens)
    pin = lambda bits: torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).pin_memory()
    k_new, v_new = H.rand_bits(rng, (batch, hkv, d)), H.rand_bits(rng, (batch, hkv, d))
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(256, dtype=np.float32))
    out_host = torch.zeros(world, batch, per_q, d, dtype=torch.bfloat16).pin_memory()
    dk, dv = H.bf16_tensor(k_l, dev), H.bf16_tensor(v_l, dev)
    session.step(pin(q_l), pin(k_new[:, rank * per_kv:(rank + 1) * per_kv]),
                 pin(v_new[:, rank * per_kv:(rank + 1) * per_kv]), H.bf16_tensor(w, dev), dk, dv,
                 layout_l, lens, out_host, block_table=torch.from_numpy(table).to(dev), comm=comm)
    session.close()
    gathered_bits = out_host.view(torch.int16).numpy().view(np.uint16)
    all_bits = [None] * world
    dist.all_gather_object(all_bits, gathered_bits.tobytes())
    assert all(b == all_bits[0] for b in all_bits), "ranks disagree on the gathered output"
    assert np.isfinite(out_host.float().numpy()).all()

    comm.close()
    dist.destroy_process_group()
    if rank == 0:
        print("multi_gpu_worker ok")


if __name__ == "__main__":
    main()
