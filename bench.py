"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode-layer pass over one batch: QK-Norm + RoPE + KV append for the new
token, attention over the whole KV cache and, on N > 1 GPUs, the all-gather of the output.
The headline workload is the Qwen3-32B-shaped long-context case: 64 query / 8 KV heads,
head_dim 128, batch 4, 131072 cached positions per sequence, BF16, the cache paged in
256-token pool blocks; KV heads are split over the N GPUs (strong scaling). All inputs are
seeded synthetic N(0, 1) tensors.

Rank 0 prints one JSON line: `value` is microseconds per layer with everything resident in
HBM (CUDA-graph replay of K steps, CUDA events, max over ranks); `e2e` is the same through
gqa_session_step with host buffers (H2D of the new token's rows, kernels, D2H of the output,
every step); `roofline` is for the streaming attention kernels alone; `cpu_baseline` times the
CPU oracle on a bounded sample of the same workload.

--impl reference times the reference's CPU attention path, restated in oracle/gqa_oracle.c
(the reference's own CPU sources need Armadillo and glog, which are not installed, and its
score computation is commented out), with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HEAD_DIM = 128
BLOCK_TOKENS = 256
MIN_RESIDENT_BYTES = 1 << 30  # distinct KV bytes cycled per GPU, several times the 126 MB L2


def _ragged_lengths(batch: int = 16, lo: int = 256, hi: int = 8192, seed: int = 20260614 + 4):
    import random
    rnd = random.Random(seed)
    return [rnd.randint(lo, hi) for _ in range(batch)]


# name: (query heads, kv heads, per-sequence cached lengths, cache layout, dtype)
WORKLOADS = {
    "qwen3-32b-bf16-b4-ctx131072": (64, 8, [131072] * 4, "pool", "bf16"),
    "qwen3-32b-bf16-b1-ctx131072": (64, 8, [131072], "pool", "bf16"),
    "qwen3-8b-bf16-b16-ragged256-8192": (32, 8, _ragged_lengths(), "pool", "bf16"),
    "qwen3-4b-bf16-b1-ctx32768": (32, 8, [32768], "reference", "bf16"),
    "qwen3-4b-bf16-b1-ctx1024": (32, 8, [1024], "reference", "bf16"),
    "qwen3-0.6b-f32-b1-ctx512": (16, 8, [512], "reference", "f32"),
}
DEFAULT_WORKLOAD = "qwen3-32b-bf16-b4-ctx131072"
# Rows of the output projection (the model's hidden size), by model name prefix.
HIDDEN = {"qwen3-32b": 5120, "qwen3-8b": 4096, "qwen3-4b": 2560, "qwen3-0.6b": 1024}


def algorithmic_bytes(hq: int, hkv: int, lens, elem: int = 2) -> int:
    """K and V read once per KV head, q read, out written."""
    return sum(2 * l * hkv * HEAD_DIM * elem for l in lens) + 2 * len(lens) * hq * HEAD_DIM * elem


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs.

    Reads through NVML (read-only queries, about every millisecond, so that even a timed
    region of a few milliseconds is covered); falls back to polling nvidia-smi.
    """

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40),
               ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.index = index
        self.clocks = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None

    def _nvml_loop(self, nvml, handle):
        while not self._stop.is_set():
            try:
                self.clocks.append(float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)))
                mask = nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                for name, bit in self.REASONS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(0.001)

    def _smi_loop(self):
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={fields}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        names = [n for n, _ in self.REASONS]
        while not self._stop.is_set():
            line = proc.stdout.readline()
            if not line:
                break
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                self.clocks.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:]):
                if flag.lower().startswith("active"):
                    self.reasons.add(name)
        proc.terminate()

    def __enter__(self):
        try:
            import pynvml as nvml
            nvml.nvmlInit()
            # NVML counts physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices.
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in visible.split(",") if v.strip().isdigit()]
            physical = int(ids[self.index]) if self.index < len(ids) else self.index
            handle = nvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._nvml_loop, args=(nvml, handle), daemon=True)
        except Exception:
            self._thread = threading.Thread(target=self._smi_loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=3)

    def summary(self) -> dict:
        clocks = sorted(self.clocks)
        # The clock under load: idle samples before and after the region sit at the low end.
        busy = clocks[len(clocks) // 2:] if clocks else []
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(clocks)}


# DRAM traffic per algorithmic byte of the streaming kernel, from one ncu capture
# (profiles/ncu_full_gqa_decode_stream_bf16_b1_ctx131072.md: 536.94 MB read + 3.83 MB written
# for 536.90 MB algorithmic). Traffic grows in proportion to the keys processed, so the
# capture of the batch-1 case is scaled by the algorithmic bytes of the workload timed here.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = (536.942336 + 3.828480) / 536.903680


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU attention on a bounded sample
# ---------------------------------------------------------------------------------------------
def cpu_sample_us_per_layer(hq: int, hkv: int, lens, reps: int, warmup: int) -> dict:
    """Times the longest sequence (all heads) on all host threads and scales by total keys."""
    batch = len(lens)
    length = max(lens)
    scale = sum(lens) / length
    import numpy as np
    from oracle import oracle

    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import cases

    rng = np.random.default_rng(5)
    sample_len = length
    kv_dim = hkv * HEAD_DIM

    def normal_bf16(n: int) -> "np.ndarray":
        out = np.empty(n, dtype=np.uint16)
        piece = 1 << 24
        for start in range(0, n, piece):
            m = min(piece, n - start)
            out[start:start + m] = cases.to_bf16_bits(rng.standard_normal(m, dtype=np.float32))
        return out

    k = normal_bf16(sample_len * kv_dim)
    v = normal_bf16(sample_len * kv_dim)
    q = normal_bf16(hq * HEAD_DIM).reshape(1, hq, HEAD_DIM)
    threads = oracle.use_all_cores()
    times = []
    for i in range(warmup + reps):
        t0 = time.perf_counter()
        oracle.gqa_decode(q, k, v, [sample_len], hkv=hkv, stride_block=sample_len * kv_dim,
                          stride_token=kv_dim, stride_head=HEAD_DIM, block_tokens=sample_len,
                          accum=0, threads=0)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    per_seq = sum(times) / len(times)
    return {"value": per_seq * scale * 1e6, "unit": "us/layer", "cores": threads, "kind": "port",
            "sample": f"1 of {batch} sequences ({hq} q heads, {hkv} kv heads, {sample_len} keys, "
                      f"FP32 math on BF16-rounded values), all {threads} host threads, scaled "
                      f"x{scale:.3g} by key count",
            "seconds_per_sample": per_seq}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    hq, hkv, lens, _, _ = WORKLOADS[args.workload]
    batch, length = len(lens), max(lens)
    steps = max(1, min(args.steps, 5))
    res = cpu_sample_us_per_layer(hq, hkv, lens, reps=steps, warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "gqa_decode_attn_us_per_layer", "value": res["value"],
        "unit": "us/layer", "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": res["value"] / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "num_q_heads": hq, "num_kv_heads": hkv,
                   "batch": batch, "kv_len": length, "note": "CPU oracle port of the reference's "
                   "FP32 CPU attention; each step is the bounded sample described in cpu_baseline"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "us/layer", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import llminfer_b200 as gqa

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        ident = [gqa.ShardComm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        comm = gqa.ShardComm(ident[0], world, rank)
        if args.gather == "peer":
            # Needs CUDA IPC between the ranks' processes; every rank falls back to NCCL
            # together if any of them cannot set it up.
            try:
                comm.enable_peer_gather(4 << 20)
                ok = 1
            except gqa.GqaError:
                ok = 0
            flag = torch.tensor([ok], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                args.gather = "nccl"
                comm.disable_peer_gather()

    hq_total, hkv_total, lens, layout_kind, dtype_name = WORKLOADS[args.workload]
    batch = len(lens)
    seq_parallel = args.partition == "sequence" and world > 1
    if seq_parallel:
        # Every rank holds all heads and 1/world of every sequence's keys (whole chunks).
        if not args.attn_only or args.gather != "peer":
            raise SystemExit("--partition sequence needs --attn-only and the peer windows")
        hq, hkv = hq_total, hkv_total
        lens = [max(32, l // world // 32 * 32) for l in lens]
    else:
        shard = gqa.shard_plan(hq_total, hkv_total, world, rank)
        hq, hkv = shard["num_local_q_heads"], shard["num_local_kv_heads"]
    tdtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    elem = 2 if dtype_name == "bf16" else 4
    gen = torch.Generator(device=dev)
    gen.manual_seed(20260614 + rank)

    def randn_fill(t: "torch.Tensor") -> None:
        flat, piece = t.view(-1), 1 << 26
        for start in range(0, flat.numel(), piece):
            n = min(piece, flat.numel() - start)
            flat[start:start + n] = torch.randn(n, device=dev, generator=gen).to(tdtype)

    positions = [l - 1 for l in lens]  # the new token is the last cached position
    if layout_kind == "pool":
        blocks_per_seq = -(-max(lens) // BLOCK_TOKENS)
        seq_blocks = [-(-l // BLOCK_TOKENS) for l in lens]
        blocks_per_slot = sum(seq_blocks)
        slot_bytes = 2 * blocks_per_slot * hkv * BLOCK_TOKENS * HEAD_DIM * elem
        slots = max(1, -(-MIN_RESIDENT_BYTES // slot_bytes))
        layout = gqa.layout_pool(slots * blocks_per_slot, BLOCK_TOKENS, hkv)
        cache_shape = (slots * blocks_per_slot * hkv * BLOCK_TOKENS * HEAD_DIM,)
        cpu_gen = torch.Generator().manual_seed(7)
        tables = []
        for s_ in range(slots):
            perm = (torch.randperm(blocks_per_slot, generator=cpu_gen) + s_ * blocks_per_slot).tolist()
            table = torch.full((batch, blocks_per_seq), -1, dtype=torch.int32)
            for b, nb in enumerate(seq_blocks):
                table[b, :nb] = torch.tensor([perm.pop() for _ in range(nb)], dtype=torch.int32)
            tables.append(table.to(dev))
        layout_note = f"paged pool, {BLOCK_TOKENS}-token blocks, shuffled block order"
    else:
        assert batch == 1
        max_seq_len = lens[0]
        slot_bytes = 2 * max_seq_len * hkv * HEAD_DIM * elem
        slots = max(1, -(-MIN_RESIDENT_BYTES // slot_bytes))
        if lens[0] <= 1024:
            slots = 36  # the Qwen3-4B layer count: 36 independent caches, one per step
        layout = gqa.layout_reference(slots, max_seq_len, hkv)
        cache_shape = (slots, max_seq_len, hkv * HEAD_DIM)
        blocks_per_seq = 0
        tables = [None] * slots
        layout_note = "reference cache [layer, max_seq_len, kv_dim], one layer per step"
    k_pool = torch.empty(cache_shape, dtype=tdtype, device=dev)
    v_pool = torch.empty(cache_shape, dtype=tdtype, device=dev)
    randn_fill(k_pool)
    randn_fill(v_pool)
    q_raw = torch.randn(batch, hq, HEAD_DIM, device=dev, generator=gen).to(tdtype)
    k_new = torch.randn(batch, hkv, HEAD_DIM, device=dev, generator=gen).to(tdtype)
    v_new = torch.randn(batch, hkv, HEAD_DIM, device=dev, generator=gen).to(tdtype)
    weight = (1.0 + 0.05 * torch.randn(2 * HEAD_DIM, device=dev, generator=gen)).to(torch.bfloat16)
    q_rot = torch.empty_like(q_raw)
    out = torch.empty(batch, hq, HEAD_DIM, dtype=tdtype, device=dev)
    gathered = torch.empty(world, batch, hq, HEAD_DIM, dtype=tdtype, device=dev)
    positions_dev = torch.tensor(positions, dtype=torch.int32, device=dev)
    sin_table = torch.empty(max(lens), HEAD_DIM // 2, dtype=torch.float32, device=dev)
    cos_table = torch.empty_like(sin_table)
    gqa.sin_cos_cache(sin_table, cos_table, HEAD_DIM)
    lens_dev = torch.tensor(lens, dtype=torch.int32, device=dev)
    workspace = gqa.binding.workspace_for(batch, hq, hkv, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    paged = layout_kind == "pool"
    has_front = dtype_name == "bf16"  # the front stage is a BF16 kernel
    plan = gqa.decode_plan(dtype=2 if dtype_name == "bf16" else 1, batch=batch, num_q_heads=hq,
                           num_kv_heads=hkv, layout=layout, seq_lens=lens, paged=paged,
                           blocks_per_seq=blocks_per_seq, device_lens=paged,
                           sm_count=torch.cuda.get_device_properties(dev).multi_processor_count,
                           workspace_bytes=workspace.numel() * 4)

    def attention(slot: int) -> None:
        # Ahead of each attention call are the front stage (writes the newest rows only) and
        # the previous layer's kernels (other caches): older rows may be prefetched early.
        kw = dict(num_kv_heads=hkv, layout=layout, seq_lens=lens, workspace=workspace,
                  status=status, early_prefetch=True)
        if paged:
            kw.update(seq_lens_dev=lens_dev, block_table=tables[slot])
        else:
            kw.update(fixed_block=slot)
        q_in = q_rot if has_front else q_raw
        if comm is None:
            gqa.decode(q_in, k_pool, v_pool, out, **kw)
        elif seq_parallel:
            gqa.decode_seqpar(comm, q_in, k_pool, v_pool, out, **kw)
        else:
            gqa.decode_sharded(comm, gathered, q_in, k_pool, v_pool, out, **kw)

    def step(slot: int) -> None:
        if has_front:
            kw = dict(block_table=tables[slot], positions_dev=positions_dev) if paged else dict(
                fixed_block=slot)
            gqa.qk_norm_rope_append(q_raw, k_new, v_new, weight, k_pool, v_pool, layout=layout,
                                    positions=positions, q_out=q_rot, sin_cache=sin_table,
                                    cos_cache=cos_table, **kw)
        attention(slot)

    def barrier() -> None:
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_graph(fn, steps: int, warmup: int) -> float:
        """Warm-up eagerly, capture `steps` calls in one CUDA graph, time one replay."""
        for i in range(warmup):
            fn(i % slots)
        barrier()
        if args.no_graph:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(steps):
                fn(i % slots)
            stop.record()
            barrier()
            return max_over_ranks(start.elapsed_time(stop))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(steps):
                fn(i % slots)
        graph.replay()  # untimed: first replay uploads the graph
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        barrier()
        return max_over_ranks(start.elapsed_time(stop))

    steps, warmup = args.steps, max(args.warmup, 3)
    with ClockSampler(local_rank) as clocks:
        total_ms = timed_graph(step, steps, warmup)
        attn_ms = timed_graph(attention, steps, warmup)
    clock_info = clocks.summary()
    us_per_layer = total_ms * 1e3 / steps
    attn_us = attn_ms * 1e3 / steps
    assert int(status.item()) == 0, "a bounded device wait ran out"

    # ---- the step behind attention: output projection + residual ---------------------------
    # Reported beside the headline, never inside it. Weights are cycled over more copies than
    # L2 holds; sharded runs exchange the per-KV-head sums through the peer windows.
    oproj_info = None
    qkv_info = None
    if dtype_name == "bf16" and (comm is None or args.gather == "peer") and not seq_parallel:
        hidden = HIDDEN[args.workload.split("-bf16")[0]]
        weight_bytes = hidden * hq * HEAD_DIM * 2
        copies = max(2, -(-(256 << 20) // weight_bytes))
        o_weights = [torch.randn(hidden, hq * HEAD_DIM, device=dev, dtype=torch.bfloat16) / 64
                     for _ in range(copies)]
        resid = torch.zeros(batch, hidden, dtype=torch.bfloat16, device=dev)
        o_ws = gqa.oproj_workspace(hidden, hkv, dev)
        calls = [0]

        def oproj(_slot: int) -> None:
            gqa.oproj_residual(out, o_weights[calls[0] % copies], resid, num_kv_heads=hkv,
                               workspace=o_ws, comm=comm, status=status)
            calls[0] += 1

        torch.cuda.synchronize()
        o_us = timed_graph(oproj, steps, warmup) * 1e3 / steps
        assert int(status.item()) == 0, "a bounded device wait ran out"
        peak_gbs, _ = measured_peak_gbs()
        o_gbs = weight_bytes / (o_us * 1e-6) / 1e9
        oproj_info = {"us_per_layer": o_us, "hidden": hidden, "weight_bytes_per_gpu": weight_bytes,
                      "achieved_gbs": o_gbs, "frac_of_measured_peak": o_gbs / peak_gbs,
                      "exchange": "per-KV-head sums over the peer windows" if comm else "none"}
        del o_weights

        # The step in front: packed QKV projection of this rank's heads (nothing to exchange).
        rows = (hq + 2 * hkv) * HEAD_DIM
        qkv_bytes = rows * hidden * 2
        copies = max(2, -(-(256 << 20) // qkv_bytes))
        qkv_weights = [torch.randn(rows, hidden, device=dev, dtype=torch.bfloat16) / 64
                       for _ in range(copies)]
        x_in = torch.randn(batch, hidden, device=dev, dtype=torch.bfloat16)
        qkv_ws = gqa.qkv_workspace(hidden, hq, hkv, dev)
        q_tmp = torch.empty(batch, hq, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        k_tmp = torch.empty(batch, hkv, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        v_tmp = torch.empty_like(k_tmp)

        def qkv(_slot: int) -> None:
            gqa.qkv_gemv(x_in, qkv_weights[calls[0] % copies], q_tmp, k_tmp, v_tmp,
                         workspace=qkv_ws, status=status)
            calls[0] += 1

        torch.cuda.synchronize()
        qkv_us = timed_graph(qkv, steps, warmup) * 1e3 / steps
        assert int(status.item()) == 0, "a bounded device wait ran out"
        qkv_gbs = qkv_bytes / (qkv_us * 1e-6) / 1e9
        qkv_info = {"us_per_layer": qkv_us, "hidden": hidden, "weight_bytes_per_gpu": qkv_bytes,
                    "achieved_gbs": qkv_gbs, "frac_of_measured_peak": qkv_gbs / peak_gbs}
        del qkv_weights

    # ---- end to end through the host-buffer entry point -----------------------------------
    if args.attn_only:
        peak, peak_kind = measured_peak_gbs()
        achieved = algorithmic_bytes(hq, hkv, lens, elem) / (attn_us * 1e-6) / 1e9
        if rank == 0:
            print(json.dumps({"attention_only_us_per_layer": attn_us, "us_per_layer": us_per_layer,
                              "roofline": {"achieved": achieved, "frac": achieved / peak},
                              "plan": plan}))
        if comm is not None:
            comm.close()
            dist.destroy_process_group()
        return
    if not has_front:
        raise SystemExit("the end-to-end leg needs the BF16 front stage; use --attn-only")
    session = gqa.Session(batch, hq, hkv, max(lens))
    pin = lambda t: t.cpu().pin_memory()
    q_host, k_host, v_host = pin(q_raw), pin(k_new), pin(v_new)
    out_host = torch.empty(world if comm else 1, batch, hq, HEAD_DIM, dtype=torch.bfloat16).pin_memory()
    def e2e_step(i: int) -> None:
        session.step(q_host, k_host, v_host, weight, k_pool, v_pool, layout, positions,
                     out_host, block_table=tables[i % slots],
                     fixed_block=0 if paged else i % slots, comm=comm)
    for i in range(warmup):
        e2e_step(i)
    barrier()
    with ClockSampler(local_rank) as e2e_clocks:
        t0 = time.perf_counter()
        for i in range(steps):
            e2e_step(i)
        barrier()
        e2e_us = max_over_ranks((time.perf_counter() - t0) * 1e3) * 1e3 / steps
    session.close()
    e2e_clock_info = e2e_clocks.summary()
    clock_info["reasons"] = sorted(set(clock_info["reasons"]) | set(e2e_clock_info["reasons"]))
    clock_info["samples_e2e"] = e2e_clock_info["samples"]
    h2d = (hq + 2 * hkv) * HEAD_DIM * 2 * batch + 8 * batch
    d2h = out_host.numel() * 2

    # Front stage, streaming kernel, combine; the gather is a fourth launch unless the combine
    # kernel carries it (peer gather, split units, every combine CTA resident at once).
    peer = comm is not None and args.gather == "peer"
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    fused_gather = (peer and plan["needs_combine"] and batch * hq <= min(160, sms)
                    and os.environ.get("GQA_FUSED_GATHER", "1")[:1] != "0")
    launches_per_step = 3 + (1 if world > 1 and not fused_gather else 0)
    gather_note = ""
    if world > 1:
        gather_note = (", peer-store all-gather over NVLink inside the combine kernel"
                       if fused_gather else f", {args.gather} all-gather over NVLink")

    peak, peak_kind = measured_peak_gbs()
    rank_bytes = algorithmic_bytes(hq, hkv, lens, elem)
    achieved = rank_bytes / (attn_us * 1e-6) / 1e9
    line = {
        "metric": "gqa_decode_attn_us_per_layer", "value": us_per_layer, "unit": "us/layer",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": us_per_layer / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": args.workload, "num_q_heads": hq_total, "num_kv_heads": hkv_total,
                   "head_dim": HEAD_DIM, "batch": batch, "kv_len": max(lens),
                   "kv_len_total": sum(lens), "kv_layout": layout_note,
                   "parallelism": f"kv-head-parallel x{world}",
                   "l2": f"inputs larger than L2: {slots} cache slot(s) of "
                         f"{slot_bytes / 2**20:.0f} MiB cycled per GPU",
                   "step": "qk-norm+rope+append, split attention, lse combine"
                           + gather_note,
                   "split_chunks": plan["split_chunks"], "ctas": plan["num_ctas"],
                   "items": plan["num_items"]},
        "hbm_tbs_aggregate": achieved * world / 1e3,
        "attention_only_us_per_layer": attn_us,
        "roofline": {"bound": "hbm", "kernel": "gqa_decode_stream_bf16 (+ lse combine)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "frac_of_8tbs_nominal": achieved / 8000.0,
                     "algorithmic_bytes_per_launch": rank_bytes,
                     "traffic": int(rank_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE),
                     "traffic_source": "ncu capture of the batch-1 case, scaled by bytes"},
        "e2e": {"value": e2e_us, "unit": "us/layer", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * steps,
        "next_rows": {"oproj_residual": oproj_info, "qkv_gemv": qkv_info},
        "clocks": clock_info,
    }
    if rank == 0 and world == 1 and args.sweep:
        # The other BASELINE configurations, attention kernels only, each in its own process.
        sweep = {}
        for name in WORKLOADS:
            if name == args.workload:
                continue
            run = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", name,
                                  "--attn-only", "--no-cpu", "--steps", str(steps)],
                                 capture_output=True, text=True)
            try:
                got = json.loads(run.stdout.strip().splitlines()[-1])
                sweep[name] = {"attention_only_us_per_layer": got["attention_only_us_per_layer"],
                               "gbs": got["roofline"]["achieved"]}
            except (IndexError, ValueError, KeyError):
                sweep[name] = {"error": run.stderr[-200:]}
        line["context_sweep"] = sweep
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_sample_us_per_layer(hq_total, hkv_total, lens, reps=2, warmup=1)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        print(json.dumps(line))
    if comm is not None:
        comm.close()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=tuple(WORKLOADS), default=DEFAULT_WORKLOAD)
    ap.add_argument("--gather", choices=("peer", "nccl"), default="peer",
                    help="N > 1: gather the output with peer stores over NVLink or with NCCL")
    ap.add_argument("--partition", choices=("heads", "sequence"), default="heads",
                    help="N > 1: KV heads per GPU (default) or a slice of every sequence per GPU")
    ap.add_argument("--sweep", action="store_true",
                    help="N = 1: also time the attention kernels on the other workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager launches instead of a CUDA-graph replay (profiler runs)")
    ap.add_argument("--attn-only", action="store_true",
                    help="tuning runs: skip the end-to-end and CPU legs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
