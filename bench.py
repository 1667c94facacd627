"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode-layer pass over one batch: QK-Norm + RoPE + KV append for the new
token, attention over the whole KV cache and, on N > 1 GPUs, the all-gather of the output.
The headline workload is the Qwen3-32B-shaped long-context case: 64 query / 8 KV heads,
head_dim 128, batch 4, 131072 cached positions per sequence, BF16, the cache paged in
256-token pool blocks; KV heads are split over the N GPUs (strong scaling). All inputs are
seeded synthetic N(0, 1) tensors.

Rank 0 prints one JSON line: `value` is microseconds per layer with everything resident in
HBM: a CUDA graph of K steps is replayed many times (at least half a second of timed region at
N = 1, at least 100 replays at N > 1), every replay timed with CUDA events, max over ranks per
replay, and `value` is the median over the replays (`stats` carries the minimum as well).
`e2e` is the same through gqa_session_step with host buffers (H2D of the new token's rows,
kernels, D2H of the output, every step; median per step); `roofline` is for the streaming
attention kernels alone; `cpu_baseline` times the CPU oracle on a bounded sample of the same
workload, on all host threads and on one. `context_sweep` (N = 1) carries the other contexts of
the metric (1K x 36 layer caches, 32K, the ragged paged batch, the FP32 case) measured the same
way; `reference_cuda_kernel` the reference's own CUDA kernels on this GPU when the checker
library built from the reference checkout is present. `parity` checks the values behind the
numbers: the gathered output equal on every rank, one (sequence, KV head) unit against the FP64
oracle, and at N > 1 a small case sharded bit-equal to unsharded plus sequence-parallel decode
against the oracle; a failed check ends the run with a non-zero exit code.

--impl reference times the reference's CPU attention path, restated in oracle/gqa_oracle.c
(the reference's own CPU sources need Armadillo and glog, which are not installed, and its
score computation is commented out), with all host threads; every step is a bounded sample of
the workload (a slice of one sequence's keys, all heads), scaled by key count.
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
# (profiles/ncu_full_gqa_decode_stream_bf16_b1_ctx131072.md: 536.96 MB read + 3.60 MB written
# for 536.90 MB algorithmic). Traffic grows in proportion to the keys processed, so the
# capture of the batch-1 case is scaled by the algorithmic bytes of the workload timed here.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = (536.962816 + 3.600384) / 536.903680


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"




def median(values) -> float:
    vals = sorted(values)
    n = len(vals)
    return vals[n // 2] if n % 2 else 0.5 * (vals[n // 2 - 1] + vals[n // 2])


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU attention on a bounded sample
# ---------------------------------------------------------------------------------------------
class CpuSample:
    """A slice of one sequence of the workload (all heads, `keys` cached positions) for the CPU
    oracle; one call of run() is one bounded sample, scaled to the whole workload by key count."""

    def __init__(self, hq: int, hkv: int, lens, keys: int):
        import numpy as np
        from oracle import oracle

        sys.path.insert(0, str(ROOT / "tests" / "golden"))
        import cases

        self.oracle, self.hq, self.hkv = oracle, hq, hkv
        self.keys = min(keys, max(lens))
        self.scale = sum(lens) / self.keys
        self.batch = len(lens)
        rng = np.random.default_rng(5)
        kv_dim = hkv * HEAD_DIM

        def normal_bf16(n: int):
            out = np.empty(n, dtype=np.uint16)
            piece = 1 << 24
            for start in range(0, n, piece):
                m = min(piece, n - start)
                out[start:start + m] = cases.to_bf16_bits(rng.standard_normal(m, dtype=np.float32))
            return out

        self.k = normal_bf16(self.keys * kv_dim)
        self.v = normal_bf16(self.keys * kv_dim)
        self.q = normal_bf16(hq * HEAD_DIM).reshape(1, hq, HEAD_DIM)

    def run(self, threads: int) -> float:
        """Seconds for one sample on `threads` host threads (0 = all)."""
        kv_dim = self.hkv * HEAD_DIM
        t0 = time.perf_counter()
        self.oracle.gqa_decode(self.q, self.k, self.v, [self.keys], hkv=self.hkv,
                               stride_block=self.keys * kv_dim, stride_token=kv_dim,
                               stride_head=HEAD_DIM, block_tokens=self.keys, accum=0,
                               threads=threads)
        return time.perf_counter() - t0

    def describe(self, threads: int) -> str:
        return (f"{self.keys} keys of 1 of {self.batch} sequences ({self.hq} q heads, {self.hkv} kv "
                f"heads, FP32 math on BF16-rounded values), {threads} host thread(s), scaled "
                f"x{self.scale:.4g} by key count")


def cpu_rows(hq: int, hkv: int, lens, budget_s: float = 12.0) -> dict:
    """cpu_baseline (all host threads) and cpu_baseline_1thread for the bench line: each a
    bounded sample sized from a probe so that it takes a few seconds."""
    from oracle import oracle
    threads = oracle.use_all_cores()
    probe = CpuSample(hq, hkv, lens, 4096)
    probe.run(0)
    per_key_all = min(probe.run(0) for _ in range(2)) / probe.keys
    per_key_one = probe.run(1) / probe.keys
    rows = {}
    for name, nthreads, per_key in (("cpu_baseline", 0, per_key_all),
                                    ("cpu_baseline_1thread", 1, per_key_one)):
        keys = int(max(4096, min(max(lens), budget_s / 3 / per_key)))
        sample = CpuSample(hq, hkv, lens, keys // 32 * 32)
        sample.run(nthreads)
        best = min(sample.run(nthreads) for _ in range(2))
        used = threads if nthreads == 0 else 1
        rows[name] = {"value": best * sample.scale * 1e6, "unit": "us/layer", "cores": used,
                      "kind": "port", "sample": sample.describe(used)}
    return rows


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    hq, hkv, lens, _, _ = WORKLOADS[args.workload]
    batch, length = len(lens), max(lens)
    threads = oracle.use_all_cores()
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    # Every step is one bounded sample: sized from a probe so that warm-up and timed steps
    # together take about a minute, whatever --steps asks for.
    probe = CpuSample(hq, hkv, lens, 4096)
    probe.run(0)
    per_key = min(probe.run(0) for _ in range(2)) / probe.keys
    keys = int(max(2048, min(length, 60.0 / (steps + warmup) / per_key))) // 32 * 32
    sample = CpuSample(hq, hkv, lens, keys)
    for _ in range(warmup):
        sample.run(0)
    times = [sample.run(0) for _ in range(steps)]
    value = median(times) * sample.scale * 1e6
    line = {
        "impl": "reference", "metric": "gqa_decode_attn_us_per_layer", "value": value,
        "unit": "us/layer", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": value / 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "num_q_heads": hq, "num_kv_heads": hkv,
                   "head_dim": HEAD_DIM, "batch": batch, "kv_len": length,
                   "kv_len_total": sum(lens),
                   "note": "CPU oracle port of the reference's FP32 CPU attention; each step is "
                           "the bounded sample described in cpu_baseline; value = median step"},
        "stats": {"median_us": value, "min_us": min(times) * sample.scale * 1e6,
                  "samples": len(times)},
        "cpu_baseline": {"value": value, "unit": "us/layer", "cores": threads, "kind": "port",
                         "sample": sample.describe(threads)},
        "e2e": {"value": value, "unit": "us/layer", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Workload:
    """One named workload on this rank's GPU: caches, the new token's rows, and the closures
    that launch one decode-layer step over cache slot `slot` (several slots are cycled so that
    the K/V a step reads were not left in L2 by the step before)."""

    def __init__(self, gqa, name, world, rank, dev, comm, args):
        import torch
        self.gqa, self.name, self.world, self.comm, self.dev = gqa, name, world, comm, dev
        hq_total, hkv_total, lens, layout_kind, dtype_name = WORKLOADS[name]
        self.hq_total, self.hkv_total, self.dtype_name = hq_total, hkv_total, dtype_name
        self.batch = batch = len(lens)
        self.seq_parallel = args.partition == "sequence" and world > 1
        if self.seq_parallel:
            # Every rank holds all heads and 1/world of every sequence's keys (whole chunks).
            hq, hkv = hq_total, hkv_total
            lens = [max(32, l // world // 32 * 32) for l in lens]
        else:
            shard = gqa.shard_plan(hq_total, hkv_total, world, rank)
            hq, hkv = shard["num_local_q_heads"], shard["num_local_kv_heads"]
        self.hq, self.hkv, self.lens = hq, hkv, lens
        tdtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
        self.elem = elem = 2 if dtype_name == "bf16" else 4
        gen = torch.Generator(device=dev)
        gen.manual_seed(20260614 + rank)

        def randn_fill(t):
            flat, piece = t.view(-1), 1 << 26
            for start in range(0, flat.numel(), piece):
                n = min(piece, flat.numel() - start)
                flat[start:start + n] = torch.randn(n, device=dev, generator=gen).to(tdtype)

        self.positions = [l - 1 for l in lens]  # the new token is the last cached position
        self.paged = layout_kind == "pool"
        if self.paged:
            self.blocks_per_seq = -(-max(lens) // BLOCK_TOKENS)
            seq_blocks = [-(-l // BLOCK_TOKENS) for l in lens]
            blocks_per_slot = sum(seq_blocks)
            self.slot_bytes = 2 * blocks_per_slot * hkv * BLOCK_TOKENS * HEAD_DIM * elem
            self.slots = max(1, -(-MIN_RESIDENT_BYTES // self.slot_bytes))
            self.layout = gqa.layout_pool(self.slots * blocks_per_slot, BLOCK_TOKENS, hkv)
            cache_shape = (self.slots * blocks_per_slot, hkv, BLOCK_TOKENS, HEAD_DIM)
            cpu_gen = torch.Generator().manual_seed(7)
            self.tables = []
            for s_ in range(self.slots):
                perm = (torch.randperm(blocks_per_slot, generator=cpu_gen) + s_ * blocks_per_slot).tolist()
                table = torch.full((batch, self.blocks_per_seq), -1, dtype=torch.int32)
                for b, nb in enumerate(seq_blocks):
                    table[b, :nb] = torch.tensor([perm.pop() for _ in range(nb)], dtype=torch.int32)
                self.tables.append(table.to(dev))
            self.layout_note = f"paged pool, {BLOCK_TOKENS}-token blocks, shuffled block order"
        else:
            assert batch == 1
            max_seq_len = lens[0]
            self.slot_bytes = 2 * max_seq_len * hkv * HEAD_DIM * elem
            self.slots = max(1, -(-MIN_RESIDENT_BYTES // self.slot_bytes))
            if lens[0] <= 1024:
                self.slots = 36  # the Qwen3-4B layer count: 36 independent caches, one per step
            self.layout = gqa.layout_reference(self.slots, max_seq_len, hkv)
            cache_shape = (self.slots, max_seq_len, hkv * HEAD_DIM)
            self.blocks_per_seq = 0
            self.tables = [None] * self.slots
            self.layout_note = "reference cache [layer, max_seq_len, kv_dim], one layer per step"
        self.k_pool = torch.empty(cache_shape, dtype=tdtype, device=dev)
        self.v_pool = torch.empty(cache_shape, dtype=tdtype, device=dev)
        randn_fill(self.k_pool)
        randn_fill(self.v_pool)
        rn = lambda *shape: torch.randn(*shape, device=dev, generator=gen)
        self.q_raw = rn(batch, hq, HEAD_DIM).to(tdtype)
        self.k_new = rn(batch, hkv, HEAD_DIM).to(tdtype)
        self.v_new = rn(batch, hkv, HEAD_DIM).to(tdtype)
        self.weight = (1.0 + 0.05 * rn(2 * HEAD_DIM)).to(torch.bfloat16)
        self.q_rot = torch.empty_like(self.q_raw)
        self.out = torch.empty(batch, hq, HEAD_DIM, dtype=tdtype, device=dev)
        self.gathered = torch.empty(world, batch, hq, HEAD_DIM, dtype=tdtype, device=dev)
        self.positions_dev = torch.tensor(self.positions, dtype=torch.int32, device=dev)
        self.sin_table = torch.empty(max(lens), HEAD_DIM // 2, dtype=torch.float32, device=dev)
        self.cos_table = torch.empty_like(self.sin_table)
        gqa.sin_cos_cache(self.sin_table, self.cos_table, HEAD_DIM)
        self.lens_dev = torch.tensor(lens, dtype=torch.int32, device=dev)
        self.workspace = gqa.binding.workspace_for(batch, hq, hkv, dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.has_front = dtype_name == "bf16"  # the front stage is a BF16 kernel
        self.fused_front = self.has_front and args.front == "fused" and not self.seq_parallel
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.plan = gqa.decode_plan(dtype=2 if dtype_name == "bf16" else 1, batch=batch,
                                    num_q_heads=hq, num_kv_heads=hkv, layout=self.layout,
                                    seq_lens=lens, paged=self.paged,
                                    blocks_per_seq=self.blocks_per_seq, device_lens=self.paged,
                                    sm_count=self.sms, workspace_bytes=self.workspace.numel() * 4)
        self.front = gqa.FusedFront(self.k_new, self.v_new, self.weight, q_out=self.q_rot,
                                    sin_cache=self.sin_table,
                                    cos_cache=self.cos_table) if self.has_front else None

    def bytes_per_step(self) -> int:
        return algorithmic_bytes(self.hq, self.hkv, self.lens, self.elem)

    def attention(self, slot: int, fused: bool = False) -> None:
        """The attention kernels alone on already rotated queries (fused: with the front stage
        inside, on the raw rows). Ahead of each call in the stream are only kernels that write
        other caches or the newest rows, so older rows may be requested early."""
        gqa = self.gqa
        kw = dict(num_kv_heads=self.hkv, layout=self.layout, seq_lens=self.lens,
                  workspace=self.workspace, status=self.status, early_prefetch=True)
        if self.paged:
            kw.update(seq_lens_dev=self.lens_dev, block_table=self.tables[slot])
        else:
            kw.update(fixed_block=slot)
        if fused:
            kw.update(front=self.front)
        q_in = self.q_raw if (fused or not self.has_front) else self.q_rot
        if self.comm is None:
            gqa.decode(q_in, self.k_pool, self.v_pool, self.out, **kw)
        elif self.seq_parallel:
            gqa.decode_seqpar(self.comm, q_in, self.k_pool, self.v_pool, self.out, **kw)
        else:
            gqa.decode_sharded(self.comm, self.gathered, q_in, self.k_pool, self.v_pool, self.out, **kw)

    def step(self, slot: int) -> None:
        """One decode-layer step: QK-Norm + RoPE + KV append, attention, (gather)."""
        if self.fused_front:
            self.attention(slot, fused=True)
            return
        if self.has_front:
            kw = dict(block_table=self.tables[slot], positions_dev=self.positions_dev) if self.paged \
                else dict(fixed_block=slot)
            self.gqa.qk_norm_rope_append(self.q_raw, self.k_new, self.v_new, self.weight,
                                         self.k_pool, self.v_pool, layout=self.layout,
                                         positions=self.positions, q_out=self.q_rot,
                                         sin_cache=self.sin_table, cos_cache=self.cos_table, **kw)
        self.attention(slot)

    def launches_per_step(self, gather: str) -> int:
        """Kernels of this library per step: (front stage,) streaming kernel, combine; the
        gather is one more launch unless the combine kernel carries it."""
        n = 1 + (1 if self.plan["needs_combine"] and not self.cluster_merge() else 0)
        if self.has_front and not self.fused_front:
            n += 1
        if self.world > 1 and not self.seq_parallel and not self.fused_gather(gather):
            n += 1
        return n

    def cluster_merge(self) -> bool:
        """Splits merged inside thread-block clusters by the streaming kernel: no combine launch."""
        return (self.comm is None and self.plan.get("cluster_size", 0) > 0
                and os.environ.get("GQA_CLUSTER_MERGE", "1")[:1] != "0")

    def fused_gather(self, gather: str) -> bool:
        return (self.world > 1 and gather == "peer" and bool(self.plan["needs_combine"])
                and self.batch * self.hq <= min(160, self.sms)
                and os.environ.get("GQA_FUSED_GATHER", "1")[:1] != "0")

    def free(self) -> None:
        for name in ("k_pool", "v_pool", "tables"):
            setattr(self, name, None)


class Timer:
    """CUDA-graph timing shared by every measurement of the GPU arm."""

    def __init__(self, torch, dist, world, dev, no_graph):
        self.torch, self.dist, self.world, self.dev, self.no_graph = torch, dist, world, dev, no_graph

    def barrier(self) -> None:
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def run(self, fn, slots: int, steps: int, warmup: int, min_seconds: float = 0.5,
            min_replays: int = 20, max_replays: int = 400) -> dict:
        """Warm up eagerly, capture `steps` calls of fn in one CUDA graph, replay it until the
        timed region reaches `min_seconds` (between min_replays and max_replays times), every
        replay between its own pair of CUDA events. Returns us per step: median and min over
        the replays, each replay's time being the max over ranks."""
        torch = self.torch
        for i in range(warmup):
            fn(i % slots)
        self.barrier()
        if self.no_graph:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(steps):
                fn(i % slots)
            stop.record()
            self.barrier()
            us = self.max_over_ranks([start.elapsed_time(stop)])[0] * 1e3 / steps
            return {"median_us": us, "min_us": us, "replays": 1, "timed_region_s": us * steps / 1e6}
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(steps):
                fn(i % slots)
        graph.replay()  # untimed: the first replay uploads the graph
        self.barrier()
        probe = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        probe[0].record()
        graph.replay()
        probe[1].record()
        self.barrier()
        est_ms = max(self.max_over_ranks([probe[0].elapsed_time(probe[1])])[0], 1e-3)
        replays = int(min(max_replays, max(min_replays, -(-min_seconds * 1e3 // est_ms))))
        events = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
        events[0].record()
        for r in range(replays):
            graph.replay()
            events[r + 1].record()
        self.barrier()
        per_replay = self.max_over_ranks(
            [events[r].elapsed_time(events[r + 1]) for r in range(replays)])
        us = [ms * 1e3 / steps for ms in per_replay]
        return {"median_us": median(us), "min_us": min(us), "replays": replays,
                "timed_region_s": sum(per_replay) / 1e3}


def unit_against_oracle(w: "Workload", out, slot: int, b: int, hk: int) -> float:
    """Attention output of one (sequence, local KV head) unit of the workload against the FP64
    CPU oracle on the same cache contents; returns the error relative to max|out|, raises when
    the absolute error passes the BF16 tolerance (2e-2)."""
    import numpy as np
    from oracle import oracle
    torch = __import__("torch")
    g = w.hq // w.hkv
    length = w.lens[b]
    if w.paged:
        blocks = w.tables[slot][b, :-(-length // BLOCK_TOKENS)].long()
        k_unit = w.k_pool[blocks, hk].reshape(-1, HEAD_DIM)[:length]
        v_unit = w.v_pool[blocks, hk].reshape(-1, HEAD_DIM)[:length]
    else:
        k_unit = w.k_pool[slot, :length, hk * HEAD_DIM:(hk + 1) * HEAD_DIM]
        v_unit = w.v_pool[slot, :length, hk * HEAD_DIM:(hk + 1) * HEAD_DIM]
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    q_rows = w.q_rot[b:b + 1, hk * g:(hk + 1) * g]
    want = oracle.gqa_decode(bits(q_rows), bits(k_unit).reshape(-1), bits(v_unit).reshape(-1),
                             [length], hkv=1, stride_block=length * HEAD_DIM,
                             stride_token=HEAD_DIM, stride_head=HEAD_DIM, block_tokens=length)[0]
    got = out[b, hk * g:(hk + 1) * g].float().cpu().numpy()
    abs_err = float(np.max(np.abs(got - want)))
    rel = abs_err / float(np.max(np.abs(want)))
    if not (abs_err <= 2e-2 and rel <= 1e-2):
        raise SystemExit(f"parity: unit ({b}, {hk}) of {w.name} differs from the oracle: "
                         f"abs {abs_err:.3e}, relative {rel:.3e}")
    return rel


def multi_gpu_parity(gqa, comm, world: int, rank: int, dev) -> dict:
    """Small seeded cases, identical on every rank, run outside every timed region at N > 1:
    KV-head-parallel decode with an explicit split gathered over the peer windows must equal
    the unsharded decode computed on this rank's GPU bit for bit and agree with the FP64
    oracle; sequence-parallel decode must agree with the oracle and across ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from llminfer_b200 import sharding
    from oracle import oracle
    sys.path.insert(0, str(ROOT / "tests" / "golden"))
    import cases

    hq, hkv, batch, d = 64, 8, 3, HEAD_DIM
    lens = [3000, 257, 1024]
    rng = np.random.default_rng(53)
    bps = 12
    num_blocks = batch * bps
    table = rng.permutation(num_blocks).reshape(batch, bps).astype(np.int32)
    bits = lambda shape: cases.to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))
    q, k_pool, v_pool = bits((batch, hq, d)), bits((num_blocks, hkv, BLOCK_TOKENS, d)), \
        bits((num_blocks, hkv, BLOCK_TOKENS, d))
    to_dev = lambda b: torch.from_numpy(np.ascontiguousarray(b).view(np.int16)).to(dev).view(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    dtab = torch.from_numpy(table).to(dev)
    dlens = torch.tensor(lens, dtype=torch.int32, device=dev)

    def run(q_bits, k_bits, v_bits, heads_q, heads_kv, sharded):
        layout = gqa.layout_pool(num_blocks, BLOCK_TOKENS, heads_kv)
        out = torch.zeros(batch, heads_q, d, dtype=torch.bfloat16, device=dev)
        kw = dict(num_kv_heads=heads_kv, layout=layout, seq_lens=lens, seq_lens_dev=dlens,
                  block_table=dtab, workspace=gqa.binding.workspace_for(batch, heads_q, heads_kv, dev),
                  split_keys=512, status=status)
        if not sharded:
            gqa.decode(to_dev(q_bits), to_dev(k_bits), to_dev(v_bits), out, **kw)
            torch.cuda.synchronize()
            return out
        gathered = torch.zeros(world, batch, heads_q, d, dtype=torch.bfloat16, device=dev)
        for _ in range(2):  # both halves of the peer windows
            gqa.decode_sharded(comm, gathered, to_dev(q_bits), to_dev(k_bits), to_dev(v_bits), out, **kw)
            torch.cuda.synchronize()
        return sharding.unshard_output(gathered)

    full = run(q, k_pool, v_pool, hq, hkv, sharded=False)
    pq, pkv = hq // world, hkv // world
    whole = run(q[:, rank * pq:(rank + 1) * pq], k_pool[:, rank * pkv:(rank + 1) * pkv],
                v_pool[:, rank * pkv:(rank + 1) * pkv], pq, pkv, sharded=True)
    bit_equal = bool(torch.equal(whole.view(torch.int16), full.view(torch.int16)))
    okw = dict(hkv=hkv, stride_block=hkv * BLOCK_TOKENS * d, stride_token=d,
               stride_head=BLOCK_TOKENS * d, block_tokens=BLOCK_TOKENS, block_table=table)
    want = oracle.gqa_decode(q, k_pool.reshape(-1), v_pool.reshape(-1), lens, **okw)
    err = lambda got, ref: float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
    sharded_rel = err(whole.float().cpu().numpy(), want)

    # Sequence-parallel: every rank holds all heads and every world-th block; one sequence is
    # so short that ranks 1.. hold no key of it (an empty slice).
    sp_lens = [3000, 200, 2048]
    rows, local = sharding.sequence_slice(sp_lens, table, BLOCK_TOKENS, world, rank)
    out_sp = torch.zeros(batch, hq, d, dtype=torch.bfloat16, device=dev)
    gqa.decode_seqpar(comm, to_dev(q), to_dev(k_pool), to_dev(v_pool), out_sp, num_kv_heads=hkv,
                      layout=gqa.layout_pool(num_blocks, BLOCK_TOKENS, hkv), seq_lens=local,
                      seq_lens_dev=torch.tensor(local, dtype=torch.int32, device=dev),
                      block_table=torch.tensor(rows, dtype=torch.int32, device=dev),
                      workspace=gqa.binding.workspace_for(batch, hq, hkv, dev), status=status)
    torch.cuda.synchronize()
    want_sp = oracle.gqa_decode(q, k_pool.reshape(-1), v_pool.reshape(-1), sp_lens, **okw)
    seqpar_rel = err(out_sp.float().cpu().numpy(), want_sp)
    sums = [None] * world
    dist.all_gather_object(sums, (int(out_sp.view(torch.int16).long().sum().item()),
                                  int(whole.view(torch.int16).long().sum().item())))
    ranks_equal = all(s == sums[0] for s in sums)
    ok = (bit_equal and ranks_equal and sharded_rel <= 1e-2 and seqpar_rel <= 1e-2
          and int(status.item()) == 0)
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    return {"sharded_bit_equal": bit_equal, "sharded_rel_err": sharded_rel,
            "seqpar_rel_err": seqpar_rel, "small_cases_ranks_equal": ranks_equal,
            "all_ranks_ok": all(flags)}


def reference_cuda_rows(torch, dev, peak_gbs: float) -> dict:
    """The reference's own CUDA kernels (kernel::mha_kernel_cu, kernel::fused_gemv_add_kernel_cu),
    built from the reference checkout into oracle/_ref/libref_attn.so, timed on this GPU for the
    configurations they can run (BF16, one sequence, contiguous cache, <= 32768 keys with an
    enlarged workspace; one token for the projection). A comparison row, never the product."""
    import ctypes as C
    lib_path = ROOT / "oracle" / "_ref" / "libref_attn.so"
    if not lib_path.exists():
        return {"unavailable": "oracle/_ref/libref_attn.so was not built (no reference checkout)"}
    ref = C.CDLL(str(lib_path))
    ref.ref_mha_bf16.restype = C.c_int
    ref.ref_mha_bf16.argtypes = [C.c_void_p] * 4 + [C.c_int64, C.c_void_p] + [C.c_int32] * 8 + [C.c_void_p]
    ref.ref_fused_gemv_add.restype = C.c_int
    ref.ref_fused_gemv_add.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 2 + [C.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    rows = {}

    def timed(call, cycle: int, steps: int) -> float:
        for i in range(5):
            call(i % cycle)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            call(i % cycle)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / steps

    for name, hq, hkv, length, layers in (("qwen3-4b-bf16-b1-ctx1024", 32, 8, 1024, 36),
                                          ("qwen3-4b-bf16-b1-ctx4096", 32, 8, 4096, 16),
                                          ("qwen3-4b-bf16-b1-ctx32768", 32, 8, 32768, 8)):
        kv_dim = hkv * HEAD_DIM
        q = torch.randn(hq * HEAD_DIM, device=dev).to(torch.bfloat16)
        k = torch.randn(layers, length, kv_dim, device=dev).to(torch.bfloat16)
        v = torch.randn(layers, length, kv_dim, device=dev).to(torch.bfloat16)
        out = torch.zeros(hq * HEAD_DIM, dtype=torch.bfloat16, device=dev)
        ws_floats = hq * ((length + 31) // 32) * 130
        ws = torch.zeros(ws_floats, dtype=torch.float32, device=dev)

        def call(layer: int) -> None:
            rc = ref.ref_mha_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), ws.data_ptr(), ws_floats,
                                  out.data_ptr(), layers, layer, length - 1, kv_dim, hq // hkv, hq,
                                  HEAD_DIM, length, stream)
            assert rc == 0, rc

        us = timed(call, layers, 4 * layers)
        gbs = algorithmic_bytes(hq, hkv, [length]) / us / 1e3
        rows[name] = {"us_per_layer": us, "gbs": gbs, "frac_of_measured_peak": gbs / peak_gbs}
        del k, v
    n, kdim, copies = 5120, 8192, 6
    x = torch.randn(kdim, device=dev).to(torch.bfloat16)
    weights = [(torch.randn(n, kdim, device=dev) / 64).to(torch.bfloat16) for _ in range(copies)]
    r = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    us = timed(lambda i: ref.ref_fused_gemv_add(x.data_ptr(), weights[i].data_ptr(), r.data_ptr(),
                                                n, kdim, stream), copies, 10 * copies)
    rows["qwen3-32b-oproj-5120x8192-1token"] = {"us_per_token": us, "gbs": n * kdim * 2 / us / 1e3}
    return rows


def projection_rows(gqa, torch, w: "Workload", timer: "Timer", steps: int, warmup: int,
                    gather: str) -> dict:
    """The steps on either side of attention, reported beside the headline, never inside it.
    Weights are cycled over more copies than L2 holds; sharded runs exchange the per-KV-head
    sums of the output projection through the peer windows."""
    comm, dev, hq, hkv, batch = w.comm, w.dev, w.hq, w.hkv, w.batch
    hidden = HIDDEN[w.name.split("-bf16")[0]]
    peak_gbs, _ = measured_peak_gbs()
    weight_bytes = hidden * hq * HEAD_DIM * 2
    copies = max(2, -(-(256 << 20) // weight_bytes))
    o_weights = [torch.randn(hidden, hq * HEAD_DIM, device=dev, dtype=torch.bfloat16) / 64
                 for _ in range(copies)]
    resid = torch.zeros(batch, hidden, dtype=torch.bfloat16, device=dev)
    o_ws = gqa.oproj_workspace(hidden, hkv, dev)
    calls = [0]

    def oproj(_slot: int) -> None:
        gqa.oproj_residual(w.out, o_weights[calls[0] % copies], resid, num_kv_heads=hkv,
                           workspace=o_ws, comm=comm, status=w.status)
        calls[0] += 1

    torch.cuda.synchronize()
    o_stat = timer.run(oproj, 1, steps, warmup, min_seconds=0.1)
    o_us = o_stat["median_us"]
    o_gbs = weight_bytes / (o_us * 1e-6) / 1e9
    rows = {"oproj_residual": {
        "us_per_layer": o_us, "min_us": o_stat["min_us"], "hidden": hidden,
        "weight_bytes_per_gpu": weight_bytes, "achieved_gbs": o_gbs,
        "frac_of_measured_peak": o_gbs / peak_gbs,
        "exchange": "per-KV-head sums over the peer windows" if comm else "none"}}
    del o_weights

    # The step in front: packed QKV projection of this rank's heads (nothing to exchange).
    n_rows = (hq + 2 * hkv) * HEAD_DIM
    qkv_bytes = n_rows * hidden * 2
    copies = max(2, -(-(256 << 20) // qkv_bytes))
    qkv_weights = [torch.randn(n_rows, hidden, device=dev, dtype=torch.bfloat16) / 64
                   for _ in range(copies)]
    x_in = torch.randn(batch, hidden, device=dev, dtype=torch.bfloat16)
    qkv_ws = gqa.qkv_workspace(hidden, hq, hkv, dev)
    q_tmp = torch.empty(batch, hq, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    k_tmp = torch.empty(batch, hkv, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    v_tmp = torch.empty_like(k_tmp)

    def qkv(_slot: int) -> None:
        gqa.qkv_gemv(x_in, qkv_weights[calls[0] % copies], q_tmp, k_tmp, v_tmp,
                     workspace=qkv_ws, status=w.status)
        calls[0] += 1

    torch.cuda.synchronize()
    q_stat = timer.run(qkv, 1, steps, warmup, min_seconds=0.1)
    qkv_us = q_stat["median_us"]
    qkv_gbs = qkv_bytes / (qkv_us * 1e-6) / 1e9
    rows["qkv_gemv"] = {"us_per_layer": qkv_us, "min_us": q_stat["min_us"], "hidden": hidden,
                        "weight_bytes_per_gpu": qkv_bytes, "achieved_gbs": qkv_gbs,
                        "frac_of_measured_peak": qkv_gbs / peak_gbs}
    assert int(w.status.item()) == 0, "a bounded device wait ran out"
    return rows


def multi_token_row(gqa, torch, w: "Workload", timer: "Timer", steps: int, warmup: int) -> dict:
    """Four query tokens per sequence against the same caches in one pass (the reference would
    run four decode steps): reported beside the headline."""
    tokens = 4 if w.hq // w.hkv <= 4 else 2
    lens = w.lens
    q = torch.randn(w.batch, tokens, w.hq, HEAD_DIM, device=w.dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    ws = gqa.binding.workspace_for(w.batch, w.hq * tokens, w.hkv, w.dev)

    def call(slot: int) -> None:
        kw = dict(num_kv_heads=w.hkv, layout=w.layout, seq_lens=lens, workspace=ws,
                  status=w.status, early_prefetch=True)
        if w.paged:
            kw.update(seq_lens_dev=w.lens_dev, block_table=w.tables[slot])
        else:
            kw.update(fixed_block=slot)
        gqa.decode(q, w.k_pool, w.v_pool, out, **kw)

    stat = timer.run(call, w.slots, steps, warmup, min_seconds=0.1)
    gbs = algorithmic_bytes(w.hq * tokens, w.hkv, lens, w.elem) / stat["median_us"] / 1e3
    return {"q_tokens": tokens, "us_per_layer": stat["median_us"], "min_us": stat["min_us"],
            "us_per_token": stat["median_us"] / tokens, "achieved_gbs": gbs}


def sweep_row(gqa, torch, name, timer, args, dev) -> dict:
    """One other context of the metric on this GPU, measured like the headline: the full step
    and the attention kernels alone, with the roofline fractions."""
    w = Workload(gqa, name, 1, 0, dev, None, args)
    steps = 36 if w.slots == 36 else args.steps
    row = {}
    peak, _ = measured_peak_gbs()
    if w.has_front:
        full = timer.run(w.step, w.slots, steps, max(args.warmup, 3), min_seconds=0.1)
        row.update(us_per_layer=full["median_us"], min_us=full["min_us"], replays=full["replays"])
    else:
        row.update(note="FP32 parity case (the front stage is a BF16 kernel): attention only")
    if w.has_front:
        w.step(0)  # q_rot of the last step for the attention-only leg and the oracle check
    attn = timer.run(w.attention, w.slots, steps, max(args.warmup, 3), min_seconds=0.1)
    gbs = w.bytes_per_step() / attn["median_us"] / 1e3
    row.update(attention_only_us_per_layer=attn["median_us"], attention_only_min_us=attn["min_us"],
               gbs=gbs, frac_of_measured_peak=gbs / peak, frac_of_8tbs_nominal=gbs / 8000.0,
               algorithmic_bytes=w.bytes_per_step(), split_chunks=w.plan["split_chunks"],
               ctas=w.plan["num_ctas"], cluster_size=w.plan.get("cluster_size", 0) if w.cluster_merge() else 0,
               even_cut=w.plan.get("even_cut", 0), layers_cycled=w.slots,
               launches_per_step=w.launches_per_step("peer"))
    if w.has_front:
        w.attention(0)
        torch.cuda.synchronize()
        row["unit_rel_err_vs_oracle"] = unit_against_oracle(w, w.out, 0, w.batch - 1, w.hkv - 1)
    assert int(w.status.item()) == 0, "a bounded device wait ran out"
    w.free()
    del w
    torch.cuda.empty_cache()
    return row


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
    if args.partition == "sequence" and world > 1 and (not args.attn_only or args.gather != "peer"):
        raise SystemExit("--partition sequence needs --attn-only and the peer windows")

    timer = Timer(torch, dist, world, dev, args.no_graph)
    w = Workload(gqa, args.workload, world, rank, dev, comm, args)
    steps, warmup = args.steps, max(args.warmup, 3)
    min_replays = 100 if world > 1 else 20
    with ClockSampler(local_rank) as clocks:
        total = timer.run(w.step, w.slots, steps, warmup, min_replays=min_replays)
        if w.has_front:
            w.step(0)
        attn = timer.run(w.attention, w.slots, steps, warmup, min_replays=min_replays)
    clock_info = clocks.summary()
    us_per_layer, attn_us = total["median_us"], attn["median_us"]
    assert int(w.status.item()) == 0, "a bounded device wait ran out"
    peak, peak_kind = measured_peak_gbs()
    rank_bytes = w.bytes_per_step()
    achieved = rank_bytes / (attn_us * 1e-6) / 1e9

    if args.attn_only:
        if rank == 0:
            print(json.dumps({"attention_only_us_per_layer": attn_us, "us_per_layer": us_per_layer,
                              "min_us": total["min_us"], "attention_only_min_us": attn["min_us"],
                              "roofline": {"achieved": achieved, "frac": achieved / peak},
                              "front": "fused" if w.fused_front else "separate", "plan": w.plan}))
        if comm is not None:
            comm.close()
            dist.destroy_process_group()
        return
    if not w.has_front:
        raise SystemExit("the end-to-end leg needs the BF16 front stage; use --attn-only")

    # ---- parity of the values behind the numbers -------------------------------------------
    w.step(0)
    torch.cuda.synchronize()
    result = w.gathered if comm is not None else w.out.unsqueeze(0)
    checksum = int(result.view(torch.int16).long().sum().item())
    parity = {"unit_rel_err": unit_against_oracle(w, w.out, 0, w.batch - 1, w.hkv - 1),
              "unit": f"sequence {w.batch - 1}, local kv head {w.hkv - 1} of every rank vs the "
                      f"FP64 oracle (abs <= 2e-2, relative to max|out| <= 1e-2)"}
    if comm is not None:
        sums = [None] * world
        dist.all_gather_object(sums, checksum)
        parity["ranks_equal"] = all(s == sums[0] for s in sums)
        mine = w.gathered[rank]
        parity["own_slot_equals_local_output"] = bool(torch.equal(mine.view(torch.int16),
                                                                  w.out.view(torch.int16)))
        if args.gather == "peer":
            parity.update(multi_gpu_parity(gqa, comm, world, rank, dev))
        ok = parity["ranks_equal"] and parity["own_slot_equals_local_output"] and \
            parity.get("all_ranks_ok", True)
        if not ok:
            if rank == 0:
                print(json.dumps({"parity": parity, "error": "multi-GPU parity check failed"}))
            raise SystemExit(3)

    next_rows = {}
    if comm is None or args.gather == "peer":
        next_rows = projection_rows(gqa, torch, w, timer, steps, warmup, args.gather)
        if comm is None:
            next_rows["multi_token"] = multi_token_row(gqa, torch, w, timer, steps, warmup)

    # ---- end to end through the host-buffer entry point -----------------------------------
    session = gqa.Session(w.batch, w.hq, w.hkv, max(w.lens))
    pin = lambda t: t.cpu().pin_memory()
    q_host, k_host, v_host = pin(w.q_raw), pin(w.k_new), pin(w.v_new)
    out_host = torch.empty(world if comm else 1, w.batch, w.hq, HEAD_DIM, dtype=torch.bfloat16).pin_memory()

    def e2e_step(i: int) -> None:
        session.step(q_host, k_host, v_host, w.weight, w.k_pool, w.v_pool, w.layout, w.positions,
                     out_host, block_table=w.tables[i % w.slots],
                     fixed_block=0 if w.paged else i % w.slots, comm=comm)

    for i in range(warmup):
        e2e_step(i)
    timer.barrier()
    # Enough steps for a steady figure: at least the driver's K, at least 0.2 s.
    e2e_steps = min(4000, max(steps, int(0.2e6 / max(us_per_layer, 1.0))))
    per_step, parts = [], []
    with ClockSampler(local_rank) as e2e_clocks:
        t_begin = time.perf_counter()
        for i in range(e2e_steps):
            t0 = time.perf_counter()
            e2e_step(i)
            per_step.append((time.perf_counter() - t0) * 1e6)
            parts.append(session.last_timing())
        timer.barrier()
        wall_us = (time.perf_counter() - t_begin) * 1e6 / e2e_steps
    # Steps are collective at N > 1 (every rank needs everybody's rows): the slowest rank sets
    # the pace, so the per-step figure is the max over ranks of each rank's median.
    e2e_us = timer.max_over_ranks([median(per_step)])[0]
    e2e_mean = timer.max_over_ranks([wall_us])[0]
    breakdown = timer.max_over_ranks(
        [median([p[key] for p in parts]) / 1e3 for key in ("stage_ns", "launch_ns", "wait_ns", "copy_out_ns")])
    w.step((e2e_steps - 1) % w.slots)  # the device path on the cache slot of the last e2e step
    torch.cuda.synchronize()
    same_as_graph = bool(torch.equal(out_host.view(torch.int16),
                                     result.cpu().view(torch.int16).reshape(out_host.shape)))
    parity["e2e_output_equals_device_path"] = same_as_graph
    session.close()
    e2e_clock_info = e2e_clocks.summary()
    clock_info["reasons"] = sorted(set(clock_info["reasons"]) | set(e2e_clock_info["reasons"]))
    clock_info["samples_e2e"] = e2e_clock_info["samples"]
    h2d = (w.hq + 2 * w.hkv) * HEAD_DIM * 2 * w.batch + 8 * w.batch
    d2h = out_host.numel() * 2

    launches_per_step = w.launches_per_step(args.gather)
    gather_note = ""
    if world > 1:
        gather_note = (", peer-store all-gather over NVLink inside the combine kernel"
                       if w.fused_gather(args.gather) else f", {args.gather} all-gather over NVLink")
    front_note = ("qk-norm+rope+append inside the attention kernel" if w.fused_front
                  else "qk-norm+rope+append")
    line = {
        "metric": "gqa_decode_attn_us_per_layer", "value": us_per_layer, "unit": "us/layer",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": us_per_layer / 1e3,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": args.workload, "num_q_heads": w.hq_total, "num_kv_heads": w.hkv_total,
                   "head_dim": HEAD_DIM, "batch": w.batch, "kv_len": max(w.lens),
                   "kv_len_total": sum(w.lens), "kv_layout": w.layout_note,
                   "parallelism": f"kv-head-parallel x{world}",
                   "l2": f"inputs larger than L2: {w.slots} cache slot(s) of "
                         f"{w.slot_bytes / 2**20:.0f} MiB cycled per GPU",
                   "step": f"{front_note}, split attention, lse combine" + gather_note,
                   "split_chunks": w.plan["split_chunks"], "ctas": w.plan["num_ctas"],
                   "items": w.plan["num_items"]},
        "stats": {"median_us": total["median_us"], "min_us": total["min_us"],
                  "replays": total["replays"], "timed_region_s": total["timed_region_s"],
                  "attention_only_median_us": attn["median_us"],
                  "attention_only_min_us": attn["min_us"],
                  "how": f"CUDA graph of {steps} steps replayed; one CUDA-event pair per replay; "
                         f"max over ranks per replay; median and min over replays"},
        "hbm_tbs_aggregate": achieved * world / 1e3,
        "attention_only_us_per_layer": attn_us,
        "roofline": {"bound": "hbm", "kernel": "gqa_decode_stream_bf16 (+ lse combine)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "frac_of_8tbs_nominal": achieved / 8000.0,
                     "algorithmic_bytes_per_launch": rank_bytes,
                     "traffic": int(rank_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE),
                     "traffic_source": "ncu capture of the batch-1 case, scaled by bytes"},
        "e2e": {"value": e2e_us, "unit": "us/layer", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps, "mean_us": e2e_mean,
                "how": "median host time per gqa_session_step call, max over ranks",
                "breakdown_us": dict(zip(("stage", "launch", "wait", "copy_out"), breakdown))},
        "gpu_launches": launches_per_step * steps * total["replays"],
        "gpu_launches_per_step": launches_per_step,
        "parity": parity,
        "next_rows": next_rows,
        "clocks": clock_info,
    }
    if rank == 0 and world == 1 and not args.no_sweep:
        w.free()
        torch.cuda.empty_cache()
        sweep = {}
        for name in WORKLOADS:
            if name not in (args.workload, "qwen3-32b-bf16-b1-ctx131072"):
                sweep[name] = sweep_row(gqa, torch, name, timer, args, dev)
        line["context_sweep"] = sweep
        line["reference_cuda_kernel"] = reference_cuda_rows(torch, dev, peak)
    if rank == 0 and world == 1 and not args.no_cpu:
        line.update(cpu_rows(w.hq_total, w.hkv_total, w.lens))
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
    ap.add_argument("--front", choices=("fused", "separate"), default="fused",
                    help="QK-Norm + RoPE + KV append inside the attention kernel, or as its own launch")
    ap.add_argument("--no-sweep", action="store_true",
                    help="N = 1: skip the other contexts and the reference-kernel rows")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline legs")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager launches instead of CUDA-graph replays (profiler runs)")
    ap.add_argument("--attn-only", action="store_true",
                    help="tuning runs: skip the end-to-end, parity, sweep and CPU legs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
