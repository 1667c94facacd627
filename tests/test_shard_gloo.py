"""World-size-2 test of the KV-head-parallel host logic on CPU (gloo): each rank attends with its
own kv heads (the CPU oracle stands in for the GPU kernel), the outputs are all-gathered in the
layout gqa_decode_sharded produces, and the reassembled result must equal the unsharded one."""
import os
import socket
import sys
import traceback
from pathlib import Path

# Spawned workers re-import this module without pytest's conftest: set the paths here.
_ROOT = Path(__file__).resolve().parent.parent
for _p in (_ROOT, _ROOT / "tests", _ROOT / "tests" / "golden"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_queue) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from llminfer_b200 import sharding
        from oracle import oracle
        hq, hkv, batch, length, d = 16, 4, 3, 70, 128
        rng = np.random.default_rng(3)  # same data on every rank
        q = cases.to_bf16_bits(rng.standard_normal((batch, hq, d), dtype=np.float32))
        k = cases.to_bf16_bits(rng.standard_normal((batch, length, hkv * d), dtype=np.float32))
        v = cases.to_bf16_bits(rng.standard_normal((batch, length, hkv * d), dtype=np.float32))
        lens = [70, 33, 1]
        full = oracle.gqa_decode(q, k.reshape(-1), v.reshape(-1), lens, hkv=hkv,
                                 stride_block=length * hkv * d, stride_token=hkv * d,
                                 stride_head=d, block_tokens=length,
                                 block_table=np.arange(batch, dtype=np.int32)[:, None])
        hq_l, hkv_l = sharding.local_heads(hq, hkv, world, rank)
        as_t = lambda a: torch.from_numpy(a.astype(np.int32))
        q_l = sharding.shard_heads(as_t(q), hq, world, rank).numpy().astype(np.uint16)
        k_l = sharding.shard_heads(as_t(k), hkv, world, rank).numpy().astype(np.uint16)
        v_l = sharding.shard_heads(as_t(v), hkv, world, rank).numpy().astype(np.uint16)
        assert q_l.shape == (batch, hq_l, d) and k_l.shape == (batch, length, hkv_l * d)
        local = oracle.gqa_decode(q_l, k_l.reshape(-1), v_l.reshape(-1), lens, hkv=hkv_l,
                                  stride_block=length * hkv_l * d, stride_token=hkv_l * d,
                                  stride_head=d, block_tokens=length,
                                  block_table=np.arange(batch, dtype=np.int32)[:, None])
        pieces = [torch.empty(batch, hq_l, d) for _ in range(world)]
        dist.all_gather(pieces, torch.from_numpy(local))
        gathered = torch.stack(pieces)  # [rank, batch, local_q_heads, d], as ncclAllGather lays it
        whole = sharding.unshard_output(gathered).numpy()
        result_queue.put((rank, bool(np.array_equal(whole, full))))
    except Exception:
        result_queue.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_head_parallel_gather_reassembles_the_full_output(built_lib):
    world = 2
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {0: True, 1: True}


def test_sequence_slices_partition_every_sequence(built_lib):
    """Block-interleaved slices for the sequence-parallel decode: over all ranks every key is
    held exactly once, only a rank's last block can be partly filled, and a rank without keys
    of a sequence gets an empty slice (length 0)."""
    from llminfer_b200 import sharding
    block_tokens, lens = 256, [3000, 2100, 2048, 257]
    table = [[100 * b + i for i in range(12)] for b in range(len(lens))]
    for nranks in (1, 2, 4):
        lens_n, table_n = lens, table  # at 4 ranks the 257-key sequence leaves two ranks empty
        seen = [[] for _ in lens_n]
        total = [0] * len(lens_n)
        for rank in range(nranks):
            rows, local = sharding.sequence_slice(lens_n, table_n, block_tokens, nranks, rank)
            for b, (row, keys) in enumerate(zip(rows, local)):
                held = -(-keys // block_tokens)
                assert len(row) == 12 and all(v == 0 for v in row[held:])
                seen[b] += row[:held]
                total[b] += keys
        assert total == lens_n
        for b, length in enumerate(lens_n):
            assert sorted(seen[b]) == table_n[b][:-(-length // block_tokens)]
    rows, local = sharding.sequence_slice([257], [table[0]], block_tokens, 4, 3)
    assert local == [0] and rows == [[0] * 12]
