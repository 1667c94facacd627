"""Partition helpers on the host side. KV-head-parallel: which heads a rank owns, how to cut
a full cache into the rank's shard, and how the gathered output maps back to the full head
order. Sequence-parallel: which blocks of a paged sequence a rank holds."""
from __future__ import annotations

import torch

from .binding import shard_plan


def shard_heads(x: torch.Tensor, num_heads: int, nranks: int, rank: int, head_dim: int = 128):
    """Rank's slice of a tensor whose last dimension is [num_heads * head_dim] or whose last two
    are [num_heads, head_dim]."""
    per = num_heads // nranks
    if x.shape[-1] == num_heads * head_dim:
        lead = x.shape[:-1]
        return x.reshape(*lead, num_heads, head_dim)[..., rank * per:(rank + 1) * per, :] \
                .reshape(*lead, per * head_dim).contiguous()
    assert x.shape[-2] == num_heads and x.shape[-1] == head_dim
    return x[..., rank * per:(rank + 1) * per, :].contiguous()


def unshard_output(gathered: torch.Tensor) -> torch.Tensor:
    """[nranks, batch, local_q_heads, head_dim] (what the all-gather produces) ->
    [batch, nranks * local_q_heads, head_dim] in the full model's head order."""
    nranks, batch, local, dim = gathered.shape
    return gathered.permute(1, 0, 2, 3).reshape(batch, nranks * local, dim)


def local_heads(num_q_heads: int, num_kv_heads: int, nranks: int, rank: int):
    plan = shard_plan(num_q_heads, num_kv_heads, nranks, rank)
    return plan["num_local_q_heads"], plan["num_local_kv_heads"]


def sequence_slice(seq_lens, block_table, block_tokens: int, nranks: int, rank: int):
    """Block-interleaved slice of paged sequences for gqa_decode_seqpar: rank r holds logical
    blocks r, r + nranks, ... of every sequence.

    seq_lens: keys per sequence; block_table: [batch][blocks_per_seq] physical block ids in
    logical order (nested lists or an array). Returns (local_table, local_lens): the rank's
    block table, padded with zeros to the original width, and the number of keys in its
    blocks. Only the globally last block of a sequence can be partly filled, and it is the
    last block of the rank that holds it, so a local sequence is an ordinary one. A rank that
    holds no block of a sequence (a sequence shorter than `nranks` blocks) gets length 0 for
    it: gqa_decode_seqpar and gqa_decode_partial take that as an empty slice.
    """
    local_table, local_lens = [], []
    for length, row in zip(seq_lens, block_table):
        row = [int(v) for v in row]
        blocks = -(-int(length) // block_tokens)
        mine = list(range(rank, blocks, nranks))
        keys = sum(min(block_tokens, int(length) - i * block_tokens) for i in mine)
        local_table.append([row[i] for i in mine] + [0] * (len(row) - len(mine)))
        local_lens.append(keys)
    return local_table, local_lens
