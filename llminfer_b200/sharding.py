"""KV-head-parallel helpers on the host side: which heads a rank owns, how to cut a full cache
into the rank's shard, and how the gathered output maps back to the full head order."""
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
