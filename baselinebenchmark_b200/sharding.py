"""Multi-GPU drivers for the operator: one process per GPU, torch.distributed for
the plumbing.  The reference has no multi-device path at all (no collective
call site; its native kernel is rendered with enable_cp=False,
backends/_mthreads/ops/moba/native_moba.py:69), so both modes are additions that
keep the single-device results bit for bit.

* Unit sharding.  Routing and attention never cross a sequence
  (routing.py:1109-1119) or a KV-head group (routing.py:1089,
  attention.py:649-650), so the (sequence, KV-head group) units of a batch are
  independent: `unit_shard` gives every rank a contiguous block of them and no
  data-path collective is needed.

* Context parallelism for one very long sequence.  Every rank owns a contiguous
  token range.  A query needs the mean key of every earlier chunk and the K/V of
  the chunks it selects, which over millions of (token, head) rows means every
  earlier chunk: K and V are all-gathered into local memory (NCCL over NVLink
  on GPUs), after which each rank runs the operator on its own query window.
  Per-(query, chunk) arithmetic is unchanged, so routing is bit-identical to a
  single-device run.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch


def unit_shard(num_sequences: int, num_kv_heads: int, world_size: int, rank: int) -> List[Tuple[int, int]]:
    """(sequence, kv head) units of `rank`: units are numbered sequence-major and
    dealt out in contiguous blocks, the first `total % world_size` ranks taking one more."""
    total = num_sequences * num_kv_heads
    base, extra = divmod(total, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return [(u // num_kv_heads, u % num_kv_heads) for u in range(lo, hi)]


def shard_slices(units: Sequence[Tuple[int, int]], cu_seqlens: Sequence[int], group: int):
    """For each unit the token slice and the q / kv head slices of the full tensors."""
    out = []
    for seq, kvh in units:
        out.append((slice(int(cu_seqlens[seq]), int(cu_seqlens[seq + 1])),
                    slice(kvh * group, (kvh + 1) * group), slice(kvh, kvh + 1)))
    return out


def context_window(total_tokens: int, chunk: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous, chunk-aligned token range of `rank` for one sequence of
    `total_tokens`: whole chunks are dealt out as evenly as possible, earlier ranks
    taking the remainder; the last rank also takes the partial tail chunk."""
    nchunks = -(-total_tokens // chunk)
    base, extra = divmod(nchunks, world_size)
    lo_c = rank * base + min(rank, extra)
    hi_c = lo_c + base + (1 if rank < extra else 0)
    return min(lo_c * chunk, total_tokens), min(hi_c * chunk, total_tokens)


def _default_forward(q, k, v, cu, max_seqlen, chunk, topk, q_token_begin):
    from .parallel import moba_forward
    return moba_forward(q, k, v, cu, max_seqlen, chunk, topk, q_token_begin=q_token_begin)[0]


def moba_context_parallel(q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                          total_tokens: int, moba_chunk_size: int, moba_topk: int,
                          group=None, forward: Optional[Callable] = None) -> torch.Tensor:
    """MoBA forward of ONE sequence of `total_tokens` split over the ranks of
    `group` by `context_window`.  Each rank passes the q/k/v rows of its own
    window and receives the output rows of that window.

    K and V are all-gathered (ragged windows are padded to the longest one);
    every kernel afterwards reads local memory only.  `forward` replaces the
    CUDA operator (tests run the host logic on CPU with the oracle)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    windows = [context_window(total_tokens, moba_chunk_size, world, r) for r in range(world)]
    lo, hi = windows[rank]
    if q_local.shape[0] != hi - lo or k_local.shape[0] != hi - lo or v_local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} must hold tokens [{lo}, {hi}), got {q_local.shape[0]} rows")
    longest = max(h - l for l, h in windows)
    hkv, d = k_local.shape[1], k_local.shape[2]

    def gather(x):
        pad = torch.zeros((longest, hkv, d), dtype=x.dtype, device=x.device)
        pad[: x.shape[0]] = x
        parts = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(parts, pad, group=group)
        return torch.cat([parts[r][: windows[r][1] - windows[r][0]] for r in range(world)], 0)

    k_full, v_full = gather(k_local), gather(v_local)
    cu = torch.tensor([0, total_tokens], dtype=torch.int32, device=q_local.device)
    if hi == lo:
        return q_local.new_empty(q_local.shape)
    fn = forward or _default_forward
    return fn(q_local, k_full, v_full, cu, total_tokens, moba_chunk_size, moba_topk, lo)
