"""Incremental prefill and decode of ONE growing sequence on top of `moba_forward_cached`.

The reference's MoBA operator has no incremental mode: `parallel_moba` takes whole sequences
and recomputes every chunk mean on each call (backends/_mthreads/ops/moba/parallel.py:306-311).
Here the K/V rows, the chunk means and the position live on the device between calls; a call
appends any number of tokens - a prefill block or a single decode token - and returns their
attention rows, which equal the rows of a one-shot run over the final sequence bit for bit
(a query only sees keys at or before its own position, and a chunk's mean only its own keys).
"""
from typing import Optional

import torch

from . import parallel


class IncrementalMoba:
    """K/V cache of one sequence with cached chunk means.

    `capacity` tokens of K and V ([capacity, Hkv, D]) and ceil(capacity / chunk) chunk means are
    allocated once.  `append(q, k, v)` stores the new K/V rows behind the `length` tokens already
    there and runs the operator on the query window [length, length + n) over the prefix; the
    means of chunks completed by earlier calls are read from the cache, the others recomputed.
    Nothing is read back to the host: the position is kept on both sides."""

    def __init__(self, capacity: int, num_kv_heads: int, head_dim: int, moba_chunk_size: int, moba_topk: int,
                 dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None,
                 attend_impl: Optional[int] = None):
        if capacity <= 0:
            raise ValueError(f"capacity must be positive, got {capacity}")
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.capacity, self.chunk, self.topk, self.attend_impl = capacity, moba_chunk_size, moba_topk, attend_impl
        self.k = torch.empty(capacity, num_kv_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        slots = (capacity + moba_chunk_size - 1) // moba_chunk_size
        self.means = torch.zeros(slots, num_kv_heads, head_dim, dtype=dtype, device=device)
        self.cu = torch.zeros(2, dtype=torch.int32, device=device)
        self.length = 0

    def reset(self) -> None:
        self.length = 0

    def append(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, return_selected: bool = False):
        """q [n, Hq, D], k / v [n, Hkv, D]: the next n >= 1 tokens.  Returns their rows [n, Hq, D];
        with `return_selected` also the chunks they selected, (out, selected[hist, Hq, n] int32)."""
        n, begin = q.shape[0], self.length
        if k.shape[0] != n or v.shape[0] != n:
            raise ValueError(f"q, k and v must hold the same number of new tokens, got {n}, {k.shape[0]}, {v.shape[0]}")
        if n == 0 or begin + n > self.capacity:
            raise ValueError(f"cannot append {n} tokens at position {begin} of a cache of {self.capacity}")
        end = begin + n
        self.k[begin:end].copy_(k)
        self.v[begin:end].copy_(v)
        self.cu[1:].fill_(end)
        # a call on a prefix of `begin` tokens left final means in the slots of all chunks but the
        # prefix's last one (the last chunk of a sequence is no candidate and is not computed)
        cached = (begin - 1) // self.chunk if begin > 0 else 0
        out, _, sel = parallel.moba_forward(q, self.k[:end], self.v[:end], self.cu, self.capacity, self.chunk,
                                            self.topk, attend_impl=self.attend_impl, q_token_begin=begin,
                                            means_cache=self.means, cached_slots=cached,
                                            return_selected=return_selected)
        self.length = end
        return (out, sel) if return_selected else out
