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
  earlier chunk.  Each rank computes the means of its own chunks and all means
  are exchanged (a few hundred KB); the gating then runs while the K and V rows
  of the EARLIER ranks arrive in local memory (NCCL send/recv over NVLink; later
  ranks' rows are never needed by a causal query and are not sent).  The dense
  stage waits for the rows.  Per-(query, chunk) arithmetic is unchanged, so
  routing and outputs are bit-identical to a single-device run.
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


def agree(ok: bool, group=None, what: str = "arguments") -> None:
    """Collective check before a rank enters the exchange: every rank reports whether its own
    arguments are valid and ALL ranks raise if any of them is not, instead of the valid ranks
    waiting in a collective the invalid one never joins."""
    import torch.distributed as dist
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag.item()) == 0:
        raise ValueError(f"context parallel: a rank reported invalid {what}" + ("" if ok else " (this rank)"))


class ContextParallel:
    """Context-parallel MoBA forward of ONE sequence on the GPUs of `group` through the C ABI
    (moba_cp_forward): rank r owns the tokens of `context_window(..., r)`.

    The object holds what stays the same from call to call: the full-length K / V buffers (each
    rank writes its own rows into `k_rows` / `v_rows`, views of those buffers, or passes them to
    `forward`), the communication stream and the NCCL communicator of the group (torch's own,
    ProcessGroupNCCL._comm_ptr).  Shapes are agreed on collectively when the object is built, so
    a rank with inconsistent arguments makes every rank raise there and the steps can stay free
    of host synchronisation."""

    def __init__(self, total_tokens: int, num_kv_heads: int, head_dim: int, chunk: int, dtype, device, group=None):
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.total, self.chunk = total_tokens, chunk
        windows = [context_window(total_tokens, chunk, self.world, r) for r in range(self.world)]
        self.bounds = (C.c_int64 * (self.world + 1))(*([w[0] for w in windows] + [total_tokens]))
        self.lo, self.hi = windows[self.rank]
        same = torch.tensor([total_tokens, num_kv_heads, head_dim, chunk], dtype=torch.int64, device=device)
        lo, hi = same.clone(), same.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
        agree(bool((lo == hi).all()), group, "sequence length, heads, head_dim or chunk size")
        self.k_full = torch.empty(total_tokens, num_kv_heads, head_dim, dtype=dtype, device=device)
        self.v_full = torch.empty_like(self.k_full)
        self.k_rows, self.v_rows = self.k_full[self.lo:self.hi], self.v_full[self.lo:self.hi]
        self.cu = torch.tensor([0, total_tokens], dtype=torch.int32, device=device)
        self.comm_stream = torch.cuda.Stream(device)
        pg = group if group is not None else dist.distributed_c10d._get_default_group()
        self.comm = pg._get_backend(torch.device(device))._comm_ptr()
        self._lib = _lib

    def forward(self, q_local, moba_topk: int, k_local=None, v_local=None, *, out=None, workspace=None,
                events=None, return_selected: bool = False):
        """Output rows of this rank's window.  `k_local` / `v_local`, when given, are copied into
        place first; otherwise the caller has written `k_rows` / `v_rows`."""
        import ctypes as C
        from . import parallel
        _lib = self._lib
        if q_local.shape[0] != self.hi - self.lo:
            raise ValueError(f"rank {self.rank} must pass the {self.hi - self.lo} query rows of tokens "
                             f"[{self.lo}, {self.hi}), got {q_local.shape[0]}")
        if k_local is not None:
            self.k_rows.copy_(k_local)
            self.v_rows.copy_(v_local)
        out = torch.empty_like(q_local) if out is None else out
        if self.hi == self.lo:
            return (out, None) if return_selected else out
        prob = parallel.make_problem(q_local, self.k_full, self.v_full, out, self.cu, self.total, self.chunk,
                                     moba_topk, q_token_begin=self.lo)
        need = C.c_size_t(0)
        _lib.check(_lib.lib().moba_cp_workspace_size(C.byref(prob), C.byref(need)))
        ws = workspace if workspace is not None and workspace.numel() >= need.value else \
            torch.empty(need.value, dtype=torch.uint8, device=q_local.device)
        sel = None
        if return_selected:
            dims = _lib.Dims()
            _lib.check(_lib.lib().moba_problem_dims(C.byref(prob), C.byref(dims)))
            sel = torch.empty((max(dims.hist, 0), q_local.shape[1], q_local.shape[0]), dtype=torch.int32,
                              device=q_local.device)
        arr = (C.c_void_p * 6)(*[e.cuda_event for e in events]) if events is not None else None
        with torch.cuda.device(q_local.device):
            rc = _lib.lib().moba_cp_forward(
                C.byref(prob), self.comm, self.rank, self.world, self.bounds, q_local.data_ptr(),
                self.k_full.data_ptr(), self.v_full.data_ptr(), self.cu.data_ptr(), out.data_ptr(), None,
                sel.data_ptr() if sel is not None and sel.numel() else None, ws.data_ptr(), ws.numel(),
                torch.cuda.current_stream(q_local.device).cuda_stream, self.comm_stream.cuda_stream, arr)
        _lib.check(rc)
        self.workspace = ws                      # keeps the buffer alive while the call runs
        return (out, sel) if return_selected else out

    def finish(self, timeout_s: float = 60.0) -> None:
        """Host-side wait for the calls queued so far with a deadline: polls the stream and the
        communicator's asynchronous error state; on an error or when the deadline passes the
        communicator is aborted (ncclCommAbort) and RuntimeError raised, so that a rank whose peer
        never joined gets its stream back instead of waiting forever."""
        import ctypes as C
        import time
        done = torch.cuda.Event()
        done.record()
        deadline = time.monotonic() + timeout_s
        state = C.c_int32(0)
        while not done.query():
            self._lib.check(self._lib.lib().moba_cp_poll(self.comm, C.byref(state)))
            if state.value not in (0, 7) or time.monotonic() > deadline:      # 7: ncclInProgress
                self._lib.lib().moba_cp_abort(self.comm)
                raise RuntimeError(f"context-parallel exchange failed (NCCL state {state.value}) or timed out "
                                   f"after {timeout_s} s; the communicator was aborted")
            time.sleep(0.001)


def _default_forward(q, k, v, cu, max_seqlen, chunk, topk, q_token_begin):
    from .parallel import moba_forward
    return moba_forward(q, k, v, cu, max_seqlen, chunk, topk, q_token_begin=q_token_begin)[0]


def moba_context_parallel(q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                          total_tokens: int, moba_chunk_size: int, moba_topk: int,
                          group=None, forward: Optional[Callable] = None) -> torch.Tensor:
    """MoBA forward of ONE sequence of `total_tokens` split over the ranks of
    `group` by `context_window`.  Each rank passes the q/k/v rows of its own
    window and receives the output rows of that window.

    All ranks first agree that every rank's rows match its window (a rank with a wrong shape
    makes every rank raise ValueError rather than leaving the others in a collective).  On CUDA
    tensors the call then goes through `ContextParallel` (the C ABI's moba_cp_forward: means
    exchanged first, K/V rows of earlier ranks received while the gating runs, no padding and no
    concatenation).  `forward` replaces the operator for host-logic tests: K and V are then
    all-gathered with the group's backend (ragged windows padded to the longest) and `forward`
    is called on the full tensors."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    windows = [context_window(total_tokens, moba_chunk_size, world, r) for r in range(world)]
    lo, hi = windows[rank]
    ok = q_local.shape[0] == hi - lo and k_local.shape[0] == hi - lo and v_local.shape[0] == hi - lo
    agree(ok, group, f"row counts (rank {rank} must hold tokens [{lo}, {hi}))")
    if forward is None and q_local.is_cuda:
        cp = ContextParallel(total_tokens, k_local.shape[1], k_local.shape[2], moba_chunk_size, k_local.dtype,
                             q_local.device, group)
        return cp.forward(q_local, moba_topk, k_local, v_local)
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
