"""Host-side mirror of the reference operator
``parallel_moba(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)``
(backends/_mthreads/ops/moba/parallel.py:377-457) on top of the C ABI.

Same seven positional arguments, same validation order and exception types as
parallel.py:410-443, same caller contract for the inference path
(parallel.py:270-274): ``cu_seqlens`` starts at 0, increases strictly and ends
at ``q.shape[0]``; ``max_seqlen`` is at least the longest sequence; neither is
read back to the host.  torch is used for device memory and the current stream
only; all computation happens inside libmoba_b200.so and there is no fallback:
an unsupported configuration raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib

__all__ = ["parallel_moba", "moba_attn_varlen", "moba_forward", "make_problem", "workspace_bytes"]

#: head dims of the reference's benchmark suite (benchmarks/moba_compare.py:63, :70)
HEAD_DIMS = (64, 96, 128, 256)


def _validate(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, windowed: bool = False) -> None:
    """parallel.py:410-446, message for message where it matters to callers.
    `windowed`: q holds a window of the packed tokens, so its token count may differ from k's."""
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3:
        raise ValueError("q, k, and v must have shape [tokens, heads, head_dim]")
    if k.shape != v.shape:
        raise ValueError(f"k and v must have identical shapes, got {k.shape} and {v.shape}")
    if (q.shape[0] != k.shape[0] and not windowed) or q.shape[2] != k.shape[2]:
        raise ValueError(
            f"q and k/v must have the same token count and head dimension, got q={q.shape}, k={k.shape}")
    if q.device != k.device or q.device != v.device or q.device.type != "cuda":
        raise ValueError("q, k, and v must be accelerator tensors on the same device")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise TypeError("q, k, and v must have the same dtype")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"only float16 and bfloat16 are supported, got {q.dtype}")
    if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must be a one-dimensional tensor of length >= 2")
    if cu_seqlens.device != q.device or cu_seqlens.dtype != torch.int32:
        raise TypeError("cu_seqlens must be an int32 tensor on the q device")
    if not isinstance(max_seqlen, int) or max_seqlen <= 0:
        raise ValueError(f"max_seqlen must be a positive int, got {max_seqlen}")
    if not isinstance(moba_chunk_size, int) or moba_chunk_size <= 0:
        raise ValueError(f"moba_chunk_size must be a positive int, got {moba_chunk_size}")
    if not isinstance(moba_topk, int) or moba_topk < 1:
        raise ValueError(f"moba_topk must be a positive int, got {moba_topk}")
    if moba_topk > 64:
        raise ValueError(f"moba_topk must be <= 64 to match FlashMoBA, got {moba_topk}")
    if q.shape[0] == 0 or q.shape[1] == 0 or k.shape[1] == 0 or q.shape[2] == 0:
        raise ValueError("q, k, and v dimensions must be non-zero")
    if q.shape[1] % k.shape[1] != 0:
        raise ValueError(f"q heads ({q.shape[1]}) must be divisible by kv heads ({k.shape[1]})")
    if q.shape[2] > 256:
        raise ValueError(f"head_dim must be <= 256 to match FlashMoBA, got {q.shape[2]}")
    # limits of this build (no fallback by design)
    if q.shape[2] not in HEAD_DIMS:
        raise NotImplementedError(f"this build supports head_dim {HEAD_DIMS} only")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.stride(2) != 1:
            raise NotImplementedError(f"{name} must be contiguous in its last dimension")


def default_attend_impl(head_dim: int) -> int:
    """The tcgen05 dense stage for every supported head_dim (its own kernel at 256)."""
    return _lib.ATTEND_TCGEN05 if head_dim in HEAD_DIMS else _lib.ATTEND_MMA_SYNC


def make_problem(q, k, v, out, cu_seqlens, max_seqlen, chunk, topk, attend_impl=None,
                 q_token_begin=None):
    """struct moba_problem for these tensors.  With `q_token_begin` set, q/out hold the
    packed tokens [q_token_begin, q_token_begin + q.shape[0]) and k/v all of them."""
    return _lib.Problem(
        q_token_begin=q_token_begin or 0, q_tokens=q.shape[0] if q_token_begin is not None else 0,
        dtype=1 if q.dtype == torch.float16 else 0,
        total_tokens=k.shape[0], batch=cu_seqlens.numel() - 1, num_q_heads=q.shape[1],
        num_kv_heads=k.shape[1], head_dim=q.shape[2], max_seqlen=max_seqlen, chunk_size=chunk,
        topk=topk, attend_impl=default_attend_impl(q.shape[2]) if attend_impl is None else attend_impl,
        q_stride_token=q.stride(0), q_stride_head=q.stride(1),
        k_stride_token=k.stride(0), k_stride_head=k.stride(1),
        v_stride_token=v.stride(0), v_stride_head=v.stride(1),
        o_stride_token=out.stride(0), o_stride_head=out.stride(1))


def workspace_bytes(problem, limit: Optional[int] = None) -> int:
    """Workspace for one pass over all heads, or, with `limit`, the largest useful size not
    above it (never below the one-kv-head minimum): the library then runs kv-head groups in turn."""
    size = C.c_size_t(0)
    _lib.check(_lib.lib().moba_workspace_size(C.byref(problem), C.byref(size)))
    if limit is None or size.value <= limit:
        return int(size.value)
    least = C.c_size_t(0)
    _lib.check(_lib.lib().moba_workspace_size_min(C.byref(problem), C.byref(least)))
    return max(int(least.value), int(limit))


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch for one call, taken from torch's caching allocator like the reference's own
    per-call buffers (parallel.py:283-374): the allocator orders reuse by stream, so calls on
    unordered streams never share a buffer, and a buffer allocated while a CUDA graph is
    being captured belongs to that graph's memory pool and stays valid for its replays."""
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def moba_forward(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, *,
                 return_lse: bool = False, return_selected: bool = False,
                 attend_impl: Optional[int] = None, workspace: Optional[torch.Tensor] = None,
                 q_token_begin: Optional[int] = None, workspace_limit: Optional[int] = None,
                 means_cache: Optional[torch.Tensor] = None, cached_slots: int = 0
                 ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Runs the operator and optionally returns the final LSE [Hq, T] (fp32) and
    the routing decision selected[hist, Hq, T] (int32, -1 padded).

    `q_token_begin` (context parallelism, incremental prefill, decode): q holds only the
    packed tokens [q_token_begin, q_token_begin + q.shape[0]), a window that may start and
    end at any token, while k, v and cu_seqlens describe every token; outputs cover the
    window and equal the rows of the run over all tokens bit for bit.  `workspace_limit` (bytes) bounds the scratch memory: the kv heads
    are then processed in groups, with identical results.  Scratch memory is allocated per
    call through torch's caching allocator unless `workspace` (a uint8 tensor the caller
    keeps alive and does not share between unordered streams) is given.

    `means_cache` (incremental prefill and decode, see incremental.IncrementalMoba): a [slots, Hkv, D] tensor the caller keeps between calls;
    slots below `cached_slots` are taken from it, the others are computed and stored into it
    (moba_forward_cached in include/moba_b200.h has the rule for `cached_slots`)."""
    _validate(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, windowed=q_token_begin is not None)
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    prob = make_problem(q, k, v, out, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, attend_impl,
                        q_token_begin)
    dims = _lib.Dims()
    _lib.check(_lib.lib().moba_problem_dims(C.byref(prob), C.byref(dims)))
    need = workspace_bytes(prob, workspace_limit)
    ws = workspace if workspace is not None else _workspace(q.device, need)
    lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device) if return_lse else None
    sel = None
    if return_selected:
        sel = torch.empty((max(dims.hist, 0), q.shape[1], q.shape[0]), dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        common = (C.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(),
                  lse.data_ptr() if lse is not None else None,
                  sel.data_ptr() if sel is not None and sel.numel() else None)
        if means_cache is not None:
            if means_cache.shape != (dims.slots, k.shape[1], k.shape[2]) or means_cache.dtype != k.dtype \
                    or not means_cache.is_contiguous():
                raise ValueError(f"means_cache must be a contiguous {k.dtype} tensor of shape "
                                 f"{(dims.slots, k.shape[1], k.shape[2])}")
            rc = _lib.lib().moba_forward_cached(*common, means_cache.data_ptr(), cached_slots,
                                                ws.data_ptr(), ws.numel() * ws.element_size(), stream)
        else:
            rc = _lib.lib().moba_forward(*common, ws.data_ptr(), ws.numel() * ws.element_size(), stream)
    _lib.check(rc)
    return out, lse, sel


def moba_backward(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, out, lse, selected, dout,
                  attend_impl=None):
    """Gradients (dq, dk, dv) of the operator for the output gradient `dout`, given what
    `moba_forward(..., return_lse=True, return_selected=True)` returned
    (MixedAttention.backward, parallel.py:149-250: merged LSE and output, constant selection).
    `attend_impl` picks the dq and dk/dv kernels: tcgen05 by default, mma.sync when asked for."""
    _validate(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
    dout = dout.contiguous()
    if attend_impl is None:
        attend_impl = default_attend_impl(q.shape[2])
    prob = make_problem(q, k, v, out, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk, attend_impl)
    need = C.c_size_t(0)
    _lib.check(_lib.lib().moba_backward_workspace_size(C.byref(prob), C.byref(need)))
    ws = _workspace(q.device, need.value)
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        rc = _lib.lib().moba_backward(
            C.byref(prob), q.data_ptr(), k.data_ptr(), v.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(),
            lse.data_ptr(), selected.data_ptr() if selected is not None and selected.numel() else None,
            dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            ws.data_ptr(), ws.numel() * ws.element_size(), stream)
    _lib.check(rc)
    return dq, dk, dv


class _MobaFunction(torch.autograd.Function):
    """Training path: forward through the same kernels as inference, keeping the LSE and the
    routing decision for the backward (the reference's MixedAttention, parallel.py:59-250)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk):
        out, lse, sel = moba_forward(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk,
                                     return_lse=True, return_selected=True)
        ctx.save_for_backward(q, k, v, cu_seqlens, out, lse, sel)
        ctx.args = (max_seqlen, moba_chunk_size, moba_topk)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, cu_seqlens, out, lse, sel = ctx.saved_tensors
        dq, dk, dv = moba_backward(q, k, v, cu_seqlens, *ctx.args, out, lse, sel, dout)
        return dq, dk, dv, None, None, None, None


def parallel_moba(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                  max_seqlen: int, moba_chunk_size: int, moba_topk: int) -> torch.Tensor:
    """Causal variable-length MoBA forward, signature of parallel.py:377-385.

    Like the reference (parallel.py:447-456) the inference dataflow is taken when autograd is
    off; with autograd on and an input that requires grad the call goes through an
    autograd.Function whose backward runs `moba_backward`.
    """
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        _validate(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
        return _MobaFunction.apply(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
    return moba_forward(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)[0]


@torch.library.custom_op("moba_b200::moba_attn_varlen", mutates_args=(), device_types="cuda")
def _moba_attn_varlen_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                         max_seqlen: int, moba_chunk_size: int, moba_topk: int) -> torch.Tensor:
    return moba_forward(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)[0]


@_moba_attn_varlen_op.register_fake
def _(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk):
    return torch.empty_like(q)


def moba_attn_varlen(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk):
    """The operator under the name the benchmark contract uses; a registered
    torch custom op (``torch.ops.moba_b200.moba_attn_varlen``)."""
    _validate(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
    return _moba_attn_varlen_op(q, k, v, cu_seqlens, max_seqlen, moba_chunk_size, moba_topk)
