"""Helpers shared by the GPU tests: staged calls through the C ABI."""
import ctypes as C

import numpy as np
import torch

from baselinebenchmark_b200 import _lib, parallel


def to_dev(*tensors):
    return [t.cuda() for t in tensors]


def problem_for(q, k, v, cu, max_seqlen, chunk, topk, impl=None):
    out = torch.empty_like(q)
    return parallel.make_problem(q, k, v, out, cu, max_seqlen, chunk, topk, impl), out


def dims_of(prob):
    d = _lib.Dims()
    _lib.check(_lib.lib().moba_problem_dims(C.byref(prob), C.byref(d)))
    return d


def stream():
    return torch.cuda.current_stream().cuda_stream


def metadata(prob, cu):
    d = dims_of(prob)
    cu_chunk = torch.empty(d.slots + 1, dtype=torch.int32, device="cuda")
    chunk_end = torch.empty(d.slots, dtype=torch.int32, device="cuda")
    valid = torch.empty(d.slots, dtype=torch.int8, device="cuda")
    _lib.check(_lib.lib().moba_chunk_metadata(C.byref(prob), cu.data_ptr(), cu_chunk.data_ptr(),
                                              chunk_end.data_ptr(), valid.data_ptr(), stream()))
    return cu_chunk, chunk_end, valid


def means(prob, k, cu):
    d = dims_of(prob)
    m = torch.empty(d.slots, prob.num_kv_heads, prob.head_dim, dtype=k.dtype, device="cuda")
    _lib.check(_lib.lib().moba_chunk_means(C.byref(prob), k.data_ptr(), cu.data_ptr(), m.data_ptr(), stream()))
    return m


def gate(prob, q, m, cu):
    d = dims_of(prob)
    sel = torch.empty(max(d.hist, 0), prob.num_q_heads, prob.total_tokens, dtype=torch.int32, device="cuda")
    counts = torch.zeros(d.lists, dtype=torch.int32, device="cuda")
    if d.hist > 0:
        _lib.check(_lib.lib().moba_gate_topk(C.byref(prob), q.data_ptr(), m.data_ptr(), cu.data_ptr(),
                                             sel.data_ptr(), counts.data_ptr(), stream()))
    return sel, counts


def gate_stats(prob, q, m, cu, flags=0):
    """moba_gate_topk_stats: (selected, list counts, stats int32[4] as numpy)."""
    d = dims_of(prob)
    tq = prob.q_tokens if prob.q_tokens > 0 else prob.total_tokens
    sel = torch.full((max(d.hist, 0), prob.num_q_heads, tq), -9, dtype=torch.int32, device="cuda")
    counts = torch.zeros(d.lists, dtype=torch.int32, device="cuda")
    stats = torch.zeros(4, dtype=torch.int32, device="cuda")
    if d.hist > 0:
        _lib.check(_lib.lib().moba_gate_topk_stats(C.byref(prob), q.data_ptr(), m.data_ptr(), cu.data_ptr(),
                                                   sel.data_ptr(), counts.data_ptr(), stats.data_ptr(), flags,
                                                   stream()))
    torch.cuda.synchronize()
    return sel, counts, stats.cpu().numpy()


def compact(prob, cu, sel, counts, tile_rows):
    d = dims_of(prob)
    offsets = torch.empty(d.lists + 1, dtype=torch.int32, device="cuda")
    tiles = torch.empty(d.lists + 1, dtype=torch.int32, device="cuda")
    cursors = torch.empty(d.lists, dtype=torch.int32, device="cuda")
    row_list = torch.full((max(d.hist, 0) * d.rows,), -7, dtype=torch.int32, device="cuda")
    plse = torch.zeros(d.rows * d.partials, 2, dtype=torch.float32, device="cuda")   # {lse, 1 / scale}
    _lib.check(_lib.lib().moba_compact_routes(
        C.byref(prob), cu.data_ptr(), sel.data_ptr(), counts.data_ptr(), offsets.data_ptr(), tiles.data_ptr(),
        cursors.data_ptr(), row_list.data_ptr(), plse.data_ptr(), tile_rows, stream()))
    return offsets, tiles, row_list, plse


def rel_stats(out, ref):
    diff = (out.double() - ref.double()).abs()
    return diff.max().item(), diff.mean().item()
