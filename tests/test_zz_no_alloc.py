"""GPU: the workspace-free routing entry point.

moba_route_static serves callers that cannot provide scratch memory when they
call (fixed memory pools, call sites where allocation is forbidden): it keeps
the chunk means in an array built into the library.  The test calls it through
the C ABI twice in a row, on two different problems, and requires the selected
chunks to be identical to those of the ordinary entry points
(moba_chunk_means + moba_gate_topk with caller-owned buffers); the second call
reuses the array the first one filled, so stale contents would show up there.
It also checks that an oversized problem is refused instead of overrunning the
array.  The file sorts last so a run that stops at the first failure has
already executed every other test.
"""
import ctypes as C

import pytest
import torch

from baselinebenchmark_b200 import _lib, parallel
from oracle import moba_oracle as O
from tests import gpu_util as G

pytestmark = pytest.mark.gpu


def _route_static(prob, q, k, cu, hist):
    tq = prob.q_tokens if prob.q_tokens > 0 else prob.total_tokens
    sel = torch.full((hist, prob.num_q_heads, tq), -9, dtype=torch.int32, device="cuda")
    rc = _lib.lib().moba_route_static(C.byref(prob), q.data_ptr(), k.data_ptr(), cu.data_ptr(), sel.data_ptr(),
                                      G.stream())
    _lib.check(rc)
    return sel


# (seq_lens, Hq, Hkv, head_dim, chunk, topk, dtype); the second case has 261 chunks and K = 64
CASES = [
    ((1500, 900), 8, 2, 128, 128, 4, torch.bfloat16),
    ((4161,), 4, 4, 128, 16, 64, torch.bfloat16),
    ((700, 333), 4, 2, 64, 64, 5, torch.float16),
]


def test_route_static_matches_workspace_path_twice():
    for lens, hq, hkv, d, chunk, topk, dtype in CASES:
        q, k, v, cu = O.make_inputs(list(lens), hq, hkv, d, chunk, seed=len(lens) + chunk, dtype=dtype)
        qd, kd = q.cuda(), k.cuda()
        cud = torch.from_numpy(cu).cuda()
        prob, _ = G.problem_for(qd, kd, kd, cud, max(lens), chunk, topk)
        hist = G.dims_of(prob).hist
        want, _ = G.gate(prob, qd, G.means(prob, kd, cud), cud)
        got = _route_static(prob, qd, kd, cud, hist)
        torch.cuda.synchronize()
        assert torch.equal(got, want)                                    # integer routing: exact
        # and against the CPU oracle, not only against the sibling entry points
        cu_chunk, _, valid, mc = O.chunk_slots(cu, max(lens), chunk)
        sel_o = O.select_chunks(q, O.chunk_means(k, cu_chunk, valid, chunk), cu, max(lens), chunk, hist)
        assert (got.cpu().numpy() == sel_o).all()


def test_route_static_on_a_query_window():
    """Context-parallel callers pass a window of the queries (q_token_begin / q_tokens) and all
    of K: the selection of the window must equal the same rows of the whole-problem selection."""
    lens, hq, hkv, chunk, topk = (2048,), 4, 2, 128, 4
    q, k, v, cu = O.make_inputs(list(lens), hq, hkv, 128, chunk, seed=17)
    qd, kd = q.cuda(), k.cuda()
    cud = torch.from_numpy(cu).cuda()
    prob, _ = G.problem_for(qd, kd, kd, cud, 2048, chunk, topk)
    hist = G.dims_of(prob).hist
    whole = _route_static(prob, qd, kd, cud, hist)
    lo, hi = 5 * chunk, 11 * chunk
    qw = qd[lo:hi].contiguous()
    wprob = parallel.make_problem(qw, kd, kd, torch.empty_like(qw), cud, 2048, chunk, topk, q_token_begin=lo)
    part = _route_static(wprob, qw, kd, cud, hist)
    torch.cuda.synchronize()
    assert torch.equal(part, whole[:, :, lo:hi])


def test_route_static_refuses_oversized_problem():
    # 2 Mi elements = 16384 (slot, kv head) pairs of 128; ask for more without touching the device
    prob = _lib.Problem(total_tokens=1 << 20, batch=1, num_q_heads=32, num_kv_heads=32, head_dim=128,
                        max_seqlen=1 << 20, chunk_size=1024, topk=4, attend_impl=0,
                        q_stride_token=4096, q_stride_head=128, k_stride_token=4096, k_stride_head=128,
                        v_stride_token=4096, v_stride_head=128, o_stride_token=4096, o_stride_head=128)
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = _lib.lib().moba_route_static(C.byref(prob), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                      dummy.data_ptr(), G.stream())
    assert rc == -8
    assert b"built-in scratch" in _lib.lib().moba_b200_strerror(rc)
