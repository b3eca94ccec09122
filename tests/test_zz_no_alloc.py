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

from baselinebenchmark_b200 import _lib
from oracle import moba_oracle as O
from tests import gpu_util as G

pytestmark = pytest.mark.gpu


def _route_static(prob, q, k, cu, hist):
    sel = torch.full((hist, prob.num_q_heads, prob.total_tokens), -9, dtype=torch.int32, device="cuda")
    rc = _lib.lib().moba_route_static(C.byref(prob), q.data_ptr(), k.data_ptr(), cu.data_ptr(), sel.data_ptr(),
                                      G.stream())
    _lib.check(rc)
    return sel


def test_route_static_matches_workspace_path_twice():
    cases = [((1500, 900), 8, 2, 128, 4), ((4161,), 4, 4, 16, 64)]       # second: 261 chunks, K = 64
    for lens, hq, hkv, chunk, topk in cases:
        q, k, v, cu = O.make_inputs(list(lens), hq, hkv, 128, chunk, seed=len(lens) + chunk)
        qd, kd = q.cuda(), k.cuda()
        cud = torch.from_numpy(cu).cuda()
        prob, _ = G.problem_for(qd, kd, kd, cud, max(lens), chunk, topk)
        hist = G.dims_of(prob).hist
        want, _ = G.gate(prob, qd, G.means(prob, kd, cud), cud)
        got = _route_static(prob, qd, kd, cud, hist)
        torch.cuda.synchronize()
        assert torch.equal(got, want)                                    # integer routing: exact


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
