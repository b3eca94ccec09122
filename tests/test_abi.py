"""CPU: the C-ABI library builds, loads and exports every symbol that
include/moba_b200.h declares; argument validation follows parallel.py:410-443.
No compute entry point is called here."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from baselinebenchmark_b200 import _lib, build, parallel

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def _problem(**kw):
    base = dict(total_tokens=4096, batch=1, num_q_heads=8, num_kv_heads=8, head_dim=128, max_seqlen=4096,
                chunk_size=512, topk=3, attend_impl=0, q_stride_token=1024, q_stride_head=128,
                k_stride_token=1024, k_stride_head=128, v_stride_token=1024, v_stride_head=128,
                o_stride_token=1024, o_stride_head=128)
    base.update(kw)
    return _lib.Problem(**base)


def test_header_symbols_are_exported(lib):
    header = (ROOT / "include" / "moba_b200.h").read_text()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(moba_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.moba_b200_abi_version() == 3


def test_problem_check_codes(lib):
    ok = _problem()
    assert lib.moba_problem_check(C.byref(ok)) == 0
    assert lib.moba_problem_check(C.byref(_problem(num_q_heads=6, num_kv_heads=4))) == -1   # not divisible
    assert lib.moba_problem_check(C.byref(_problem(topk=0))) == -5
    assert lib.moba_problem_check(C.byref(_problem(topk=65))) == -5
    wide = dict(q_stride_token=2048, q_stride_head=256, k_stride_token=2048, k_stride_head=256,
                v_stride_token=2048, v_stride_head=256, o_stride_token=2048, o_stride_head=256)
    assert lib.moba_problem_check(C.byref(_problem(head_dim=256, **wide))) == 0             # its own tcgen05 kernel
    assert lib.moba_problem_check(C.byref(_problem(head_dim=512))) == -1                    # parallel.py:445
    assert lib.moba_problem_check(C.byref(_problem(max_seqlen=0))) == -1
    assert lib.moba_problem_check(C.byref(_problem(q_stride_head=132))) == -6
    assert lib.moba_problem_check(None) == -4
    assert b"topk" in lib.moba_b200_strerror(-5)


def test_head_dims_and_dtypes_accepted(lib):
    for d in (64, 96, 256):
        stride = dict(q_stride_token=8 * d, q_stride_head=d, k_stride_token=8 * d, k_stride_head=d,
                      v_stride_token=8 * d, v_stride_head=d, o_stride_token=8 * d, o_stride_head=d)
        assert lib.moba_problem_check(C.byref(_problem(head_dim=d, attend_impl=1, **stride))) == 0      # mma.sync stage
        assert lib.moba_problem_check(C.byref(_problem(head_dim=d, attend_impl=0, **stride))) == 0
    assert lib.moba_problem_check(C.byref(_problem(head_dim=32, attend_impl=1))) == -2
    assert lib.moba_problem_check(C.byref(_problem(dtype=1))) == 0                           # fp16
    assert lib.moba_problem_check(C.byref(_problem(dtype=2))) == -2
    assert lib.moba_problem_check(C.byref(_problem(reserved=1))) == -2


def test_query_windows_at_any_token_are_accepted(lib):
    """A query window may start and end at any token (decode: one token at the end of the prefix);
    its workspace is sized by the window, not by the prefix."""
    whole, one, odd = C.c_size_t(0), C.c_size_t(0), C.c_size_t(0)
    assert lib.moba_workspace_size(C.byref(_problem()), C.byref(whole)) == 0
    assert lib.moba_workspace_size(C.byref(_problem(q_token_begin=4095, q_tokens=1)), C.byref(one)) == 0
    assert lib.moba_workspace_size(C.byref(_problem(q_token_begin=7, q_tokens=1001)), C.byref(odd)) == 0
    assert 0 < one.value < odd.value < whole.value
    assert lib.moba_problem_check(C.byref(_problem(q_token_begin=4095, q_tokens=2))) == -1     # past the last token
    assert lib.moba_problem_check(C.byref(_problem(q_token_begin=3, q_tokens=0))) == -1


def test_backward_argument_checks(lib):
    need = C.c_size_t(0)
    assert lib.moba_backward_workspace_size(C.byref(_problem(attend_impl=1)), C.byref(need)) == 0
    fwd = C.c_size_t(0)
    assert lib.moba_workspace_size(C.byref(_problem(attend_impl=1)), C.byref(fwd)) == 0
    # the forward keeps its partial rows in fp16, the backward its dq contributions in fp32
    # (same shape: rows x partials x head_dim); + delta and lse per row
    packed = 2 * (2 * 4096 * 8 + 64) * 128 * 2                      # Q and dO rows of the routed lists (hist 2)
    assert need.value == fwd.value + 4096 * 8 * 3 * 128 * 2 + 2 * 4096 * 8 * 4 + packed
    assert lib.moba_backward_workspace_size(C.byref(_problem(q_token_begin=0, q_tokens=512)), C.byref(need)) == -2
    wide = dict(q_stride_token=2048, q_stride_head=256, k_stride_token=2048, k_stride_head=256,
                v_stride_token=2048, v_stride_head=256, o_stride_token=2048, o_stride_head=256)
    assert lib.moba_backward_workspace_size(C.byref(_problem(head_dim=256, attend_impl=1, **wide)), C.byref(need)) == 0
    assert lib.moba_backward(C.byref(_problem()), *([None] * 12), 0, None) == -4             # null pointers


def test_misaligned_pointers_are_refused_before_any_launch(lib):
    """q, k, v and the means are read with 16-byte loads (and K/V through TMA descriptors): a
    base pointer that is not 16-byte aligned returns MOBA_E_ALIGN from every entry point that
    would dereference it.  The check comes before anything touches a device, so fake addresses do."""
    ok, off = 0x10000, 0x10002
    prob = C.byref(_problem())
    assert lib.moba_forward(prob, off, ok, ok, ok, ok, None, None, ok, 1 << 40, None) == -6
    assert lib.moba_forward(prob, ok, ok, off, ok, ok, None, None, ok, 1 << 40, None) == -6
    assert lib.moba_chunk_means(prob, off, ok, ok, None) == -6
    assert lib.moba_chunk_means(prob, ok, ok, off, None) == -6
    assert lib.moba_gate_topk(prob, off, ok, ok, ok, None, None) == -6
    assert lib.moba_gate_topk(prob, ok, off, ok, ok, None, None) == -6
    assert lib.moba_gate_topk_stats(prob, off, ok, ok, ok, None, None, 0, None) == -6
    assert lib.moba_route_static(prob, off, ok, ok, ok, None) == -6
    assert lib.moba_route_static(prob, ok, off, ok, ok, None) == -6
    need = C.c_size_t(0)
    assert lib.moba_backward_workspace_size(prob, C.byref(need)) == 0
    for bad in range(3):                                                 # q, k, v in turn
        ptrs = [ok, ok, ok]
        ptrs[bad] = off
        assert lib.moba_backward(prob, *ptrs, ok, ok, ok, ok, ok, ok, ok, ok, ok, need.value, None) == -6


def test_launch_limits_are_refused_by_the_problem_check(lib):
    """Shapes the launchers could not run are refused up front instead of failing at launch:
    more sequences than a grid dimension holds, and dense-stage work items beyond int32."""
    assert lib.moba_problem_check(C.byref(_problem(batch=65536, total_tokens=65536 * 16, max_seqlen=16, chunk_size=8))) == -2
    assert lib.moba_problem_check(C.byref(_problem(batch=65535, total_tokens=65535 * 16, max_seqlen=16, chunk_size=8))) == 0
    # max_seqlen far above the real lengths: slots * heads * tiles overflows the item counter
    big = _problem(batch=4096, total_tokens=1 << 20, max_seqlen=1 << 22, chunk_size=256, num_q_heads=128, num_kv_heads=1)
    assert lib.moba_problem_check(C.byref(big)) == -2
    # the largest chunk table (16384 chunks per sequence) with top-k 64 still fits the gating kernel
    stride = dict(q_stride_token=2048, q_stride_head=256, k_stride_token=2048, k_stride_head=256,
                  v_stride_token=2048, v_stride_head=256, o_stride_token=2048, o_stride_head=256)
    wide = _problem(total_tokens=16384 * 16, max_seqlen=16384 * 16, chunk_size=16, topk=64, head_dim=256, attend_impl=1, **stride)
    assert lib.moba_problem_check(C.byref(wide)) == 0


def test_dims_follow_reference_formulas(lib):
    d = _lib.Dims()
    assert lib.moba_problem_dims(C.byref(_problem()), C.byref(d)) == 0
    assert (d.chunks_per_seq, d.slots, d.hist, d.partials, d.rows, d.lists) == (8, 8, 2, 3, 4096 * 8, 64)
    assert lib.moba_problem_dims(C.byref(_problem(topk=1)), C.byref(d)) == 0
    assert (d.hist, d.partials) == (0, 1)
    assert lib.moba_problem_dims(C.byref(_problem(max_seqlen=300, topk=64)), C.byref(d)) == 0
    assert (d.chunks_per_seq, d.hist) == (1, 0)                                             # parallel.py:303


def test_workspace_size_and_null_handling(lib):
    size = C.c_size_t(0)
    assert lib.moba_workspace_size(C.byref(_problem()), C.byref(size)) == 0
    assert 4096 * 8 * 3 * 128 * 2 < size.value < 4096 * 8 * 3 * 128 * 4     # fp16 partial rows dominate
    assert lib.moba_workspace_size(C.byref(_problem()), None) == -4
    # null tensors are rejected before anything touches a device
    assert lib.moba_forward(C.byref(_problem()), None, None, None, None, None, None, None, None, 0, None) == -4
    assert lib.moba_attend_tile_rows(_lib.ATTEND_TCGEN05) == 256
    assert lib.moba_attend_tile_rows(_lib.ATTEND_MMA_SYNC) == 128
    assert [lib.moba_attend_tile_rows_for(_lib.ATTEND_TCGEN05, d) for d in (64, 96, 128, 256)] == [256, 256, 256, 128]
    assert lib.moba_attend_tile_rows_for(_lib.ATTEND_MMA_SYNC, 256) == 128
    assert lib.moba_problem_tile_rows(C.byref(_problem())) == 256                       # chunk 512
    assert lib.moba_problem_tile_rows(C.byref(_problem(chunk_size=128))) == 128         # short items: their own kernel
    assert lib.moba_problem_tile_rows(C.byref(_problem(chunk_size=128, attend_impl=1))) == 128
    assert lib.moba_problem_tile_rows(C.byref(_problem(topk=0))) == -5


def _cpu_args(t=64, hq=4, hkv=2, d=128, dtype=torch.bfloat16):
    q = torch.zeros(t, hq, d, dtype=dtype)
    k = torch.zeros(t, hkv, d, dtype=dtype)
    return q, k, k.clone(), torch.tensor([0, t], dtype=torch.int32)


def test_host_validation_mirrors_reference():
    q, k, v, cu = _cpu_args()
    with pytest.raises(ValueError, match="accelerator tensors"):
        parallel.parallel_moba(q, k, v, cu, 64, 32, 2)          # CPU tensors, parallel.py:416-417
    with pytest.raises(ValueError, match="shape \\[tokens, heads, head_dim\\]"):
        parallel.parallel_moba(q[0], k, v, cu, 64, 32, 2)
    with pytest.raises(ValueError, match="identical shapes"):
        parallel.parallel_moba(q, k, v[:, :1], cu, 64, 32, 2)
    with pytest.raises(ValueError, match="same token count"):
        parallel.parallel_moba(q[:32], k, v, cu, 64, 32, 2)


def test_host_validation_value_checks(monkeypatch):
    """Checks that come after the device check, exercised on fake 'cuda' metadata."""
    q, k, v, cu = _cpu_args()

    class Dev:
        type = "cuda"

        def __eq__(self, other):
            return True

        def __ne__(self, other):
            return False

    class T:
        def __init__(self, t):
            self._t = t
            self.device = Dev()

        def __getattr__(self, name):
            return getattr(self._t, name)

    fq, fk, fv, fcu = T(q), T(k), T(v), T(cu)
    with pytest.raises(TypeError, match="same dtype"):
        parallel._validate(fq, T(k.half()), fv, fcu, 64, 32, 2)
    with pytest.raises(TypeError, match="only float16 and bfloat16"):
        parallel._validate(T(q.float()), T(k.float()), T(v.float()), fcu, 64, 32, 2)
    with pytest.raises(TypeError, match="int32"):
        parallel._validate(fq, fk, fv, T(cu.long()), 64, 32, 2)
    with pytest.raises(ValueError, match="max_seqlen"):
        parallel._validate(fq, fk, fv, fcu, 0, 32, 2)
    with pytest.raises(ValueError, match="moba_chunk_size"):
        parallel._validate(fq, fk, fv, fcu, 64, 0, 2)
    with pytest.raises(ValueError, match="moba_topk must be a positive int"):
        parallel._validate(fq, fk, fv, fcu, 64, 32, 0)
    with pytest.raises(ValueError, match="<= 64"):
        parallel._validate(fq, fk, fv, fcu, 64, 32, 65)
    with pytest.raises(ValueError, match="divisible"):
        parallel._validate(T(q[:, :3]), fk, fv, fcu, 64, 32, 2)
    parallel._validate(T(q.half()), T(k.half()), T(v.half()), fcu, 64, 32, 2)      # float16 is built
    parallel._validate(T(q[..., :64]), T(k[..., :64]), T(v[..., :64]), fcu, 64, 32, 2)   # head_dim 64 is built
    with pytest.raises(NotImplementedError):
        parallel._validate(T(q[..., :32]), T(k[..., :32]), T(v[..., :32]), fcu, 64, 32, 2)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libmoba_b200.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.lib()
