"""CPU: the context-parallel entry points' argument checks and the failure-handling pair
moba_cp_poll / moba_cp_abort, against a stand-in NCCL library (tests/fake_nccl.c) so that no
GPU and no real communicator is involved.  Each case runs in a child process because the
library binds NCCL once per process."""
import ctypes as C
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from baselinebenchmark_b200 import _lib, build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfakenccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(out), str(ROOT / "tests" / "fake_nccl.c")], check=True)
    build.build()
    return out


def _child(code, env):
    full = dict(os.environ, **env)
    res = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], cwd=ROOT, env=full, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return res.stdout.strip().splitlines()


def _window_problem(**kw):
    base = dict(total_tokens=4096, batch=1, num_q_heads=8, num_kv_heads=2, head_dim=128, max_seqlen=4096,
                chunk_size=512, topk=3, attend_impl=0, q_stride_token=1024, q_stride_head=128,
                k_stride_token=256, k_stride_head=128, v_stride_token=256, v_stride_head=128,
                o_stride_token=1024, o_stride_head=128, q_token_begin=2048, q_tokens=2048)
    base.update(kw)
    return _lib.Problem(**base)


def test_argument_checks_come_before_any_collective(fake_nccl):
    lib = _lib.lib()
    size = C.c_size_t(0)
    assert lib.moba_cp_workspace_size(C.byref(_window_problem()), C.byref(size)) == 0 and size.value > 0
    assert lib.moba_cp_workspace_size(C.byref(_window_problem(q_tokens=0, q_token_begin=0)), C.byref(size)) == -1
    assert lib.moba_cp_workspace_size(C.byref(_window_problem(batch=2)), C.byref(size)) == -1
    ok = 0x10000
    good = (C.c_int64 * 3)(0, 2048, 4096)
    args = lambda prob, rank, bounds, k=ok: (C.byref(prob), ok, rank, 2, bounds, ok, k, ok, ok, ok, None, None, ok,  # noqa: E731
                                             1 << 40, None, None, None)
    # window of `p` is rank 1's: calling as rank 0 is a shape error; so are unaligned or uncovered bounds
    assert lib.moba_cp_forward(*args(_window_problem(), 0, good)) == -1
    assert lib.moba_cp_forward(*args(_window_problem(), 1, (C.c_int64 * 3)(0, 2000, 4096))) == -1
    assert lib.moba_cp_forward(*args(_window_problem(), 1, (C.c_int64 * 3)(0, 2048, 4000))) == -1
    assert lib.moba_cp_forward(*args(_window_problem(), 1, good, k=ok + 2)) == -6
    assert lib.moba_cp_forward(*args(_window_problem(k_stride_token=512), 1, good)) == -2     # K not contiguous
    assert lib.moba_cp_forward(C.byref(_window_problem()), None, 1, 2, good, ok, ok, ok, ok, ok, None, None, ok, 1 << 40,
                               None, None, None) == -4


def test_poll_reports_the_async_state_and_abort_reaches_nccl(fake_nccl, tmp_path):
    log = tmp_path / "calls.log"
    code = """
        import ctypes as C
        from baselinebenchmark_b200 import _lib
        lib = _lib.lib()
        state = C.c_int32(-1)
        print(lib.moba_cp_poll(0x1234, C.byref(state)), state.value)
        print(lib.moba_cp_abort(0x1234))
        print(lib.moba_cp_poll(None, C.byref(state)))
    """
    out = _child(code, {"MOBA_NCCL_LIB": str(fake_nccl), "FAKE_NCCL_ASYNC_ERROR": "3", "FAKE_NCCL_LOG": str(log)})
    assert out == ["0 3", "0", "-4"]
    assert log.read_text().split() == ["abort"]


def test_missing_nccl_library_is_an_error_code(fake_nccl, tmp_path):
    # a library file without the entry points: binding fails, the calls return MOBA_E_NCCL
    empty = tmp_path / "libempty.so"
    src = tmp_path / "empty.c"
    src.write_text("int nothing_here(void) { return 0; }\n")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(empty), str(src)], check=True)
    code = """
        import ctypes as C
        from baselinebenchmark_b200 import _lib
        lib = _lib.lib()
        state = C.c_int32(0)
        print(lib.moba_cp_poll(0x1234, C.byref(state)))
        print(lib.moba_b200_strerror(-9).decode())
    """
    out = _child(code, {"MOBA_NCCL_LIB": str(empty)})
    assert out[0] == "-9" and "NCCL" in out[1]
