"""Generate tests/golden/forward_*.npz by executing the reference's own MoBA package
(backends/_mthreads/ops/moba) end to end on CPU with the Triton interpreter: the inference
forward `_moba_attn_varlen_inference` (parallel.py:253-374: slot tables, own-chunk attention,
chunk means, top-k, route building, routed attention, LSE merge) and the training path
`parallel_moba` under autograd with its backward (parallel.py:59-250, attention.py:163-369).
Run in the build container only (needs the reference checkout; about a minute per case):

    TRITON_INTERPRET=1 python tests/golden/make_forward_golden.py /path/to/reference

The reference files are loaded unmodified.  Three stand-ins on the harness side make them run
without the vendor stack:
  * `triton.language.extra.musa.libdevice` (absent from stock Triton) is replaced by jitted
    wrappers of tl.exp / tl.log / tl.log2 / tl.exp2, the functions attention.py calls
    (attention.py:47-50, :155, :706, :853-857);
  * autotuned kernels (attention.py:775-789, routing.py gather kernel) are launched with their
    first configuration: the autotuner needs a GPU driver, and the configurations differ in
    tile width and warps only, not in the values computed;
  * `is_accelerator_tensor` (routing.py:31-32) is overridden so that CPU tensors pass the
    device check of `parallel_moba`.
As for the routing fixtures, the interpreter mishandles bfloat16, so inputs are drawn, rounded
to bf16, checked to be exactly representable in float16 and the reference runs on the float16
copy: the same real numbers in both dtypes.

Recorded per case: q, k, v, dout (float16), `out_ref` of the inference path, `out_train_ref`
of the training forward, and `dq_ref`, `dk_ref`, `dv_ref` of its backward (all float16).
"""
import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

os.environ.setdefault("TRITON_INTERPRET", "1")

import triton  # noqa: E402
import triton.language as tl  # noqa: E402

CASES = {
    # name: (seq_lens, Hq, Hkv, D, chunk, topk)
    "gqa_varlen_d64": ((130, 126), 4, 2, 64, 32, 3),
    "tail_d128": ((97, 160), 2, 2, 128, 32, 4),
    "k1_local_d64": ((100,), 2, 1, 64, 32, 1),
    "mqa_k64_d64": ((200,), 4, 1, 64, 16, 64),
}


@triton.jit
def _exp(x):
    return tl.exp(x)


@triton.jit
def _exp2(x):
    return tl.exp2(x)


@triton.jit
def _log(x):
    return tl.log(x)


@triton.jit
def _log2(x):
    return tl.log2(x)


class _FirstConfig:
    """Launches an autotuned kernel with one fixed configuration."""

    def __init__(self, fn, **meta):
        self.fn, self.meta = fn, meta

    def __getitem__(self, grid):
        return lambda *args, **kwargs: self.fn[grid](*args, **kwargs, **self.meta)


def load_reference(ref_root: Path):
    from triton.runtime.autotuner import Autotuner
    fake = types.ModuleType("triton.language.extra.musa")
    fake.libdevice = types.SimpleNamespace(exp=_exp, exp2=_exp2, log=_log, log2=_log2)
    sys.modules["triton.language.extra.musa"] = fake
    pkg = ref_root / "backends/_mthreads/ops/moba"
    spec = importlib.util.spec_from_file_location("_ref_moba", pkg / "__init__.py",
                                                  submodule_search_locations=[str(pkg)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    mods = [sys.modules["_ref_moba." + n] for n in ("parallel", "attention", "routing", "native_moba")]
    for m in mods:
        for name, obj in list(vars(m).items()):
            if isinstance(obj, Autotuner):
                setattr(m, name, _FirstConfig(obj.fn, **obj.configs[0].kwargs))
        if hasattr(m, "is_accelerator_tensor"):
            m.is_accelerator_tensor = lambda t: True
    return mods[0]


def make_case(seq_lens, hq, hkv, d, chunk, seed):
    g = torch.Generator().manual_seed(seed)
    total = sum(seq_lens)
    q = torch.randn(total, hq, d, generator=g)
    k = torch.randn(total, hkv, d, generator=g)
    v = torch.randn(total, hkv, d, generator=g)
    dout = torch.randn(total, hq, d, generator=g)
    start = 0
    for n in seq_lens:
        nck = (n + chunk - 1) // chunk
        off = torch.randn(nck, hkv, d, generator=g) * 0.5
        k[start:start + n] += off.repeat_interleave(chunk, 0)[:n]
        start += n
    outs = []
    for x in (q, k, v, dout):
        x = x.bfloat16()
        x = torch.where(x.float().abs() < 2.0 ** -14, torch.zeros_like(x), x)   # float16 normal range
        assert (x.half().float() == x.float()).all()
        outs.append(x.half())
    cu = np.concatenate([[0], np.cumsum(seq_lens)]).astype(np.int32)
    return (*outs, cu)


def main():
    ref_root = Path(sys.argv[1])
    par = load_reference(ref_root)
    out_dir = Path(__file__).parent
    for i, (name, (lens, hq, hkv, d, chunk, topk)) in enumerate(CASES.items()):
        q, k, v, dout, cu = make_case(lens, hq, hkv, d, chunk, 100 + i)
        cut = torch.from_numpy(cu)
        with torch.no_grad():
            out = par._moba_attn_varlen_inference(q, k, v, cut, max(lens), chunk, topk)
        qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
        out_train = par.parallel_moba(qg, kg, vg, cut, max(lens), chunk, topk)
        out_train.backward(dout)
        np.savez_compressed(
            out_dir / f"forward_{name}.npz",
            seq_lens=np.asarray(lens), hq=hq, hkv=hkv, d=d, chunk=chunk, topk=topk, cu_seqlens=cu,
            q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=dout.numpy(),
            out_ref=out.numpy(), out_train_ref=out_train.detach().numpy(),
            dq_ref=qg.grad.numpy(), dk_ref=kg.grad.numpy(), dv_ref=vg.grad.numpy())
        print(name, "done", tuple(out.shape), flush=True)


if __name__ == "__main__":
    main()
