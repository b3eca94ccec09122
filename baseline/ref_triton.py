"""Loads the reference's own MoBA package (installed by baseline/install_ref.py) on a CUDA
device and runs its inference path through its Triton kernels: the path the reference takes
on every device that is not a Moore Threads MP31 (`native_moba._supported` is false there,
native_moba.py:29-32, so `routed` and `varlen` fall through to attention.py, :120-124,
:143-146).

Test and measurement infrastructure only; the product never imports this module.

The reference files are loaded unmodified.  One stand-in makes them importable off the
vendor stack: `triton.language.extra.musa` (absent from stock Triton, imported by
attention.py:20) is provided as a module whose `libdevice` is Triton's CUDA libdevice, the
same functions under the same names.  The reference indexes with int32
(routing.py:1094-1100): callers keep T * Hq * D below 2^31 per call.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref" / "moba"
_mods = None


def available() -> str | None:
    """None when the reference can be loaded here, otherwise the reason it cannot."""
    if not (REF_DIR / "parallel.py").exists():
        return f"{REF_DIR} is missing (python baseline/install_ref.py <reference checkout>)"
    try:
        import torch
        import triton  # noqa: F401
    except Exception as exc:  # pragma: no cover
        return f"triton / torch not importable: {exc}"
    if not torch.cuda.is_available():
        return "no CUDA device"
    return None


def load():
    """(parallel, routing, attention) modules of the reference package."""
    global _mods
    if _mods is not None:
        return _mods
    why = available()
    if why:
        raise RuntimeError(why)
    from triton.language.extra.cuda import libdevice
    fake = types.ModuleType("triton.language.extra.musa")
    fake.libdevice = libdevice
    sys.modules.setdefault("triton.language.extra.musa", fake)
    spec = importlib.util.spec_from_file_location("_ref_moba_cuda", REF_DIR / "__init__.py",
                                                  submodule_search_locations=[str(REF_DIR)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    _mods = tuple(sys.modules[f"{spec.name}.{n}"] for n in ("parallel", "routing", "attention"))
    return _mods


def routing(q, k, cu_seqlens, max_seqlen, chunk, topk, means=None):
    """The reference's slot tables, chunk means and selected chunks for these CUDA tensors
    (routing.py:595-632, :740-775, :1185-1262).  `means` replaces its own chunk means as the
    input of its top-k kernel.  Returns (chunk_means, selected[hist, Hq, T]) or (means, None)
    when nothing is selected."""
    import torch
    par, rt, _ = load()
    with torch.inference_mode():
        cu_chunk, chunk_end, _, valid, mc = rt._build_dense_chunk_metadata_triton(cu_seqlens, max_seqlen, chunk)
        hist = min(topk - 1, mc - 1)
        own = rt._compute_dense_chunk_means_triton(k, cu_chunk, valid, chunk)
        if hist <= 0:
            return own, None
        sel = rt._compute_selected_chunks_batched_streaming_triton(
            q, own if means is None else means, chunk_end, cu_seqlens, max_seqlen, mc, hist)
    return own, sel


def forward(q, k, v, cu_seqlens, max_seqlen, chunk, topk):
    """The reference's inference forward (parallel.py:253-374)."""
    import torch
    par, _, _ = load()
    with torch.inference_mode():
        return par._moba_attn_varlen_inference(q, k, v, cu_seqlens, max_seqlen, chunk, topk)


def time_forward(q, k, v, cu_seqlens, max_seqlen, chunk, topk, warmup=2, iters=5):
    """Median milliseconds per call of the reference forward, CUDA events, after `warmup`
    calls (the first one compiles the kernels)."""
    import statistics
    import torch
    for _ in range(warmup):
        forward(q, k, v, cu_seqlens, max_seqlen, chunk, topk)
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        forward(q, k, v, cu_seqlens, max_seqlen, chunk, topk)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)
