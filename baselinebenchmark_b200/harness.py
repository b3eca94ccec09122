"""Latency harness for the operator, CUDA edition of the reference's
benchmarks/moba_compare.py protocol: inputs built outside the timed region
(seed 42, randn, moba_compare.py:103-109), one untimed first call, `--warmup`
calls, then `--rounds` x `--iterations` timed calls with perf_counter + device
synchronisation per call (:111-128); median / mean / p99 per case in one JSON
report (:39-44).  Like the original it performs no correctness check.

    python -m baselinebenchmark_b200.harness --case cfg2 --rounds 1 --iterations 3
    python -m baselinebenchmark_b200.harness --suite --output results.json
    python -m baselinebenchmark_b200.harness --case cfg3-seq --decode 64      # latency of decode steps

`--suite` runs the reference's case list (moba_compare.py:59-99); a case outside
what this build supports (bf16 or fp16; head_dim 64, 96, 128, 256) would be
reported as skipped.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from dataclasses import asdict, dataclass
from itertools import accumulate

import torch

from . import native_moba
from .parallel import moba_backward, moba_forward, parallel_moba


@dataclass(frozen=True)
class Case:
    name: str
    seq_lens: tuple
    q_heads: int = 16
    kv_heads: int = 16
    head_dim: int = 128
    chunk_size: int = 128
    topk: int = 8
    dtype: str = "bfloat16"
    key_offsets: bool = False      # BASELINE.json configs add a per-chunk offset to the keys


BASELINE_CASES = {
    "cfg0": Case("cfg0", (4096,), 8, 8, 128, 512, 3, key_offsets=True),
    "cfg1": Case("cfg1", (6144, 2560, 7168, 3584), 32, 32, 128, 512, 3, key_offsets=True),
    "cfg2": Case("cfg2", (32768,), 32, 8, 128, 4096, 12, key_offsets=True),
    "cfg3-unit": Case("cfg3-unit", (131072,), 4, 1, 128, 4096, 8, key_offsets=True),
    "cfg3-seq": Case("cfg3-seq", (131072,), 32, 8, 128, 4096, 8, key_offsets=True),     # one of the 16 sequences
}


def reference_suite():
    """The workload list of benchmarks/moba_compare.py:59-99 (same shapes, same names)."""
    cases = [Case(f"length-{n}", (n, n)) for n in (512, 2048, 4096, 8192, 16384)]
    cases += [Case(f"batch-{b}", (4096,) * b) for b in (1, 4)]
    cases += [Case(f"dim-{d}", (4096, 4096), head_dim=d) for d in (64, 96, 256)]
    cases += [Case(f"chunk-{c}", (4096, 4096), chunk_size=c) for c in (64, 256, 512)]
    cases += [Case(f"topk-{k}", (4096, 4096), topk=k) for k in (2, 4, 16)]
    cases += [Case("gqa-16q-4kv", (4096, 4096), kv_heads=4), Case("mqa-16q-1kv", (4096, 4096), kv_heads=1),
              Case("heads-4", (4096, 4096), q_heads=4, kv_heads=4)]
    cases += [Case("fp16-d128", (4096, 4096), dtype="float16"),
              Case("fp16-d64", (4096, 4096), head_dim=64, dtype="float16"),
              Case("fp16-gqa", (4096, 4096), kv_heads=4, dtype="float16")]
    cases += [Case("chunk-boundaries", (127, 128, 129), q_heads=4, kv_heads=4), Case("one-token-tail", (4097, 4097)),
              Case("varlen-gqa", (200, 400, 648), q_heads=8, kv_heads=2), Case("varlen-long", (1023, 4097, 8191)),
              Case("fp16-varlen", (127, 513, 2049), q_heads=8, kv_heads=2, head_dim=64, dtype="float16")]
    cases += [Case(f"long-gqa-{n}", (n,), q_heads=32, kv_heads=8) for n in (32768, 65536)]
    cases += [Case(f"long-c{c}-k{k}", (32768,), q_heads=32, kv_heads=8, chunk_size=c, topk=k)
              for c, k in ((512, 8), (1024, 8), (512, 16))]
    cases += [Case("tokens16k-b1", (16384,)), Case("tokens16k-b8", (2048,) * 8),
              Case("tokens16k-varlen", (1024, 2048, 4096, 9216))]
    cases += [Case(f"length-{n}", (n, n)) for n in (4096, 8192, 16384, 32768, 65536)]
    cases += [Case("topk-1", (4096, 4096), topk=1), Case("topk64-saturated", (512, 512), topk=64),
              Case("topk64-long-gqa", (32768,), q_heads=32, kv_heads=8, topk=64)]
    unique = {}
    for case in cases:
        key = (case.seq_lens, case.q_heads, case.kv_heads, case.head_dim, case.chunk_size, case.topk, case.dtype)
        unique.setdefault(key, case)
    return list(unique.values())


def summary(samples):
    out = {"mean_ms": statistics.mean(samples), "median_ms": statistics.median(samples), "count": len(samples)}
    if len(samples) >= 100:
        out["p99_ms"] = sorted(samples)[int(0.99 * (len(samples) - 1))]
    return out


def make_inputs(case: Case, device):
    torch.manual_seed(42)
    dtype = getattr(torch, case.dtype)
    total = sum(case.seq_lens)
    q = torch.randn(total, case.q_heads, case.head_dim, device=device, dtype=dtype)
    k = torch.randn(total, case.kv_heads, case.head_dim, device=device, dtype=dtype)
    v = torch.randn_like(k)
    if case.key_offsets:
        start = 0
        for n in case.seq_lens:
            nck = -(-n // case.chunk_size)
            off = (torch.randn(nck, case.kv_heads, case.head_dim, device=device) * 0.5).to(dtype)
            k[start:start + n] += off.repeat_interleave(case.chunk_size, 0)[:n]
            start += n
    cu = torch.tensor([0, *accumulate(case.seq_lens)], device=device, dtype=torch.int32)
    return q, k, v, cu


def supported(case: Case) -> bool:
    return case.dtype in ("bfloat16", "float16") and case.head_dim in (64, 96, 128, 256)


def run_case(case: Case, args, device):
    if not supported(case):
        return {**asdict(case), "status": "skipped", "reason": "this build: head_dim 64, 96, 128, 256"}
    q, k, v, cu = make_inputs(case, device)
    call = (q, k, v, cu, max(case.seq_lens), case.chunk_size, case.topk)
    if args.decode:
        return run_decode_case(case, args, call)
    if args.backward:
        return run_backward_case(case, args, call)
    if args.stage == "gating":
        return run_gating_case(case, args, call)
    with torch.inference_mode():
        parallel_moba(*call)
        torch.cuda.synchronize()
        samples = []
        for _ in range(args.rounds):
            for _ in range(args.warmup):
                parallel_moba(*call)
            torch.cuda.synchronize()
            for _ in range(args.iterations):
                t0 = time.perf_counter()
                result = parallel_moba(*call)
                torch.cuda.synchronize()
                samples.append((time.perf_counter() - t0) * 1e3)
                del result
    tokens = sum(case.seq_lens)
    stats = summary(samples)
    return {**asdict(case), "status": "measured", "q_shape": list(q.shape), "kv_shape": list(k.shape),
            "native_sparse_path_eligible": bool(native_moba._supported(q)) and case.topk > 1
            and max(case.seq_lens) > case.chunk_size,
            "latency": stats, "tokens_per_s": tokens / (stats["median_ms"] * 1e-3)}


def run_gating_case(case: Case, args, call):
    """Latency of the gating stage alone through the staged C entry points (chunk means, then
    scores + mask + top-k: routing.py:740-775, :1185-1262), with the counters of the gating
    kernel's decision paths."""
    import ctypes as C
    from . import _lib
    from .parallel import make_problem
    q, k, v, cu, max_seqlen, chunk, topk = call
    prob = make_problem(q, k, v, q, cu, max_seqlen, chunk, topk)          # no output tensor: q stands in for its strides
    dims = _lib.Dims()
    _lib.check(_lib.lib().moba_problem_dims(C.byref(prob), C.byref(dims)))
    if dims.hist <= 0:
        return {**asdict(case), "status": "skipped", "reason": "nothing to select (top-k 1 or one chunk)"}
    means = torch.empty(dims.slots, k.shape[1], k.shape[2], dtype=k.dtype, device=k.device)
    sel = torch.empty(dims.hist, q.shape[1], q.shape[0], dtype=torch.int32, device=q.device)
    counts = torch.zeros(dims.lists, dtype=torch.int32, device=q.device)
    stats = torch.zeros(4, dtype=torch.int32, device=q.device)
    lib = _lib.lib()

    def call_once(with_stats=False):
        st = torch.cuda.current_stream().cuda_stream
        counts.zero_()
        _lib.check(lib.moba_chunk_means(C.byref(prob), k.data_ptr(), cu.data_ptr(), means.data_ptr(), st))
        _lib.check(lib.moba_gate_topk_stats(C.byref(prob), q.data_ptr(), means.data_ptr(), cu.data_ptr(), sel.data_ptr(),
                                            counts.data_ptr(), stats.data_ptr() if with_stats else None, 0, st))

    call_once(True)
    torch.cuda.synchronize()
    st = stats.cpu().tolist()
    samples = []
    for _ in range(args.rounds):
        for _ in range(args.warmup):
            call_once()
        torch.cuda.synchronize()
        for _ in range(args.iterations):
            t0 = time.perf_counter()
            call_once()
            torch.cuda.synchronize()
            samples.append((time.perf_counter() - t0) * 1e3)
    rows = q.shape[0] * q.shape[1]
    return {**asdict(case), "status": "measured", "pass": "gating", "latency": summary(samples), "rows": rows,
            "rows_rechecked": st[0], "rows_ranked_over_all_candidates": st[3],
            "largest_estimate_error_over_bound": st[1] / 65536.0, "bound_violations": st[2]}


def run_decode_case(case: Case, args, call):
    """Latency of single-token decode steps at the end of the case's sequence (incremental.py):
    the prefix is prefilled in one untimed call; then `--decode` steps are timed one by one
    (perf_counter + synchronize per step, like the other cases) and as many again back to back
    between two CUDA events, which gives the device time of a step without the host's launches."""
    from .incremental import IncrementalMoba
    q, k, v, _, _, chunk, topk = call
    n, warm = args.decode, min(args.warmup, 8)
    total = case.seq_lens[0]
    if len(case.seq_lens) != 1 or total <= 2 * n + warm:
        return {**asdict(case), "status": "skipped", "reason": "--decode wants one sequence longer than the steps"}
    with torch.inference_mode():
        inc = IncrementalMoba(total, case.kv_heads, case.head_dim, chunk, topk, dtype=q.dtype, device=q.device)
        at = total - 2 * n - warm
        inc.append(q[:at], k[:at], v[:at])

        def step(t):
            return inc.append(q[t:t + 1], k[t:t + 1], v[t:t + 1])

        for _ in range(warm):
            step(at)
            at += 1
        torch.cuda.synchronize()
        samples = []
        for _ in range(n):
            t0 = time.perf_counter()
            step(at)
            torch.cuda.synchronize()
            samples.append((time.perf_counter() - t0) * 1e3)
            at += 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            step(at)
            at += 1
        e1.record()
        torch.cuda.synchronize()
    return {**asdict(case), "status": "measured", "pass": "decode", "prefix_tokens": total - 2 * n,
            "latency": summary(samples), "back_to_back_ms_per_step": e0.elapsed_time(e1) / n}


def run_backward_case(case: Case, args, call):
    """Latency of `moba_backward` alone (gradients of the training path, parallel.py:149-250)
    on what one forward with LSE and selection returned; same timing protocol."""
    q = call[0]
    with torch.inference_mode():
        out, lse, sel = moba_forward(*call, return_lse=True, return_selected=True)
        dout = torch.randn_like(q)
        samples = []
        for _ in range(args.rounds):
            for _ in range(max(args.warmup, 1)):
                moba_backward(*call, out, lse, sel, dout)
            torch.cuda.synchronize()
            for _ in range(args.iterations):
                t0 = time.perf_counter()
                grads = moba_backward(*call, out, lse, sel, dout)
                torch.cuda.synchronize()
                samples.append((time.perf_counter() - t0) * 1e3)
                del grads
    return {**asdict(case), "status": "measured", "pass": "backward", "latency": summary(samples)}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", action="append", choices=sorted(BASELINE_CASES), help="BASELINE.json workload(s)")
    ap.add_argument("--suite", action="store_true", help="the reference's 40-case list")
    ap.add_argument("--only", action="append", help="with --suite: only the cases of this name (repeatable)")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iterations", type=int, default=25)
    ap.add_argument("--rounds", type=int, default=4)
    ap.add_argument("--backward", action="store_true", help="time moba_backward instead of the forward")
    ap.add_argument("--decode", type=int, default=0, metavar="N",
                    help="time N single-token decode steps at the end of the sequence instead of the prefill")
    ap.add_argument("--stage", choices=["all", "gating"], default="all",
                    help="gating: time chunk means + scores + top-k alone (staged entry points)")
    ap.add_argument("--output")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    device = torch.device("cuda", torch.cuda.current_device())
    suite = reference_suite() if args.suite else []
    if args.only:
        unknown = set(args.only) - {c.name for c in suite}
        if unknown:
            raise SystemExit(f"--only: not in the suite: {sorted(unknown)}")
        suite = [c for c in suite if c.name in args.only]
    cases = [BASELINE_CASES[c] for c in (args.case or [])] + suite
    if not cases:
        cases = [BASELINE_CASES["cfg0"]]
    report = {"schema_version": 4, "timing": "perf_counter + device synchronize per call; inference only",
              "correctness_checked": False, "device": torch.cuda.get_device_name(device),
              "arguments": {"warmup": args.warmup, "iterations": args.iterations, "rounds": args.rounds},
              "cases": []}
    for case in cases:
        res = run_case(case, args, device)
        report["cases"].append(res)
        lat = res.get("latency", {})
        print(f"{case.name:>20}  {res['status']:>8}  median {lat.get('median_ms', float('nan')):9.4f} ms", flush=True)
        torch.cuda.empty_cache()
    text = json.dumps(report, indent=2)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text + "\n")
    return report


if __name__ == "__main__":
    main()
    sys.exit(0)
