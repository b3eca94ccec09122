#!/usr/bin/env python
"""Benchmark of the B200 MoBA prefill forward.

    python bench.py --gpus N --steps K --warmup W            (N > 1: under torchrun)
    python bench.py --impl reference --gpus N --steps K --warmup W

Workload (BASELINE.json configs[3], "batched GQA prefill sharded by (sequence,
KV-head group)"): 16 sequences of 131072 tokens with 32 query / 8 KV heads,
head_dim 128, bf16, chunk 4096, top-k 8, causal = 128 independent (sequence,
KV-head group) units.  The WHOLE config runs at every N (strong scaling): rank r
holds 16 / N sequences with all their heads and processes them two sequences (16
units) per operator call, 8 / N calls per step, no collective.  Inputs are
synthetic: q, k, v ~ N(0,1) plus a N(0, 0.5^2) offset per (sequence, chunk, kv
head) on the keys, generated on the device from a seed.

Printed JSON (one line, rank 0): tokens/s with inputs resident in HBM (`value`),
the same through the C ABI with pinned HOST buffers (`e2e`), the dense-stage
roofline from CUDA events recorded between the kernels of the timed steps, the
CPU baseline, clocks sampled during the timed region, and under `also`: the 32K
GQA prefill (configs[2]) with its backward, the million-token context-parallel
prefill (configs[4]) on the same N GPUs, and the reference's own Triton path
timed on this GPU when its copy is present (baseline/install_ref.py).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEQ_LEN = 131072
NUM_SEQS = 16             # BASELINE.json configs[3]
SEQS_PER_CALL = 2         # sequences per operator call (16 units: 18 GB of partial results)
HQ, HKV, D, CHUNK, TOPK = 32, 8, 128, 4096, 8
KERNELS_PER_CALL = 6      # chunk_mean, gate_topk, scan_lists, scatter_routes, attend, merge
# dram__bytes_read.sum + dram__bytes_write.sum of one attend_tc5_kernel launch on configs[2]
# (32768 tokens x 32 heads, 8 partial results per row), from an ncu capture of that launch
ATTEND_TRAFFIC_CFG2 = 2.610216e9 + 1.323296e9
PARTIALS = min(TOPK - 1, SEQ_LEN // CHUNK - 1) + 1


def cdiv(a, b):
    return (a + b - 1) // b


def attention_flops(seq_lens, hq, d, chunk, topk):
    pairs = 0
    for n in seq_lens:
        for j in range(cdiv(n, chunk)):
            ln = min(chunk, n - j * chunk)
            pairs += ln * (ln + 1) // 2 + ln * min(topk - 1, j) * chunk
    return 4.0 * d * hq * pairs


def gating_roofline(ms, pk):
    """Gating stage (chunk means + scores + top-k) against the HBM roofline: algorithmic bytes =
    read Q and K once, write and re-read the chunk means, write the selection."""
    tokens = SEQS_PER_CALL * SEQ_LEN
    slots = SEQS_PER_CALL * (SEQ_LEN // CHUNK)
    nbytes = 2 * tokens * HQ * D + 2 * tokens * HKV * D + 2 * 2 * slots * HKV * D + 4 * (PARTIALS - 1) * HQ * tokens
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "algorithmic_bytes": nbytes, "ms": ms, "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s",
            "frac": gbs / pk["hbm"], "per": "operator call (2 sequences)"}


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return dict(burst=float(p["bf16_tflops"]), sustained=float(p["bf16_tflops_sustained"]),
                    hbm=float(p["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def make_inputs_device(seq_lens, hq, hkv, d, chunk, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    total = sum(seq_lens)
    q = torch.randn(total, hq, d, generator=g, device=device, dtype=torch.float32).bfloat16()
    k = torch.empty(total, hkv, d, device=device, dtype=torch.bfloat16)
    v = torch.randn(total, hkv, d, generator=g, device=device, dtype=torch.float32).bfloat16()
    start = 0
    for n in seq_lens:                      # keys: N(0,1) + one offset vector per (chunk, kv head)
        kk = torch.randn(n, hkv, d, generator=g, device=device, dtype=torch.float32)
        off = torch.randn(cdiv(n, chunk), hkv, d, generator=g, device=device, dtype=torch.float32) * 0.5
        kk += off.repeat_interleave(chunk, 0)[:n]
        k[start:start + n] = kk.bfloat16()
        start += n
    cu = torch.tensor(np.concatenate([[0], np.cumsum(seq_lens)]), dtype=torch.int32, device=device)
    return q, k, v, cu


class Runner:
    """Holds problem, workspace and events for repeated calls through the C ABI."""

    def __init__(self, q, k, v, cu, max_seqlen, chunk, topk, q_token_begin=None, ws=None, out=None):
        from baselinebenchmark_b200 import _lib, parallel
        self.lib, self._lib = _lib.lib(), _lib
        self.q, self.k, self.v, self.cu = q, k, v, cu
        self.out = torch.empty_like(q) if out is None else out
        self.prob = parallel.make_problem(q, k, v, self.out, cu, max_seqlen, chunk, topk,
                                          q_token_begin=q_token_begin)
        need = parallel.workspace_bytes(self.prob)
        self.ws = ws if ws is not None and ws.numel() >= need else torch.empty(need, dtype=torch.uint8, device=q.device)

    def step(self, events=None):
        stream = torch.cuda.current_stream().cuda_stream
        if events is None:
            rc = self.lib.moba_forward(C.byref(self.prob), self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                                       self.cu.data_ptr(), self.out.data_ptr(), None, None, self.ws.data_ptr(),
                                       self.ws.numel(), stream)
        else:
            arr = (C.c_void_p * 6)(*[e.cuda_event for e in events])
            rc = self.lib.moba_forward_events(C.byref(self.prob), self.q.data_ptr(), self.k.data_ptr(),
                                              self.v.data_ptr(), self.cu.data_ptr(), self.out.data_ptr(), None, None,
                                              self.ws.data_ptr(), self.ws.numel(), stream, arr)
        self._lib.check(rc)


class MultiRunner:
    """A step made of several operator calls that share one workspace (the calls of a rank's
    share of config 3, or the query windows of config 4 a rank runs in turn)."""

    def __init__(self, runners):
        self.runners = runners

    def step(self, events=None):
        for i, r in enumerate(self.runners):
            r.step(None if events is None else events[i])


def new_events(n):
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
    for e in evs:
        e.record()                          # materialises the cudaEvent_t handle
    return evs


def timed_steps(runner, steps, warmup, barrier, calls=1):
    """Times `steps` steps after `warmup`; returns (total ms, mean stage ms per call [5])."""
    multi = isinstance(runner, MultiRunner)
    for _ in range(warmup):
        runner.step()
    per_step = [[new_events(6) for _ in range(calls)] for _ in range(steps)]
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    for evs in per_step:
        runner.step(evs if multi else evs[0])
    torch.cuda.synchronize()
    barrier()
    total_ms = per_step[0][0][0].elapsed_time(per_step[-1][-1][5])
    stage_ms = [[evs[i].elapsed_time(evs[i + 1]) for i in range(5)] for step in per_step for evs in step]
    return total_ms, np.asarray(stage_ms).mean(0)


def pin_to_gpu_numa_node(index):
    """Best effort: run this process on the CPUs next to its GPU, so that the pinned host buffers
    of the end-to-end leg are allocated (first touch) on the NUMA node the GPU hangs off and the
    copies of eight ranks do not all cross the same socket link.  The CPU list comes from the
    driver's topology table (`nvidia-smi topo -m`, column "CPU Affinity").  Returns the list it
    pinned to (as text) or None."""
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
        header = None
        for line in out.splitlines():
            clean = line.replace("\x1b[4m", "").replace("\x1b[0m", "")
            cells = [c.strip() for c in clean.split("\t")]
            if header is None and any(c == "CPU Affinity" for c in cells):
                header = cells
                continue
            if header is not None and cells and cells[0] == f"GPU{index}":
                spec = cells[header.index("CPU Affinity")]
                cpus = set()
                for part in spec.split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
                cpus &= os.sched_getaffinity(0)
                if cpus:
                    os.sched_setaffinity(0, cpus)
                    return spec
                return None
    except Exception:
        pass
    return None


class HostRunner:
    """The same operator through moba_forward_host: pinned host tensors in, pinned host result
    out.  A step is `calls` calls (the rank's share of the config, two sequences per call); the
    host side keeps one two-sequence slab of inputs and one of results and every call copies
    its inputs from the former and its result into the latter, so the bytes crossing PCIe per
    step are those of the whole share while the pinned memory stays at 5.4 GB per rank.
    Calls alternate between two (stream, workspace) pairs, the way a host that feeds the
    operator continuously would: the entry point is re-entrant for distinct pairs, so the first
    copies in of a call run while the call before it computes and its last copy out while the
    next one does (the copies out of all calls pass through one copy stream of the library, in
    order, so the shared result slab is written by one copy at a time)."""

    def __init__(self, prob, q, k, v, cu, calls):
        from baselinebenchmark_b200 import _lib
        self.lib, self._lib, self.prob, self.calls = _lib.lib(), _lib, prob, calls
        size = C.c_size_t(0)
        _lib.check(self.lib.moba_workspace_size_host(C.byref(self.prob), C.byref(size)))
        self.ws = [torch.empty(size.value, dtype=torch.uint8, device=q.device) for _ in range(2)]
        self.streams = [torch.cuda.Stream(device=q.device) for _ in range(2)]
        self.hq, self.hk, self.hv = (torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (q, k, v))
        for h, t in ((self.hq, q), (self.hk, k), (self.hv, v)):
            h.copy_(t)
        self.hcu = cu.cpu().pin_memory()
        self.hout = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
        self.h2d = calls * sum(t.numel() * t.element_size() for t in (self.hq, self.hk, self.hv, self.hcu))
        self.d2h = calls * self.hout.numel() * self.hout.element_size()
        self.issued = 0

    def begin(self):
        """The two streams start after what is queued on the current stream (the start event)."""
        for s in self.streams:
            s.wait_stream(torch.cuda.current_stream())

    def step(self):
        for _ in range(self.calls):
            i = self.issued & 1
            self.issued += 1
            rc = self.lib.moba_forward_host(C.byref(self.prob), self.hq.data_ptr(), self.hk.data_ptr(),
                                            self.hv.data_ptr(), self.hcu.data_ptr(), self.hout.data_ptr(), None, None,
                                            self.ws[i].data_ptr(), self.ws[i].numel(), self.streams[i].cuda_stream)
            self._lib.check(rc)

    def end(self):
        """The current stream (the stop event) waits for the last copy out of both streams."""
        for s in self.streams:
            torch.cuda.current_stream().wait_stream(s)


def cpu_sample(threads):
    """CPU baseline on a bounded sample of the workload: one whole (sequence,
    KV-head group) unit of the 128, about 15 s on 16 host threads."""
    from oracle import moba_cpu, moba_oracle
    torch.set_num_threads(threads)
    q, k, v, cu = moba_oracle.make_inputs([SEQ_LEN], HQ // HKV, 1, D, CHUNK, seed=7)
    t0 = time.perf_counter()
    _, done = moba_cpu.moba_forward_cpu(q, k, v, cu, SEQ_LEN, CHUNK, TOPK)
    dt = time.perf_counter() - t0
    # a benchmark token carries all 32 query heads; the sample evaluated 4 of them
    tokens_equiv = int(done.sum()) * (HQ // HKV) / HQ
    return tokens_equiv / dt, dt, ("one whole (sequence, KV-group) unit of the 128: 131072 tokens, 4 query heads, "
                                   "1 kv head; rate counted in whole tokens (32 heads)")


def reference_arm(args, rank):
    """The reference has no CPU implementation of this path and its kernels need a
    vendor device; the arm times the oracle's PyTorch-CPU port on the host cores."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rates, secs = [], []
    sample = ""
    for i in range(args.warmup + args.steps):
        r, dt, sample = cpu_sample(threads)
        if i >= args.warmup:
            rates.append(r); secs.append(dt)
    value = sum(rates) / len(rates)
    line = {
        "impl": "reference", "metric": "MoBA prefill tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(secs) / len(secs), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


CP_TOKENS, CP_TOPK, CP_WINDOWS = 1048576, 16, 8


def context_block(steps, warmup, rank, world, local, dev, dist):
    """BASELINE.json configs[4]: one sequence of 1048576 tokens, 32/8 heads, chunk 4096, top-k 16,
    as 8 contiguous query windows of 131072 tokens.  With 8 GPUs every rank owns one window and
    its K/V rows (with 4 or 2: two or four windows each) and a step = exchange of K and V over
    NCCL + the operator on the rank's windows.  With 1 GPU the partial results of all eight
    windows do not fit, so the rank runs the windows in turn on K and V that are resident in
    full (no exchange): the same work, which gives the 1 -> 8 curve its base.  Returns the dict
    for `also` (all ranks must call; rank 0 gets the numbers)."""
    from baselinebenchmark_b200 import sharding
    per_rank = CP_WINDOWS // world if world <= CP_WINDOWS else 0
    if per_rank == 0:
        return None
    win = CP_TOKENS // CP_WINDOWS
    tq = win * per_rank
    exchange = world >= 2
    q, k_loc, v_loc, _ = make_inputs_device([tq], HQ, HKV, D, CHUNK, 46000 + rank, dev)
    out = torch.empty_like(q)
    if exchange:
        # one call per step over the rank's whole token range; its own K/V rows live in place
        cp = sharding.ContextParallel(CP_TOKENS, HKV, D, CHUNK, torch.bfloat16, dev)
        cp.k_rows.copy_(k_loc)
        cp.v_rows.copy_(v_loc)
        del k_loc, v_loc
        calls = 1
        state = {"ws": None}

        def step(evs=None):
            cp.forward(q, CP_TOPK, out=out, workspace=state["ws"], events=None if evs is None else evs[0])
            state["ws"] = cp.workspace
    else:
        cu = torch.tensor([0, CP_TOKENS], dtype=torch.int32, device=dev)
        k_full = torch.empty(CP_TOKENS, HKV, D, dtype=torch.bfloat16, device=dev)
        v_full = torch.empty_like(k_full)
        for w in range(CP_WINDOWS):                          # resident K/V: any values of the right distribution
            _, kk, vv, _ = make_inputs_device([win], 1, HKV, D, CHUNK, 46100 + w, dev)
            k_full[w * win:(w + 1) * win], v_full[w * win:(w + 1) * win] = kk, vv
        runners, ws = [], None
        for w in range(per_rank):
            lo = (rank * per_rank + w) * win
            r = Runner(q[w * win:(w + 1) * win], k_full, v_full, cu, CP_TOKENS, CHUNK, CP_TOPK, q_token_begin=lo, ws=ws,
                       out=out[w * win:(w + 1) * win])
            ws = r.ws
            runners.append(r)
        multi = MultiRunner(runners)
        calls = per_rank
        step = multi.step

    for _ in range(warmup):
        step()
    per_step = [[new_events(6) for _ in range(calls)] for _ in range(steps)]
    e0, e1 = new_events(2)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        e0.record()
        for evs in per_step:
            step(evs)
        e1.record()
        torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    all_calls = [evs for st in per_step for evs in st]
    mine = [e0.elapsed_time(e1) / steps,
            sum(evs[0].elapsed_time(evs[5]) for evs in all_calls) / steps,   # operator (with the wait for K/V, if any)
            sum(evs[0].elapsed_time(evs[2]) for evs in all_calls) / steps,   # means (+ their exchange) + gating
            sum(evs[3].elapsed_time(evs[4]) for evs in all_calls) / steps,   # dense stage
            sum(evs[2].elapsed_time(evs[3]) for evs in all_calls) / steps]   # compaction + wait for K/V rows
    t = torch.tensor(mine, dtype=torch.float64, device=dev)
    tmax, tmin = t.clone(), t.clone()
    if dist is not None:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
    step_ms, op_ms, gate_ms, dense_ms, compact_wait_ms = (float(x) for x in tmax)
    flops = attention_flops([CP_TOKENS], HQ, D, CHUNK, CP_TOPK)
    pk = peaks()
    return {
        "workload": "BASELINE.json configs[4]: 1 sequence x 1048576 tokens, 32 q / 8 kv heads, head_dim 128, chunk "
                    f"4096, top-k 16, causal; 8 query windows of 131072 tokens, {per_rank} per GPU on {world} GPU(s); "
                    + ("through moba_cp_forward: chunk means exchanged, then K and V rows of the earlier ranks "
                       "received over NCCL on a side stream while the gating runs" if exchange else
                       "K and V resident in full, no exchange; the windows run in turn (the partial results of all "
                       "eight at once would not fit)"),
        "n_gpus": world, "steps": steps, "warmup": warmup, "scaling": "strong",
        "tokens_per_s": CP_TOKENS / (step_ms * 1e-3), "ms_per_step": step_ms,
        "tflops_effective": flops / (step_ms * 1e-3) / 1e12,
        "frac_of_bf16_peak": flops / (step_ms * 1e-3) / 1e12 / (pk["sustained"] * world),
        "operator_ms": op_ms, "gate_ms": gate_ms, "dense_ms": dense_ms,
        "compaction_and_kv_wait_ms": compact_wait_ms,
        "compaction_and_kv_wait_note": "between the gating and the dense stage: route compaction plus, with an "
                                       "exchange, whatever of the K/V transfer outlasted the gating",
        "per_rank_step_ms": {"max": float(tmax[0]), "min": float(tmin[0])},
        "per_rank_dense_ms": {"max": float(tmax[3]), "min": float(tmin[3])},
        "gpu_launches": KERNELS_PER_CALL * calls * steps, "clocks": clocks.summary(),
    }


def workload_config(n_gpus):
    per = NUM_SEQS // n_gpus
    return {"workload": "BASELINE.json configs[3], the whole config at every N (strong scaling): 16 sequences x 131072 "
                        "tokens, 32 q / 8 kv heads, head_dim 128, chunk 4096, top-k 8, causal = 128 (sequence, "
                        f"KV-head group) units; {per} sequences ({per * HKV} units) per GPU at {n_gpus} GPU(s), "
                        f"{SEQS_PER_CALL} sequences per operator call",
            "tokens_per_gpu": SEQ_LEN * per, "calls_per_step": per // SEQS_PER_CALL,
            "parallelism": f"units x{n_gpus}, no collective",
            "l2": "inputs (3 GiB per operator call) exceed the 126 MB L2"}


def reference_triton_block(dev):
    """Informational: the reference's own Triton path (what it runs off Moore Threads hardware)
    on this GPU, next to this build, on configs[2] and three cases of its benchmark list."""
    try:
        from baseline import ref_triton
    except Exception as exc:                                  # noqa: BLE001
        return {"unavailable": f"{exc}"}
    why = ref_triton.available()
    if why:
        return {"unavailable": why}
    from baselinebenchmark_b200 import harness, parallel
    cases = [harness.BASELINE_CASES["cfg2"]] + [c for c in harness.reference_suite()
                                                 if c.name in ("length-16384", "long-gqa-32768", "long-c512-k8")]
    out = {}
    for case in cases:
        try:
            q, k, v, cu = harness.make_inputs(case, dev)
            call = (q, k, v, cu, max(case.seq_lens), case.chunk_size, case.topk)
            ref_ms = ref_triton.time_forward(*call, warmup=2, iters=5)
            with torch.inference_mode():
                for _ in range(3):
                    parallel.parallel_moba(*call)
                e0, e1 = new_events(2)
                e0.record()
                for _ in range(10):
                    parallel.parallel_moba(*call)
                e1.record()
                torch.cuda.synchronize()
            ours_ms = e0.elapsed_time(e1) / 10
            out[case.name] = {"reference_triton_ms": ref_ms, "this_build_ms": ours_ms, "speedup": ref_ms / ours_ms}
        except Exception as exc:                              # noqa: BLE001
            out[case.name] = {"error": str(exc)[:200]}
        torch.cuda.empty_cache()
    return out


_JSON_FD = None


def emit(line: dict) -> None:
    """The one JSON line goes to the original stdout; everything else that
    libraries print there (NCCL's version banner) is sent to stderr."""
    data = (json.dumps(line) + "\n").encode()
    os.write(_JSON_FD if _JSON_FD is not None else 1, data)


def main():
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-also", action="store_true", help="skip the extra measurements under `also`")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--context-steps", type=int, default=3)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    if NUM_SEQS % (world * SEQS_PER_CALL) != 0:
        raise SystemExit("bench.py runs on 1, 2, 4 or 8 GPUs (16 sequences, two per call)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = pin_to_gpu_numa_node(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    from baselinebenchmark_b200 import build
    build.build()
    # the rank's sequences, generated two at a time (the generator works in fp32)
    my_seqs = NUM_SEQS // world
    calls = my_seqs // SEQS_PER_CALL
    call_lens = [SEQ_LEN] * SEQS_PER_CALL
    call_tokens = sum(call_lens)
    q = torch.empty(my_seqs * SEQ_LEN, HQ, D, dtype=torch.bfloat16, device=dev)
    k = torch.empty(my_seqs * SEQ_LEN, HKV, D, dtype=torch.bfloat16, device=dev)
    v = torch.empty_like(k)
    out = torch.empty_like(q)
    cu = None
    for c in range(calls):
        sl = slice(c * call_tokens, (c + 1) * call_tokens)
        q[sl], k[sl], v[sl], cu = make_inputs_device(call_lens, HQ, HKV, D, CHUNK, 45000 + rank * 8 + c, dev)
    runners, ws = [], None
    for c in range(calls):
        sl = slice(c * call_tokens, (c + 1) * call_tokens)
        r = Runner(q[sl], k[sl], v[sl], cu, SEQ_LEN, CHUNK, TOPK, ws=ws, out=out[sl])
        ws = r.ws
        runners.append(r)
    runner = MultiRunner(runners)
    with ClockSampler(local) as clocks:
        total_ms, stage_ms = timed_steps(runner, args.steps, args.warmup, barrier, calls)
    total_ms = max_over_ranks(total_ms)
    attend_ms = max_over_ranks(float(stage_ms[3]))
    tokens = NUM_SEQS * SEQ_LEN * args.steps
    value = tokens / (total_ms * 1e-3)
    flops_call = attention_flops(call_lens, HQ, D, CHUNK, TOPK)
    flops_total = flops_call * (NUM_SEQS // SEQS_PER_CALL)
    pk = peaks()

    # end to end: pinned host buffers in, pinned host result out, copies inside the timed region
    prob = runners[0].prob
    sl0 = slice(0, call_tokens)
    del runner, runners, ws, r
    torch.cuda.empty_cache()
    host = HostRunner(prob, q[sl0], k[sl0], v[sl0], cu, calls)
    host.begin()
    for _ in range(2 if calls == 1 else 1):                  # untimed: both (stream, workspace) pairs once
        host.step()
    host.end()
    torch.cuda.synchronize()
    barrier()
    e0, e1 = new_events(2)
    torch.cuda.synchronize()
    e0.record()
    host.begin()
    for _ in range(args.e2e_steps):
        host.step()
    host.end()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    e2e_value = NUM_SEQS * SEQ_LEN * args.e2e_steps / (e2e_ms * 1e-3)
    h2d, d2h = host.h2d, host.d2h
    del host, q, k, v, out
    torch.cuda.empty_cache()

    also = {}
    if not args.no_also:
        if rank == 0:
            q2, k2, v2, cu2 = make_inputs_device([32768], 32, 8, 128, 4096, 44, dev)
            r2 = Runner(q2, k2, v2, cu2, 32768, 4096, 12)
            ms2, st2 = timed_steps(r2, 20, 5, lambda: None)
            ms2 /= 20
            f2 = attention_flops([32768], 32, 128, 4096, 12)
            also["configs[2] 32K GQA prefill (1 GPU, 32768 tokens, 32/8 heads, chunk 4096, top-k 12)"] = {
                "ms_per_call": ms2, "tokens_per_s": 32768 / (ms2 * 1e-3), "tflops": f2 / (ms2 * 1e-3) / 1e12,
                "frac_of_measured_burst_peak": f2 / (ms2 * 1e-3) / 1e12 / pk["burst"],
                "dense_stage_ms": float(st2[3]), "dense_stage_tflops": f2 / (float(st2[3]) * 1e-3) / 1e12,
                "stage_ms": {"means": float(st2[0]), "gate_topk": float(st2[1]), "compact": float(st2[2]),
                             "attend": float(st2[3]), "merge": float(st2[4])}}
            # the training path on the same configuration: forward with LSE and selection, then moba_backward
            from baselinebenchmark_b200 import parallel as _par
            del r2
            out2, lse2, sel2 = _par.moba_forward(q2, k2, v2, cu2, 32768, 4096, 12, return_lse=True, return_selected=True)
            dout2 = torch.randn_like(q2)
            for _ in range(2):
                _par.moba_backward(q2, k2, v2, cu2, 32768, 4096, 12, out2, lse2, sel2, dout2)
            b0, b1 = new_events(2)
            b0.record()
            for _ in range(3):
                _par.moba_backward(q2, k2, v2, cu2, 32768, 4096, 12, out2, lse2, sel2, dout2)
            b1.record()
            torch.cuda.synchronize()
            bwd_ms = b0.elapsed_time(b1) / 3
            also["configs[2] backward (training path, dq and dk/dv kernels on tcgen05)"] = {
                "ms_per_call": bwd_ms, "tflops_on_2.5x_forward_flops": 2.5 * f2 / bwd_ms / 1e9}
            del q2, k2, v2, out2, lse2, sel2, dout2
            torch.cuda.empty_cache()
            # decode: one sequence of configs[3] prefilled in one call, then single-token steps with the
            # K/V rows and chunk means cached on the device (incremental.py)
            from baselinebenchmark_b200.incremental import IncrementalMoba
            q3, k3, v3, _ = make_inputs_device([SEQ_LEN], HQ, HKV, D, CHUNK, 47000, dev)
            n_dec, n_warm = 64, 8
            inc = IncrementalMoba(SEQ_LEN, HKV, D, CHUNK, TOPK, device=dev)
            at = SEQ_LEN - n_dec - n_warm
            inc.append(q3[:at], k3[:at], v3[:at])
            for _ in range(n_warm):
                inc.append(q3[at:at + 1], k3[at:at + 1], v3[at:at + 1])
                at += 1
            d0, d1 = new_events(2)
            d0.record()
            for _ in range(n_dec):
                inc.append(q3[at:at + 1], k3[at:at + 1], v3[at:at + 1])
                at += 1
            d1.record()
            torch.cuda.synchronize()
            dec_ms = d0.elapsed_time(d1) / n_dec
            also["decode (1 GPU, one sequence of configs[3]: single-token steps on a cached prefix)"] = {
                "prefix_tokens": SEQ_LEN - n_dec, "steps": n_dec, "ms_per_token": dec_ms,
                "tokens_per_s": 1e3 / dec_ms,
                "note": "steps issued back to back from Python, CUDA events around all of them; every step "
                        "returns the bits of the prefill's row"}
            del q3, k3, v3, inc
            torch.cuda.empty_cache()
        barrier()
        ctx = context_block(args.context_steps, 1, rank, world, local, dev, dist)
        if rank == 0 and ctx is not None:
            also["configs[4] context parallel"] = ctx
        torch.cuda.empty_cache()
        if rank == 0 and world == 1:
            also["reference_triton_b200"] = reference_triton_block(dev)
    barrier()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        rate, dt, sample = cpu_sample(threads)
        cpu = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample,
               "seconds": dt}

    if rank == 0:
        achieved = flops_call / (attend_ms * 1e-3) / 1e12
        line = {
            "metric": "MoBA prefill tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(world),
            "tflops_effective": flops_total * args.steps / (total_ms * 1e-3) / 1e12,
            "frac_of_bf16_peak": flops_total * args.steps / (total_ms * 1e-3) / 1e12 / (pk["sustained"] * world),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms / args.e2e_steps, "steps": args.e2e_steps,
                    "host_buffers": "per rank one pinned two-sequence slab of inputs (3.2 GB) and one of results "
                                    "(2.1 GB), copied in and out by every call of every step; calls alternate "
                                    "between two (stream, workspace) pairs, so the copies of a call overlap the "
                                    "kernels of its neighbours",
                    "cpus_of_rank0": numa},
            "gpu_launches": KERNELS_PER_CALL * calls * args.steps,
            "roofline": {"kernel": "attend_tc5_kernel", "bound": "tensor", "achieved": achieved,
                         "peak": pk["sustained"], "unit": "TFLOP/s", "frac": achieved / pk["sustained"],
                         "peak_kind": f"{pk['source']} cuBLAS bf16, sustained (kernel timed inside a long step); "
                                      f"burst {pk['burst']}", "frac_of_burst": achieved / pk["burst"],
                         "flops_per_launch": flops_call, "ms_per_launch": attend_ms,
                         "launches_per_step": calls,
                         "traffic": ATTEND_TRAFFIC_CFG2 * (call_tokens * HQ * PARTIALS) / (32768 * 32 * 8),
                         "traffic_unit": "bytes of DRAM read + write per launch, scaled from one ncu capture of "
                                         "configs[2] (3.934e9 B for 32768 x 32 rows x 8 partial results) by "
                                         "rows x partial results: the traffic is fp16 partial writes and Q gathers"},
            "stage_ms": {"means": float(stage_ms[0]), "gate_topk": float(stage_ms[1]), "compact": float(stage_ms[2]),
                         "attend": float(stage_ms[3]), "merge": float(stage_ms[4]), "per": "operator call"},
            "gating": gating_roofline(float(stage_ms[0]) + float(stage_ms[1]), pk),
            "cpu_baseline": cpu, "clocks": clocks.summary(), "also": also,
        }
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
