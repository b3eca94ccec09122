"""Generate tests/golden/routing_*.npz by executing the reference's own routing
kernels (backends/_mthreads/ops/moba/routing.py) on CPU with the Triton
interpreter.  Run in the build container only (needs the reference checkout):

    TRITON_INTERPRET=1 python tests/golden/make_routing_golden.py /path/to/reference

Recorded per case: the inputs (bf16 bit patterns), and the reference outputs of
  _build_dense_chunk_metadata_triton                   (routing.py:595-632)
  _compute_dense_chunk_means_triton                    (routing.py:740-775)
  _compute_selected_chunks_batched_streaming_triton    (routing.py:1185-1262)
  _build_sparse_routes_device_triton                   (routing.py:1642-1718)

The interpreter mishandles bfloat16 (fp32->bf16 is a truncation and negative
bf16 inputs lose their sign), while float16 goes through numpy and is exact.
The reference accepts both dtypes (parallel.py:420-421), so the fixtures are
made like this: inputs are drawn, rounded to bf16, and every value is checked
to be exactly representable in float16; the reference kernels then run on the
float16 copy of those same numbers.  Products and sums are identical real
numbers in both dtypes, so the recorded routing is the routing of the bf16
inputs.  Only the rounding of the stored chunk means depends on the dtype:
`means_ref_f16` holds the reference's float16 means (compared with the oracle
run in float16), and the top-k kernel is driven with bf16-rounded means
supplied from outside (`means_rne`: float64 sum, rounded to fp32, then to bf16,
exact in float16), whose output `selected_ref` is the routing golden vector.
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

os.environ.setdefault("TRITON_INTERPRET", "1")

CASES = {
    # name: (seq_lens, Hq, Hkv, D, chunk, topk, max_seqlen or None, kind)
    "varlen_gqa_c64":   ((257, 193), 4, 2, 64, 64, 3, None, "randn"),
    "tail_c32_k64":     ((300, 33, 96), 2, 2, 128, 32, 64, None, "randn"),
    "slack_maxlen":     ((130, 70), 4, 2, 128, 32, 4, 192, "randn"),
    "separated_k64":    ((257, 193), 4, 2, 64, 64, 64, None, "separated"),
    "ties_zero":        ((192, 129), 4, 2, 64, 64, 3, None, "zeros"),
}


def load_routing(ref_root: Path):
    path = ref_root / "backends/_mthreads/ops/moba/routing.py"
    spec = importlib.util.spec_from_file_location("_ref_routing", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def make_case(seq_lens, hq, hkv, d, chunk, kind, seed):
    g = torch.Generator().manual_seed(seed)
    total = sum(seq_lens)
    if kind == "randn":
        q = torch.randn(total, hq, d, generator=g)
        k = torch.randn(total, hkv, d, generator=g)
        start = 0
        for n in seq_lens:
            nck = (n + chunk - 1) // chunk
            off = torch.randn(nck, hkv, d, generator=g) * 0.5
            k[start:start + n] += off.repeat_interleave(chunk, 0)[:n]
            start += n
    elif kind == "separated":          # test_moba_topk.py:68-82
        q = torch.full((total, hq, d), 0.125)
        q[:, 1::2] *= -1
        k = torch.empty(total, hkv, d)
        start = 0
        for n in seq_lens:
            for pos in range(n):
                k[start + pos].fill_((pos // chunk + 1) / 128)
            start += n
    else:                              # all-zero scores: every candidate ties
        q = torch.zeros(total, hq, d)
        k = torch.zeros(total, hkv, d)
    q, k = q.bfloat16(), k.bfloat16()
    # flush the few values that float16 cannot hold exactly (|x| < 2^-16)
    q = torch.where(q.float().abs() < 2.0 ** -16, torch.zeros_like(q), q)
    k = torch.where(k.float().abs() < 2.0 ** -16, torch.zeros_like(k), k)
    assert (q.half().float() == q.float()).all() and (k.half().float() == k.float()).all()
    return q, k


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_routing_golden.py <path to the reference checkout>")
    ref_root = Path(sys.argv[1])
    routing = load_routing(ref_root)
    out_dir = Path(__file__).resolve().parent
    for seed, (name, (lens, hq, hkv, d, chunk, topk, max_len, kind)) in enumerate(CASES.items()):
        q, k = make_case(lens, hq, hkv, d, chunk, kind, 1000 + seed)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
        max_seqlen = max_len or max(lens)
        cu_chunk, chunk_end, _, valid, mc = routing._build_dense_chunk_metadata_triton(cu, max_seqlen, chunk)
        hist = min(topk - 1, mc - 1)
        q16, k16 = q.half(), k.half()
        means_ref = routing._compute_dense_chunk_means_triton(k16, cu_chunk, valid, chunk)
        # round-to-nearest means computed outside the interpreter
        means64 = torch.zeros(valid.numel(), hkv, d, dtype=torch.float64)
        for s in range(valid.numel()):
            if valid[s]:
                means64[s] = k[int(cu_chunk[s]):int(cu_chunk[s]) + chunk].double().sum(0) / chunk
        means_rne = means64.float().bfloat16()
        assert (means_rne.half().float() == means_rne.float()).all()
        rec = dict(
            seq_lens=np.asarray(lens), hq=hq, hkv=hkv, d=d, chunk=chunk, topk=topk,
            max_seqlen=max_seqlen, mc=mc, hist=hist,
            q_bits=q.view(torch.int16).numpy(), k_bits=k.view(torch.int16).numpy(),
            cu_seqlens=cu.numpy(), cu_chunk=cu_chunk.numpy(), chunk_end=chunk_end.numpy(),
            valid_hist=valid.numpy(),
            means_ref_f16=means_ref.numpy(),
            means_rne_bits=means_rne.view(torch.int16).numpy(),
        )
        if hist > 0:
            sel = routing._compute_selected_chunks_batched_streaming_triton(
                q16, means_rne.half(), chunk_end, cu, max_seqlen, mc, hist)
            rec["selected_ref"] = sel.numpy()
            block_m = 64
            (query_indices, route_positions, expert_offsets, desc_experts, desc_starts) = \
                routing._build_sparse_routes_device_triton(sel, valid.numel(), hq, q.shape[0], block_m)
            rec.update(query_indices=query_indices.numpy(), route_positions=route_positions.numpy(),
                       expert_offsets=expert_offsets.numpy(), descriptor_experts=desc_experts.numpy(),
                       descriptor_starts=desc_starts.numpy(), block_m=block_m)
        np.savez_compressed(out_dir / f"routing_{name}.npz", **rec)
        print(name, "mc", mc, "hist", hist, "T", q.shape[0], flush=True)


if __name__ == "__main__":
    main()
