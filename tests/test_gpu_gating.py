"""GPU: the gating kernel's two decision paths.

The kernel estimates every score of a row on the tensor core and evaluates in the
contract order (oracle.moba_oracle._tree_dot) only the candidates whose rank the estimate
cannot settle.  Whatever path a row takes, `selected` must equal the oracle's bit for bit;
the statistics output shows how many rows took which path and how far the estimate was
from the exact score relative to the bound the kernel assumes."""
import zlib

import numpy as np
import pytest
import torch

from oracle import moba_oracle as O
from tests import gpu_util as G

pytestmark = pytest.mark.gpu

DTYPES = [pytest.param(torch.bfloat16, id="bf16"), pytest.param(torch.float16, id="fp16")]
NORMAL, FORCE_EXACT, FORCE_RECHECK = 0, 1, 2

# (name, head_dim, seq_lens, Hq, Hkv, chunk, topk)
CASES = [
    ("d128_gqa", 128, (700, 333, 1290), 8, 2, 128, 4),
    ("d128_many_chunks", 128, (4161,), 4, 2, 16, 8),
    ("d128_k64_many_chunks", 128, (4161,), 4, 2, 16, 64),
    ("d64_tail_k64", 64, (513, 2049), 4, 2, 32, 64),
    ("d96_gqa", 96, (127, 128, 129, 900), 8, 2, 64, 5),
    ("d256_mqa", 256, (900,), 4, 1, 64, 8),
    ("g3_odd_group", 128, (1000, 500), 6, 2, 64, 4),
]


def _oracle_selection(q, k, cu, max_seqlen, chunk, topk):
    cu_chunk, _, valid, mc = O.chunk_slots(cu, max_seqlen, chunk)
    hist = O.historical_topk(topk, mc)
    means = O.chunk_means(k, cu_chunk, valid, chunk)
    return means, O.select_chunks(q, means, cu, max_seqlen, chunk, hist)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_every_decision_path_gives_the_oracle_selection(case, dtype):
    name, d, lens, hq, hkv, chunk, topk = case
    q, k, v, cu = O.make_inputs(list(lens), hq, hkv, d, chunk, zlib.crc32(name.encode()) % 1000, dtype=dtype)
    means_o, sel_o = _oracle_selection(q, k, cu, max(lens), chunk, topk)
    qd, kd = q.cuda(), k.cuda()
    cud = torch.from_numpy(cu).cuda()
    prob, _ = G.problem_for(qd, kd, kd, cud, max(lens), chunk, topk)
    m = G.means(prob, kd, cud)
    assert torch.equal(m.cpu().view(torch.int16), means_o.view(torch.int16))
    rows_with_candidates = sum(max(n - chunk, 0) for n in lens) * hq
    for flags in (NORMAL, FORCE_EXACT, FORCE_RECHECK):
        sel, counts, stats = G.gate_stats(prob, qd, m, cud, flags)
        np.testing.assert_array_equal(sel.cpu().numpy(), sel_o, err_msg=f"flags={flags}")
        assert counts.sum().item() == (sel_o >= 0).sum()
        assert stats[2] == 0, f"estimate outside its bound on {stats[2]} rows (flags={flags})"
        if flags == FORCE_EXACT:
            assert stats[3] == rows_with_candidates and stats[0] == 0
        if flags == FORCE_RECHECK:
            assert stats[0] + stats[3] == rows_with_candidates
            # the tensor-core estimate stays far inside the bound the kernel assumes
            assert stats[1] < 0.25 * 65536, stats
        if flags == NORMAL and topk <= 8:
            # near-ties among a few selected chunks are rare on random inputs: most rows are settled by the
            # estimate (with 63 selected chunks most rows have some pair of scores within the bound)
            assert stats[0] + stats[3] < 0.25 * rows_with_candidates + 64, stats


def _gate_with_means(q, means, lens, chunk, topk, hkv):
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    mc = O.cdiv(max(lens), chunk)
    hist = O.historical_topk(topk, mc)
    sel_o = O.select_chunks(q, means, cu, max(lens), chunk, hist)
    qd, md = q.cuda(), means.cuda()
    cud = torch.from_numpy(cu).cuda()
    kdummy = torch.zeros(q.shape[0], hkv, q.shape[2], dtype=q.dtype, device="cuda")
    prob, _ = G.problem_for(qd, kdummy, kdummy, cud, max(lens), chunk, topk)
    out = {}
    for flags in (NORMAL, FORCE_EXACT, FORCE_RECHECK):
        sel, _, stats = G.gate_stats(prob, qd, md, cud, flags)
        np.testing.assert_array_equal(sel.cpu().numpy(), sel_o, err_msg=f"flags={flags}")
        assert stats[2] == 0
        out[flags] = stats
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("topk", [8, 64])
def test_exact_ties_and_one_ulp_near_ties_across_many_candidates(dtype, topk):
    """Adversarial means: 300 candidate chunks whose scores tie exactly (identical mean
    vectors), tie in groups, differ in the last bit of one input element, or are all +-0.
    The lower chunk must win every tie and the order of the near-ties must be the contract's."""
    g = torch.Generator().manual_seed(7 + topk)
    chunk, nchunks, hq, hkv, d = 8, 301, 4, 2, 128
    lens = [chunk * nchunks]
    t = lens[0]
    q = torch.randn(t, hq, d, generator=g).to(dtype)
    base = (torch.randn(hkv, d, generator=g) * 0.5).to(dtype)

    # 1. every chunk has the same mean: all scores of a row tie exactly
    same = base[None].repeat(nchunks, 1, 1).contiguous()
    stats = _gate_with_means(q, same, lens, chunk, topk, hkv)
    assert stats[NORMAL][0] + stats[NORMAL][3] > 0.9 * (t - chunk) * hq        # nothing is settled by the estimate

    # 2. five distinct means repeated: ties in groups of sixty
    five = (torch.randn(5, hkv, d, generator=g) * 0.5).to(dtype)
    _gate_with_means(q, five[torch.arange(nchunks) % 5].contiguous(), lens, chunk, topk, hkv)

    # 3. one element one ulp up or down per chunk: scores differ by about 2^-9 |q_i m_i| relative
    bits = same.clone().view(torch.int16)
    dim = torch.randint(0, d, (nchunks,), generator=g)
    step = torch.randint(0, 3, (nchunks,), generator=g).to(torch.int16) - 1
    bits[torch.arange(nchunks), :, dim] += step[:, None]
    _gate_with_means(q, bits.view(dtype), lens, chunk, topk, hkv)

    # 4. zero means of either sign (scores +0.0 and -0.0: +0.0 ranks first, routing.py:778-784)
    zeros = torch.zeros(nchunks, hkv, d, dtype=dtype)
    zeros.view(torch.int16)[1::2] = -32768                                    # -0.0
    _gate_with_means(q, zeros, lens, chunk, topk, hkv)

    # 5. zero query rows mixed in
    q0 = q.clone()
    q0[::3] = 0
    _gate_with_means(q0, bits.view(dtype), lens, chunk, topk, hkv)


def test_long_candidate_lists_sampled():
    """More candidates than one tensor-core tile holds (625 > 256), top-k 8 and 64, against the
    oracle on sampled tokens; all three decision paths."""
    lens, hq, hkv, chunk = [40000], 4, 2, 64
    q, k, v, cu = O.make_inputs(lens, hq, hkv, 128, chunk, seed=99)
    cu_chunk, _, valid, mc = O.chunk_slots(cu, lens[0], chunk)
    means_o = O.chunk_means(k, cu_chunk, valid, chunk)
    rng = np.random.default_rng(5)
    rows = sorted(set(rng.integers(0, lens[0], 600).tolist()) | {63, 64, 65, 16383, 16384, 16447, 39999})
    qd, kd = q.cuda(), k.cuda()
    cud = torch.from_numpy(cu).cuda()
    for topk in (8, 64):
        hist = O.historical_topk(topk, mc)
        sel_o = O.select_chunks(q, means_o, cu, lens[0], chunk, hist, rows=rows)
        prob, _ = G.problem_for(qd, kd, kd, cud, lens[0], chunk, topk)
        m = G.means(prob, kd, cud)
        for flags in (NORMAL, FORCE_RECHECK, FORCE_EXACT):
            sel, _, stats = G.gate_stats(prob, qd, m, cud, flags)
            np.testing.assert_array_equal(sel.cpu().numpy()[:, :, rows], sel_o[:, :, rows], err_msg=f"{topk} {flags}")
            assert stats[2] == 0
