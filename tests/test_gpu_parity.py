"""GPU parity tests: every stage of the CUDA path, called through the C ABI,
against the CPU oracle on the same seeded inputs.

Routing (slot tables, chunk means, selected chunks) must be bit-exact.
Outputs must be within max-abs 2e-2 and mean-abs 2e-3 of the fp32 evaluation of
the same selection (BASELINE.json north_star); the reference's own limits are
max < 0.04, mean < 4e-4 against float64 (test_moba_topk.py:117-118)."""
import ctypes as C
import glob
import zlib
from pathlib import Path

import numpy as np
import pytest
import torch

from baselinebenchmark_b200 import _lib, parallel
from oracle import moba_oracle as O
from tests import gpu_util as G

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS = 2e-2, 2e-3
IMPLS = [pytest.param(_lib.ATTEND_TCGEN05, id="tcgen05"), pytest.param(_lib.ATTEND_MMA_SYNC, id="mma_sync")]
DTYPES = [pytest.param(torch.bfloat16, id="bf16"), pytest.param(torch.float16, id="fp16")]
GOLDEN = sorted(glob.glob(str(Path(__file__).parent / "golden" / "routing_*.npz")))

# (name, seq_lens, Hq, Hkv, chunk, topk, max_seqlen or None)
SMALL_CASES = [
    ("mha_c128", (1024,), 4, 4, 128, 3, None),
    ("gqa_varlen", (700, 333, 1290), 8, 2, 128, 4, None),
    ("tail_one_token", (513, 257), 4, 2, 256, 3, None),
    ("chunk_boundaries", (127, 128, 129), 4, 4, 64, 8, None),
    ("short_seqs_one_chunk", (100, 60), 4, 1, 128, 8, None),
    ("slack_maxlen", (520, 130), 8, 2, 64, 5, 1024),
    ("k64_saturated", (512, 512), 4, 2, 32, 64, None),
    ("k1_local_only", (600, 300), 4, 2, 128, 1, None),
    ("many_chunks_k64", (4161,), 4, 2, 16, 64, None),
    ("mqa", (900,), 8, 1, 128, 3, None),
]


def _case_inputs(lens, hq, hkv, chunk, seed, dtype=torch.bfloat16, d=128):
    return O.make_inputs(list(lens), hq, hkv, d, chunk, seed, dtype=dtype)


# the other head dims of the reference's suite (moba_compare.py:63, :70, :77):
# (name, head_dim, seq_lens, Hq, Hkv, chunk, topk)
HEAD_DIM_CASES = [
    ("d64_gqa_varlen", 64, (700, 333, 1290), 8, 2, 128, 4),
    ("d64_tail_k64", 64, (513, 2049), 4, 2, 32, 64),
    ("d96_mha", 96, (1024, 300), 4, 4, 128, 3),
    ("d96_gqa", 96, (127, 128, 129, 900), 8, 2, 64, 5),
    ("d256_gqa", 256, (640, 257), 4, 2, 128, 3),
    ("d256_mqa", 256, (900,), 4, 1, 64, 8),
    ("d256_c512", 256, (2048, 700), 8, 2, 512, 3),          # items of several key tiles
    ("d256_c1024_mqa", 256, (3000,), 4, 1, 1024, 4),
]


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.split("routing_")[-1][:-4])
def test_golden_routing_through_cuda(path):
    """Reference-generated golden vectors (head_dim 64 and 128) through the CUDA gating stage."""
    z = np.load(path)
    q = torch.from_numpy(z["q_bits"]).view(torch.bfloat16).cuda()
    k = torch.from_numpy(z["k_bits"]).view(torch.bfloat16).cuda()
    cu = torch.from_numpy(z["cu_seqlens"]).cuda()
    prob, _ = G.problem_for(q, k, k, cu, int(z["max_seqlen"]), int(z["chunk"]), int(z["topk"]))
    cu_chunk, chunk_end, valid = G.metadata(prob, cu)
    np.testing.assert_array_equal(cu_chunk.cpu().numpy(), z["cu_chunk"])
    np.testing.assert_array_equal(chunk_end.cpu().numpy(), z["chunk_end"])
    np.testing.assert_array_equal(valid.cpu().numpy(), z["valid_hist"])
    m = G.means(prob, k, cu)
    np.testing.assert_array_equal(m.cpu().view(torch.int16).numpy(), z["means_rne_bits"])
    sel, _ = G.gate(prob, q, m, cu)
    np.testing.assert_array_equal(sel.cpu().numpy(), z["selected_ref"])


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.split("routing_")[-1][:-4])
def test_golden_routing_through_cuda_fp16(path):
    """The same fixtures in float16, the dtype the reference kernels produced them in: the
    float16 chunk means must equal the reference kernel's own output bit for bit, and the
    selection from the means the reference's top-k kernel was given must equal its output."""
    z = np.load(path)
    q = torch.from_numpy(z["q_bits"]).view(torch.bfloat16).half().cuda()
    k = torch.from_numpy(z["k_bits"]).view(torch.bfloat16).half().cuda()
    cu = torch.from_numpy(z["cu_seqlens"]).cuda()
    prob, _ = G.problem_for(q, k, k, cu, int(z["max_seqlen"]), int(z["chunk"]), int(z["topk"]))
    assert prob.dtype == 1
    m = G.means(prob, k, cu)
    np.testing.assert_array_equal(m.cpu().numpy(), z["means_ref_f16"])
    given = torch.from_numpy(z["means_rne_bits"]).view(torch.bfloat16).half().cuda()
    sel, _ = G.gate(prob, q, given, cu)
    np.testing.assert_array_equal(sel.cpu().numpy(), z["selected_ref"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", SMALL_CASES, ids=lambda c: c[0])
def test_routing_bit_exact(case, dtype):
    name, lens, hq, hkv, chunk, topk, max_len = case
    q, k, v, cu = _case_inputs(lens, hq, hkv, chunk, seed=zlib.crc32(name.encode()) % 1000, dtype=dtype)
    max_seqlen = max_len or max(lens)
    cu_chunk_o, chunk_end_o, valid_o, mc = O.chunk_slots(cu, max_seqlen, chunk)
    hist = O.historical_topk(topk, mc)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    prob, _ = G.problem_for(qd, kd, vd, cud, max_seqlen, chunk, topk)
    cu_chunk, chunk_end, valid = G.metadata(prob, cud)
    np.testing.assert_array_equal(cu_chunk.cpu().numpy(), cu_chunk_o)
    np.testing.assert_array_equal(chunk_end.cpu().numpy(), chunk_end_o)
    np.testing.assert_array_equal(valid.cpu().numpy(), valid_o)
    means_o = O.chunk_means(k, cu_chunk_o, valid_o, chunk)
    m = G.means(prob, kd, cud)
    assert torch.equal(m.cpu().view(torch.int16), means_o.view(torch.int16))
    if hist <= 0:
        return
    sel_o = O.select_chunks(q, means_o, cu, max_seqlen, chunk, hist)
    sel, counts = G.gate(prob, qd, m, cud)
    np.testing.assert_array_equal(sel.cpu().numpy(), sel_o)
    # list sizes: rows routed to each (slot, kv head)
    g = hq // hkv
    want = np.zeros((len(valid_o), hkv), dtype=np.int64)
    for h in range(hq):
        ids = sel_o[:, h, :].ravel()
        np.add.at(want[:, h // g], ids[ids >= 0], 1)
    np.testing.assert_array_equal(counts.cpu().numpy().reshape(-1, hkv), want)
    # compaction: every routed (row, rank) appears exactly once, in the list of its slot
    for tile_rows in (128, 256):
        offsets, tiles, row_list, plse = G.compact(prob, cud, sel, counts, tile_rows)
        offsets, tiles, row_list = offsets.cpu().numpy(), tiles.cpu().numpy(), row_list.cpu().numpy()
        assert offsets[0] == 0 and offsets[-1] == (sel_o >= 0).sum()
        np.testing.assert_array_equal(np.diff(offsets), want.ravel())
        np.testing.assert_array_equal(np.diff(tiles), -(-want.ravel() // tile_rows))
        npart = hist + 1
        used = row_list[:offsets[-1]]
        assert len(np.unique(used)) == len(used)
        rank = used % npart - 1
        row = used // npart
        tok, head = row // hq, row % hq
        slot_of_entry = sel_o[rank, head, tok]
        list_id = np.repeat(np.arange(len(want.ravel())), want.ravel())
        np.testing.assert_array_equal(slot_of_entry * hkv + head // g, list_id)
        # ranks without a chunk are marked -inf for the merge
        plse = plse.cpu().numpy()[:, 0].reshape(-1, npart)
        empty = np.transpose(sel_o < 0, (2, 1, 0)).reshape(-1, hist)        # [row, rank]
        assert np.all(np.isneginf(plse[:, 1:][empty])) and np.all(plse[:, 1:][~empty] == 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", HEAD_DIM_CASES, ids=lambda c: c[0])
def test_other_head_dims(case, dtype):
    """head_dim 64, 96 and 256: chunk means and selection bit-exact, output within tolerance
    on both dense stages."""
    name, d, lens, hq, hkv, chunk, topk = case
    q, k, v, cu = _case_inputs(lens, hq, hkv, chunk, zlib.crc32(name.encode()) % 1000, dtype=dtype, d=d)
    max_seqlen = max(lens)
    ref, ref_lse, sel_o = O.moba_forward(q, k, v, cu, max_seqlen, chunk, topk, dtype=torch.float32)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    prob, _ = G.problem_for(qd, kd, vd, cud, max_seqlen, chunk, topk)
    assert prob.attend_impl == _lib.ATTEND_TCGEN05
    cu_chunk_o, _, valid_o, _ = O.chunk_slots(cu, max_seqlen, chunk)
    means_o = O.chunk_means(k, cu_chunk_o, valid_o, chunk)
    m = G.means(prob, kd, cud)
    assert torch.equal(m.cpu().view(torch.int16), means_o.view(torch.int16))
    for impl in (_lib.ATTEND_TCGEN05, _lib.ATTEND_MMA_SYNC):
        out, lse, sel = parallel.moba_forward(qd, kd, vd, cud, max_seqlen, chunk, topk, return_lse=True,
                                              return_selected=True, attend_impl=impl)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(sel.cpu().numpy(), sel_o)
        mx, mean = G.rel_stats(out.cpu(), ref)
        assert mx < MAX_ABS and mean < MEAN_ABS, (impl, mx, mean)
        assert (lse.cpu() - ref_lse).abs().max().item() < 2e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("case", SMALL_CASES, ids=lambda c: c[0])
def test_forward_matches_fp32_evaluation(case, impl, dtype):
    name, lens, hq, hkv, chunk, topk, max_len = case
    q, k, v, cu = _case_inputs(lens, hq, hkv, chunk, seed=zlib.crc32(name.encode()) % 1000, dtype=dtype)
    max_seqlen = max_len or max(lens)
    ref, ref_lse, sel_o = O.moba_forward(q, k, v, cu, max_seqlen, chunk, topk, dtype=torch.float32)
    qd, kd, vd = G.to_dev(q, k, v)
    out, lse, sel = parallel.moba_forward(qd, kd, vd, torch.from_numpy(cu).cuda(), max_seqlen, chunk, topk,
                                          return_lse=True, return_selected=True, attend_impl=impl)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(sel.cpu().numpy(), sel_o)
    assert torch.isfinite(out.float()).all()
    mx, mean = G.rel_stats(out.cpu(), ref)
    assert mx < MAX_ABS and mean < MEAN_ABS, (mx, mean)
    assert (lse.cpu() - ref_lse).abs().max().item() < 2e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("jump", [4.0, 24.0, 140.0])
@pytest.mark.parametrize("d", [128, 256])
def test_scores_rising_late_in_a_chunk(impl, dtype, jump, d):
    """Keys whose scores lie far above everything seen earlier in the same chunk (by `jump`
    in units of log2 after scaling): the running reference of the softmax has to follow,
    whatever shortcut a kernel takes on tiles that look ordinary."""
    t, hq, hkv, chunk, topk = 1536, 4, 2, 512, 3
    g = torch.Generator().manual_seed(int(jump))
    q = torch.ones(t, hq, d) * 0.25
    k = torch.randn(t, hkv, d, generator=g) * 0.05
    v = torch.randn(t, hkv, d, generator=g)
    amp = jump / (0.25 * d * d ** -0.5 * 1.4426950408889634)          # q.k * scale * log2(e) == jump
    for start in (300, 700, 1400):                                     # late in chunk 0, 1 and 2
        k[start:start + 3] = amp
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    cu = np.array([0, t], dtype=np.int32)
    ref, ref_lse, sel_o = O.moba_forward(q, k, v, cu, t, chunk, topk, dtype=torch.float32)
    out, lse, sel = parallel.moba_forward(*G.to_dev(q, k, v), torch.from_numpy(cu).cuda(), t, chunk, topk,
                                          return_lse=True, return_selected=True, attend_impl=impl)
    np.testing.assert_array_equal(sel.cpu().numpy(), sel_o)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    mx, mean = G.rel_stats(out.cpu(), ref)
    assert mx < MAX_ABS and mean < MEAN_ABS, (mx, mean)
    assert (lse.cpu() - ref_lse).abs().max().item() < 2e-3 * max(1.0, jump / 8)


@pytest.mark.parametrize("impl", IMPLS)
def test_topk1_chunk_local_exact(impl):
    """test_moba_topk.py:30-57 with head_dim 128: exact equality required."""
    lengths, chunk = (192, 129), 64
    total = sum(lengths)
    q = torch.zeros(total, 4, 128, dtype=torch.bfloat16)
    k = torch.zeros(total, 2, 128, dtype=torch.bfloat16)
    v = torch.empty_like(k)
    expected = torch.empty_like(q)
    full = torch.empty_like(q)
    start = 0
    for b, n in enumerate(lengths):
        for pos in range(n):
            val = (pos // chunk + 1) * (1 if b == 0 else -1)
            v[start + pos].fill_(val)
            expected[start + pos].fill_(val)
        for pos in range(n):
            full[start + pos] = v[start:start + pos + 1].float().mean(0).repeat_interleave(2, dim=0).bfloat16()
        start += n
    cu = torch.tensor([0, lengths[0], total], dtype=torch.int32).cuda()
    out = parallel.moba_forward(q.cuda(), k.cuda(), v.cuda(), cu, max(lengths), chunk, 1, attend_impl=impl)[0].cpu()
    torch.testing.assert_close(out, expected, rtol=0, atol=0)
    assert (out.float() - full.float()).abs().max().item() > 0.5


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("lengths,topk", [((257, 193), 2), ((257, 193), 64), ((4161,), 64)])
def test_separated_scores_against_float64(lengths, topk, impl):
    """test_moba_topk.py:60-118 with head_dim 128, limits max < 0.04, mean < 4e-4."""
    chunk, hq, hkv, dim = 64, 4, 2, 128
    total = sum(lengths)
    qc = torch.full((total, hq, dim), 0.125, dtype=torch.bfloat16)
    qc[:, 1::2] *= -1
    kc = torch.empty(total, hkv, dim, dtype=torch.bfloat16)
    start = 0
    for n in lengths:
        for pos in range(n):
            kc[start + pos].fill_((pos // chunk + 1) / 128)
        start += n
    vc = torch.randn(total, hkv, dim, generator=torch.Generator().manual_seed(42)).bfloat16()
    bounds = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    out = parallel.moba_forward(qc.cuda(), kc.cuda(), vc.cuda(), torch.from_numpy(bounds).cuda(), max(lengths),
                                chunk, topk, attend_impl=impl)[0].cpu().double()
    errors = []
    for b, n in enumerate(lengths):
        s = int(bounds[b])
        keys, values = kc[s:s + n], vc[s:s + n].double()
        means = torch.stack([keys[t:t + chunk].double().mean(0).bfloat16().double() for t in range(0, n, chunk)])
        positions = {0, n - 1}
        positions.update(range(0, n, max(1, n // 32)))
        for edge in range(chunk, n, chunk):
            positions.update((edge - 1, edge))
        for pos in sorted(positions):
            cur = pos // chunk
            for head in range(hq):
                kvh = head // (hq // hkv)
                query = qc[s + pos, head].double()
                scores = means[:cur, kvh] @ query
                chosen = torch.topk(scores, min(topk - 1, cur)).indices.tolist()
                idx = [i for blk in chosen for i in range(blk * chunk, (blk + 1) * chunk)]
                idx += list(range(cur * chunk, pos + 1))
                logits = (keys[idx, kvh].double() @ query) * dim ** -0.5
                errors.append((out[s + pos, head] - logits.softmax(0) @ values[idx, kvh]).abs())
    diff = torch.stack(errors)
    assert torch.isfinite(diff).all()
    assert diff.max().item() < 0.04 and diff.mean().item() < 4e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", IMPLS)
def test_config0_full(impl, dtype):
    """BASELINE.json configs[0]: 4096 tokens, 8/8 heads, chunk 512, top-k 3."""
    cfg = O.CONFIGS[0]
    lens = O.config_lengths(0)
    q, k, v, cu = O.make_inputs(lens, cfg["hq"], cfg["hkv"], cfg["d"], cfg["chunk"], seed=42, dtype=dtype)
    ref, ref_lse, sel_o = O.moba_forward(q, k, v, cu, max(lens), cfg["chunk"], cfg["topk"])
    out, lse, sel = parallel.moba_forward(*G.to_dev(q, k, v), torch.from_numpy(cu).cuda(), max(lens), cfg["chunk"],
                                          cfg["topk"], return_lse=True, return_selected=True, attend_impl=impl)
    np.testing.assert_array_equal(sel.cpu().numpy(), sel_o)
    mx, mean = G.rel_stats(out.cpu(), ref)
    assert mx < MAX_ABS and mean < MEAN_ABS, (mx, mean)
    assert (lse.cpu() - ref_lse).abs().max().item() < 2e-3


def _sampled_check(q, k, v, cu, max_seqlen, chunk, topk, out, sel, nsample, seed):
    """Routing bit-exact on sampled tokens (all heads); outputs of sampled rows vs float64."""
    rng = np.random.default_rng(seed)
    t_total, hq, _ = q.shape
    toks = set(rng.integers(0, t_total, nsample).tolist())
    for b in range(len(cu) - 1):                                    # sequence and chunk edges
        toks.update({int(cu[b]), int(cu[b + 1]) - 1})
        for e in range(int(cu[b]) + chunk, int(cu[b + 1]), chunk * max(1, (int(cu[b + 1]) - int(cu[b])) // chunk // 4)):
            toks.update({e - 1, e})
    toks = sorted(toks)
    cu_chunk, _, valid, mc = O.chunk_slots(cu, max_seqlen, chunk)
    hist = O.historical_topk(topk, mc)
    means = O.chunk_means(k, cu_chunk, valid, chunk)
    sel_o = O.select_chunks(q, means, cu, max_seqlen, chunk, hist, rows=toks)
    np.testing.assert_array_equal(sel[:, :, toks], sel_o[:, :, toks])
    rows = [(t, int(h)) for t in toks[:: max(1, len(toks) // 48)] for h in rng.integers(0, hq, 2)]
    ref, _ = O.attend_rows(q, k, v, cu, max_seqlen, chunk, sel_o, rows)
    got = torch.stack([out[t, h] for t, h in rows]).double()
    diff = (got - ref).abs()
    return diff.max().item(), diff.mean().item()


@pytest.mark.parametrize("impl", IMPLS)
def test_config1_varlen_sampled(impl):
    """BASELINE.json configs[1]: 4 seeded lengths in [1024, 8192], 32/32 heads, chunk 512, top-k 3."""
    cfg = O.CONFIGS[1]
    lens = O.config_lengths(1)
    q, k, v, cu = O.make_inputs(lens, cfg["hq"], cfg["hkv"], cfg["d"], cfg["chunk"], seed=43)
    out, _, sel = parallel.moba_forward(*G.to_dev(q, k, v), torch.from_numpy(cu).cuda(), max(lens), cfg["chunk"],
                                        cfg["topk"], return_selected=True, attend_impl=impl)
    assert torch.isfinite(out.float()).all()
    mx, mean = _sampled_check(q, k, v, cu, max(lens), cfg["chunk"], cfg["topk"], out.cpu(), sel.cpu().numpy(), 96, 1)
    assert mx < MAX_ABS and mean < MEAN_ABS, (mx, mean)


def test_config2_long_gqa_sampled():
    """BASELINE.json configs[2]: 32768 tokens, 32/8 heads, chunk 4096, top-k 12 (every earlier chunk is selected)."""
    cfg = O.CONFIGS[2]
    lens = O.config_lengths(2)
    q, k, v, cu = O.make_inputs(lens, cfg["hq"], cfg["hkv"], cfg["d"], cfg["chunk"], seed=44)
    out, _, sel = parallel.moba_forward(*G.to_dev(q, k, v), torch.from_numpy(cu).cuda(), max(lens), cfg["chunk"],
                                        cfg["topk"], return_selected=True)
    assert torch.isfinite(out.float()).all()
    sel = sel.cpu().numpy()
    # hist = 7 = all earlier chunks: the selected set of a query in chunk j is {0..j-1}
    for j in (1, 3, 7):
        got = np.sort(sel[:, 5, j * 4096 + 17])
        assert got[got >= 0].tolist() == list(range(j))
    mx, mean = _sampled_check(q, k, v, cu, max(lens), cfg["chunk"], cfg["topk"], out.cpu(), sel, 48, 2)
    assert mx < MAX_ABS and mean < MEAN_ABS, (mx, mean)


def test_implementations_agree_and_are_deterministic():
    q, k, v, cu = _case_inputs((2048, 1111), 8, 2, 256, seed=5)
    args = (*G.to_dev(q, k, v), torch.from_numpy(cu).cuda(), 2048, 256, 4)
    a = parallel.moba_forward(*args, attend_impl=_lib.ATTEND_TCGEN05)[0]
    b = parallel.moba_forward(*args, attend_impl=_lib.ATTEND_TCGEN05)[0]
    c = parallel.moba_forward(*args, attend_impl=_lib.ATTEND_MMA_SYNC)[0]
    assert torch.equal(a, b)                                    # run-to-run bit identical
    assert (a.float() - c.float()).abs().max().item() < 2e-2


def test_causality_and_batch_isolation():
    """SEMANTICS.md:38: changing Q/K/V after a prefix, and a later sequence, leaves the prefix outputs unchanged."""
    lens = (1500, 900)
    q, k, v, cu = _case_inputs(lens, 8, 2, 128, seed=9)
    cud = torch.from_numpy(cu).cuda()
    base = parallel.moba_forward(*G.to_dev(q, k, v), cud, 1500, 128, 4)[0].cpu()
    cut = 777
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    g = torch.Generator().manual_seed(1)
    for t in (q2, k2, v2):
        t[cut:] = torch.randn(t[cut:].shape, generator=g).bfloat16()
    pert = parallel.moba_forward(*G.to_dev(q2, k2, v2), cud, 1500, 128, 4)[0].cpu()
    assert torch.equal(base[:cut], pert[:cut])
    assert not torch.equal(base[cut:], pert[cut:])


def test_strided_inputs():
    """q/k/v given as slices of a fused projection (token stride larger than heads*dim)."""
    t, hq, hkv = 1024, 8, 2
    g = torch.Generator().manual_seed(3)
    fused = torch.randn(t, hq + 2 * hkv, 128, generator=g).bfloat16().cuda()
    q, k, v = fused[:, :hq], fused[:, hq:hq + hkv], fused[:, hq + hkv:]
    cu = torch.tensor([0, 600, t], dtype=torch.int32).cuda()
    a = parallel.moba_forward(q, k, v, cu, 600, 128, 3)[0]
    b = parallel.moba_forward(q.contiguous(), k.contiguous(), v.contiguous(), cu, 600, 128, 3)[0]
    assert torch.equal(a, b)


def test_public_operator_names():
    import baselinebenchmark_b200 as pkg
    from baselinebenchmark_b200 import native_moba
    q, k, v, cu = _case_inputs((512,), 4, 2, 128, seed=11)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    with torch.inference_mode():
        a = pkg.parallel_moba(qd, kd, vd, cud, 512, 128, 3)
        b = pkg.moba_attn_varlen(qd, kd, vd, cud, 512, 128, 3)
        c = torch.ops.moba_b200.moba_attn_varlen(qd, kd, vd, cud, 512, 128, 3)
    assert torch.equal(a, b) and torch.equal(a, c)
    assert native_moba._supported(qd)
    assert native_moba._supported(qd.half())
    assert pkg.parallel_moba(qd.half(), kd.half(), vd.half(), cud, 512, 128, 3).dtype == torch.float16
    assert native_moba._supported(qd[..., :64]) and not native_moba._supported(qd[..., :96])
    assert pkg.parallel_moba(qd[..., :64], kd[..., :64], vd[..., :64], cud, 512, 128, 3).shape == qd[..., :64].shape
    with pytest.raises(NotImplementedError):
        pkg.parallel_moba(qd[..., :32], kd[..., :32], vd[..., :32], cud, 512, 128, 3)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("d,dtype", [(128, torch.bfloat16), (64, torch.float16)], ids=["d128_bf16", "d64_fp16"])
def test_query_window_equals_full_run(impl, d, dtype):
    """Context-parallel building block: the operator run on a chunk-aligned query
    window, with K/V of the whole sequence, returns exactly the rows of the full run."""
    lens = (2048, 1280)
    q, k, v, cu = _case_inputs(lens, 8, 2, 128, seed=21, dtype=dtype, d=d)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    full, full_lse, full_sel = parallel.moba_forward(qd, kd, vd, cud, 2048, 128, 4, return_lse=True,
                                                     return_selected=True, attend_impl=impl)
    for lo, hi in [(0, 1024), (1024, 2048), (2048, 2048 + 1280), (512, 2560)]:
        out, lse, sel = parallel.moba_forward(qd[lo:hi].contiguous(), kd, vd, cud, 2048, 128, 4, return_lse=True,
                                              return_selected=True, attend_impl=impl, q_token_begin=lo)
        assert torch.equal(sel, full_sel[:, :, lo:hi])
        assert torch.equal(out, full[lo:hi])
        assert torch.equal(lse, full_lse[:, lo:hi])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("d,chunk,topk", [(128, 512, 3), (128, 128, 4), (64, 1024, 2), (256, 512, 3), (96, 256, 3)],
                         ids=["d128_c512", "d128_c128", "d64_c1024", "d256_c512", "d96_c256"])
def test_query_window_at_any_token_equals_full_run(impl, d, chunk, topk):
    """Decode building block: a query window may start and end at ANY token - inside a chunk,
    inside a row tile, across a sequence boundary, a single token - and still returns exactly the
    rows, LSE and selection of the full run (own-chunk tiles keep their place in the chunk and
    compute only their rows inside the window)."""
    lens = (2500, 1300)
    total = sum(lens)
    q, k, v, cu = _case_inputs(lens, 8, 2, chunk, seed=27, d=d)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    full, full_lse, full_sel = parallel.moba_forward(qd, kd, vd, cud, 2500, chunk, topk, return_lse=True,
                                                     return_selected=True, attend_impl=impl)
    windows = [(0, 1), (1, 2), (777, 778), (130, 1999), (chunk - 1, chunk + 1), (2499, 2501), (2300, 2900),
               (total - 1, total), (2500 + 255, 2500 + 257), (3, total - 5)]
    for lo, hi in windows:
        out, lse, sel = parallel.moba_forward(qd[lo:hi].contiguous(), kd, vd, cud, 2500, chunk, topk, return_lse=True,
                                              return_selected=True, attend_impl=impl, q_token_begin=lo)
        torch.cuda.synchronize()
        assert torch.equal(sel, full_sel[:, :, lo:hi]), (lo, hi)
        assert torch.equal(out, full[lo:hi]), (lo, hi)
        assert torch.equal(lse, full_lse[:, lo:hi]), (lo, hi)


@pytest.mark.parametrize("d,chunk,topk,impl", [(128, 256, 4, None), (128, 512, 3, None), (256, 512, 3, None),
                                               (64, 128, 3, _lib.ATTEND_MMA_SYNC)],
                         ids=["d128_c256", "d128_c512", "d256_c512", "d64_c128_mma"])
def test_decode_token_by_token_equals_one_shot(d, chunk, topk, impl):
    """IncrementalMoba: an unaligned prefill block, 40 decode steps of one token, a second block
    and more single tokens (crossing chunk boundaries on the way) give the rows of the one-shot
    run over the final sequence bit for bit; the means cache ends as the oracle's means."""
    from baselinebenchmark_b200.incremental import IncrementalMoba
    total, capacity, hq, hkv = 1500, 2048, 8, 2
    q, k, v, cu = _case_inputs((total,), hq, hkv, chunk, seed=31, d=d)
    qd, kd, vd = G.to_dev(q, k, v)
    full = parallel.moba_forward(qd, kd, vd, torch.from_numpy(cu).cuda(), capacity, chunk, topk, attend_impl=impl)[0]
    inc = IncrementalMoba(capacity, hkv, d, chunk, topk, dtype=qd.dtype, attend_impl=impl)
    steps = [700] + [1] * 40 + [300] + [1] * 30 + [total - 1070]
    assert sum(steps) == total
    at = 0
    for n in steps:
        out = inc.append(qd[at:at + n], kd[at:at + n], vd[at:at + n])
        torch.cuda.synchronize()
        assert torch.equal(out, full[at:at + n]), (at, n)
        at += n
    assert inc.length == total
    cu_chunk, _, valid, mc = O.chunk_slots(cu, capacity, chunk)
    want = O.chunk_means(k, cu_chunk, valid, chunk)
    done = (total - 1) // chunk                        # chunks behind the last one hold final means
    assert torch.equal(inc.means[:done].cpu().view(torch.int16), want[:done].view(torch.int16))


def test_host_buffer_entry_point_matches_device_call():
    """moba_forward_host (pinned host tensors, pipelined query windows) returns the bits of moba_forward."""
    import ctypes as C
    lens = (3000, 1100, 2048)
    q, k, v, cu = _case_inputs(lens, 8, 2, 128, seed=33)
    cud = torch.from_numpy(cu).cuda()
    ref, ref_lse, ref_sel = parallel.moba_forward(*G.to_dev(q, k, v), cud, 3000, 128, 4, return_lse=True,
                                                  return_selected=True)
    hq, hk, hv = q.pin_memory(), k.pin_memory(), v.pin_memory()
    hcu = torch.from_numpy(cu).pin_memory()
    prob, _ = G.problem_for(q.cuda(), k.cuda(), v.cuda(), cud, 3000, 128, 4)
    size = C.c_size_t(0)
    _lib.check(_lib.lib().moba_workspace_size_host(C.byref(prob), C.byref(size)))
    ws = torch.empty(size.value, dtype=torch.uint8, device="cuda")
    for extra in (False, True):
        hout = torch.zeros_like(q).pin_memory()
        hlse = torch.zeros(8, sum(lens), dtype=torch.float32).pin_memory() if extra else None
        hsel = torch.zeros(3, 8, sum(lens), dtype=torch.int32).pin_memory() if extra else None
        for _ in range(2):                                   # back-to-back calls share the staging buffers
            _lib.check(_lib.lib().moba_forward_host(
                C.byref(prob), hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), hcu.data_ptr(), hout.data_ptr(),
                hlse.data_ptr() if extra else None, hsel.data_ptr() if extra else None,
                ws.data_ptr(), ws.numel(), G.stream()))
        torch.cuda.synchronize()
        assert torch.equal(hout, ref.cpu())
        if extra:
            assert torch.equal(hlse, ref_lse.cpu()) and torch.equal(hsel, ref_sel.cpu())


def test_host_calls_in_flight_on_two_streams_keep_their_results():
    """moba_forward_host is re-entrant for distinct (stream, workspace, result buffer) sets: six
    calls on two different problems, alternating between two streams without any host
    synchronisation in between (the copies of one call then overlap the kernels of the other and
    share the library's two copy streams), each leave the bits of the device call."""
    import ctypes as C
    sets = []
    for i, (lens, topk) in enumerate((((3000, 1100, 2048), 4), ((2500, 3100), 3))):
        q, k, v, cu = _case_inputs(lens, 8, 2, 128, seed=61 + i)
        cud = torch.from_numpy(cu).cuda()
        ref = parallel.moba_forward(*G.to_dev(q, k, v), cud, max(lens), 128, topk)[0].cpu()
        prob, _ = G.problem_for(q.cuda(), k.cuda(), v.cuda(), cud, max(lens), 128, topk)
        size = C.c_size_t(0)
        _lib.check(_lib.lib().moba_workspace_size_host(C.byref(prob), C.byref(size)))
        sets.append(dict(prob=prob, ref=ref, host=[t.pin_memory() for t in (q, k, v, torch.from_numpy(cu))],
                         out=torch.zeros_like(q).pin_memory(), stream=torch.cuda.Stream(),
                         ws=torch.empty(size.value, dtype=torch.uint8, device="cuda")))
    torch.cuda.synchronize()
    for _ in range(3):
        for s in sets:
            hq, hk, hv, hcu = s["host"]
            _lib.check(_lib.lib().moba_forward_host(
                C.byref(s["prob"]), hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), hcu.data_ptr(), s["out"].data_ptr(),
                None, None, s["ws"].data_ptr(), s["ws"].numel(), s["stream"].cuda_stream))
    torch.cuda.synchronize()
    for s in sets:
        assert torch.equal(s["out"], s["ref"])


def test_config3_unit_sampled():
    """BASELINE.json configs[3], one of its 128 (sequence, KV-head group) units at full size:
    131072 tokens, 4 query heads sharing 1 KV head, chunk 4096, top-k 8."""
    cfg = O.CONFIGS[3]
    q, k, v, cu = O.make_inputs([131072], 4, 1, 128, cfg["chunk"], seed=45)
    out, _, sel = parallel.moba_forward(*G.to_dev(q, k, v), torch.from_numpy(cu).cuda(), 131072, cfg["chunk"],
                                        cfg["topk"], return_selected=True)
    assert torch.isfinite(out.float()).all()
    mx, mean = _sampled_check(q, k, v, cu, 131072, cfg["chunk"], cfg["topk"], out.cpu(), sel.cpu().numpy(), 64, 3)
    assert mx < MAX_ABS and mean < MEAN_ABS, (mx, mean)


def test_config4_window_sampled():
    """BASELINE.json configs[4] as one of its 8 ranks sees it, for one KV-head group: K/V of
    the whole 1048576-token sequence, queries of the window [5/8, 6/8), chunk 4096, top-k 16
    (255 candidate chunks, 15 selected)."""
    cfg = O.CONFIGS[4]
    total, chunk, topk = 1048576, cfg["chunk"], cfg["topk"]
    q, k, v, cu = O.make_inputs([total], 4, 1, 128, chunk, seed=46)
    lo, hi = 5 * total // 8, 6 * total // 8
    out, _, sel = parallel.moba_forward(q[lo:hi].cuda(), k.cuda(), v.cuda(), torch.from_numpy(cu).cuda(), total,
                                        chunk, topk, return_selected=True, q_token_begin=lo)
    assert torch.isfinite(out.float()).all()
    out, sel = out.cpu(), sel.cpu().numpy()
    rng = np.random.default_rng(4)
    toks = sorted(set(rng.integers(lo, hi, 40).tolist()) | {lo, hi - 1, lo + chunk - 1, lo + chunk})
    cu_chunk, _, valid, mc = O.chunk_slots(cu, total, chunk)
    hist = O.historical_topk(topk, mc)
    assert (mc, hist) == (256, 15)
    means = O.chunk_means(k, cu_chunk, valid, chunk)
    sel_o = O.select_chunks(q, means, cu, total, chunk, hist, rows=toks)
    np.testing.assert_array_equal(sel[:, :, [t - lo for t in toks]], sel_o[:, :, toks])
    rows = [(t, int(h)) for t in toks[::4] for h in rng.integers(0, 4, 2)]
    ref, _ = O.attend_rows(q, k, v, cu, total, chunk, sel_o, rows)
    got = torch.stack([out[t - lo, h] for t, h in rows]).double()
    diff = (got - ref).abs()
    assert diff.max().item() < MAX_ABS and diff.mean().item() < MEAN_ABS


def test_decode_on_config4_prefix_sampled():
    """BASELINE.json configs[4] geometry for one KV-head group at full length: a cache of 1048576
    tokens (chunk 4096, top-k 16: 255 candidate chunks, 15 selected) is prefilled in eight blocks,
    the last one 24 tokens short, and the last 24 tokens are decoded one by one.  Their selection
    against the oracle bit for bit, their rows against float64."""
    from baselinebenchmark_b200.incremental import IncrementalMoba
    cfg = O.CONFIGS[4]
    total, chunk, topk, steps = 1048576, cfg["chunk"], cfg["topk"], 24
    q, k, v, cu = O.make_inputs([total], 4, 1, 128, chunk, seed=47)
    qd, kd, vd = G.to_dev(q, k, v)
    inc = IncrementalMoba(total, 1, 128, chunk, topk)
    at = 0
    for n in [total // 8] * 7 + [total // 8 - steps]:
        out = inc.append(qd[at:at + n], kd[at:at + n], vd[at:at + n])
        at += n
    assert torch.isfinite(out.float()).all()
    del out
    outs, sels = [], []
    for _ in range(steps):
        o, s = inc.append(qd[at:at + 1], kd[at:at + 1], vd[at:at + 1], return_selected=True)
        outs.append(o)
        sels.append(s)
        at += 1
    assert at == total == inc.length
    out = torch.cat(outs, 0).cpu()
    sel = torch.cat(sels, 2).cpu().numpy()
    toks = list(range(total - steps, total))
    cu_chunk, _, valid, mc = O.chunk_slots(cu, total, chunk)
    hist = O.historical_topk(topk, mc)
    assert (mc, hist) == (256, 15)
    means = O.chunk_means(k, cu_chunk, valid, chunk)
    sel_o = O.select_chunks(q, means, cu, total, chunk, hist, rows=toks)
    np.testing.assert_array_equal(sel, sel_o[:, :, toks])
    rows = [(t, h) for t in toks[::3] for h in range(4)]
    ref, _ = O.attend_rows(q, k, v, cu, total, chunk, sel_o, rows)
    got = torch.stack([out[t - (total - steps), h] for t, h in rows]).double()
    diff = (got - ref).abs()
    assert diff.max().item() < MAX_ABS and diff.mean().item() < MEAN_ABS


@pytest.mark.parametrize("d,dtype", [(128, torch.bfloat16), (64, torch.float16), (96, torch.bfloat16)],
                         ids=["d128_bf16", "d64_fp16", "d96_bf16"])
def test_bounded_workspace_runs_head_groups(d, dtype):
    """A workspace below the one-pass size makes the library process kv-head groups in turn;
    results, LSE and selection are the bits of the one-pass run."""
    import ctypes as C
    q, k, v, cu = _case_inputs((1536, 1000), 16, 4, 128, seed=41, dtype=dtype, d=d)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    ref, ref_lse, ref_sel = parallel.moba_forward(qd, kd, vd, cud, 1536, 128, 4, return_lse=True, return_selected=True)
    prob, _ = G.problem_for(qd, kd, vd, cud, 1536, 128, 4)
    full, least = C.c_size_t(0), C.c_size_t(0)
    _lib.check(_lib.lib().moba_workspace_size(C.byref(prob), C.byref(full)))
    _lib.check(_lib.lib().moba_workspace_size_min(C.byref(prob), C.byref(least)))
    assert least.value * 3 < full.value
    for limit in (least.value, least.value * 2 + 4096, (full.value * 3) // 4):
        out, lse, sel = parallel.moba_forward(qd, kd, vd, cud, 1536, 128, 4, return_lse=True, return_selected=True,
                                              workspace=torch.empty(limit, dtype=torch.uint8, device="cuda"))
        assert torch.equal(out, ref) and torch.equal(lse, ref_lse) and torch.equal(sel, ref_sel)
    with pytest.raises(_lib.MobaError):
        parallel.moba_forward(qd, kd, vd, cud, 1536, 128, 4,
                              workspace=torch.empty(least.value - 256, dtype=torch.uint8, device="cuda"))


# --------------------------------------------------------------------------
# training path (backward)
# --------------------------------------------------------------------------
BACKWARD_CASES = [
    ("bwd_mha_c128", 128, (1024,), 4, 4, 128, 3),
    ("bwd_gqa_varlen", 128, (700, 333, 1290), 8, 2, 128, 4),
    ("bwd_tails", 128, (513, 257, 129), 4, 2, 64, 5),
    ("bwd_k1_local", 128, (600, 300), 4, 2, 128, 1),
    ("bwd_mqa_k8", 128, (900,), 8, 1, 64, 8),
    ("bwd_d64", 64, (700, 333), 8, 2, 128, 4),
    ("bwd_d96", 96, (640,), 4, 4, 64, 3),
    ("bwd_d96_gqa", 96, (900, 257), 8, 2, 128, 4),
    ("bwd_d256", 256, (700, 333), 4, 2, 128, 3),              # mma.sync kernels whichever implementation is asked for
    ("bwd_d256_mqa_c512", 256, (1500,), 4, 1, 512, 3),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", BACKWARD_CASES, ids=lambda c: c[0])
def test_backward_matches_float64_autograd(case, dtype):
    """dq, dk, dv against float64 autograd through the dense evaluation of the same selection.
    Tolerance: the reference's forward bound scaled to the gradients (max-abs error below 4 %
    of the largest gradient entry, mean-abs error below 0.4 % of it)."""
    name, d, lens, hq, hkv, chunk, topk = case
    q, k, v, cu = _case_inputs(lens, hq, hkv, chunk, zlib.crc32(name.encode()) % 1000, dtype=dtype, d=d)
    g = torch.Generator().manual_seed(11)
    dout = torch.randn(q.shape, generator=g).to(dtype)
    max_seqlen = max(lens)
    qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
    cud = torch.from_numpy(cu).cuda()
    out = parallel.parallel_moba(qd, kd, vd, cud, max_seqlen, chunk, topk)
    assert out.requires_grad
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    _, _, sel_o = O.moba_forward(q, k, v, cu, max_seqlen, chunk, topk)
    rq, rk, rv = O.attend_grads(q, k, v, cu, max_seqlen, chunk, sel_o, dout)
    for name_, got, ref in (("dq", qd.grad, rq), ("dk", kd.grad, rk), ("dv", vd.grad, rv)):
        got = got.double().cpu()
        assert torch.isfinite(got).all(), name_
        ref_max = ref.abs().max().item()
        err = (got - ref).abs()
        assert err.max().item() < 0.04 * ref_max and err.mean().item() < 0.004 * ref_max, \
            (name_, err.max().item(), err.mean().item(), ref_max)


def test_backward_run_to_run_and_no_grad_for_inference():
    """dq is bit-identical run to run (a row's keys are visited in a fixed order); dk and dv add
    the rows of a routed list in the order the compaction's atomics produced, so they agree to
    the last bits only (the reference's lists are unordered too, routing.py:1586-1591)."""
    q, k, v, cu = _case_inputs((700, 333, 1290), 8, 2, 128, seed=3)
    cud = torch.from_numpy(cu).cuda()
    dout = torch.randn(q.shape, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    grads = []
    for _ in range(2):
        qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
        parallel.parallel_moba(qd, kd, vd, cud, 1290, 128, 4).backward(dout)
        grads.append((qd.grad.clone(), kd.grad.clone(), vd.grad.clone()))
    assert torch.equal(grads[0][0], grads[1][0])
    for a, b in zip(grads[0][1:], grads[1][1:]):
        assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -7 * a.float().abs().max().item()
    with torch.no_grad():
        assert not parallel.parallel_moba(q.cuda(), k.cuda(), v.cuda(), cud, 1290, 128, 4).requires_grad


def test_backward_config2_dq_sampled_and_dkdv_finite():
    """BASELINE.json configs[2] at full size: dq of sampled rows against float64, dk / dv finite
    and of the expected magnitude (their exact check runs on the small shapes above)."""
    cfg = O.CONFIGS[2]
    lens = O.config_lengths(2)
    q, k, v, cu = O.make_inputs(lens, cfg["hq"], cfg["hkv"], cfg["d"], cfg["chunk"], seed=44)
    dout = torch.randn(q.shape, generator=torch.Generator().manual_seed(7)).bfloat16()
    qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
    cud = torch.from_numpy(cu).cuda()
    out, lse, sel = parallel.moba_forward(qd.detach(), kd.detach(), vd.detach(), cud, max(lens), cfg["chunk"],
                                          cfg["topk"], return_lse=True, return_selected=True)
    dq, dk, dv = parallel.moba_backward(qd.detach(), kd.detach(), vd.detach(), cud, max(lens), cfg["chunk"],
                                        cfg["topk"], out, lse, sel, dout.cuda())
    torch.cuda.synchronize()
    assert torch.isfinite(dq.float()).all() and torch.isfinite(dk.float()).all() and torch.isfinite(dv.float()).all()
    rng = np.random.default_rng(3)
    rows = [(int(rng.integers(0, q.shape[0])), int(rng.integers(0, q.shape[1]))) for _ in range(24)]
    rows += [(0, 0), (q.shape[0] - 1, q.shape[1] - 1), (4095, 3), (4096, 5)]
    ref = O.dq_rows(q, k, v, cu, max(lens), cfg["chunk"], sel.cpu().numpy(), dout, rows)
    got = torch.stack([dq[t, h].double().cpu() for t, h in rows])
    err = (got - ref).abs()
    scale = ref.abs().max().item()
    assert err.max().item() < 0.04 * scale and err.mean().item() < 0.004 * scale, (err.max().item(), err.mean().item(), scale)
    # every key receives gradient from the later queries of its own chunk at least
    assert dv.float().abs().sum(-1).min().item() > 0


# the last case has 2502 route lists: more than the dq kernel keeps of the tile prefix in shared memory
AGREE_CASES = BACKWARD_CASES + [("bwd_many_lists", 64, (20010,), 2, 2, 16, 4)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", AGREE_CASES, ids=lambda c: c[0])
def test_backward_kernels_agree(case, dtype):
    """The tcgen05 and the mma.sync gradient kernels evaluate the same sums with P and dS
    rounded to the input dtype and fp32 accumulation: they agree up to the summation order
    and the exponential's approximation, i.e. within a rounding step or two of the result."""
    name, d, lens, hq, hkv, chunk, topk = case
    q, k, v, cu = _case_inputs(lens, hq, hkv, chunk, zlib.crc32(name.encode()) % 1000, dtype=dtype, d=d)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    cud = torch.from_numpy(cu).cuda()
    dout = torch.randn(q.shape, generator=torch.Generator().manual_seed(13)).to(dtype).cuda()
    out, lse, sel = parallel.moba_forward(q, k, v, cud, max(lens), chunk, topk, return_lse=True, return_selected=True)
    res = [parallel.moba_backward(q, k, v, cud, max(lens), chunk, topk, out, lse, sel, dout, attend_impl=impl)
           for impl in (_lib.ATTEND_TCGEN05, _lib.ATTEND_MMA_SYNC)]
    torch.cuda.synchronize()
    a, b = res[0][0].float(), res[1][0].float()
    assert torch.isfinite(a).all()
    scale = b.abs().max().item()
    assert (a - b).abs().max().item() <= 0.01 * scale
    assert (a != b).float().mean().item() < 0.5
    for x, y in zip(res[0][1:], res[1][1:]):
        assert torch.isfinite(x.float()).all()
        assert (x.float() - y.float()).abs().max().item() <= 0.01 * y.float().abs().max().item()


# --------------------------------------------------------------------------
# CUDA path against outputs of the reference package itself (tests/golden/forward_*.npz)
# --------------------------------------------------------------------------
FORWARD_GOLDEN = sorted(glob.glob(str(Path(__file__).parent / "golden" / "forward_*.npz")))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", FORWARD_GOLDEN, ids=lambda p: p.split("forward_")[-1][:-4])
def test_reference_outputs_and_gradients_through_cuda(path, dtype):
    """Forward and backward on the fixture inputs (exact in bf16 and fp16) against what the
    reference's own kernels returned for them: output within max-abs 2e-2 / mean-abs 2e-3
    (BASELINE.json north_star), gradients within 4 % / 0.4 % of the largest entry."""
    z = np.load(path)
    lens = [int(x) for x in z["seq_lens"]]
    q, k, v, dout = (torch.from_numpy(z[n]).to(dtype).cuda() for n in ("q", "k", "v", "dout"))
    assert (q.float().cpu() == torch.from_numpy(z["q"]).float()).all()          # same numbers in both dtypes
    cud = torch.from_numpy(z["cu_seqlens"]).cuda()
    qd, kd, vd = (x.requires_grad_(True) for x in (q, k, v))
    out = parallel.parallel_moba(qd, kd, vd, cud, max(lens), int(z["chunk"]), int(z["topk"]))
    out.backward(dout)
    torch.cuda.synchronize()
    for name in ("out_ref", "out_train_ref"):
        mx, mean = G.rel_stats(out.detach().cpu(), torch.from_numpy(z[name]).float())
        assert mx < MAX_ABS and mean < MEAN_ABS, (name, mx, mean)
    for name, got in (("dq_ref", qd.grad), ("dk_ref", kd.grad), ("dv_ref", vd.grad)):
        ref = torch.from_numpy(z[name]).double()
        err = (got.double().cpu() - ref).abs()
        scale = ref.abs().max().item()
        assert err.max().item() < 0.04 * scale and err.mean().item() < 0.004 * scale, (name, err.max().item(), scale)


def test_forward_is_capturable_in_a_cuda_graph():
    """The reference's inference path reads nothing back to the host so that it can be captured
    (parallel.py:270-274); the same holds here: capture once, replay on new inputs."""
    q, k, v, cu = _case_inputs((700, 333, 1290), 8, 2, 128, seed=21)
    q2, k2, v2, _ = _case_inputs((700, 333, 1290), 8, 2, 128, seed=22)
    cud = torch.from_numpy(cu).cuda()
    sq, sk, sv = q.cuda(), k.cuda(), v.cuda()                 # static input buffers of the graph
    side = torch.cuda.Stream()
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(2):                                      # warm-up: workspace, kernel attributes
            parallel.parallel_moba(sq, sk, sv, cud, 1290, 128, 4)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), torch.no_grad():
        out = parallel.parallel_moba(sq, sk, sv, cud, 1290, 128, 4)
    for a, b, c in ((q, k, v), (q2, k2, v2)):
        sq.copy_(a); sk.copy_(b); sv.copy_(c)
        graph.replay()
        torch.cuda.synchronize()
        with torch.no_grad():
            eager = parallel.parallel_moba(sq, sk, sv, cud, 1290, 128, 4)
        assert torch.equal(out, eager)


def test_bounded_wait_gives_up_and_the_merge_poisons_the_output():
    """A device-side wait that nothing satisfies runs out after its limit (1 ms here), sets the
    status word and returns; the merge then writes NaN instead of partial results.  The failure
    is made by a barrier nobody arrives on: no fault, no trap, no unbounded spin, and the context
    stays usable (a normal forward afterwards is checked)."""
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.check(_lib.lib().moba_selftest_bounded_wait(status.data_ptr(), 1000, G.stream()))
    t1.record()
    torch.cuda.synchronize()
    assert status[0].item() != 0
    assert 0.9 < t0.elapsed_time(t1) < 50.0                                # waited its millisecond, not the 2 s default
    assert _lib.lib().moba_selftest_bounded_wait(status.data_ptr(), 0, G.stream()) == -1
    # merge of arbitrary finite partials under that status: NaN everywhere
    q, k, v, cu = _case_inputs((512,), 4, 2, 128, seed=1)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    prob, out = G.problem_for(qd, kd, vd, cud, 512, 128, 3)
    d = G.dims_of(prob)
    pout = torch.randn(d.rows * d.partials * 128, dtype=torch.float16, device="cuda")
    plse = torch.randn(d.rows * d.partials, 2, dtype=torch.float32, device="cuda")      # {lse, 1 / scale}
    _lib.check(_lib.lib().moba_merge(C.byref(prob), pout.data_ptr(), plse.data_ptr(), status.data_ptr(), out.data_ptr(),
                                     None, G.stream()))
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()
    status.zero_()
    _lib.check(_lib.lib().moba_merge(C.byref(prob), pout.data_ptr(), plse.data_ptr(), status.data_ptr(), out.data_ptr(),
                                     None, G.stream()))
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    good = parallel.moba_forward(qd, kd, vd, cud, 512, 128, 3)[0]
    assert torch.isfinite(good.float()).all()


def test_incremental_prefill_with_a_means_cache_equals_one_shot():
    """Prefill of one sequence in three chunk-aligned increments, each call seeing a longer K/V
    prefix and taking the means of the chunks completed earlier from a caller-held cache: outputs
    and selections equal the one-shot run bit for bit, and so does the cache in the end."""
    total, hq, hkv, chunk, topk = 3072, 8, 2, 256, 4
    q, k, v, cu = _case_inputs((total,), hq, hkv, chunk, seed=12)
    qd, kd, vd = G.to_dev(q, k, v)
    full, _, full_sel = parallel.moba_forward(qd, kd, vd, torch.from_numpy(cu).cuda(), total, chunk, topk,
                                              return_selected=True)
    mc = total // chunk
    cache = torch.full((mc, hkv, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    cached = 0
    for lo, hi in ((0, 1024), (1024, 1792), (1792, 3072)):
        cu_i = torch.tensor([0, hi], dtype=torch.int32, device="cuda")
        out, _, sel = parallel.moba_forward(qd[lo:hi], kd[:hi], vd[:hi], cu_i, total, chunk, topk, return_selected=True,
                                            q_token_begin=lo, means_cache=cache, cached_slots=cached)
        torch.cuda.synchronize()
        assert torch.equal(out, full[lo:hi]) and torch.equal(sel, full_sel[:, :, lo:hi]), (lo, hi)
        cached = hi // chunk - 1                      # the prefix's last chunk is not final yet
    cu_chunk, _, valid, _ = O.chunk_slots(cu, total, chunk)
    want = O.chunk_means(k, cu_chunk, valid, chunk)
    assert torch.equal(cache.cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("cfg_id,seed", [(1, 43), (2, 44)])
def test_config_selection_full_tensor(cfg_id, seed):
    """BASELINE.json configs[1] and configs[2]: the WHOLE selected-chunk tensor (every token,
    head and rank, 1.2 M and 7.3 M entries), the chunk means and the list sizes against the
    oracle, bit for bit."""
    cfg = O.CONFIGS[cfg_id]
    lens = O.config_lengths(cfg_id)
    q, k, v, cu = O.make_inputs(lens, cfg["hq"], cfg["hkv"], cfg["d"], cfg["chunk"], seed=seed)
    cu_chunk, _, valid, mc = O.chunk_slots(cu, max(lens), cfg["chunk"])
    hist = O.historical_topk(cfg["topk"], mc)
    means_o = O.chunk_means(k, cu_chunk, valid, cfg["chunk"])
    sel_o = O.select_chunks(q, means_o, cu, max(lens), cfg["chunk"], hist)
    qd, kd = q.cuda(), k.cuda()
    cud = torch.from_numpy(cu).cuda()
    prob, _ = G.problem_for(qd, kd, kd, cud, max(lens), cfg["chunk"], cfg["topk"])
    m = G.means(prob, kd, cud)
    assert torch.equal(m.cpu().view(torch.int16), means_o.view(torch.int16))
    sel, counts = G.gate(prob, qd, m, cud)
    assert np.array_equal(sel.cpu().numpy(), sel_o)
    assert counts.sum().item() == (sel_o >= 0).sum()


@pytest.mark.parametrize("case", [("long_items", (2048, 900), 8, 2, 128, 512, 4),
                                  ("short_items", (1500, 700), 8, 2, 128, 128, 5),
                                  ("d256", (1024, 300), 4, 2, 256, 128, 3),
                                  ("mma_sync", (1024, 300), 4, 2, 64, 128, 3)], ids=lambda c: c[0])
def test_stage_entry_points_chain_to_the_forward_result(case):
    """moba_chunk_means -> moba_gate_topk -> moba_compact_routes -> moba_attend -> moba_merge with
    caller-held buffers (work items of moba_problem_tile_rows rows, fp16 partial rows, {lse,
    1 / scale} pairs) give bit for bit what moba_forward gives: the three tcgen05 kernels and
    the mma.sync one."""
    name, lens, hq, hkv, d, chunk, topk = case
    q, k, v, cu = _case_inputs(lens, hq, hkv, chunk, seed=11, d=d)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    impl = _lib.ATTEND_MMA_SYNC if name == "mma_sync" else _lib.ATTEND_TCGEN05
    prob, out = G.problem_for(qd, kd, vd, cud, max(lens), chunk, topk, impl)
    lib = _lib.lib()
    dims = G.dims_of(prob)
    tile_rows = lib.moba_problem_tile_rows(C.byref(prob))
    assert tile_rows == (256 if name == "long_items" else 128)
    m = G.means(prob, kd, cud)
    sel, counts = G.gate(prob, qd, m, cud)
    offsets, tiles, row_list, plse = G.compact(prob, cud, sel, counts, tile_rows)
    pout = torch.empty(dims.rows * dims.partials * d, dtype=torch.float16, device="cuda")
    work = torch.zeros(2, dtype=torch.int32, device="cuda")
    _lib.check(lib.moba_attend(C.byref(prob), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), cud.data_ptr(),
                               counts.data_ptr(), offsets.data_ptr(), tiles.data_ptr(), row_list.data_ptr(),
                               pout.data_ptr(), plse.data_ptr(), work.data_ptr(), G.stream()))
    lse = torch.empty(hq, sum(lens), dtype=torch.float32, device="cuda")
    _lib.check(lib.moba_merge(C.byref(prob), pout.data_ptr(), plse.data_ptr(), work[1:].data_ptr(), out.data_ptr(),
                              lse.data_ptr(), G.stream()))
    torch.cuda.synchronize()
    assert work[1].item() == 0
    want, want_lse, want_sel = parallel.moba_forward(qd, kd, vd, cud, max(lens), chunk, topk, return_lse=True,
                                                     return_selected=True, attend_impl=impl)
    assert torch.equal(sel, want_sel)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert torch.equal(lse, want_lse)
