"""CPU: pins the oracle's routing restatement against outputs of the
reference's own routing kernels (tests/golden/routing_*.npz, produced by
tests/golden/make_routing_golden.py) and against the reference's procedural
known-answer tests (backends/_mthreads/tests/test_moba_topk.py)."""
import glob

import numpy as np
import pytest
import torch

from oracle import moba_oracle as O

GOLDEN = sorted(glob.glob(str(__import__("pathlib").Path(__file__).parent / "golden" / "routing_*.npz")))


def _load(path):
    z = np.load(path)
    q = torch.from_numpy(z["q_bits"]).view(torch.bfloat16)
    k = torch.from_numpy(z["k_bits"]).view(torch.bfloat16)
    return z, q, k


def test_golden_files_present():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.split("routing_")[-1][:-4])
def test_chunk_slots_match_reference(path):
    z, _, _ = _load(path)
    cu_chunk, chunk_end, valid, mc = O.chunk_slots(z["cu_seqlens"], int(z["max_seqlen"]), int(z["chunk"]))
    assert mc == int(z["mc"])
    np.testing.assert_array_equal(cu_chunk, z["cu_chunk"])
    np.testing.assert_array_equal(chunk_end, z["chunk_end"])
    np.testing.assert_array_equal(valid, z["valid_hist"])
    assert O.historical_topk(int(z["topk"]), mc) == int(z["hist"])


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.split("routing_")[-1][:-4])
def test_chunk_means_match_reference(path):
    z, _, k = _load(path)
    cu_chunk, _, valid, _ = O.chunk_slots(z["cu_seqlens"], int(z["max_seqlen"]), int(z["chunk"]))
    # bf16 means against a float64 sum rounded once
    means = O.chunk_means(k, cu_chunk, valid, int(z["chunk"]))
    np.testing.assert_array_equal(means.view(torch.int16).numpy(), z["means_rne_bits"])
    # the same numbers in float16 against the reference kernel's float16 output
    means16 = O.chunk_means(k.half(), cu_chunk, valid, int(z["chunk"]))
    np.testing.assert_array_equal(means16.numpy(), z["means_ref_f16"])


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.split("routing_")[-1][:-4])
def test_selected_chunks_match_reference(path):
    z, q, _ = _load(path)
    hist = int(z["hist"])
    if hist <= 0:
        pytest.skip("no historical chunk")
    means = torch.from_numpy(z["means_rne_bits"]).view(torch.bfloat16)
    sel = O.select_chunks(q, means, z["cu_seqlens"], int(z["max_seqlen"]), int(z["chunk"]), hist)
    np.testing.assert_array_equal(sel, z["selected_ref"])


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.split("routing_")[-1][:-4])
def test_reference_route_lists_hold_the_same_rows(path):
    """The reference groups routed rows by (slot, q head) (routing.py:1326); the
    multiset of (row, slot) pairs must equal the oracle's selection."""
    z, _, _ = _load(path)
    if int(z["hist"]) <= 0:
        pytest.skip("no historical chunk")
    hq = int(z["hq"])
    sel = z["selected_ref"]
    offs, qi = z["expert_offsets"], z["query_indices"]
    got = set()
    for e in range(len(offs) - 1):
        for pos in range(offs[e], offs[e + 1]):
            got.add((int(qi[pos]), e // hq, e % hq))
    want = set()
    hist, _, t_total = sel.shape
    for r in range(hist):
        for h in range(hq):
            for t in np.nonzero(sel[r, h] >= 0)[0]:
                want.add((int(t) * hq + h, int(sel[r, h, t]), h))
    assert got == want


def test_tie_break_prefers_lower_slot():
    # all scores equal: the lowest slots win, in increasing order (SEMANTICS.md:55)
    z, q, _ = _load([p for p in GOLDEN if "ties_zero" in p][0])
    sel = z["selected_ref"]
    cu = z["cu_seqlens"]
    mc, chunk = int(z["mc"]), int(z["chunk"])
    for b in range(len(cu) - 1):
        for t in range(cu[b], cu[b + 1]):
            cur = (t - cu[b]) // chunk
            want = [b * mc + i if i < cur else -1 for i in range(sel.shape[0])]
            assert sel[:, 0, t].tolist() == want


# ---- the reference's known-answer tests, run on the oracle -------------------
def test_topk1_is_chunk_local():
    """test_moba_topk.py:30-57: zero q/k, V constant per chunk, K = 1."""
    lengths, chunk = (192, 129), 64
    total = sum(lengths)
    q = torch.zeros(total, 4, 64, dtype=torch.bfloat16)
    k = torch.zeros(total, 2, 64, dtype=torch.bfloat16)
    v = torch.empty_like(k)
    expected = torch.empty_like(q)
    start = 0
    for b, n in enumerate(lengths):
        for pos in range(n):
            val = (pos // chunk + 1) * (1 if b == 0 else -1)
            v[start + pos].fill_(val)
            expected[start + pos].fill_(val)
        start += n
    cu = np.array([0, lengths[0], total], dtype=np.int32)
    out, _, sel = O.moba_forward(q, k, v, cu, max(lengths), chunk, 1)
    assert sel.shape[0] == 0
    torch.testing.assert_close(out.bfloat16(), expected, rtol=0, atol=0)


@pytest.mark.parametrize("lengths,topk", [((257, 193), 2), ((257, 193), 64), ((1100,), 64)])
def test_separated_scores_against_float64(lengths, topk):
    """test_moba_topk.py:60-118 with its float64 procedure written out
    independently of the oracle's own evaluation code."""
    chunk, hq, hkv, dim = 64, 4, 2, 64
    total = sum(lengths)
    dtype = torch.bfloat16
    qc = torch.full((total, hq, dim), 0.125, dtype=dtype)
    qc[:, 1::2] *= -1
    kc = torch.empty(total, hkv, dim, dtype=dtype)
    start = 0
    for n in lengths:
        for pos in range(n):
            kc[start + pos].fill_((pos // chunk + 1) / 128)
        start += n
    vc = torch.randn(total, hkv, dim, generator=torch.Generator().manual_seed(42)).to(dtype)
    bounds = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    actual, _, _ = O.moba_forward(qc, kc, vc, bounds, max(lengths), chunk, topk)
    actual = actual.double()
    errors = []
    for b, n in enumerate(lengths):
        s = int(bounds[b])
        keys, values = kc[s:s + n], vc[s:s + n].double()
        means = torch.stack([keys[t:t + chunk].double().mean(0).to(dtype).double() for t in range(0, n, chunk)])
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
                errors.append((actual[s + pos, head] - logits.softmax(0) @ values[idx, kvh]).abs())
    diff = torch.stack(errors)
    assert torch.isfinite(diff).all()
    assert diff.max().item() < 0.04 and diff.mean().item() < 4e-4


def test_reference_tile_numerics_agree_with_exact_evaluation():
    """attention.py:116-155 + :849-889 restated (bf16 P, per-branch flash, LSE
    merge) stays within the reference's published error of the exact softmax."""
    q, k, v, cu = O.make_inputs([640], 2, 1, 128, 128, seed=7)
    out, lse, sel = O.moba_forward(q, k, v, cu, 640, 128, 3, dtype=torch.float64)
    for (t, h) in [(639, 0), (300, 1), (129, 0)]:
        outs, lses = [], []
        own0 = (t // 128) * 128
        o, l = O.branch_flash(q[t, h], k[own0:t + 1, 0], v[own0:t + 1, 0])
        outs.append(o), lses.append(l)
        for r in range(sel.shape[0]):
            s = int(sel[r, h, t])
            if s >= 0:
                o, l = O.branch_flash(q[t, h], k[s * 128:(s + 1) * 128, 0], v[s * 128:(s + 1) * 128, 0])
                outs.append(o), lses.append(l)
        merged, mlse = O.merge_lse(outs, lses)
        assert np.abs(merged - out[t, h].numpy()).max() < 0.0063
        assert abs(float(mlse) - float(lse[h, t])) < 1e-3


# --------------------------------------------------------------------------
# the whole operator and its backward against the reference package run end to end
# (tests/golden/forward_*.npz, produced by tests/golden/make_forward_golden.py)
# --------------------------------------------------------------------------
FORWARD_GOLDEN = sorted(glob.glob(str(__import__("pathlib").Path(__file__).parent / "golden" / "forward_*.npz")))


def _load_forward(path):
    z = np.load(path)
    t = {n: torch.from_numpy(z[n]) for n in ("q", "k", "v", "dout", "out_ref", "out_train_ref", "dq_ref", "dk_ref", "dv_ref")}
    return z, t


def test_forward_golden_files_present():
    assert len(FORWARD_GOLDEN) >= 4


@pytest.mark.parametrize("path", FORWARD_GOLDEN, ids=lambda p: p.split("forward_")[-1][:-4])
def test_oracle_forward_matches_reference_output(path):
    """Oracle (contract routing + fp32 evaluation) against the output of the reference's
    inference path and of its training forward, both float16: float16 rounding of the output
    (2^-11 relative) plus the float16 rounding of P inside the reference kernels."""
    z, t = _load_forward(path)
    lens = [int(x) for x in z["seq_lens"]]
    out, _, _ = O.moba_forward(t["q"], t["k"], t["v"], z["cu_seqlens"], max(lens), int(z["chunk"]), int(z["topk"]))
    for name in ("out_ref", "out_train_ref"):
        err = (out - t[name].float()).abs()
        assert err.max().item() < 4e-3 and err.mean().item() < 2e-4, (name, err.max().item(), err.mean().item())


@pytest.mark.parametrize("path", FORWARD_GOLDEN, ids=lambda p: p.split("forward_")[-1][:-4])
def test_oracle_gradients_match_reference_backward(path):
    """float64 autograd of the oracle's evaluation against the gradients the reference's
    backward kernels produced (float16)."""
    z, t = _load_forward(path)
    lens = [int(x) for x in z["seq_lens"]]
    _, _, sel = O.moba_forward(t["q"], t["k"], t["v"], z["cu_seqlens"], max(lens), int(z["chunk"]), int(z["topk"]))
    dq, dk, dv = O.attend_grads(t["q"], t["k"], t["v"], z["cu_seqlens"], max(lens), int(z["chunk"]), sel, t["dout"])
    for name, got in (("dq_ref", dq), ("dk_ref", dk), ("dv_ref", dv)):
        ref = t[name].double()
        err = (got - ref).abs()
        scale = ref.abs().max().item()
        assert err.max().item() < 4e-3 * scale and err.mean().item() < 2e-4 * scale, (name, err.max().item(), scale)


def test_rows_of_a_prefix_equal_rows_of_the_whole_sequence():
    """What incremental prefill and decode rest on, stated on the oracle: the rows of a prefix
    of the sequence - selection, output and LSE - are those of the whole sequence.  A query only
    sees keys at or before its own position, only chunks before its own are candidates, and a
    complete chunk's mean depends on its own keys alone; the prefix's last, possibly partial,
    chunk is nobody's candidate yet.  max_seqlen is the capacity in every call so that the
    slots and the number of selected chunks keep their meaning.  The selection is compared
    exactly; outputs and LSE to 1e-5 (the oracle's fp32 matrix products sum in an order that
    depends on the shapes)."""
    total, capacity, chunk, topk = 700, 1024, 64, 4
    q, k, v, cu = O.make_inputs([total], 4, 2, 64, chunk, seed=19)
    out, lse, sel = O.moba_forward(q, k, v, cu, capacity, chunk, topk)
    for t in (1, 63, 64, 65, 300, 511, 699):
        cu_t = np.array([0, t], dtype=np.int32)
        out_t, lse_t, sel_t = O.moba_forward(q[:t], k[:t], v[:t], cu_t, capacity, chunk, topk)
        assert np.array_equal(sel_t, sel[:, :, :t]), t
        assert torch.allclose(out_t, out[:t], rtol=0, atol=1e-5), t
        assert torch.allclose(lse_t, lse[:, :t], rtol=0, atol=1e-5), t
