"""GPU: the CUDA path against the reference's own Triton kernels on the same device.

The reference package (backends/_mthreads/ops/moba, copied unmodified by
baseline/install_ref.py) runs its inference path in bfloat16 on the B200: slot tables and
chunk means (routing.py:595-632, :740-775), scores and top-k (:1185-1262), and the whole
forward (parallel.py:253-374: own-chunk attention, routed attention, LSE merge).  Compared on
BASELINE.json configs 0, 1 and 2 in full and on one (sequence, KV-head group) unit of
config 3 (131072 tokens), each call below the reference's int32 index range.

What is asserted
  * chunk means: every element within one bf16 unit of the reference's (both are roundings of
    fp32 sums in different orders); the count of differing elements is reported;
  * selected chunks with IDENTICAL means (the reference's means fed to both top-k kernels):
    every (token, head) row whose ordered selection differs is audited against float64 scores.
    The reference scores with tl.dot (routing.py:1132-1136), this build in its fixed fp32
    order; both sum 128 exact products in fp32, so two scores closer than
    REL_BOUND * (sum_i |q_i m_i| of the two candidates) may legitimately rank either way.
    The test fails on any disagreement whose float64 gap is larger than that;
  * selected chunks end to end (each side with its own means): audited the same way, each
    side against the float64 scores of its own means;
  * outputs: on rows whose selections agree, max-abs and mean-abs difference to the
    reference's bf16 output (the reference rounds its running output to bf16 after every
    rank pass, parallel.py:333, :363-373; this build rounds once).
The module is skipped when the reference copy or Triton is unavailable.
"""
import numpy as np
import pytest
import torch

from baselinebenchmark_b200 import parallel
from baseline import ref_triton as R
from oracle import moba_oracle as O
from tests import gpu_util as G

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(R.available() is not None, reason=str(R.available()))]

#: relative size of an fp32 summation error of 128 exact products that either kernel may make
#: (this build's gating kernel assumes the same figure for the tensor core, csrc/gate.cu)
REL_BOUND = 4e-5

# (name, seq_lens, Hq, Hkv, chunk, topk, seed)
CASES = [
    ("cfg0", O.config_lengths(0), 8, 8, 512, 3, 42),
    ("cfg1", O.config_lengths(1), 32, 32, 512, 3, 43),
    ("cfg2", O.config_lengths(2), 32, 8, 4096, 12, 44),
    ("cfg3_unit", [131072], 4, 1, 4096, 8, 45),
]


def _audit(q, means, cu, chunk, mc, sel, other):
    """Rows where `sel` and `other` differ: is `sel` an ordering the float64 scores of `means`
    allow within REL_BOUND?  Returns (rows differing, worst gap / allowed gap)."""
    hq, hkv = q.shape[1], means.shape[1]
    g = hq // hkv
    diff = (sel != other).any(0).nonzero().tolist()                     # [head, token]
    cu_l = cu.tolist()
    worst = 0.0
    for h, t in diff[:4000]:
        b = int(np.searchsorted(cu_l, t, side="right") - 1)
        ncand = (t - cu_l[b]) // chunk
        slots = b * mc + torch.arange(ncand, device=q.device)
        m = means[slots, h // g].double()
        qq = q[t, h].double()
        s64 = m @ qq
        mag = m.abs() @ qq.abs()
        mine = sel[:, h, t]
        mine = (mine[mine >= 0] - b * mc).long()
        assert mine.numel() == min(sel.shape[0], ncand)
        rest = torch.ones(ncand, dtype=torch.bool, device=q.device)
        rest[mine] = False
        chain = torch.cat([mine, rest.nonzero().flatten()[s64[rest].argsort(descending=True)[:1]]])
        for a, c in zip(chain[:-1].tolist(), chain[1:].tolist()):      # each entry must not lose to the next
            allowed = REL_BOUND * (mag[a] + mag[c]).item() + 1e-30
            worst = max(worst, (s64[c] - s64[a]).item() / allowed)
    return len(diff), worst


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_routing_and_outputs_against_reference_triton(case, record_property):
    name, lens, hq, hkv, chunk, topk, seed = case
    q, k, v, cu = O.make_inputs(list(lens), hq, hkv, 128, chunk, seed=seed)
    qd, kd, vd = G.to_dev(q, k, v)
    cud = torch.from_numpy(cu).cuda()
    max_seqlen = max(lens)
    mc = O.cdiv(max_seqlen, chunk)
    prob, _ = G.problem_for(qd, kd, vd, cud, max_seqlen, chunk, topk)

    ours_means = G.means(prob, kd, cud)
    ref_means, ref_sel = R.routing(qd, kd, cud, max_seqlen, chunk, topk)
    # chunk means: roundings of the same sums in different fp32 orders
    a, b = ours_means.view(torch.int16).int(), ref_means.view(torch.int16).int()
    means_differ = int((a != b).sum())
    assert ((a - b).abs() <= 1).all(), "chunk means differ by more than one bf16 unit"

    # identical means on both sides
    _, ref_sel_same = R.routing(qd, kd, cud, max_seqlen, chunk, topk, means=ref_means)
    ours_same, _ = G.gate(prob, qd, ref_means, cud)
    n_same, worst_ours = _audit(qd, ref_means, cud.cpu(), chunk, mc, ours_same, ref_sel_same)
    _, worst_ref = _audit(qd, ref_means, cud.cpu(), chunk, mc, ref_sel_same, ours_same)
    assert worst_ours <= 1.0 and worst_ref <= 1.0, (n_same, worst_ours, worst_ref)

    # end to end, each side with its own means
    out, _, ours_sel = parallel.moba_forward(qd, kd, vd, cud, max_seqlen, chunk, topk, return_selected=True)
    n_e2e, w1 = _audit(qd, ours_means, cud.cpu(), chunk, mc, ours_sel, ref_sel)
    _, w2 = _audit(qd, ref_means, cud.cpu(), chunk, mc, ref_sel, ours_sel)
    assert w1 <= 1.0 and w2 <= 1.0, (n_e2e, w1, w2)

    ref_out = R.forward(qd, kd, vd, cud, max_seqlen, chunk, topk)
    agree = ~(ours_sel != ref_sel).any(0).T                              # [T, Hq]
    d = (out.float() - ref_out.float()).abs()[agree]
    mx, mean = d.max().item(), d.mean().item()
    rows = q.shape[0] * hq
    summary = dict(case=name, rows=rows, means_elements_differing=means_differ,
                   rows_differing_same_means=n_same, rows_differing_end_to_end=n_e2e,
                   worst_gap_over_bound=max(worst_ours, worst_ref, w1, w2), out_max_abs=mx, out_mean_abs=mean)
    record_property("reference_triton", summary)
    print("reference_triton", summary)
    assert mx < 0.06 and mean < 1e-3, summary
