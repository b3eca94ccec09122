"""Timed CPU baseline of the MoBA forward.  TEST / BENCHMARK INFRASTRUCTURE ONLY.

The reference ships no CPU implementation of MoBA; its only pure-PyTorch MoBA
computation is the sampled float64 check of
backends/_mthreads/tests/test_moba_topk.py:92-113 (chunk means rounded to the
input dtype, top-(K-1) of the earlier chunks, one softmax over the own chunk up
to the query plus the selected chunks).  This module is that computation
vectorised with PyTorch CPU ops in fp32 so it can be timed on all host cores:
it spends exactly the algorithmic FLOPs (own chunk + selected chunks only) by
grouping query rows per selected chunk and merging the partial softmaxes by
their log-sum-exp.  Nothing in the shipped package imports it.
"""
from __future__ import annotations

import numpy as np
import torch


def moba_forward_cpu(q, k, v, cu_seqlens, max_seqlen: int, chunk: int, topk: int, query_chunks=None):
    """Returns (out fp32 [T,Hq,D], computed bool[T]).

    `query_chunks` (iterable of chunk indices, per sequence) restricts the
    queries that are evaluated; keys and chunk means are always complete.
    """
    t_total, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    scale = d ** -0.5
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    mc = -(-max_seqlen // chunk)
    hist = min(topk - 1, mc - 1)
    out = torch.zeros(t_total, hq, d, dtype=torch.float32)
    done = torch.zeros(t_total, dtype=torch.bool)
    kf, vf = k.float(), v.float()
    for b in range(len(cu) - 1):
        s0, s1 = int(cu[b]), int(cu[b + 1])
        n = s1 - s0
        nck = -(-n // chunk)
        nfull = n // chunk if n % chunk else nck - 1              # chunks that can be selected
        means = None
        if hist > 0 and nfull > 0:
            means = kf[s0:s0 + nfull * chunk].view(nfull, chunk, hkv, d).mean(1).to(q.dtype).float()
        for j in range(nck):
            if query_chunks is not None and j not in query_chunks:
                continue
            a, e = s0 + j * chunk, min(s0 + (j + 1) * chunk, s1)
            qc = q[a:e].float()                                   # [n_j, Hq, D]
            nj = e - a
            done[a:e] = True
            for h in range(hq):
                kh = h // g
                qh = qc[:, h]
                # own chunk, token-causal
                logits = (qh @ kf[a:e, kh].T) * scale
                logits.masked_fill_(torch.ones(nj, nj, dtype=torch.bool).triu_(1), float("-inf"))
                m = logits.max(1).values
                p = torch.exp(logits - m[:, None])
                l = p.sum(1)
                acc = p @ vf[a:e, kh]
                nsel = min(hist, j)
                if nsel > 0:
                    scores = qh @ means[:j, kh].T                 # [n_j, j]
                    sel = torch.topk(scores, nsel, dim=1).indices
                    member = torch.zeros(nj, j, dtype=torch.bool)
                    member.scatter_(1, sel, True)
                    for c in range(j):
                        rows = member[:, c].nonzero().squeeze(1)
                        if rows.numel() == 0:
                            continue
                        kc = kf[s0 + c * chunk:s0 + (c + 1) * chunk, kh]
                        vc = vf[s0 + c * chunk:s0 + (c + 1) * chunk, kh]
                        lg = (qh[rows] @ kc.T) * scale
                        m_new = torch.maximum(m[rows], lg.max(1).values)
                        alpha = torch.exp(m[rows] - m_new)
                        pc = torch.exp(lg - m_new[:, None])
                        l[rows] = l[rows] * alpha + pc.sum(1)
                        acc[rows] = acc[rows] * alpha[:, None] + pc @ vc
                        m[rows] = m_new
                out[a:e, h] = acc / l[:, None]
    return out, done
