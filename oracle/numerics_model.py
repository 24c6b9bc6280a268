"""CPU model of the rounding points of a bf16-staged fused prefill pipeline.  TEST
INFRASTRUCTURE ONLY — never on a product code path.

The fp32 chain of ``oracle/chain_oracle.py`` (the reference's ``src/mega_attention/
reference/fused.py:215-221``) rounds once, at the very end.  A kernel that stages its
intermediates the way the reference's device code does (fused_fa_oproj_ar.py:848-999:
fp32 scores and softmax statistics, P cast to bf16 before ``P V``, the attention output
stored to O_scratch as bf16; :1001-1104: fp32 GEMM accumulation, bf16 partial in C_sym;
:1105-1142: fp32 sum of the ranks' bf16 partials, one cast) cannot reproduce the chain bit
for bit; this model computes what such a pipeline gives when everything between the
rounding points is exact fp32, so a test can tell "the kernel is as accurate as its
staging allows" from "the kernel has a defect":

* per (sequence, q head, 128-row tile): key blocks of 128 from the last visible one down to
  block 0, scores in fp32, running row maximum, ``P = bf16(exp2((s - m) * scale * log2 e))``,
  row sum of the un-rounded exponentials in fp32, ``O += P V`` in fp32, rescale when the
  maximum moves;
* ``O / l`` rounded to bf16 (O_scratch);
* ``O_scratch @ W_o`` in fp32, rounded to bf16 (the rank's partial);
* tp > 1: fp32 sum of the bf16 partials, rounded to bf16.
"""
from __future__ import annotations

import numpy as np
import torch

M_TILE = 128
LOG2E = 1.4426950408889634


def _cu(lens):
    out = np.zeros(len(lens) + 1, dtype=np.int64)
    out[1:] = np.cumsum(np.asarray(lens, dtype=np.int64))
    return out


def attention_model(Q, K, V, seqlens_q, seqlens_k=None, softmax_scale=None):
    """bf16 ``O [tot_q, H, D]`` of the staged pipeline (fp32 statistics, bf16 P, fp32 O)."""
    seqlens_k = seqlens_q if seqlens_k is None else seqlens_k
    H, Hkv, D = Q.shape[1], K.shape[1], Q.shape[2]
    group = H // Hkv
    scale = float(D) ** -0.5 if softmax_scale is None else float(softmax_scale)
    sl2 = scale * LOG2E
    cq, ck = _cu(seqlens_q), _cu(seqlens_k)
    out = torch.zeros(Q.shape, dtype=torch.bfloat16)
    for b in range(len(seqlens_q)):
        q0, q1, k0, k1 = int(cq[b]), int(cq[b + 1]), int(ck[b]), int(ck[b + 1])
        lq, lk = q1 - q0, k1 - k0
        offset = lk - lq
        for mb in range(-(-lq // M_TILE)):
            r0 = mb * M_TILE
            rows = min(M_TILE, lq - r0)
            nblk = min(-(-lk // M_TILE), -(-((mb + 1) * M_TILE + offset) // M_TILE))
            qpos = torch.arange(r0, r0 + rows)[:, None] + offset
            q = Q[q0 + r0:q0 + r0 + rows].float().transpose(0, 1)          # [H, rows, D]
            m = torch.full((H, rows), float("-inf"))
            l = torch.zeros(H, rows)
            acc = torch.zeros(H, rows, D)
            for j in range(nblk - 1, -1, -1):
                c0, c1 = j * M_TILE, min((j + 1) * M_TILE, lk)
                k = K[k0 + c0:k0 + c1].float().transpose(0, 1).repeat_interleave(group, 0)
                v = V[k0 + c0:k0 + c1].float().transpose(0, 1).repeat_interleave(group, 0)
                s = torch.matmul(q, k.transpose(1, 2))                       # [H, rows, cols]
                keep = torch.arange(c0, c1)[None, :] <= qpos
                s = s.masked_fill(~keep[None], float("-inf"))
                m_new = torch.maximum(m, s.max(dim=2).values)
                m_safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                alpha = torch.where(torch.isinf(m), torch.zeros_like(m),
                                    torch.exp2((m - m_safe) * sl2))
                e = torch.exp2((s - m_safe[..., None]) * sl2)                # exp2(-inf) = 0
                l = l * alpha + e.sum(dim=2)
                acc = acc * alpha[..., None] + torch.matmul(e.to(torch.bfloat16).float(), v)
                m = m_new
            o = acc / l.clamp_min(1e-30)[..., None]
            out[q0 + r0:q0 + r0 + rows] = o.transpose(0, 1).to(torch.bfloat16)
    return out


def chain_model(Q, K, V, W_o, seqlens_q, seqlens_k=None, softmax_scale=None):
    """One rank: ``(O_scratch values bf16 [tot_q,H,D], partial bf16 [tot_q,hidden])``."""
    O = attention_model(Q, K, V, seqlens_q, seqlens_k, softmax_scale)
    Y = (O.float().reshape(O.shape[0], -1) @ W_o.float()).to(torch.bfloat16)
    return O, Y


def allreduce_model(partials_bf16):
    """fp32 sum of the ranks' bf16 partials, one cast (what the switch reduction gives)."""
    acc = partials_bf16[0].float().clone()
    for p in partials_bf16[1:]:
        acc += p.float()
    return acc.to(torch.bfloat16)
