"""CPU statement of the rotary position embedding of the producer side (TEST
INFRASTRUCTURE: imported by tests only, never by the product path).

The reference has no implementation of this op (README.md:41-44 of the reference lists the
"QKV-proj / RoPE producer" as not built): **parity unpinned** with respect to the reference.
It is pinned instead to the textbook definition — multiplication of the pairs (x[d], x[d+64])
by exp(i * pos * w_d) — evaluated in float64 (``tests/test_producer_oracle_cpu.py``).
"""
import numpy as np
import torch


def inv_freq_fp32(theta=10000.0):
    return 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128.0))


def rope_oracle(q, k, seqlens_q, seqlens_k=None, theta=10000.0):
    """q [tot_q, H, 128], k [tot_k, Hkv, 128] bf16 -> rotated copies.  Rotate-half convention,
    fp32 frequencies, angles and products, one rounding; K: last q_len rows of each sequence."""
    seqlens_k = seqlens_q if seqlens_k is None else seqlens_k
    w = inv_freq_fp32(theta)
    qo, ko = q.clone(), k.clone()

    def rot(x, pos):                      # x [n, h, 128] bf16, pos [n] int
        ang = pos.to(torch.float32)[:, None] * w[None, :]          # fp32 product
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        x1, x2 = x[..., :64].float(), x[..., 64:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(torch.bfloat16)

    q0 = k0 = 0
    for lq, lk in zip(seqlens_q, seqlens_k):
        pos = torch.arange(lk - lq, lk)
        qo[q0:q0 + lq] = rot(q[q0:q0 + lq], pos)
        ko[k0 + lk - lq:k0 + lk] = rot(k[k0 + lk - lq:k0 + lk], pos)
        q0 += lq
        k0 += lk
    return qo, ko
