"""Small parity cases shared by the fixture generator and the tests.

The matrix follows the reference's single-GPU fused test
(tests/fused/test_fused_single_card.py:162-182): complete prefill with tail tiles,
several sequences, a ragged last super-group, GQA, and chunked prefill (q < k) with
aligned / unaligned offsets — at smaller head counts so the fixtures stay small.
Inputs are N(0,1) bf16 drawn from CPU generators seeded ``seed + {0,1,2,3}``.
"""
import hashlib

import torch

D = 128

# name: (seqlens_q, H_local, hidden, q_per_kv, seqlens_k or None, seed)
CASES = {
    "uniform_128":     ([128],           2, 256, 1, None,            11),
    "varlen_200":      ([200],           2, 256, 1, None,            12),
    "vm44_300":        ([300],           2, 256, 1, None,            13),
    "multi_seq":       ([200, 64, 130],  2, 384, 1, None,            14),
    "ragged_hidden":   ([200, 130],      2, 640, 1, None,            15),
    "gqa_q2":          ([200, 64, 130],  4, 256, 2, None,            16),
    "gqa_q4_vm44":     ([300],           4, 200, 4, None,            17),
    "chunk_aligned":   ([128],           2, 256, 1, [384],           18),
    "chunk_unaligned": ([128],           2, 256, 1, [316],           19),
    "chunk_multitile": ([300],           2, 256, 1, [700],           20),
    "chunk_multiseq":  ([200, 64, 130],  2, 384, 1, [512, 64, 260],  21),
    "chunk_gqa_q4":    ([200, 300],      4, 256, 4, [328, 700],      22),
    # the CPU-runnable benchmark configuration: B=3, 8 q / 1 kv heads, hidden 1024
    "c1":              ([64, 200, 256],  8, 1024, 8, None,           0),
}


def _randn(shape, seed, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)


def make_inputs(name):
    sq, H, hidden, qpk, sk, seed = CASES[name]
    sk = sq if sk is None else sk
    Hkv = H // qpk
    base = seed * 1000
    Q = _randn((sum(sq), H, D), base + 0)
    K = _randn((sum(sk), Hkv, D), base + 1)
    V = _randn((sum(sk), Hkv, D), base + 2)
    W = _randn((H * D, hidden), base + 3, float(H * D) ** -0.5)
    return Q, K, V, W


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    return h.hexdigest()
