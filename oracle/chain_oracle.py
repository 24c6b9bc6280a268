"""CPU oracle for the fused prefill path.  TEST INFRASTRUCTURE ONLY — never on a
product code path; it is the checker, not the thing measured or shipped.

Restates, in explicit fp32 tensor arithmetic, the algorithm of the reference's
``src/mega_attention/reference/fused.py``:

* ``fa_oracle``        follows ``fa_reference``        (fused.py:80-117)
* ``o_scratch_oracle`` follows ``o_scratch_reference`` (fused.py:178-193)
* ``oproj_oracle``     follows ``oproj_reference``     (fused.py:197-204)
* ``allreduce_oracle`` follows ``allreduce_reference`` (fused.py:207-212) with the
  cross-rank sum taken over a list of per-rank partials instead of a process group
* ``full_chain_oracle`` follows ``full_chain_reference`` (fused.py:215-221)

The reference delegates the attention math to ``torch.nn.functional.
scaled_dot_product_attention`` (PyTorch, unpinned in the reference's pyproject; 2.11.0
in this image) with an explicit boolean mask on fp32 tensors.  Here the published
definition is written out: ``softmax(scale * Q K^T + mask) V`` with the mask keeping
``kpos <= qpos + (k_len - q_len)`` (causal, aligned bottom-right).

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference module itself
(imported from the reference tree by ``tests/golden/make_golden.py``); the CPU tests
check this file against them.
"""
from __future__ import annotations

import numpy as np
import torch

M_TILE = 128


def _cu(lens):
    out = np.zeros(len(lens) + 1, dtype=np.int64)
    out[1:] = np.cumsum(np.asarray(lens, dtype=np.int64))
    return out


def fa_oracle(Q, K, V, seqlens_q, seqlens_k=None, softmax_scale=None):
    """Causal varlen GQA attention in fp32.

    ``Q [tot_q, H, D]``, ``K/V [tot_k, H_kv, D]`` packed per sequence; q head ``h`` reads
    kv head ``h // (H // H_kv)``.  Returns ``O [tot_q, H, D]`` fp32.
    """
    seqlens_k = seqlens_q if seqlens_k is None else seqlens_k
    H, Hkv, D = Q.shape[1], K.shape[1], Q.shape[2]
    assert H % Hkv == 0
    group = H // Hkv
    scale = float(D) ** -0.5 if softmax_scale is None else float(softmax_scale)
    cq, ck = _cu(seqlens_q), _cu(seqlens_k)
    O = torch.zeros(Q.shape, dtype=torch.float32)
    for b in range(len(seqlens_q)):
        q0, q1, k0, k1 = int(cq[b]), int(cq[b + 1]), int(ck[b]), int(ck[b + 1])
        lq, lk = q1 - q0, k1 - k0
        if lq == 0:
            continue
        keep = (torch.arange(lk)[None, :] <= torch.arange(lq)[:, None] + (lk - lq))
        for h in range(H):
            q = Q[q0:q1, h].float()
            k = K[k0:k1, h // group].float()
            v = V[k0:k1, h // group].float()
            s = (q @ k.T) * scale
            s = s.masked_fill(~keep, float("-inf"))
            s = s - s.max(dim=1, keepdim=True).values
            p = torch.exp(s)
            O[q0:q1, h] = (p / p.sum(dim=1, keepdim=True)) @ v
    return O


def make_paged_kv(K, V, seqlens_k, page_size=128, num_pages=None, shuffle=True, seed=0):
    """Scatter packed ``K/V [tot_k, H_kv, D]`` into a paged cache (follows ``make_paged_kv``,
    fused.py:121-175, with the same generators so the result is identical on the CPU).

    Returns ``(K_cache, V_cache [num_pages, 128, H_kv, D], page_table [B, max_pps] int32,
    cache_seqlens [B] int32)``.  Physical pages are a seeded permutation; every slot that
    holds no valid token (tail of a last page, unused pages) is filled with finite random
    values, so only masking - not zero fill - keeps them out of the result.
    """
    assert page_size == 128
    lens = [int(x) for x in seqlens_k]
    B = len(lens)
    Hkv, D = K.shape[1], K.shape[2]
    pages_per_seq = [(s + page_size - 1) // page_size for s in lens]
    total = int(sum(pages_per_seq))
    if num_pages is None:
        num_pages = total
    assert num_pages >= total
    g = torch.Generator(device="cpu").manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist() if shuffle else list(range(num_pages))
    gk = torch.Generator(device="cpu").manual_seed(seed + 11)
    Kc = torch.randn(num_pages, page_size, Hkv, D, dtype=K.dtype, generator=gk) * 0.2
    Vc = torch.randn(num_pages, page_size, Hkv, D, dtype=K.dtype, generator=gk) * 0.2
    table = torch.zeros(B, max(max(pages_per_seq) if B else 0, 1), dtype=torch.int32)
    nxt, off = 0, 0
    for b in range(B):
        for i in range(pages_per_seq[b]):
            phys = perm[nxt]
            nxt += 1
            table[b, i] = phys
            lo, hi = i * page_size, min((i + 1) * page_size, lens[b])
            Kc[phys, :hi - lo] = K[off + lo:off + hi]
            Vc[phys, :hi - lo] = V[off + lo:off + hi]
        off += lens[b]
    return Kc, Vc, table, torch.tensor(lens, dtype=torch.int32)


def tile_coords(seqlens_q):
    """``(q_tile_start, valid_m)`` per flattened 128-row tile (row_desc.py:96-104)."""
    out = []
    cq = _cu(seqlens_q)
    for b, lq in enumerate(seqlens_q):
        for mb in range(-(-int(lq) // M_TILE)):
            out.append((int(cq[b]) + mb * M_TILE, min(M_TILE, int(lq) - mb * M_TILE)))
    return out


def o_scratch_oracle(O, seqlens_q):
    """Pack ``O [tot_q,H,D]`` into ``[num_row_tiles,128,H,D]``; tail rows stay zero."""
    tiles = tile_coords(seqlens_q)
    out = torch.zeros(len(tiles), M_TILE, O.shape[1], O.shape[2], dtype=torch.float32)
    for t, (start, vm) in enumerate(tiles):
        out[t, :vm] = O[start:start + vm]
    return out


def oproj_oracle(O, W_o):
    """``Y_partial [tot_q, hidden] = concat_heads(O) @ W_o`` in fp32; ``W_o [H*D, hidden]``."""
    return O.float().reshape(O.shape[0], -1) @ W_o.float()


def allreduce_oracle(partials):
    """fp32 sum over the per-rank partials, then one cast to bf16."""
    acc = partials[0].float().clone()
    for p in partials[1:]:
        acc += p.float()
    return acc.to(torch.bfloat16)


def full_chain_oracle(Q, K, V, W_o, seqlens_q, seqlens_k=None, softmax_scale=None):
    """One rank: returns ``(O fp32, Y_partial fp32, Y_final bf16)``."""
    O = fa_oracle(Q, K, V, seqlens_q, seqlens_k, softmax_scale)
    Yp = oproj_oracle(O, W_o)
    return O, Yp, allreduce_oracle([Yp])


def untile_csym(csym, seqlens_q, hidden):
    """``csym [R,128,num_out,128]`` -> ``[tot_q, hidden]`` over the valid region
    (the de-tiling of benchmarks/bench_fused_fa_oproj_ar.py:263-269)."""
    tiles = tile_coords(seqlens_q)
    R, _, num_out, nt = csym.shape
    flat = csym.reshape(R, M_TILE, num_out * nt)
    out = torch.empty(int(sum(int(x) for x in seqlens_q)), hidden, dtype=csym.dtype)
    for t, (start, vm) in enumerate(tiles):
        out[start:start + vm] = flat[t, :vm, :hidden]
    return out


def err_rel(got, ref):
    """``max|got - ref| / max|ref|`` in fp32 (bench_fused_fa_oproj_ar.py:259-270)."""
    g, r = got.float(), ref.float()
    return float((g - r).abs().max() / r.abs().max().clamp_min(1e-30))


def bf16_half_ulp(x):
    """Half a bf16 unit-in-the-last-place at the magnitude of ``x`` (8 significant bits)."""
    a = x.float().abs().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(a)) - 8.0)


def err_beyond_rounding(got, ref_fp32, extra_half_ulps=0.0, partials=None, extra_slack=None):
    """``max(|got - ref| - r) / max|ref|`` where ``r`` is the rounding a bf16 result
    necessarily carries: half a bf16 ulp of the reference value (plus
    ``extra_half_ulps`` more half-ulps when the reference was itself rounded to bf16, plus
    half a bf16 ulp of every per-rank partial in ``partials``: with tensor parallelism the
    path stages each rank's partial in bf16 before the in-switch fp32 reduction).

    ``err_rel`` against an fp32 reference cannot go below 2^-9..2^-8 of the maximum for
    any bf16-valued result, whatever computed it; this is the part of the error the
    computation itself is answerable for.
    """
    g, r = got.float(), ref_fp32.float()
    slack = bf16_half_ulp(r) * (1.0 + extra_half_ulps)
    for part in (partials or ()):
        slack = slack + bf16_half_ulp(part)
    if extra_slack is not None:          # the partials' half-ulps, already summed elsewhere
        slack = slack + extra_slack.float()
    excess = ((g - r).abs() - slack).clamp_min(0.0)
    return float(excess.max() / r.abs().max().clamp_min(1e-30))
