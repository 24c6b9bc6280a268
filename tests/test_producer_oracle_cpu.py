"""The RoPE oracle against the textbook complex rotation in float64."""
import numpy as np
import torch

from oracle.producer_oracle import inv_freq_fp32, rope_oracle


def test_rope_oracle_is_the_complex_rotation_and_leaves_the_kv_prefix_alone():
    g = torch.Generator().manual_seed(9)
    sq, sk = [70, 33], [70, 161]
    q = torch.randn(sum(sq), 3, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(sk), 2, 128, generator=g).to(torch.bfloat16)
    qo, ko = rope_oracle(q, k, sq, sk)
    w = inv_freq_fp32().double().numpy()
    # second sequence: queries at positions 128..160, K prefix rows 0..127 untouched
    assert torch.equal(ko[70:70 + 128], k[70:70 + 128])
    for i in (0, 17, 32):
        pos = 128 + i
        x = q[70 + i, 1].double().numpy()
        z = (x[:64] + 1j * x[64:]) * np.exp(1j * pos * w)
        ref = torch.from_numpy(np.concatenate([z.real, z.imag])).to(torch.bfloat16)
        d = (qo[70 + i, 1].float() - ref.float()).abs()
        assert bool((d <= ref.float().abs() * 2.0 ** -7 + 1e-6).all())
        xk = k[70 + pos, 0].double().numpy()
        zk = (xk[:64] + 1j * xk[64:]) * np.exp(1j * pos * w)
        refk = torch.from_numpy(np.concatenate([zk.real, zk.imag])).to(torch.bfloat16)
        assert bool(((ko[70 + pos, 0].float() - refk.float()).abs() <= refk.float().abs() * 2.0 ** -7 + 1e-6).all())
    # first sequence (q = k): position = row
    x = q[5, 0].double().numpy()
    z = (x[:64] + 1j * x[64:]) * np.exp(1j * 5 * w)
    ref = torch.from_numpy(np.concatenate([z.real, z.imag])).to(torch.bfloat16)
    assert bool(((qo[5, 0].float() - ref.float()).abs() <= ref.float().abs() * 2.0 ** -7 + 1e-6).all())
