"""The consumer oracle (residual add + RMSNorm) against PyTorch's own rms_norm."""
import torch

from oracle.consumer_oracle import residual_rmsnorm_oracle


def test_consumer_oracle_is_pytorchs_rms_norm_on_the_bf16_residual_stream():
    g = torch.Generator().manual_seed(5)
    for tot, hidden, eps in ((37, 256, 1e-6), (5, 4096, 1e-5), (3, 16384, 1e-6)):
        y = torch.randn(tot, hidden, generator=g).to(torch.bfloat16)
        r = (torch.randn(tot, hidden, generator=g) * 3).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
        out, h = residual_rmsnorm_oracle(y, r, w, eps)
        assert torch.equal(h, (y.float() + r.float()).to(torch.bfloat16))
        ref = torch.nn.functional.rms_norm(h.float(), (hidden,), w.float(), eps)
        # same definition; the products may associate differently: at most one bf16 ulp apart
        d = (out.float() - ref.to(torch.bfloat16).float()).abs()
        assert bool((d <= ref.abs() * 2.0 ** -7 + 1e-30).all())
        assert float((d == 0).float().mean()) > 0.98
