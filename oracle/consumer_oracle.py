"""CPU statement of the residual-add + RMSNorm consumer (TEST INFRASTRUCTURE: imported by
tests only, never by the product path).

The reference has no implementation of this op (it lists it as the step after its fused
kernel, README.md:41-44 of the reference), so there is nothing of the reference's to pin it
to: **parity unpinned** with respect to the reference.  It is pinned to PyTorch's own
definition instead: ``tests/test_consumer_oracle_cpu.py`` checks it against
``torch.nn.functional.rms_norm`` (fp32) on the bf16 residual stream.
"""
import torch


def residual_rmsnorm_oracle(y, residual, weight, eps=1e-6):
    """y, residual [tot, hidden] bf16; weight [hidden] bf16.  Returns (normed, new_residual),
    both bf16: h = bf16(y + residual) in fp32 arithmetic; normed = bf16(h * rsqrt(mean(h^2) +
    eps) * weight) with h, the statistics and the products in fp32."""
    h = (y.float() + residual.float()).to(torch.bfloat16)
    hf = h.float()
    rstd = torch.rsqrt((hf * hf).mean(dim=-1, keepdim=True) + eps)
    return ((hf * rstd) * weight.float()).to(torch.bfloat16), h
