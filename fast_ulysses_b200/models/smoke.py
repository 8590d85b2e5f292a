"""One tiny forward+backward of the flagship path (the fused sequence-parallel attention block and
a DiT block around it) on the current device, used by the repository's smoke entry point."""

from __future__ import annotations

import torch


def model_smoke() -> None:
    import fast_ulysses_b200 as fu
    from fast_ulysses_b200.models.dit import DiTStack
    from fast_ulysses_b200.ops import gemm

    g = fu.UlyssesGroup(device=torch.device("cuda", torch.cuda.current_device()))
    torch.manual_seed(0)
    stack = DiTStack(g, depth=1, hidden=256, heads=2, ffn=512, grid=(2, 8, 16))
    x = torch.randn(1, 256, 256, device=g.device).bfloat16().requires_grad_()
    y = stack(x)
    y.float().square().mean().backward()
    torch.cuda.synchronize()
    gemm.check_errors()
    g.check()
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    g.destroy()
