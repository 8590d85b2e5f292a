"""Sequence-parallel DiT attention block: the fused path against the same block on one rank.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/sp_attention.py

Counterpart of the reference's examples/dit_attention.py (nn.Linear + SDPA around two
all_to_all_4d calls, output and input-gradient max-abs-diff < 5e-2, then five AdamW steps). Here
the block is ``UlyssesSelfAttention``: QKV projection, RMSNorm, RoPE and the head scatter are one
kernel, attention is the tcgen05 kernel, the output projection pulls from the peers itself.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import fast_ulysses_b200 as fu
from fast_ulysses_b200.models.attention import UlyssesSelfAttention, reference_attention


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(
        os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    group = fu.UlyssesGroup(device=torch.device("cuda", local))
    grid, hidden, heads = (4, 16, 16), 1024, 8  # 1024 tokens
    total = grid[0] * grid[1] * grid[2]
    torch.manual_seed(0)  # same weights and data on every rank
    attn = UlyssesSelfAttention(group, hidden, heads, grid=grid)
    x_full = torch.randn(1, total, hidden, device="cuda").bfloat16()
    s = total // world
    x = x_full[:, rank * s:(rank + 1) * s].clone().requires_grad_()

    y = attn(x)
    y.float().square().mean().backward()
    xr = x_full.float().requires_grad_()
    yr = reference_attention(xr, attn.w_qkv, attn.gamma_q, attn.gamma_k, attn.w_o, attn.b_o, heads, grid)
    yr.square().mean().backward()
    d_out = (y.float() - yr[:, rank * s:(rank + 1) * s]).abs().max().item()
    d_grad = (x.grad.float() - xr.grad[:, rank * s:(rank + 1) * s]).abs().max().item()
    print(f"rank {rank}: max |out diff| {d_out:.3e}, max |input-grad diff| {d_grad:.3e}")
    assert d_out < 5e-2 and d_grad < 5e-2

    opt = torch.optim.AdamW(attn.parameters(), lr=1e-3)
    for step in range(5):
        opt.zero_grad()
        loss = attn(x.detach()).float().square().mean()
        loss.backward()
        if world > 1:  # weights are replicated, the sequence is sharded: sum the partial gradients
            for p in attn.parameters():
                dist.all_reduce(p.grad)
        opt.step()
        if rank == 0:
            print(f"step {step}: loss {loss.item():.5f}")
    group.check()
    group.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
