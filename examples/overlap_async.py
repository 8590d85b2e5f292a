"""The asynchronous exchange beside compute: forms of the call, transports, and who owns what.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/overlap_async.py          # GPUs, NCCL
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/overlap_async.py --cpu    # dry run on gloo

Shows, on q/k/v-shaped tensors, the three ways to receive the result of ``all_to_all_4d_async``
(a fresh tensor, a window lent by the group, a symmetric buffer of your own), the two transports
(the exchange kernel on a third of the SMs; the copy engines, which hold no SM while the peer
copies run), and the rule for the input: with the default ``stage=True`` it may be overwritten the
moment the call returns. Every result is checked against the synchronous call.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import fast_ulysses_b200 as fu


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true", help="gloo ranks on the CPU executor: same API, no speed")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(
        os.environ.get("LOCAL_RANK", 0))
    if args.cpu:
        dist.init_process_group("gloo")
        device = torch.device("cpu")
    else:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
    group = fu.UlyssesGroup(device="cpu" if args.cpu else device)
    torch.manual_seed(rank)
    s_local, heads, d = 256, 4 * world, 128
    q = torch.randn(1, s_local, heads, d, device=device).bfloat16()
    work = torch.randn(512, 512, device=device)
    want = group.all_to_all_4d(q).clone()

    for transport in ("kernel", "copy_engine"):
        group.set_async_transport(transport)  # a local choice: ranks may differ
        # 1. a fresh tensor (window + copy-out). The input is staged, so it is ours again at once.
        x = q.clone()
        h = group.all_to_all_4d_async(x)
        x.zero_()  # allowed: the call took its own copy
        busy = work @ work  # compute that the exchange runs beside
        assert torch.equal(h.wait(), want), (transport, "fresh tensor")
        # 2. a window lent by the group: nothing is copied out. At most four lent results may be
        #    alive at once, and every rank must drop them at the same point of its program.
        lent = group.all_to_all_4d_async(q, lend=True, stage=False)  # stage=False: we promise not to write q
        busy = busy + work @ work
        assert torch.equal(lent.wait(), want), (transport, "lent window")
        del lent
        # 3. a symmetric buffer of our own (collective allocation, reusable across calls): the
        #    peers write it directly and it stays ours.
        if not args.cpu:
            out = group.empty_output(q)
            group.all_to_all_4d_async(q, out=out, stage=False).wait()
            assert torch.equal(out, want), (transport, "own symmetric buffer")
        if rank == 0:
            print(f"transport {transport}: fresh tensor, lent window"
                  f"{'' if args.cpu else ', own symmetric buffer'}: all equal to the synchronous call")
    group.check()  # raises if any device-side wait ran out of time
    group.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
