"""Worker of the two-GPU test of the expert-parallel MoE combine; run under torch.distributed.run with
two ranks (one GPU each).  Each rank holds half of the experts; prints one JSON line from rank 0."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402
from wuda_b200 import moe  # noqa: E402
from test_moe_ep2_gpu import local_sum, make, u16  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")            # bootstrap only: the data path never touches it
    tokens, experts, k, dim, inter = 64, 16, 4, 1024, 512
    w1, w3, w2, x, idx, rw = make(11, tokens, experts, k, dim, inter)      # identical on both ranks
    half = experts // 2
    sl = slice(rank * half, (rank + 1) * half)
    weights = moe.RoutedExperts(w1[sl], w3[sl], w2[sl], 4.0 / 2688, 3.0 / 2688)
    link = moe.EP2Link(tokens, dim)
    runner = moe.MoERunner(weights, tokens, k, expert_first=rank * half, experts_total=experts, link=link)
    shared = torch.randn(tokens, dim, generator=torch.Generator().manual_seed(2)).bfloat16()
    ys = []
    for _ in range(3):                          # three calls: both inbox sets and their reuse
        ys.append(runner.forward(x.cuda(), rw.cuda(), idx.cuda(), shared=shared.cuda() if rank == 0 else None).clone())
    torch.cuda.synchronize()
    part = local_sum(runner, tokens, k)
    if rank == 0:
        part = (part + oracle.bf16_to_f32(u16(shared))).astype(np.float32)
    got = u16(ys[-1])
    gathered = [None, None]
    dist.all_gather_object(gathered, (got.tobytes(), part.tobytes(), int(runner.status.item())))
    dist.barrier()
    link.close()
    if rank == 0:
        parts = [np.frombuffer(g[1], np.float32).reshape(tokens, dim) for g in gathered]
        total = oracle.f32_to_bf16((parts[0] + parts[1]).astype(np.float32))
        # one rank holding all experts: the same rows, summed in another order
        full = moe.MoERunner(moe.RoutedExperts(w1, w3, w2, 4.0 / 2688, 3.0 / 2688), tokens, k)
        y1 = full.forward(x.cuda(), rw.cuda(), idx.cuda(), shared=shared.cuda()).float().cpu().numpy()
        f = oracle.bf16_to_f32(got)
        print(json.dumps({"status": [g[2] for g in gathered], "ranks_identical": gathered[0][0] == gathered[1][0],
                          "calls_identical": all(torch.equal(ys[0], y) for y in ys),
                          "equals_sum_of_parts": bool(np.array_equal(got, total)),
                          "close_to_one_rank": bool(np.all(np.abs(f - y1) <= 2.0 ** -6 * np.abs(y1) + 1e-2 * np.abs(y1).max()))}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
