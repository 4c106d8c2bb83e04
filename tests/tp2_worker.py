"""Worker of the two-GPU test of the fused TP2 all-reduce GEMM; run under torch.distributed.run
with two ranks (one GPU each).  Prints one JSON line from rank 0."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
import wuda_b200 as wuda  # noqa: E402
from wuda_b200 import workloads  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")            # bootstrap only: the data path never touches it
    results = {}
    for (m, n, k) in ((64, 7168, 16384), (5, 2112, 4096), (128, 1024, 2048)):
        case = workloads.make_gemm_fp8_case(m, n, k, seed=1234 + m)      # identical on both ranks
        kl = k // 2
        sl = slice(rank * kl, (rank + 1) * kl)
        a = torch.from_numpy(np.ascontiguousarray(case["a"][:, sl])).cuda().view(torch.float8_e4m3fn)
        w = torch.from_numpy(np.ascontiguousarray(case["w"][:, sl])).cuda().view(torch.float8_e4m3fn)
        sb = slice(rank * kl // 128, (rank + 1) * kl // 128)
        a_s = torch.from_numpy(np.ascontiguousarray(case["a_s"][:, sb])).cuda()
        w_s = torch.from_numpy(np.ascontiguousarray(case["w_s"][:, sb])).cuda()
        link = wuda.TP2Link(m, n)
        status = wuda.device_status_word()
        outs = []
        for _ in range(3):                        # three calls: both inbox sets and their reuse
            outs.append(link.fp8_gemm(a, a_s, w, w_s, status_word=status).clone())
        torch.cuda.synchronize()
        got = outs[-1].cpu().view(torch.int16).numpy().view(np.uint16)
        same_calls = all(torch.equal(outs[0], o) for o in outs)
        parts = [oracle.gemm_fp8_blockscaled(case["a"][:, s_], case["a_s"][:, b_], case["w"][:, s_], case["w_s"][:, b_],
                                             out_bf16=False)
                 for s_, b_ in ((slice(0, kl), slice(0, kl // 128)), (slice(kl, k), slice(kl // 128, k // 128)))]
        ref = parts[0] + parts[1]
        f = oracle.bf16_to_f32(got)
        ok = bool(np.all(np.abs(f - ref) <= 1e-2 * np.abs(ref) + 1e-3 * np.sqrt(np.mean(ref.astype(np.float64) ** 2))))
        gathered = [None, None]
        dist.all_gather_object(gathered, got.tobytes())
        results["%dx%dx%d" % (m, n, k)] = {"ok": ok, "status": int(status.item()), "calls_identical": bool(same_calls),
                                           "ranks_identical": gathered[0] == gathered[1]}
        dist.barrier()
        link.close()
    if rank == 0:
        print(json.dumps(results))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
