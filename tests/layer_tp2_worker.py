"""Worker of the two-GPU test of the whole decode layer on a tensor-parallel pair; run under
torch.distributed.run with two ranks (one GPU each).  Prints one JSON line from rank 0."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import wuda_b200 as wuda  # noqa: E402
from wuda_b200 import moe  # noqa: E402
from wuda_b200.layer_setup import build_random_layer  # noqa: E402

SMALL = dict(topk=512, experts=32, inter=512, moe_topk=4)


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")            # bootstrap only: the data path never touches it
    batch, context = 6, 1500
    tp_link = wuda.TP2Link(batch, 7168, device_sequence=True)
    ep_link = moe.EP2Link(batch, 7168, device_sequence=True)
    layer, slots, x = build_random_layer(batch, context, rank=rank, world=2, tp_link=tp_link, ep_link=ep_link, seed=5,
                                         **SMALL)
    layer.prepare(slots)
    layer.capture(x, batch)                    # one eager pass + the capture pass: calls 1 and 2 of each link
    outs = []
    for _ in range(3):                         # replays: the links number their calls on the device
        dist.barrier()
        outs.append(layer.replay().clone())
        torch.cuda.synchronize()
    status = 0
    try:
        layer.check_status()
    except Exception:
        status = int(layer.attn.status.item()) or int(layer.runner.status.item())
    out = outs[-1].float().cpu()
    gathered = [None, None]
    dist.all_gather_object(gathered, (out.numpy().tobytes(), status))
    res = None
    if rank == 0:
        single, slots1, x1 = build_random_layer(batch, context, seed=5, **SMALL)
        single.prepare(slots1)
        ref = single.launch(x1, batch).float().cpu()
        single.check_status()
        res = {"status": [g[1] for g in gathered], "ranks_identical": gathered[0][0] == gathered[1][0],
               "replays_identical": all(torch.equal(outs[0], o) for o in outs),
               "finite": bool(torch.isfinite(out).all()),
               "rel_err_vs_one_gpu": float((out - ref).norm() / ref.norm())}
        print(json.dumps(res))
    dist.barrier()
    tp_link.close()
    ep_link.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
