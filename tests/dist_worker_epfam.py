"""Worker for the expert-parallel family tests (spawned by test_ep.py): trains a mixture-of-experts family (``EP_TEST_FAMILY``,
default olmoe) with its experts split over the ranks; every rank feeds its own data; writes the summed loss curve."""
import dataclasses
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path, device_kind = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = device_kind == "cuda"
    if gpu:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo")
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.parallel.ep import ep_group_for
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    name = os.environ.get("EP_TEST_FAMILY", "olmoe")
    fam = resolve_family(name)
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32" if not gpu else "bf16_master", ep=world)
    d = fam.derive_dims(cfg)
    lane = os.environ.get("DATAFLOW_EP_LANE") or ("p2p" if gpu else "collective")
    grp = ep_group_for(fam, cfg, rank, world, rank if gpu else None, lane, timeout_s=20.0)
    assert not hasattr(d, "Mp") or grp.C == d.Mp
    budget = float(os.environ["EP_TEST_BUDGET"]) if os.environ.get("EP_TEST_BUDGET") else None
    tr = Trainer(name, cfg, budget_gib=budget, device=rank if gpu else None, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=5,
                 groups={"ep": grp}, leeway_bytes=0)
    losses = []
    for s in range(3):
        data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 100 + rank, s)
        losses.append(tr.step(data, valid_rows=tr.T * tr.rounds * world))
    t = torch.tensor(losses, dtype=torch.float64, device="cuda" if gpu else "cpu")
    dist.all_reduce(t)
    if rank == 0:
        json.dump({"losses": t.tolist(), "lane": lane}, open(out_path, "w"))
    tr.close()
    if gpu:
        grp.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
