"""Worker for the tensor-parallel family tests (spawned by test_tp_family.py): trains the tp_mlp family on `world` ranks
and writes the summed loss curve."""
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
    from dataflow_b200.parallel.tp import TpGroup
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family("tp_mlp")
    over = dict(batch=4) if gpu else {}
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32" if not gpu else "bf16_master", tp=world, **over)
    d = fam.derive_dims(cfg)
    lane = os.environ.get("DATAFLOW_TP_LANE") or ("p2p" if gpu else "collective")
    grp = TpGroup(rank, world, rank if gpu else None, max_rows=d.Ts, max_k=d.d, max_n=d.d, lane=lane, timeout_s=20.0)
    budget = float(os.environ["TP_TEST_BUDGET"]) if os.environ.get("TP_TEST_BUDGET") else None
    tr = Trainer("tp_mlp", cfg, budget_gib=budget, device=rank if gpu else None, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=3,
                 groups={"tp": grp}, leeway_bytes=0)
    losses = []
    for s in range(3):
        full = synthetic_rounds(cfg, tr.rounds, d.T, 64, 11, s)                 # the same global data on every rank
        mine = [(tk[rank * d.Ts:(rank + 1) * d.Ts].contiguous(), tg[rank * d.Ts:(rank + 1) * d.Ts].contiguous()) for tk, tg in full]
        losses.append(tr.step(mine, valid_rows=d.T * tr.rounds))
    t = torch.tensor(losses, dtype=torch.float64, device="cuda" if gpu else "cpu")
    dist.all_reduce(t)
    if rank == 0:
        json.dump({"losses": t.tolist(), "lane": lane, "recompute": {str(k): v for k, v in tr.planned.recompute_levels.items() if v}},
                  open(out_path, "w"))
    tr.close()
    if gpu:
        grp.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
