"""Worker for the multi-process ZeRO tests (spawned by test_zero_dp.py)."""
import dataclasses
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode, out_path, device_kind = sys.argv[1], sys.argv[2], sys.argv[3]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = device_kind == "cuda"
    if gpu:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo")
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.parallel.zero import make_dp_group, zero_lower_kwargs
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="bf16_master")
    hyper = {"lr": 2e-3, "weight_decay": 0.1}
    lane = os.environ.get("DATAFLOW_DP_LANE")
    grp = make_dp_group(rank, world, rank if gpu else None, lane)
    tr = Trainer("llama3", cfg, budget_gib=None, device=rank if gpu else None, hyper=hyper, seed=5,
                 groups={"dp": grp}, lower_kwargs=zero_lower_kwargs(mode, rank, world), recompute=False)
    grp.force_stage = os.environ.get("ZERO_TEST_FORCE_STAGE") == "1"
    if mode == "fsdp":
        assert any(t.id.startswith("grad_rs_") for t in tr.program.tasks)
    losses = []
    for s in range(4):
        data = synthetic_rounds(cfg, tr.rounds, tr.T, 64, 100 + rank, s)        # each rank its own data
        losses.append(tr.step(data, valid_rows=tr.T * tr.rounds * world))
    t = torch.tensor(losses, dtype=torch.float64)
    if gpu:
        t = t.cuda()
    dist.all_reduce(t)
    # the slice this rank owns of layer 0's weights, for cross-lane comparison
    from dataflow_b200.runtime.interop import torch_view
    tr.sync_to_host()
    oid = "Ws_0" if mode in ("zero3", "fsdp") else "W_0"
    w0 = torch_view(tr.store.buffer(oid), (tr.store.sizes[oid] // 2,), "bf16", 0, None).float()
    if rank == 0:
        json.dump({"losses": t.tolist(), "w0_sum": float(w0.double().sum()), "w0_abs": float(w0.double().abs().sum())},
                  open(out_path, "w"))
    if grp.force_stage and gpu and lane == "p2p":
        assert grp.staged > 0
    tr.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
