"""Worker for the 2-GPU tensor-parallel fused-kernel tests (spawned by test_tp_fused.py)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path, bench = sys.argv[1], len(sys.argv) > 2 and sys.argv[2] == "bench"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from dataflow_b200.parallel.tp import TpGroup
    from dataflow_b200.runtime import CudaBackend
    be = CudaBackend(rank, "poll")
    rows, d, f = (2048, 8192, 28672 // world) if bench else (512, 1024, 768)
    grp = TpGroup(rank, world, rank, max_rows=rows, max_k=max(d, f), max_n=max(d, f))
    grp.attach(be)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    res = {}
    try:
        x = (torch.randn(rows, d, device="cuda", generator=g) * 0.5).bfloat16()
        w_up = (torch.randn(d, f, device="cuda", generator=g) * 0.05).bfloat16()       # this rank's column shard
        w_down = (torch.randn(f, d, device="cuda", generator=g) * 0.05).bfloat16()     # this rank's row shard
        resid = (torch.randn(rows, d, device="cuda", generator=g) * 0.5).bfloat16()
        # oracle: library collectives around fp32 matmuls
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        full = torch.cat(parts, 0).float()
        h_ref = full @ w_up.float()
        for it in range(3):                      # repeated launches exercise the growing rendezvous counters
            h = grp.ag_gemm(x, w_up)
        torch.cuda.synchronize()
        grp.check()
        res["ag_rel"] = float((h.float() - h_ref).norm() / h_ref.norm())
        hb = h_ref.bfloat16()
        part = (hb.float() @ w_down.float())
        dist.all_reduce(part)
        y_ref = part[rank * rows:(rank + 1) * rows] + resid.float()
        for it in range(3):
            y = grp.gemm_rs(hb, w_down, addend=resid)
        torch.cuda.synchronize()
        grp.check()
        res["rs_rel"] = float((y.float() - y_ref).norm() / y_ref.norm())
        if bench:
            def timed(fn, iters=10):
                for _ in range(3):
                    fn()
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t[0])
            col = TpGroup(rank, world, rank, max_rows=rows, max_k=max(d, f), max_n=max(d, f), lane="collective")
            m = rows * world
            res["ag_ms"] = timed(lambda: grp.ag_gemm(x, w_up))
            res["ag_nccl_ms"] = timed(lambda: col.ag_gemm(x, w_up))
            res["ag_tflops"] = 2.0 * m * d * f / res["ag_ms"] / 1e9
            res["rs_ms"] = timed(lambda: grp.gemm_rs(hb, w_down, addend=resid))
            res["rs_nccl_ms"] = timed(lambda: col.gemm_rs(hb, w_down, addend=resid))
            res["rs_tflops"] = 2.0 * m * d * f / res["rs_ms"] / 1e9
            grp.check()
            res["shape"] = {"rows_per_rank": rows, "d_model": d, "ffn_shard": f, "world": world}
    finally:
        allr = [None] * world
        dist.all_gather_object(allr, res)
        if rank == 0:
            json.dump({"ranks": allr}, open(out_path, "w"))
        grp.close()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
