"""Worker for the expert-parallel tests (spawned by test_ep.py): one EP MoE MLP, forward and backward, against a dense
fp32 oracle over all experts and all ranks' tokens."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def oracle(H, ids, w, W13, W2, dY):
    """fp32 autograd over the global problem."""
    H = H.float().requires_grad_(True)
    w = w.float().requires_grad_(True)
    W13 = W13.float().requires_grad_(True)
    W2 = W2.float().requires_grad_(True)
    F = W2.shape[1]
    y = torch.zeros_like(H)
    for e in range(W13.shape[0]):
        tok, k = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h13 = H[tok] @ W13[e]
        s = torch.nn.functional.silu(h13[:, :F]) * h13[:, F:]
        y = y.index_add(0, tok, (s @ W2[e]) * w[tok, k].unsqueeze(-1))
    y.backward(dY.float())
    return y.detach(), H.grad, w.grad, W13.grad, W2.grad


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def bench(out_path):
    """Timing at an OLMoE-sized layer (16384 tokens per rank, d 2048, 64 experts of width 1024, top-8): the fused
    kernels against the same data movement through NCCL all-to-all plus separate local kernels."""
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    dev = torch.device("cuda", rank)
    torch.set_grad_enabled(False)
    from dataflow_b200.ops import resolve_kernels
    from dataflow_b200.ops.eager import moe_sort, moe_topk_softmax
    from dataflow_b200.parallel.ep import EpGroup
    from dataflow_b200.runtime import CudaBackend
    T, d, F, E, K = 16384, 2048, 1024, 64, 8
    el = E // world
    gen = torch.Generator(device=dev).manual_seed(3 + rank)
    x = (torch.randn(T, d, generator=gen, device=dev) * 0.5).bfloat16()
    w, ids = moe_topk_softmax(torch.randn(T, E, generator=gen, device=dev), K)
    w13 = (torch.randn(el, d, 2 * F, generator=gen, device=dev) / d ** 0.5).bfloat16()
    w2 = (torch.randn(el, F, d, generator=gen, device=dev) / F ** 0.5).bfloat16()
    g = EpGroup(rank, world, rank, tokens=T, d_model=d, n_experts=E, top_k=K, lane="p2p", timeout_s=10.0)
    g.attach(CudaBackend(rank, "poll"))
    ks = resolve_kernels()
    plan = g.plan(ids, w)
    g.x_buffer().copy_(x)
    xb = g.x_buffer()

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
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    res = {"shape": {"tokens_per_rank": T, "d_model": d, "d_expert": F, "experts": E, "top_k": K, "world": world, "rows": g.C}}
    xp, h13 = g.dispatch_mm(xb, w13, plan)
    res["dispatch_mm_ms"] = timed(lambda: g.dispatch_mm(xb, w13, plan))
    sp = ks.swiglu_packed_fwd(h13)
    rows = g.rows_buffer()
    ks.moe_grouped_mm(sp, w2, plan.tile_expert, out=rows)
    res["combine_ms"] = timed(lambda: g.combine(rows, plan, base=x, weighted=True))
    res["grouped_mm_only_ms"] = timed(lambda: ks.moe_grouped_mm(xp, w13, plan.tile_expert, out=h13))
    # the same traffic through NCCL: permute -> all-to-all (equal splits) -> permute into the expert-major layout -> GEMM
    row_of_l, row_src_l, off_l, te_l, _ = moe_sort(ids % el, el)
    n_rows = row_src_l.numel()
    send = torch.empty(T * K, d, dtype=torch.bfloat16, device=dev)
    recv = torch.empty(T * K, d, dtype=torch.bfloat16, device=dev)
    tok_of_slot = torch.arange(T * K, device=dev, dtype=torch.int32) // K
    xp_l = torch.empty(n_rows, d, dtype=torch.bfloat16, device=dev)
    h13_l = torch.empty(n_rows, 2 * F, dtype=torch.bfloat16, device=dev)
    slot_src = torch.where(row_src_l >= 0, torch.arange(n_rows, device=dev, dtype=torch.int32) % (T * K), row_src_l).to(torch.int32)

    def base_dispatch():
        ks.moe_dispatch(x, tok_of_slot, out=send)
        dist.all_to_all_single(recv, send)
        ks.moe_dispatch(recv, slot_src, out=xp_l)
        ks.moe_grouped_mm(xp_l, w13, te_l, out=h13_l)

    res["nccl_dispatch_mm_ms"] = timed(base_dispatch)
    yp_l = torch.empty(n_rows, d, dtype=torch.bfloat16, device=dev)
    back = torch.empty(T * K, d, dtype=torch.bfloat16, device=dev)
    back_recv = torch.empty(T * K, d, dtype=torch.bfloat16, device=dev)
    row_of_slot = torch.arange(T * K, device=dev, dtype=torch.int32).view(T, K)

    def base_combine():
        ks.moe_dispatch(yp_l, row_of_l.reshape(-1), out=back)          # rows back into slot order
        dist.all_to_all_single(back_recv, back)
        return ks.moe_combine(x, back_recv, w, row_of_slot)

    res["nccl_combine_ms"] = timed(base_combine)
    g.check()
    flops = 2.0 * T * K * d * 2 * F
    res["dispatch_mm_tflops"] = flops / res["dispatch_mm_ms"] / 1e9
    res["pulled_gb_per_rank"] = T * K * d * 2 * (world - 1) / world / 1e9
    allr = [None] * world
    dist.all_gather_object(allr, res)
    if rank == 0:
        json.dump({"ranks": allr}, open(out_path, "w"))
    g.close()
    dist.barrier()
    dist.destroy_process_group()


def main():
    out_path, device_kind = sys.argv[1], sys.argv[2]
    if len(sys.argv) > 3 and sys.argv[3] == "bench":
        return bench(out_path)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = device_kind == "cuda"
    if gpu:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        dev = torch.device("cuda", rank)
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    from dataflow_b200.ops.eager import moe_topk_softmax
    from dataflow_b200.parallel.ep import EpGroup, ep_moe_backward, ep_moe_forward
    T, d, F, E, K = (1024, 512, 256, 8, 2) if gpu else (96, 64, 32, 4, 2)
    gen = torch.Generator().manual_seed(11)
    H = (torch.randn(world * T, d, generator=gen) * 0.5).bfloat16()
    logits = torch.randn(world * T, E, generator=gen)
    W13 = (torch.randn(E, d, 2 * F, generator=gen) / d ** 0.5).bfloat16()
    W2 = (torch.randn(E, F, d, generator=gen) / F ** 0.5).bfloat16()
    dY = (torch.randn(world * T, d, generator=gen) * 0.1).bfloat16()
    w_all, ids_all = moe_topk_softmax(logits, K)
    H, W13, W2, dY, w_all, ids_all = (x.to(dev) for x in (H, W13, W2, dY, w_all, ids_all))
    y_ref, dH_ref, dw_ref, dW13_ref, dW2_ref = oracle(H, ids_all, w_all, W13, W2, dY)

    lane = os.environ.get("DATAFLOW_EP_LANE") or ("p2p" if gpu else "collective")
    g = EpGroup(rank, world, rank if gpu else None, tokens=T, d_model=d, n_experts=E, top_k=K, lane=lane, timeout_s=10.0)
    if gpu:
        from dataflow_b200.runtime import CudaBackend
        g.attach(CudaBackend(rank, "poll"))
    el = E // world
    mine = slice(rank * T, (rank + 1) * T)
    w13_l, w2_l = W13[rank * el:(rank + 1) * el].contiguous(), W2[rank * el:(rank + 1) * el].contiguous()
    dw13 = torch.zeros_like(w13_l)
    dw2 = torch.zeros_like(w2_l)
    res = {}
    torch.set_grad_enabled(False)
    for it in range(2):                      # twice: rendezvous words and buffers are reused
        y, saved = ep_moe_forward(g, H[mine].contiguous(), ids_all[mine].contiguous(), w_all[mine].contiguous(), w13_l, w2_l)
        dh, dw = ep_moe_backward(g, dY[mine].contiguous(), saved, w13_l, w2_l, dw13, dw2)
        if gpu:
            torch.cuda.synchronize()
            g.check()
        res = {"y": rel(y, y_ref[mine]), "dh": rel(dh, dH_ref[mine]), "dw": rel(dw, dw_ref[mine]),
               "dW13": rel(dw13, dW13_ref[rank * el:(rank + 1) * el]), "dW2": rel(dw2, dW2_ref[rank * el:(rank + 1) * el]),
               "dropped": int(saved["plan"].dropped)}
    t = torch.tensor([res[k] for k in ("y", "dh", "dw", "dW13", "dW2")], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        json.dump({"max_rel": dict(zip(("y", "dh", "dw", "dW13", "dW2"), t.tolist())), "dropped": res["dropped"], "lane": lane},
                  open(out_path, "w"))
    g.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
