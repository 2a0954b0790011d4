"""Expert parallelism inside one NVSwitch box.

The experts of a mixture-of-experts layer are split over the ranks of a group (rank ``r`` owns experts
``[r E/P, (r + 1) E/P)``); every rank keeps its own tokens.  One layer runs as

    plan        every rank learns all routing choices (a small all-gather of ids and weights) and sorts the slots
                that chose ITS experts into the padded expert-major layout; the row every foreign slot got is
                written where the slot's owner can read it
    dispatch_mm the dispatch all-to-all fused into the grouped up-projection: copy warps of the GEMM kernel pull
                the token rows from their owners over NVLink while earlier tiles multiply
    (local)     activation, grouped down-projection — rows stay with the expert's owner
    combine     the owner of a token pulls its K rows from the experts' owners and reduces them with the routing
                weights in one kernel (combine all-to-all + weighted scatter-add, no staging, no atomics)

and the backward is the same two kernels with the roles of the matrices swapped.  A ``collective`` lane
(``torch.distributed`` all-to-all-free formulation over all-gather / all-reduce, library matmuls) is the baseline and
the oracle of the tests.

A rank's dispatched matrix has room for ``capacity_factor * tokens * top_k`` rows (rounded up to whole tiles, plus one
tile per local expert for the padding); slots past that are dropped — they contribute nothing forward or backward
— which only happens when routing is more than ``capacity_factor`` times out of balance.

The reference runs expert parallelism as NCCL send/recv pairs around separate dispatch and combine kernels
(``src/dataflow_training/model_families/dsv3/blocks.py``); it has no fused kernels.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any

from ..ops.eager import MOE_TILE_ROWS
from .group_abi import GroupCollectives

CTRL_BYTES = 1 << 12


@dataclass
class EpPlan:
    """Routing of one layer as seen by this rank."""
    ids: Any                 # (T, K) int32 global expert ids of this rank's tokens
    weights: Any             # (T, K) fp32
    row_src: Any             # (C,) int32: global token (rank * T + token) held by each local row, -1 padding
    row_slot: Any            # (C,) int64: global slot (token * K + k) of each local row, clamped to 0 on padding
    row_w: Any               # (C,) fp32 routing weight of the slot each local row serves (0 on padding)
    tile_expert: Any         # (C / tile,) int32 local expert per row tile, -1: none
    offsets_pad: Any         # (E_local + 1,) int32 padded row ranges (clamped to C)
    counts: Any              # (E,) int32 global per-expert slot counts (for the load-balance loss)
    rows_local: Any = None   # (T, K) int32 row this rank's slots got at their experts' owners, -1 dropped
    dropped: Any = None      # () int32 number of slots of this rank's experts that did not fit


class EpGroup(GroupCollectives):
    def __init__(self, rank: int, world: int, device: int | None, *, tokens: int, d_model: int, n_experts: int, top_k: int,
                 capacity_factor: float = 2.0, lane: str | None = None, timeout_s: float = 30.0, pg=None):
        """``pg``: the ``torch.distributed`` process group of the members when they are a subset of the job (a dp x ep mesh);
        ``rank`` is the rank inside it.  ``all_reduce`` (gradients of the replicated parameters) always spans the whole job:
        every rank of the job sees different tokens."""
        self.pg = pg
        if n_experts % world:
            raise ValueError(f"{n_experts} experts do not split over {world} ranks")
        self.rank, self.world, self.device = rank, world, device
        self.lane = lane or os.environ.get("DATAFLOW_EP_LANE") or ("p2p" if device is not None else "collective")
        self.timeout_s = timeout_s
        self.capacity_factor = float(capacity_factor)
        self.allow_drops = os.environ.get("DATAFLOW_EP_ALLOW_DROPS", "0") == "1"
        self.dropped_step = None          # device counter of this step's dropped slots (created with the first plan)
        self.dropped_total = 0
        self.T, self.d, self.E, self.K = int(tokens), int(d_model), int(n_experts), int(top_k)
        self.e_local = self.E // world
        slots = self.T * self.K
        want = int(min(capacity_factor * slots, world * slots))
        self.C = _up(want, MOE_TILE_ROWS) + self.e_local * MOE_TILE_ROWS
        self.slots_global = world * slots
        # symmetric workspace: control words | token rows peers read | expert rows peers read | per-row scalars | row table
        self.off_x = CTRL_BYTES
        self.off_rows = self.off_x + _up(self.T * self.d * 2)
        self.off_scal = self.off_rows + _up(self.C * self.d * 2)
        self.off_table = self.off_scal + _up(self.C * 4)
        self.ws_bytes = self.off_table + _up(self.slots_global * 4)
        self.ws: list[int] = []
        self.backend = None
        self.seq_x = 0
        self.seq_y = 0
        self.name = "ep"

    # -- set-up
    def attach(self, backend) -> None:
        if self.lane != "p2p":
            return
        import torch
        import torch.distributed as dist
        backend = getattr(backend, "backend", backend)          # a Trainer hands itself over
        if self.ws:
            return
        self.backend = backend
        self.base = backend.device_alloc_zeroed(self.ws_bytes)
        handles: list[Any] = [None] * self.world
        dist.all_gather_object(handles, backend.ipc_handle(self.base), group=self.pg)
        self.ws = [self.base if r == self.rank else backend.ipc_open(h) for r, h in enumerate(handles)]
        dev = torch.device("cuda", self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tile_flags = torch.zeros(self.C // MOE_TILE_ROWS, dtype=torch.int32, device=dev)
        self.tables_dev = torch.tensor([p + self.off_table for p in self.ws], dtype=torch.int64, device=dev)
        dist.barrier(group=self.pg)

    def close(self) -> None:
        if self.lane == "p2p" and self.backend is not None and self.ws:
            import torch
            torch.cuda.synchronize(self.device)
            for r, p in enumerate(self.ws):
                if r != self.rank:
                    self.backend.ipc_close(p)
            self.backend.device_free(self.base)
            self.ws = []

    def check(self) -> None:
        """Called once per step, after the engine has drained: raises on a kernel time-out, and on dropped token slots — a step
        that dropped slots trained a different model than the one asked for (``allow_drops`` turns that into a count)."""
        if self.lane == "p2p":
            code = int(self.err.item())
            if code:
                self.err.zero_()
                raise RuntimeError(f"fused expert-parallel kernel gave up: phase {code >> 8}, peer/rank {code & 255}")
        if self.dropped_step is not None:
            n = int(self.dropped_step.item())
            self.dropped_step.zero_()
            self.dropped_total += n
            if n and not self.allow_drops:
                raise RuntimeError(
                    f"expert-parallel dispatch dropped {n} token slots on rank {self.rank} this step: routing was more than "
                    f"{self.capacity_factor:g}x out of balance for a dispatched matrix of {self.C} rows; raise the capacity factor "
                    f"(ep_capacity; {self.world:g} can never drop) or set DATAFLOW_EP_ALLOW_DROPS=1 to train on with the loss")

    def all_reduce(self, t):
        """Sum over the group (gradients of the parameters every rank holds in full)."""
        import torch.distributed as dist
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(t)                      # the whole job, not only this group
        return t

    # -- symmetric buffers (this rank's views)
    def _view(self, off: int, shape, dtype: str):
        from ..ops import native
        return native().tensor_from_ptr(self.base + off, list(shape), dtype, self.device)

    def x_buffer(self):
        """(T, d) bf16 rows that peers pull in ``dispatch_mm``: write the layer's input (or, backward, dy) here."""
        return self._view(self.off_x, (self.T, self.d), "bf16")

    def rows_buffer(self):
        """(C, d) bf16 rows that peers pull in ``combine``: the down-projection (or, backward, dxp) writes here."""
        return self._view(self.off_rows, (self.C, self.d), "bf16")

    def scal_buffer(self):
        return self._view(self.off_scal, (self.C,), "fp32")

    # -- routing
    def plan(self, ids, weights) -> EpPlan:
        """``ids`` (T, K) int32, ``weights`` (T, K) fp32 of this rank's tokens.  No host synchronisation."""
        import torch
        import torch.distributed as dist
        from ..ops.eager import moe_sort as sort
        t, k = ids.shape
        all_ids = torch.empty(self.world * t, k, dtype=torch.int32, device=ids.device)
        all_w = torch.empty(self.world * t, k, dtype=torch.float32, device=ids.device)
        if self.world > 1:
            dist.all_gather_into_tensor(all_ids, ids.contiguous(), group=self.pg)
            dist.all_gather_into_tensor(all_w, weights.float().contiguous(), group=self.pg)
        else:
            all_ids.copy_(ids)
            all_w.copy_(weights)
        local = all_ids - self.rank * self.e_local
        mine = (local >= 0) & (local < self.e_local)
        bucket = torch.where(mine, local, torch.full_like(local, self.e_local))
        row_of, row_src, offsets_pad, tile_expert, counts_local = sort(bucket, self.e_local + 1)
        C = self.C
        keep = mine & (row_of < C)
        table = torch.where(keep, row_of, torch.full_like(row_of, -1)).to(torch.int32)
        # rows -> slots (for the routing weight of every local row)
        n_rows = row_src.numel()
        row_slot = torch.zeros(n_rows, dtype=torch.int64, device=ids.device)
        slot_idx = torch.arange(self.world * t * k, device=ids.device)
        flat_rows = row_of.reshape(-1).long()
        row_slot[flat_rows] = slot_idx
        if n_rows < C:
            pad = C - n_rows
            row_src = torch.cat([row_src, torch.full((pad,), -1, dtype=row_src.dtype, device=ids.device)])
            row_slot = torch.cat([row_slot, torch.zeros(pad, dtype=torch.int64, device=ids.device)])
            tile_expert = torch.cat([tile_expert, torch.full((pad // MOE_TILE_ROWS + 1,), -1, dtype=tile_expert.dtype, device=ids.device)])
        row_src = row_src[:C].contiguous()
        row_slot = row_slot[:C].contiguous()
        tile_expert = tile_expert[:C // MOE_TILE_ROWS]
        tile_expert = torch.where(tile_expert >= self.e_local, torch.full_like(tile_expert, -1), tile_expert).contiguous()
        # rows of the foreign bucket hold nothing this rank computes
        first_foreign = offsets_pad[self.e_local]
        rows_idx = torch.arange(C, device=ids.device)
        row_src = torch.where(rows_idx < first_foreign, row_src, torch.full_like(row_src, -1))
        row_w = torch.where(row_src >= 0, all_w.reshape(-1)[row_slot], torch.zeros((), device=ids.device))
        offsets = offsets_pad[:self.e_local + 1].clamp(max=C).to(torch.int32).contiguous()
        counts = torch.zeros(self.E, dtype=torch.int32, device=ids.device)
        counts.scatter_add_(0, all_ids.reshape(-1).long(), torch.ones(all_ids.numel(), dtype=torch.int32, device=ids.device))
        dropped = (mine & ~keep).sum().to(torch.int32)
        if self.dropped_step is None:
            self.dropped_step = torch.zeros((), dtype=torch.int32, device=ids.device)
        self.dropped_step += dropped
        plan = EpPlan(ids=ids.contiguous(), weights=weights.float().contiguous(), row_src=row_src.to(torch.int32).contiguous(),
                      row_slot=row_slot, row_w=row_w.float().contiguous(), tile_expert=tile_expert.to(torch.int32), offsets_pad=offsets,
                      counts=counts, dropped=dropped)
        plan._table = table
        if self.lane == "p2p":
            self._view(self.off_table, (self.slots_global,), "int32").copy_(table.reshape(-1))
        return plan

    # -- fused ops
    def dispatch_mm(self, x, w, plan: EpPlan, transpose_w: bool = False, out=None):
        """``x``: this rank's (T, d) rows — ideally ``x_buffer()`` itself; ``w``: this rank's experts, (E_local, d, N)
        (or (E_local, N, d) with ``transpose_w``).  Returns ``(xp (C, d), y (C, N))``: the gathered rows and their
        products.  On the first call of a layer also resolves ``plan.rows_local``."""
        import torch
        n = w.shape[1] if transpose_w else w.shape[2]
        xp = torch.empty(self.C, self.d, dtype=x.dtype, device=x.device)
        y = out if out is not None else torch.empty(self.C, n, dtype=x.dtype, device=x.device)
        if self.lane != "p2p":
            return self._dispatch_mm_collective(x, w, plan, transpose_w, xp, y)
        from ..ops import native
        from ..ops.cuda import LAUNCHES
        xb = self.x_buffer()
        if x.data_ptr() != xb.data_ptr():
            xb.copy_(x)
        self.seq_x += 1
        native().ep_dispatch_mm([p + self.off_x for p in self.ws], xp, plan.row_src, w, transpose_w, y, plan.tile_expert,
                                self.T, self.rank, self.tile_flags, [p + 0 for p in self.ws], [p + 64 for p in self.ws],
                                self.seq_x, self.timeout_s, self.err, self.done)
        LAUNCHES.total += 1
        if plan.rows_local is None:
            plan.rows_local = torch.empty(self.T, self.K, dtype=torch.int32, device=x.device)
            native().ep_pull_rows(self.tables_dev, plan.ids, plan.rows_local, self.e_local, self.rank * self.T * self.K)
            LAUNCHES.total += 1
        return xp, y

    def combine(self, rows, plan: EpPlan, base=None, weighted: bool = True, scal=None, out=None):
        """``rows``: this rank's (C, d) expert rows — ideally ``rows_buffer()`` itself.  Returns ``y`` (T, d) with
        ``y[t] = base[t] + sum_k w[t, k] rows_owner[row]`` (weights 1 when not ``weighted``); with ``scal`` (C,) fp32
        per-row values also returns the (T, K) values of this rank's slots."""
        import torch
        out = out if out is not None else torch.empty(self.T, self.d, dtype=rows.dtype, device=rows.device)
        out_s = torch.empty(self.T, self.K, dtype=torch.float32, device=rows.device) if scal is not None else None
        if self.lane != "p2p":
            return self._combine_collective(rows, plan, base, weighted, scal, out, out_s)
        from ..ops import native
        from ..ops.cuda import LAUNCHES
        rb = self.rows_buffer()
        if rows.data_ptr() != rb.data_ptr():
            rb.copy_(rows)
        if scal is not None:
            self.scal_buffer().copy_(scal)
        self.seq_y += 1
        native().ep_combine([p + self.off_rows for p in self.ws], [p + self.off_scal for p in self.ws] if scal is not None else [],
                            base, plan.weights if weighted else None, plan.ids, plan.rows_local, out, out_s, self.e_local,
                            self.rank, [p + 128 for p in self.ws], [p + 192 for p in self.ws], self.seq_y, self.timeout_s,
                            self.err, self.done)
        LAUNCHES.total += 1
        return (out, out_s) if scal is not None else out

    # -- the collective lane: same results from all-gathers and all-reduces around library ops
    def _dispatch_mm_collective(self, x, w, plan, transpose_w, xp, y):
        import torch
        import torch.distributed as dist
        from ..ops.eager import moe_grouped_mm
        all_x = torch.empty(self.world * self.T, self.d, dtype=x.dtype, device=x.device)
        if self.world > 1:
            dist.all_gather_into_tensor(all_x, x.contiguous(), group=self.pg)
        else:
            all_x.copy_(x)
        src = plan.row_src.long()
        xp.copy_(all_x[src.clamp(min=0)] * (src >= 0).unsqueeze(-1).to(x.dtype))
        moe_grouped_mm(xp, w, plan.tile_expert.cpu(), out=y, transpose_w=transpose_w)
        if plan.rows_local is None:
            lo = self.rank * self.T
            tables = [torch.empty_like(plan._table) for _ in range(self.world)]
            if self.world > 1:
                dist.all_gather(tables, plan._table.contiguous(), group=self.pg)
            else:
                tables[0] = plan._table
            owner = (plan.ids // self.e_local).long()
            stacked = torch.stack([tb[lo:lo + self.T] for tb in tables], 0)              # (P, T, K)
            plan.rows_local = stacked.gather(0, owner.unsqueeze(0)).squeeze(0).to(torch.int32)
        return xp, y

    def _combine_collective(self, rows, plan, base, weighted, scal, out, out_s):
        import torch
        import torch.distributed as dist
        all_rows = torch.empty(self.world, self.C, self.d, dtype=rows.dtype, device=rows.device)
        if self.world > 1:
            dist.all_gather_into_tensor(all_rows.view(-1, self.d), rows.contiguous(), group=self.pg)
        else:
            all_rows[0].copy_(rows)
        owner = (plan.ids // self.e_local).long()
        rl = plan.rows_local.long()
        ok = rl >= 0
        g = all_rows[owner, rl.clamp(min=0)].float() * ok.unsqueeze(-1)
        wgt = plan.weights if weighted else torch.ones_like(plan.weights)
        acc = (g * wgt.unsqueeze(-1)).sum(1)
        if base is not None:
            acc = acc + base.float()
        out.copy_(acc.to(out.dtype))
        if scal is None:
            return out
        all_s = torch.empty(self.world, self.C, dtype=torch.float32, device=rows.device)
        if self.world > 1:
            dist.all_gather_into_tensor(all_s.view(-1), scal.float().contiguous(), group=self.pg)
        else:
            all_s[0].copy_(scal)
        out_s.copy_(all_s[owner, rl.clamp(min=0)] * ok)
        return out, out_s


def _up(n: int, a: int = 1 << 12) -> int:
    return (int(n) + a - 1) // a * a


# ---------------------------------------------------------------------------------------------------------------------
# One expert-parallel MoE MLP, forward and backward, out of the group's two kernels and local grouped GEMMs.  The model
# families call these from their MoE stages; the tests compare them with a single-rank layer over all experts.

def _kernels(g: EpGroup, ks):
    if ks is not None:
        return ks
    from ..ops import resolve_kernels
    return resolve_kernels(kernel_set=None if g.lane == "p2p" else "eager")


class ExpertReplicaGradSum:
    """Block optimizer of a dp x ep mesh: the expert stacks' gradients are summed over the replicas that hold the same
    experts (group ``dp``) before the inner executable (which sums the replicated fields over the whole job) runs."""

    def __init__(self, inner, lay, group_key: str = "dp"):
        self.inner, self.lay, self.group_key = inner, lay, group_key

    def launch(self, ctx):
        from ..models.tp_mlp.blocks import ReplicatedGradSum
        layer = ctx.task.block_params.get("layer", 0)
        gl = self.lay.of_layer(layer)[1] if hasattr(self.lay, "of_layer") else self.lay.block_dw
        fields = [n for n in gl.names() if n.endswith("_experts")]
        ReplicatedGradSum(self.inner, gl, fields, self.group_key).launch(ctx)


def sum_expert_gradients_over_replicas(trainer, group_key: str = "dp") -> None:
    table = trainer.resolver.table
    table["optimizer_block"] = ExpertReplicaGradSum(table["optimizer_block"], trainer.layouts, group_key)


def ep_group_for(family, cfg, rank: int, world: int, device: int | None, lane: str | None = None, timeout_s: float = 30.0,
                 pg=None) -> EpGroup:
    """The expert-parallel group of a job that trains ``cfg`` (with ``cfg.ep == world``) of ``family`` (a ``ModelFamily``):
    reads the token / width / expert counts from the family's dims, whichever lane the family is written in."""
    d = family.derive_dims(cfg)
    x = getattr(d, "x", None)                        # reference-form families keep their config there
    if x is not None:
        if not getattr(x, "n_experts", 0):
            raise ValueError(f"{family.name}: expert parallelism needs a mixture-of-experts preset")
        n_experts, top_k = int(x.n_experts), int(x.top_k)
    else:
        if not getattr(d, "moe", False):
            raise ValueError(f"{family.name}: expert parallelism needs a mixture-of-experts preset")
        n_experts, top_k = int(d.E), int(d.topk)
    return EpGroup(rank, world, device, tokens=int(d.T), d_model=int(d.d), n_experts=n_experts, top_k=top_k,
                   capacity_factor=float(getattr(cfg, "ep_capacity", 2.0)), lane=lane, timeout_s=timeout_s, pg=pg)


def ep_moe_forward(g: EpGroup, h, ids, weights, w13, w2, base=None, ks=None):
    """``h`` (T, d) block input (normalised), ``w13`` (E_local, d, 2 F), ``w2`` (E_local, F, d).  Returns ``(y, saved)``."""
    ks = _kernels(g, ks)
    p2p = g.lane == "p2p"
    plan = g.plan(ids, weights)
    xp, h13 = g.dispatch_mm(h, w13, plan)
    sp = ks.swiglu_packed_fwd(h13)
    te = plan.tile_expert
    yp = ks.moe_grouped_mm(sp, w2, te, out=g.rows_buffer() if p2p else None)
    y = g.combine(yp, plan, base=base, weighted=True)
    # the peer-readable rows are overwritten by the next layer: the backward keeps its own copy
    return y, {"plan": plan, "xp": xp, "h13": h13, "sp": sp, "yp": yp.clone() if p2p else yp}


def ep_moe_backward(g: EpGroup, dy, saved, w13, w2, dw13, dw2, accumulate: bool = False, ks=None):
    """Returns ``(dh (T, d), d_weights (T, K) fp32)`` and writes the local experts' weight gradients."""
    ks = _kernels(g, ks)
    p2p = g.lane == "p2p"
    plan, xp, h13, sp, yp = saved["plan"], saved["xp"], saved["h13"], saved["sp"], saved["yp"]
    te = plan.tile_expert
    # d(rows): every local row receives dy of the token it serves; the down-projection's dgrad is fused with that pull
    dyp, dsp_unscaled = g.dispatch_mm(dy, w2, plan, transpose_w=True)
    # router-weight gradient <dy, y_row>, computed where the row lives
    dscal = (dyp.float() * yp.float()).sum(-1)
    rw = plan.row_w.unsqueeze(-1)
    dsp = (dsp_unscaled.float() * rw).to(dsp_unscaled.dtype)
    dyp_s = (dyp.float() * rw).to(dyp.dtype)
    ks.moe_grouped_wgrad(sp, dyp_s, plan.offsets_pad, dw2, accumulate=accumulate)
    dh13 = ks.swiglu_packed_bwd(dsp, h13)
    ks.moe_grouped_wgrad(xp, dh13, plan.offsets_pad, dw13, accumulate=accumulate)
    dxp = ks.moe_grouped_mm(dh13, w13, te, out=g.rows_buffer() if p2p else None, transpose_w=True)
    dh, dw = g.combine(dxp, plan, base=None, weighted=False, scal=dscal)
    return dh, dw
