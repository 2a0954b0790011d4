"""ZeRO data parallelism over one NVSwitch box.

Each rank owns one flat, 256-byte aligned slice of every packed weight object.
Stage 3 keeps only that slice (``Ws_*``) and its optimizer state persistent; the
full ``W_*`` is gathered once per step in front of its first use.  Stage 1 keeps
``W_*`` whole and shards the optimizer state.  Two lanes serve a group:

* ``p2p``  — the hand-written fused kernels of ``ops/csrc/comm.cu``: gradient
  reduce-scatter ⊕ fp32 accumulate ⊕ partitioned AdamW in ONE kernel that pulls the
  peers' gradients over NVLink by plain peer loads, and an all-gather by peer loads.
  Every rank's engine slab and a small control block are mapped into the peers
  through CUDA IPC handles exchanged over ``torch.distributed``.
* ``collective`` — ``torch.distributed`` reduce-scatter / all-gather + the local AdamW
  kernel: the baseline lane (NCCL on GPUs, gloo on CPU ranks) and the oracle of the
  bitwise tests.

Reference: its ZeRO-1 lanes ``blocks/adamw/rs.py:34-105`` (flat equal slices) and
``distributed/sharding.py:588-652``; ZeRO-3 is absent there.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Mapping

from ..blocks.base_blocks import _Base
from ..blocks.layouts import Field, PackedLayout
from ..blocks.optim import lr_at
from .group_abi import GroupCollectives


class CommTimeout(RuntimeError):
    """A fused communication kernel gave up waiting for a peer (the error word names phase and peer)."""


def slice_bytes(total: int, world: int) -> int:
    per = (total + world - 1) // world
    return (per + 255) // 256 * 256


def slice_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """(byte offset, byte length) of ``rank``'s slice; trailing ranks may be short or empty."""
    per = slice_bytes(total, world)
    lo = min(per * rank, total)
    hi = min(per * (rank + 1), total)
    return lo, hi - lo


def zero_opt_layout(slice_nbytes: int, master: bool = True) -> PackedLayout:
    """Optimizer state of one slice: fp32 master (optional) + fp32 first / second moments."""
    n = slice_nbytes // 2
    f = ([Field("master", (n,), "fp32")] if master else []) + [Field("m", (n,), "fp32"), Field("v", (n,), "fp32")]
    return PackedLayout(tuple(f))


def split_opt_layout(slice_nbytes: int) -> PackedLayout:
    """Optimizer state of one re-gathered (FSDP) slice: low halves of the split fp32 master + bf16 moments."""
    n = slice_nbytes // 2
    return PackedLayout((Field("mlo", (n,), "int16"), Field("m", (n,), "bf16"), Field("v", (n,), "bf16")))


def zero_lower_kwargs(mode: str, rank: int, world: int, group: str = "dp") -> dict[str, Any]:
    """``zero3``: gather each layer once per step, fused reduce-scatter + AdamW at the end of the step.
    ``fsdp``: stage 3 with re-gathering — gather in front of every use, reduce-scatter every backward into an
    fp32 slice, local split-master AdamW (6 bytes of state per parameter, divided by the world size).
    ``zero1`` / ``zero1rs``: whole weights everywhere, sharded optimizer state."""
    if mode in ("co", "dp"):
        # plain data parallelism (ZeRO-0): every rank holds everything; gradients are summed in front of the optimizer
        # (``replicate_gradients``).  Nothing changes in the lowering.
        return {}
    stage = {"zero3": 3, "fsdp": 3, "zero1": 1, "zero1rs": 1}.get(mode)
    if stage is None:
        raise KeyError(f"unknown data-parallel mode {mode!r} (fsdp | zero3 | zero1 | co)")
    # fp32 master + two fp32 moments per bf16 parameter: 12 bytes per 2 parameter bytes, 256-byte aligned planes
    z = {"stage": stage, "rank": rank, "world": world, "group": group, "opt_bytes_per_param_byte": 6.0}
    if mode == "fsdp":
        z.update(regather=True, block_opt_bytes_per_param_byte=3.0)
        return {"zero": z, "resident_params": True}
    return {"zero": z}


@dataclass
class _Slot:
    calls: int = 0


class DpGroup(GroupCollectives):
    """One data-parallel group as seen by this rank."""

    SLOTS = 512

    def __init__(self, rank: int, world: int, device: int | None, lane: str | None = None, timeout_s: float = 60.0, pg=None):
        self.rank, self.world, self.device = rank, world, device
        self.pg = pg            # process group of the members when they are a subset of the job (used by ``all_reduce``)
        self.lane = lane or ("p2p" if device is not None else "collective")
        self.timeout_s = timeout_s
        self.calls: dict[int, int] = {}
        self.slabs: list[int] = []
        self.ctrls: list[int] = []
        self.backend = None
        self.err = None
        self.done = None
        # parameter gathers: "dma" moves the bytes with the copy engines (each rank stages its shard at a fixed address behind its
        # slab first); "kernel" pulls them with SM threads from wherever the shards lie
        self.gather_mode = os.environ.get("DATAFLOW_GATHER", "auto")      # "auto" is settled in attach() from the plan
        self.comm_stream = None
        self.done_async = None
        self.async_comm = False
        self.force_stage = False       # tests: treat every published buffer as if it had overflowed the slab
        self.name = "dp"

    # -- set-up (p2p lane): map every rank's slab and control block
    def attach(self, trainer) -> None:
        if self.lane != "p2p":
            return
        import torch
        import torch.distributed as dist
        be = trainer.backend
        self.backend = be
        base, cap = trainer.session.native.fast_slab()
        if not base:
            raise RuntimeError("the p2p lane needs the engine's fast slab to exist before attach()")
        self.slab_base, self.slab_cap = base, cap
        # staging behind the managed extent (same allocation, so the peers' mapping covers it): two halves, one for
        # launches on the compute stream, one for the communication stream
        self.tail_bytes = int(trainer.session.native.fast_tail())
        self.staged = 0
        self.ctrl = be.device_alloc_zeroed(16 * self.SLOTS)
        mine = (be.ipc_handle(base), be.ipc_handle(self.ctrl))
        handles: list[Any] = [None] * self.world
        dist.all_gather_object(handles, mine)
        self.slabs, self.ctrls = [], []
        for r, (hs, hc) in enumerate(handles):
            if r == self.rank:
                self.slabs.append(base)
                self.ctrls.append(self.ctrl)
            else:
                self.slabs.append(be.ipc_open(hs))
                self.ctrls.append(be.ipc_open(hc))
        dev = torch.device("cuda", self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        # asynchronous gathers / reduce-scatters run here, off the engine's compute stream; the "last CTA"
        # counter is per stream because kernels of the two streams may overlap
        self.comm_stream = torch.cuda.Stream(device=dev)
        self.done_async = torch.zeros(1, dtype=torch.int32, device=dev)
        self.async_comm = os.environ.get("DATAFLOW_ASYNC_COMM", "1") != "0"
        if self.gather_mode == "auto":
            # The copy engines also carry the plan's host traffic.  Measured on the 8B step: at 2 GPUs the host lanes are busy half
            # of the step and gathers on the copy engines cost 11 % (prefetches fall behind); where the lanes are nearly idle the
            # copy engines are free and the SM kernel's interference with the GEMM is what costs.  So: copy engines only when the
            # planned host-to-device traffic would keep the GPU's own link busy less than a quarter of the step (8 GPUs: 6 %).
            planned = getattr(trainer, "planned", None)
            busy = 1.0
            if planned is not None and planned.makespan_us:
                busy = float((planned.transfer or {}).get("from_slow", {}).get("busy_us", planned.makespan_us)) / float(planned.makespan_us)
                hw = getattr(trainer, "hw", None)
                if hw is not None and getattr(hw, "link_gbs", 0.0):
                    busy *= float(hw.h2d_gbs) / float(hw.link_gbs)     # lane time at a shared rate -> share of what the link can do
            self.gather_mode = "dma" if busy < 0.25 else "kernel"
        dist.barrier()

    def _in_slab(self, t, nbytes: int, asynchronous: bool = False) -> int:
        """Address of ``t``'s first ``nbytes`` that the peers can read.  A buffer inside the slab is its own address;
        one that overflowed the slab (a vendor allocation the peers never mapped) is copied into the staging half of
        the calling stream first — the kernel that reads it holds the stream until every peer is done reading, so
        the next copy into the same half cannot overtake a reader."""
        ptr = t.data_ptr()
        if self.slab_base <= ptr and ptr + nbytes <= self.slab_base + self.slab_cap and not self.force_stage:
            return ptr
        half = self.tail_bytes // 2
        if nbytes > half:
            raise RuntimeError("a buffer published to peers lies outside the peer-mapped engine slab and is larger "
                               f"than the staging behind it ({nbytes} > {half} bytes)")
        from ..ops import native
        import torch
        dst_ptr = self.slab_base + self.slab_cap + (half if asynchronous else 0)
        dst = native().tensor_from_ptr(dst_ptr, [nbytes], "uint8", self.device)
        dst.copy_(t.reshape(-1).view(torch.uint8)[:nbytes])
        self.staged += 1
        return dst_ptr

    def side(self, ctx, ready_ids):
        """Context for an asynchronous launch: the communication stream, ordered after everything the compute
        stream has queued so far; on exit an event is registered for the objects ``ready_ids`` so that their next
        consumer waits for the transfer on its own stream."""
        import contextlib
        import torch

        @contextlib.contextmanager
        def scope():
            cur = torch.cuda.current_stream()
            e0 = torch.cuda.Event()
            e0.record(cur)
            self.comm_stream.wait_event(e0)
            with torch.cuda.stream(self.comm_stream):
                yield
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
            ready = ctx.run_values.setdefault("_ready", {})
            for oid in ready_ids:
                ready[oid] = ev
        return scope()

    def _stage(self, t, nbytes: int, asynchronous: bool) -> int:
        """Copy ``t``'s first ``nbytes`` into the staging half of the calling stream (behind the slab, inside the peers' mapping of
        it) and return that address — the same on every rank, in every step.  The kernel that closes a gather holds the stream
        until every peer has finished reading, so the next copy into the half cannot overtake a reader."""
        import torch
        from ..ops import native
        half = self.tail_bytes // 2
        if nbytes > half:
            return 0
        dst_ptr = self.slab_base + self.slab_cap + (half if asynchronous else 0)
        dst = native().tensor_from_ptr(dst_ptr, [nbytes], "uint8", self.device)
        dst.copy_(t.reshape(-1).view(torch.uint8)[:nbytes])
        return dst_ptr

    def _next(self, slot: int) -> tuple[int, int]:
        c = self.calls.get(slot, 0) + 1
        self.calls[slot] = c
        return c, c * (self.world - 1)

    def check(self) -> None:
        """Raise if a kernel of this group timed out (reads the error word: a host sync)."""
        if self.err is not None:
            code = int(self.err.item())
            if code:
                self.err.zero_()
                raise CommTimeout(f"fused communication kernel gave up: phase {code >> 8}, peer/rank {code & 255}")

    # -- collectives
    def rs_adamw(self, slot: int, grad, begin_elem: int, len_elem: int, master, m, v, shard_out, fields, hyper, step, K):
        """grad: flat bf16 tensor of the whole object.  Updates (master, m, v, shard_out) of this rank's slice."""
        lr = lr_at(hyper, step)
        b1, b2, eps = hyper.get("beta1", 0.9), hyper.get("beta2", 0.95), hyper.get("eps", 1e-8)
        if self.lane == "p2p":
            from ..ops import native
            from ..ops.cuda import LAUNCHES
            seq, ack = self._next(slot)
            gptr = self._in_slab(grad, grad.numel() * 2)
            native().zero_rs_adamw(self.slabs, self.ctrls, self.rank, self.SLOTS, slot, seq, ack, gptr,
                                   begin_elem, len_elem, master, m, v, shard_out.data_ptr(),
                                   [f[0] for f in fields], [f[1] for f in fields], [f[2] for f in fields],
                                   lr, b1, b2, eps, int(step), 1.0, self.timeout_s, self.err, self.done)
            LAUNCHES.total += 1
            return
        import torch
        import torch.distributed as dist
        per = slice_bytes(grad.numel() * 2, self.world) // 2
        g32 = torch.zeros(per * self.world, dtype=torch.float32, device=grad.device)
        g32[:grad.numel()] = grad.float()
        if dist.get_backend() == "gloo":
            dist.all_reduce(g32)
            acc = g32[self.rank * per:self.rank * per + len_elem].clone()
        else:
            out = torch.empty(per, dtype=torch.float32, device=grad.device)
            dist.reduce_scatter_tensor(out, g32)
            acc = out[:len_elem]
        wd_vec = torch.zeros(len_elem, dtype=torch.float32, device=grad.device)
        for b, e, wd in fields:
            lo, hi = max(b, begin_elem) - begin_elem, min(e, begin_elem + len_elem) - begin_elem
            if hi > lo:
                wd_vec[lo:hi] = wd
        m.mul_(b1).add_(acc, alpha=1 - b1)
        v.mul_(b2).addcmul_(acc, acc, value=1 - b2)
        w = master if master is not None else shard_out.float()
        upd = (m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps) + wd_vec * w
        w = w - lr * upd
        if master is not None:
            master.copy_(w)
        shard_out.copy_(w.to(shard_out.dtype))

    def rs_accum(self, slot: int, grad, begin_elem: int, len_elem: int, gacc, first: bool, asynchronous: bool = False) -> None:
        """Reduce-scatter ``grad`` (flat bf16, whole object) over the group and add this rank's slice of the sum
        into ``gacc`` (fp32, slice-sized); ``first`` overwrites instead."""
        if self.lane == "p2p":
            from ..ops import native
            from ..ops.cuda import LAUNCHES
            seq, ack = self._next(slot)
            gptr = self._in_slab(grad, grad.numel() * 2, asynchronous)
            native().zero_rs_accum(self.slabs, self.ctrls, self.rank, self.SLOTS, slot, seq, ack, gptr,
                                   begin_elem, len_elem, gacc, bool(first), self.timeout_s, self.err,
                                   self.done_async if asynchronous else self.done)
            LAUNCHES.total += 1
            return
        import torch
        import torch.distributed as dist
        g32 = grad.float()
        dist.all_reduce(g32)
        part = g32[begin_elem:begin_elem + len_elem]
        if first:
            gacc[:len_elem].copy_(part)
        else:
            gacc[:len_elem].add_(part)

    def gather(self, slot: int, shard, full, per_bytes: int, asynchronous: bool = False) -> None:
        """shard, full: uint8 tensors; ``full`` receives every rank's slice at ``rank * per_bytes``."""
        total = full.numel()
        if self.lane == "p2p":
            from ..ops import native
            from ..ops.cuda import LAUNCHES
            seq, ack = self._next(slot)
            n_mine = min(per_bytes, shard.numel())
            if self.gather_mode == "dma":
                # The bytes ride the copy engines, which need the peers' source addresses on the HOST when the copies are issued.
                # Shards live wherever the engine's allocator put them (differently on every rank, and anew after every optimizer
                # step), so every rank first copies its shard to the one address all ranks know: the staging half behind its slab.
                sptr = self._stage(shard, n_mine, asynchronous)
                if sptr:
                    offs = [sptr - self.slab_base] * self.world
                    native().param_gather_dma(self.slabs, self.ctrls, self.rank, self.SLOTS, slot, seq, ack, sptr, offs, full.data_ptr(),
                                              per_bytes, total, self.timeout_s, self.err)
                    LAUNCHES.total += 3
                    return
            sptr = self._in_slab(shard, n_mine, asynchronous)
            native().param_gather(self.slabs, self.ctrls, self.rank, self.SLOTS, slot, seq, ack, sptr,
                                  full.data_ptr(), per_bytes, total, self.timeout_s, self.err,
                                  self.done_async if asynchronous else self.done)
            LAUNCHES.total += 1
            return
        import torch
        import torch.distributed as dist
        mine = torch.zeros(per_bytes, dtype=torch.uint8, device=full.device)
        n = min(per_bytes, shard.numel())
        mine[:n] = shard[:n]
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine)
        for r, p in enumerate(parts):
            lo, ln = slice_range(total, self.world, r)
            if ln:
                full[lo:lo + ln] = p[:ln]

    def all_reduce(self, t):
        """Sum over the group (plain data parallelism: whole gradient objects in front of the optimizer)."""
        import torch.distributed as dist
        if self.world > 1:
            dist.all_reduce(t, group=self.pg)
        return t

    def close(self) -> None:
        if self.lane == "p2p" and self.backend is not None:
            for r, (s, c) in enumerate(zip(self.slabs, self.ctrls)):
                if r != self.rank:
                    self.backend.ipc_close(s)
                    self.backend.ipc_close(c)
            self.backend.device_free(self.ctrl)
            self.slabs, self.ctrls = [], []


def replicate_gradients(trainer, group_key: str = "dp") -> None:
    """ZeRO-0 ("co"): wrap every optimizer executable of ``trainer`` so that it first sums the layer's gradient object over
    the group; every rank then applies the identical update.  Replicas stay bitwise equal — which also makes this lane a
    corruption tripwire.  Ranks may run different numbers of rounds (weighted data parallelism): only the optimizer
    tasks, which every rank has in the same order, communicate."""
    from ..models.tp_mlp.blocks import ReplicatedGradSum
    table = trainer.resolver.table
    lay = trainer.layouts
    for key in list(table):
        if not key.startswith("optimizer"):
            continue
        inner = table[key]
        target = {"optimizer_embed": lay.embed_dw, "optimizer_head": lay.head_dw}.get(key)
        table[key] = _LayerAwareGradSum(inner, target, lay, group_key) if target is None else ReplicatedGradSum(inner, target, None, group_key)


class _LayerAwareGradSum:
    """``ReplicatedGradSum`` for block optimizers of families whose layers have different layouts."""

    def __init__(self, inner, layout, lay, group_key):
        self.inner, self.lay, self.group_key = inner, lay, group_key

    def launch(self, ctx):
        from ..models.tp_mlp.blocks import ReplicatedGradSum
        layer = ctx.task.block_params.get("layer", 0)
        gl = self.lay.of_layer(layer)[1] if hasattr(self.lay, "of_layer") else self.lay.block_dw
        ReplicatedGradSum(self.inner, gl, None, self.group_key).launch(ctx)


def make_dp_group(rank: int, world: int, device: int | None, lane: str | None = None, pg=None) -> DpGroup:
    lane = lane or os.environ.get("DATAFLOW_DP_LANE")
    return DpGroup(rank, world, device, lane, pg=pg)


def slot_of(target: str, layer: int | None, kind: int) -> int:
    """kind 0: gradient reduce-scatter, kind 1: parameter gather."""
    idx = 0 if target == "embed" else 1 if target == "head" else 2 + int(layer)
    return 2 * idx + kind


def wd_fields(layout: PackedLayout, wd: float, wd_all: bool = False) -> list[tuple[int, int, float]]:
    """Element ranges (bf16 elements of the flat packed object) that take weight decay."""
    offs = layout.offsets()
    out = []
    for f in layout.fields:
        if wd and (wd_all or f.kind in ("matrix", "embedding")):
            out.append((offs[f.name] // 2, (offs[f.name] + f.nbytes) // 2, float(wd)))
    return out


def _flat(buf, nbytes: int, dtype: str, device):
    from ..runtime.interop import torch_view
    item = {"bf16": 2, "uint8": 1, "fp32": 4}[dtype]
    return torch_view(buf, (nbytes // item,), dtype, 0, device if buf.location == "fast" else None)


def _group(ctx) -> DpGroup:
    name = ctx.task.comm_groups.get("dp", "dp")
    g = ctx.groups.get(name)
    if g is None:
        raise KeyError(f"task {ctx.task.id} needs peer group {name!r} but the run was started without it")
    return g


class ParamGather(_Base):
    """(Ws_X) -> (W_X): all-gather of the ranks' flat slices into the full packed weight object."""

    def run(self, ctx):
        g = _group(ctx)
        bp = ctx.task.block_params
        full_b = ctx.outputs[0]
        shard = _flat(ctx.inputs[0], ctx.inputs[0].size, "uint8", self.device)
        full = _flat(full_b, full_b.size, "uint8", self.device)
        slot = slot_of(bp.get("target", "block"), bp.get("layer"), 1)
        if g.async_comm and g.lane == "p2p" and ctx.task.id.endswith(("f", "b")) and full_b.object_id.startswith("Wg_"):
            with g.side(ctx, [full_b.object_id]):         # re-gather issued ahead of its consumer
                g.gather(slot, shard, full, slice_bytes(full_b.size, g.world), asynchronous=True)
            return
        g.gather(slot, shard, full, slice_bytes(full_b.size, g.world))


class GradReduceScatter(_Base):
    """(dW[, G]) -> ([G]): this round's full gradient, reduce-scattered and added into the rank's fp32 slice."""

    def run(self, ctx):
        g = _group(ctx)
        bp = ctx.task.block_params
        total = ctx.inputs[0].size
        lo, ln = slice_range(total, g.world, g.rank)
        first = bool(bp.get("first"))
        acc_buf = ctx.outputs[0] if first else ctx.inputs[1]
        gacc = _flat(acc_buf, acc_buf.size, "fp32", self.device)
        grad = _flat(ctx.inputs[0], total, "bf16", self.device)
        slot = slot_of(bp.get("target", "block"), bp.get("layer"), 0)
        if g.async_comm and g.lane == "p2p":
            with g.side(ctx, [ctx.inputs[0].object_id, acc_buf.object_id]):      # joined by grad_rs_join / the optimizer
                g.rs_accum(slot, grad, lo // 2, ln // 2, gacc, first, asynchronous=True)
            return
        g.rs_accum(slot, grad, lo // 2, ln // 2, gacc, first)


class CommJoin(_Base):
    """(dW, G) -> (): the point where an asynchronous reduce-scatter must be complete.  The wait itself is the
    generic input wait of ``launch``; the full gradient's last use is here, so the engine frees it after."""

    def run(self, ctx):
        return None


def local_split_step(exe, ctx, wl, grp) -> None:
    """FSDP optimizer task ``(Ws, G, O)``: split-master AdamW on this rank's slice, field by field (weight decay
    differs between matrices and vectors); no communication."""
    total = wl.size_bytes
    lo, ln = slice_range(total, grp.world, grp.rank)
    per = slice_bytes(total, grp.world)
    dev = exe.device
    n = ln // 2
    if not n:
        return
    w = _flat(ctx.inputs[0], per, "bf16", dev)
    gacc = _flat(ctx.inputs[1], ctx.inputs[1].size, "fp32", dev)
    ost = split_opt_layout(per).views(ctx.inputs[2], dev if ctx.inputs[2].location == "fast" else None)
    hy = exe.hyper
    step = int(ctx.run_args.get("step", 1))
    lr = lr_at(hy, step)
    b1, b2, eps = hy.get("beta1", 0.9), hy.get("beta2", 0.95), hy.get("eps", 1e-8)
    wd, wd_all = hy.get("weight_decay", 0.0), bool(hy.get("wd_all"))
    offs = wl.offsets()
    e0 = lo // 2
    pos = 0                                  # elements of the slice handled so far
    cuts: list[tuple[int, int, float]] = []
    for f in wl.fields:                      # fields in layout order; gaps (alignment padding) take no decay
        a, b = offs[f.name] // 2 - e0, (offs[f.name] + f.nbytes) // 2 - e0
        a, b = max(a, 0), min(b, n)
        if b <= a:
            continue
        if a > pos:
            cuts.append((pos, a, 0.0))
        cuts.append((a, b, float(wd) if (wd and (wd_all or f.kind in ("matrix", "embedding"))) else 0.0))
        pos = b
    if pos < n:
        cuts.append((pos, n, 0.0))
    for a, b, fwd in cuts:
        exe.K.adamw_split_step(w[a:b], ost["mlo"][a:b], gacc[a:b], ost["m"][a:b], ost["v"][a:b], lr, b1, b2, eps, fwd, step)


def sharded_optimizer_step(exe, ctx, wl, gl, ol, w, g, o) -> bool:
    """ZeRO optimizer task: ``(Ws|W, dW, O) -> update of this rank's slice`` (+ in-place gather at stage 1)."""
    shard = ctx.task.block_params.get("shard")
    if not shard:
        return False
    if exe.hyper.get("train_only"):
        raise NotImplementedError("a run that updates a named subset of fields (train_only) cannot shard its optimizer: "
                                  "the sharded step works on flat slices of the packed object, not on fields")
    grp = _group(ctx)
    stage, rank, world = int(shard["stage"]), grp.rank, grp.world
    bp = ctx.task.block_params
    if bp.get("local"):
        local_split_step(exe, ctx, wl, grp)
        return True
    total = wl.size_bytes
    lo, ln = slice_range(total, world, rank)
    per = slice_bytes(total, world)
    dev = exe.device
    grad = _flat(ctx.inputs[1], total, "bf16", dev)
    ost = zero_opt_layout(per).views(ctx.inputs[2], dev if ctx.inputs[2].location == "fast" else None)
    n = ln // 2
    if stage == 3:
        shard_out = _flat(ctx.inputs[0], per, "bf16", dev)[:n]
    else:
        shard_out = _flat(ctx.inputs[0], total, "bf16", dev)[lo // 2:lo // 2 + n]
    hy = exe.hyper
    fields = wd_fields(wl, hy.get("weight_decay", 0.0), bool(hy.get("wd_all")))
    step = int(ctx.run_args.get("step", 1))
    tgt = bp.get("target", "block")
    if n:
        grp.rs_adamw(slot_of(tgt, bp.get("layer"), 0), grad, lo // 2, n, ost["master"][:n], ost["m"][:n], ost["v"][:n],
                     shard_out, fields, hy, step, exe.K)
    else:
        grp.rs_adamw(slot_of(tgt, bp.get("layer"), 0), grad, 0, 0, ost["master"][:0], ost["m"][:0], ost["v"][:0],
                     shard_out, fields, hy, step, exe.K)
    if stage == 1:
        full = _flat(ctx.inputs[0], total, "uint8", dev)
        grp.gather(slot_of(tgt, bp.get("layer"), 1), full[lo:lo + ln], full, per)
    return True


def zero_initial_values(fam, cfg, program, store, seed: int, layouts, rank: int, world: int, stage: int) -> None:
    """Seeded init under ZeRO: every rank generates the same full objects one at a time (same seed,
    same order as the solo program) and keeps its slice; master = fp32 copy of the slice, moments zero."""
    import torch
    from ..runtime.executable import Buffer
    solo = fam.lower(cfg)
    keep = tuple(o for o in solo.initial_objects if o.id.startswith("W_"))
    import dataclasses
    solo = dataclasses.replace(solo, initial_objects=keep)
    pending: dict[str, Any] = {}
    regather = bool(((program.metadata or {}).get("zero") or {}).get("regather"))

    def flush():
        for oid, (t, lay) in list(pending.items()):
            name = oid[2:]
            total = lay.size_bytes
            lo, ln = slice_range(total, world, rank)
            per = slice_bytes(total, world)
            raw = t
            if stage == 3:
                dst = views_of_raw(f"Ws_{name}", per)
                dst.zero_()
                dst[:ln] = raw[lo:lo + ln]
            else:
                views_of_raw(oid, total).copy_(raw)
            if regather and name.isdigit():
                ost = split_opt_layout(per).views(store_buffer(f"O_{name}"), None)
                for plane in ("mlo", "m", "v"):         # master == weight: low halves are zero
                    ost[plane].zero_()
            else:
                ost = zero_opt_layout(per).views(store_buffer(f"O_{name}"), None)
                ost["m"].zero_()
                ost["v"].zero_()
                ost["master"].zero_()
                if ln:
                    ost["master"][:ln // 2] = raw[lo:lo + ln].view(torch.bfloat16).float()
            del pending[oid]

    store_buffer = store.buffer

    def views_of_raw(oid, nbytes):
        from ..runtime.interop import torch_view
        return torch_view(store_buffer(oid), (nbytes,), "uint8", 0, None)

    def temp_views(oid, layout):
        from ..runtime.interop import invalidate_views
        flush()
        invalidate_views()       # temp tensors may reuse an address: never serve a stale cached view
        t = torch.zeros(layout.size_bytes, dtype=torch.uint8)
        pending[oid] = (t, layout)
        return layout.views(Buffer(t.data_ptr(), t.numel(), "backing", oid), None)

    fam.initial_values(solo, cfg, temp_views, seed, layouts=layouts)
    flush()
