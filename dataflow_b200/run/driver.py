"""In-process training driver: lower → (profile) → plan → init → per-step ``execute``.

``Trainer`` is the public single-process API: it owns the backend, the session
(streams + fast slab), a pinned host *store* holding every persistent object and
the per-round token buffers, the planned Program and the resolver.  ``step()``
writes one step's tokens into the store, runs the annotated chain once and returns
the step loss read back from the ``loss_*`` objects.  Role parity: reference
``src/dataflow_training/run/driver.py:410-942`` (``init_model``, ``plan_at_budget``,
``run_engine``) — without the daemon hop, which ``dataflow_b200.service`` adds.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping

from ..core import Program
from ..lowering.planning import PlannedProgram, plan_program
from ..lowering.shaped_program import ShapedHardware, resolve_hardware
from ..models.families import resolve_family
from ..runtime import Buffer, CpuBackend, Engine, Session

GiB = 1 << 30


@dataclass
class RunResult:
    """Loss curve and timing of a run (``.save`` writes the run-curve JSON)."""
    losses: list[float] = field(default_factory=list)
    step_wall_s: list[float] = field(default_factory=list)
    tokens_per_step: int = 0
    meta: dict[str, Any] = field(default_factory=dict)

    @property
    def tokens_per_s(self) -> float:
        t = sum(self.step_wall_s)
        return self.tokens_per_step * len(self.step_wall_s) / t if t else 0.0

    def save(self, path) -> None:
        Path(path).write_text(json.dumps({"losses": self.losses, "step_wall_s": self.step_wall_s,
                                          "tokens_per_step": self.tokens_per_step, "meta": self.meta}, indent=1))


class HostStore:
    """Named extents inside one host region (pinned when the backend is CUDA)."""

    ALIGN = 4096

    def __init__(self, backend, sizes: Mapping[str, int], pinned: bool):
        self.backend = backend
        self.pinned = pinned
        self.offsets: dict[str, int] = {}
        off = 0
        for k, n in sizes.items():
            self.offsets[k] = off
            off += (int(n) + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.total = max(off, self.ALIGN)
        self.sizes = {k: int(v) for k, v in sizes.items()}
        if pinned:
            self.base = backend.pin_region(self.total, True)
        else:
            self.base = backend.alloc(1, self.total)

    def buffer(self, oid: str) -> Buffer:
        return Buffer(self.base + self.offsets[oid], self.sizes[oid], "backing", oid)

    def buffers(self) -> dict[str, Buffer]:
        return {k: self.buffer(k) for k in self.offsets}

    def close(self):
        if self.base:
            if self.pinned:
                self.backend.unpin_region(self.base, self.total)
            else:
                self.backend.free(1, self.base, self.total)
            self.base = 0


def plan_at_budget(family, cfg, budget_bytes: int | None, hw: ShapedHardware | None = None, *,
                   recompute: bool = True, measured: Mapping[str, float] | None = None,
                   leeway_bytes: int | None = None, lower_kwargs: Mapping[str, Any] | None = None) -> PlannedProgram:
    """Lower ``cfg`` and plan it under ``budget_bytes`` of device memory."""
    from ..lowering.planning import DEFAULT_PROGRAM_LEEWAY_BYTES
    from .profiling import apply_measured_costs
    fam = resolve_family(family) if isinstance(family, str) else family
    hw = hw or resolve_hardware(None)
    kw = dict(lower_kwargs or {})

    fixed_levels = kw.pop("recompute_levels", None)

    def variant(levels):
        p = fam.lower(cfg, recompute_levels=levels if levels is not None else fixed_levels, hw=hw, **kw)
        return apply_measured_costs(p, measured) if measured else p

    program = variant(None)
    return plan_program(program, budget_bytes, recompute=recompute, build_variant=variant,
                        leeway_bytes=DEFAULT_PROGRAM_LEEWAY_BYTES if leeway_bytes is None else leeway_bytes)


def _agree_across_ranks(value):
    """Every rank of a job must plan the SAME program (the same recompute choices give the same task list, hence the
    same order of collectives): planning inputs that were measured per rank are replaced by rank 0's."""
    try:
        import torch.distributed as dist
    except ImportError:
        return value
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    box = [value]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class Trainer:
    """Single-process engine training loop over one device (or the CPU backend)."""

    def __init__(self, family: str, cfg, *, budget_gib: float | None = None, device: int | None = 0,
                 hyper: Mapping[str, Any] | None = None, seed: int = 0, hw: ShapedHardware | None = None,
                 kernels=None, kernel_set: str | None = None, recompute: bool = True, profile: bool = False,
                 leeway_bytes: int | None = None, planned: PlannedProgram | None = None,
                 lower_kwargs: Mapping[str, Any] | None = None, groups: Mapping[str, Any] | None = None,
                 init: bool = True, verbose: bool = False, static_placement: bool | None = None, pool_mode: str | None = None):
        import torch
        from ..ops import resolve_kernels
        self.fam = resolve_family(family)
        self.cfg = cfg
        self.device = device
        self.verbose = verbose
        self.hyper = {"optimizer": getattr(cfg, "optimizer", "adamw"),
                      "dtype_policy": cfg.policy().to_dict() if hasattr(cfg, "policy") else "bf16", **dict(hyper or {})}
        if getattr(cfg, "trainable_patterns", ()) and "train_only" not in self.hyper:
            self.hyper["train_only"] = list(cfg.trainable_patterns)
        self.groups = dict(groups or {})
        if device is None:
            self.backend = CpuBackend()
            self.hw = hw or resolve_hardware("cpu")
            self.K = kernels or resolve_kernels(kernel_set="eager" if kernel_set is None else kernel_set)
        else:
            from ..runtime import CudaBackend
            torch.cuda.set_device(device)
            self.backend = CudaBackend(device, "poll")
            self.hw = hw or resolve_hardware(None)
            self.K = kernels or resolve_kernels(kernel_set=kernel_set)
        self.dims = self.fam.derive_dims(cfg)
        self.layouts = self.fam.family_layouts(self.dims, cfg.policy() if hasattr(cfg, "policy") else None,
                                               self.hyper["optimizer"])
        self.session = Session(self.backend)
        self.engine = Engine(self.backend, session=self.session)
        self.resolver = self.fam.build_resolver(self.dims, self.hyper, self.K, device, layouts=self.layouts)
        budget = None if budget_gib is None else int(budget_gib * GiB)
        measured = None
        t0 = time.time()
        planned_by_caller = planned
        if planned is None:
            if profile and device is not None:
                from .profiling import profile_program
                bare = self.fam.lower(cfg, hw=self.hw, **dict(lower_kwargs or {}))
                measured = profile_program(self, bare)
                measured = _agree_across_ranks(measured)
            planned = plan_at_budget(self.fam, cfg, budget, self.hw, recompute=recompute, measured=measured,
                                     leeway_bytes=leeway_bytes, lower_kwargs=lower_kwargs)
        self.planned = planned
        self.program: Program = planned.program
        self.plan_s = time.time() - t0
        self.measured = measured
        # host store: persistent objects, tokens/targets, loss landing words
        sizes: dict[str, int] = {}
        for o in self.program.initial_objects:
            if o.id not in sizes:
                sizes[o.id] = o.size_bytes
        for t in self.program.tasks:
            for out in t.outputs:
                if out.location == "backing" and out.id.startswith("loss_"):
                    sizes[out.id] = out.size_bytes
        self.store = HostStore(self.backend, sizes, pinned=device is not None)
        self.loss_ids = sorted(k for k in sizes if k.startswith("loss_"))
        self.rounds = int(self.program.metadata.get("grad_accum_rounds", 1))
        self.T = int(self.program.metadata.get("tokens_per_round", self.dims.T))
        # size the session pools once: objects only (scratch lives in the framework allocator)
        self.pool_demand = None
        keep_resident = any(loc == "fast" for loc in self.program.final_locations.values())
        if device is not None:
            self._size_pools(cfg, sizes, budget, leeway_bytes, recompute, measured, lower_kwargs, planned_by_caller is None, pool_mode, keep_resident)
        else:
            self.pool_mode = "slab"
        self.step_index = 0
        self.last_result = None
        # static placement: offsets of every device allocation of a step, computed from a dry run (runtime/placement.py)
        self.placement = None
        if static_placement is None:
            static_placement = os.environ.get("DATAFLOW_STATIC_PLACEMENT") == "1"
        if static_placement and device is not None:
            self._fit_static_extent(cfg, budget, recompute, measured, leeway_bytes, lower_kwargs, replan=planned_by_caller is None)
        self.zero = (self.program.metadata or {}).get("zero")
        if self.zero and int(self.zero.get("world", 1)) > 1 and hasattr(cfg, "policy"):
            # the sharded lanes cut the packed objects into flat slices of bf16 elements and keep fp32 state per slice
            dt = cfg.policy().for_field("w", 0)
            if dt.param != "bf16" or dt.grad != "bf16":
                raise ValueError(f"sharded data parallelism (fsdp / zero*) needs bf16 parameters and gradients (dtype policies bf16, "
                                 f"bf16_master, bf16_split_master); this run asks for {dt.param} / {dt.grad} — use --parallel co for replicas")
        # weights that end a step on the device stay there for the next one (Session.resident)
        self.keep_resident = keep_resident
        # on a device, launch up to two tasks behind an unfinished one: host dispatch hides behind device work
        self.dispatch_ahead = 2 if device is not None else 0
        for g in self.groups.values():
            if hasattr(g, "attach"):
                g.attach(self)
        if init:
            self.init_model(seed)

    # -- store views
    def views_of(self, oid: str, layout):
        return layout.views(self.store.buffer(oid), None)

    def host_tensor(self, oid: str, shape, dtype: str):
        from ..runtime.interop import torch_view
        return torch_view(self.store.buffer(oid), shape, dtype, 0, None)

    def _size_pools(self, cfg, sizes, budget, leeway_bytes, recompute, measured, lower_kwargs, may_replan: bool, pool_mode, keep_resident: bool) -> None:
        """Size the session's device and pinned pools for ``self.program`` (once, before the first step)."""
        store_bytes = sum(sizes.values())
        transient_backing = max(self.planned.peak_backing_bytes - store_bytes, 0) + (64 << 20)
        fast = self.planned.object_capacity or (self.planned.peak_fast_bytes + (256 << 20))
        # the whole object share of the budget: the room above the planned peak absorbs slab fragmentation
        # plus most of the budget's leeway share: the planner never counts on it, it only absorbs fragmentation
        # (a buffer that overflows the slab cannot be read by peers, and costs a vendor allocation)
        from ..lowering.planning import DEFAULT_PROGRAM_LEEWAY_BYTES
        lee = DEFAULT_PROGRAM_LEEWAY_BYTES if leeway_bytes is None else int(leeway_bytes)
        spare = min(lee * 3 // 4, 1 << 30) if budget is not None else 0
        zero_md = (self.program.metadata or {}).get("zero")
        tail = 0
        if zero_md and int(zero_md.get("world", 1)) > 1:
            # staging behind the slab, mapped by the peers with it: a published buffer (gradient, parameter slice)
            # that overflowed the slab is copied there first; one region per stream that publishes
            sizes_all = self.program.object_sizes()
            pub = max((b for oid, b in sizes_all.items() if oid.startswith(("dW", "W", "dEmbed", "dHead", "Embed", "Head"))), default=0)
            tail = 2 * (int(pub) + 4096)
            self.session.native.set_fast_tail(tail)
        # what the pools are really asked for, from a run of the plan on the virtual-time backend: the backing pool is
        # sized from its measured peak (the plan's backing peak minus the store's size under-counts it: the store holds
        # every persistent object for the whole run, whatever the plan's ledger says about their backing copies), and a
        # fast pool that overflows gets a plan made with a little less memory, in the pool it already has
        # ranks of a sharded run must hold the same plan.  Planning is deterministic (the same inputs give the same plan in every
        # process), so every rank would arrive at the same second plan by itself; that has not run on several GPUs, hence the switch
        sharded_ranks = int(zero_md.get("world", 1)) if zero_md else 1
        if os.environ.get("DATAFLOW_POOL_FIT", "1") != "0":
            transient_backing = self._fit_pools(cfg, sizes, int(fast) + spare, transient_backing, keep_resident, budget, recompute, measured,
                                                leeway_bytes, lower_kwargs, replan=may_replan and (sharded_ranks == 1 or os.environ.get("DATAFLOW_POOL_FIT_RANKS") == "1"))
        # pool mode: "slab" (default) is one allocation under an offset allocator; "vmm" backs the pool page by page behind
        # twice its size of virtual addresses, so fragmentation costs address room instead of failing — at the price of
        # driver calls whenever pages move.  At the 8B headline configuration (plan fills 98 % of the pool) that price was
        # 25 k page moves and 5 s per step, so the mode is opt-in: it suits plans with slack and long-lived layouts.
        mode = pool_mode or os.environ.get("DATAFLOW_POOL_MODE", "slab")
        if mode not in ("auto", "slab", "vmm"):
            raise ValueError(f"pool mode {mode!r}: auto | slab | vmm")
        peers_map_slab = bool(zero_md and int(zero_md.get("world", 1)) > 1)
        if mode == "vmm" and peers_map_slab:
            raise ValueError("pool mode 'vmm' cannot serve the sharded data-parallel lanes: their kernels read peers' slabs through "
                             "one mapping of one allocation")
        self.pool_mode = "vmm" if mode == "vmm" else "slab"           # "auto" = the default
        try:
            self.session.native.ensure_pools(int(fast) + spare, int(transient_backing), 0.0, self.pool_mode == "vmm")
        except RuntimeError as e:
            if mode == "vmm":
                raise
            if self.verbose:
                print(f"vmm pool not available ({e}); using one allocation")
            self.pool_mode = "slab"
            self.session.native.ensure_pools(int(fast) + spare, int(transient_backing), 0.0, False)

    def _fit_pools(self, cfg, store_sizes, fast_capacity: int, transient_backing: int, keep_resident: bool, budget, recompute, measured,
                   leeway_bytes, lower_kwargs, replan: bool, dispatch_ahead: int = 2, min_cut: int = 1 << 30) -> int:
        """Dry-run the plan against the pools it will get (``runtime/pool_demand.py``).  Returns the bytes to give the backing pool.
        When the fast pool overflows and ``replan`` allows it, the step is planned again with the budget lowered by the bytes
        that did not fit (at least 1 GiB), the pool keeping its size; the new plan is taken when it overflows less and its
        predicted step time is not worse by more than 1 %.  Any failure leaves the first plan and the first sizing in place."""
        from ..runtime.pool_demand import dry_run_pools
        try:
            d = dry_run_pools(self.program, store_sizes, fast_capacity, keep_resident=keep_resident, dispatch_ahead=dispatch_ahead)
        except Exception as e:          # noqa: BLE001  (a dry run that cannot finish says nothing about the real run)
            if self.verbose:
                print(f"pool dry run failed ({type(e).__name__}: {e}); pools sized from the plan's peaks")
            return transient_backing
        self.pool_demand = d
        if replan and budget is not None and d.fast_overflows:
            cut = max(int(min_cut), int(d.fast_overflow_bytes * 0.5))
            for _ in range(2):
                if cut > int(budget) // 4:                   # a quarter of the budget is no longer "a little less memory"
                    break
                try:
                    p2 = plan_at_budget(self.fam, cfg, int(budget) - cut, self.hw, recompute=recompute, measured=measured,
                                        leeway_bytes=leeway_bytes, lower_kwargs=lower_kwargs)
                    same_store = {o.id: o.size_bytes for o in p2.program.initial_objects} == {o.id: o.size_bytes for o in self.program.initial_objects}
                    if not same_store or p2.makespan_us > self.planned.makespan_us * 1.01:
                        break
                    d2 = dry_run_pools(p2.program, store_sizes, fast_capacity, keep_resident=keep_resident, dispatch_ahead=dispatch_ahead)
                except Exception:       # noqa: BLE001  (an optimisation: whatever goes wrong, the first plan stands)
                    break
                if d2.fast_overflows < d.fast_overflows:
                    if self.verbose:
                        print(f"fast pool: {d.fast_overflows} overflows per step with the first plan, {d2.fast_overflows} with a plan made for "
                              f"{cut / 2 ** 30:.2f} GiB less (predicted step {self.planned.makespan_us / 1e6:.4f} -> {p2.makespan_us / 1e6:.4f} s)")
                    self.planned, self.program, self.pool_demand, d = p2, p2.program, d2, d2
                if d.fast_overflows == 0:
                    break
                cut *= 2
        return max(transient_backing, int(d.backing_peak * 1.02) + (64 << 20))

    def _fit_static_extent(self, cfg, budget, recompute, measured, leeway_bytes, lower_kwargs, replan: bool, rounds: int = 4) -> None:
        """Static placement with a replan loop: pack the plan's allocations into the pool; when no packing fits (the plan's peak
        leaves too little room for the holes a packing needs), plan again with the budget lowered by the excess plus a margin,
        and try again.  The pool keeps the size the FIRST plan gave it, so every round gains room.  Ends with a placement
        (``self.placement``, and possibly a new ``self.program``) or with the dynamic allocator and a note.
        Role parity: reference ``src/dataflow_training/lowering/planning.py`` (``fit_static_extent``)."""
        from ..runtime.placement import PlacementError, compute_placement, plan_placement, record_lifetimes
        capacity = int(self.session.native.fast_slab()[1])
        cut = 0
        for attempt in range(rounds):
            try:
                self.placement = plan_placement(self.program, capacity)
                if self.verbose and attempt:
                    print(f"static placement fits after {attempt} replans (budget lowered by {cut / 2 ** 30:.2f} GiB)")
                return
            except PlacementError as e:
                if not replan or budget is None or attempt == rounds - 1:
                    if self.verbose:
                        print(f"static placement not used: {e}")
                    return
                top = compute_placement(record_lifetimes(self.program, 0), None).top          # what the best packing needs
                cut += max(top - capacity, 0) + (256 << 20)
                planned = plan_at_budget(self.fam, cfg, budget - cut, self.hw, recompute=recompute, measured=measured,
                                         leeway_bytes=leeway_bytes, lower_kwargs=lower_kwargs)
                ids_old = {(o.id, o.size_bytes) for o in self.program.initial_objects}
                if {(o.id, o.size_bytes) for o in planned.program.initial_objects} != ids_old:
                    if self.verbose:
                        print("static placement not used: the replanned program has other persistent objects")
                    return
                self.planned, self.program = planned, planned.program

    def init_model(self, seed: int = 0) -> None:
        """Seeded initial parameters and optimizer state.  ``hyper["init_policy"]`` (``blocks/init_policy.py``: rules by field name
        and layer, as data) overrides the fills the layouts name."""
        from ..blocks.init_policy import init_scope
        with init_scope(self.hyper.get("init_policy")):
            if self.zero:
                from ..parallel.zero import zero_initial_values
                zero_initial_values(self.fam, self.cfg, self.program, self.store, seed, self.layouts,
                                    int(self.zero["rank"]), int(self.zero["world"]), int(self.zero["stage"]))
            else:
                # a tensor-parallel family cuts the same seeded full model differently on every rank
                sliced = next((self.groups[k] for k in ("tp", "ep") if k in self.groups), None)
                kw = {"rank": sliced.rank} if sliced is not None else {}
                self.fam.initial_values(self.program, self.cfg, self.views_of, seed, layouts=self.layouts, **kw)

    # -- data
    def put_round(self, r: int, tokens, targets) -> int:
        """Copy one round's int32 ids into the store; returns the bytes written."""
        import torch
        n = int(tokens.numel())
        tk = self.host_tensor(f"tokens_0_{r}", (self.T,), "int32")
        tg = self.host_tensor(f"targets_0_{r}", (self.T,), "int32")
        tk[:n].copy_(tokens.reshape(-1).to(torch.int32))
        tg[:n].copy_(targets.reshape(-1).to(torch.int32))
        if n < self.T:
            tk[n:].zero_()
            tg[n:].fill_(-1)
        return 2 * 4 * n

    def step(self, rounds_data=None, *, seq_lens: Mapping[int, list[int]] | None = None,
             valid_rows: int | None = None, extra_args: Mapping[str, Any] | None = None) -> float:
        """One optimizer step.  ``rounds_data``: list of (tokens, targets) per round (already in the
        store if ``None``).  Returns the step loss."""
        if rounds_data is not None:
            for r, (tk, tg) in enumerate(rounds_data):
                self.put_round(r, tk, tg)
        self.step_index += 1
        if valid_rows is None:
            valid_rows = self.T * self.rounds
        args = {"step": self.step_index, "valid_rows": int(valid_rows), **dict(extra_args or {})}
        if seq_lens:
            args["seq_lens"] = dict(seq_lens)
        res = self.engine.execute(self.program, self.resolver, self.store.buffers(), run_args=args,
                                  groups=self.groups, manage_pools=self.device is None,
                                  keep_resident=self.keep_resident,
                                  dispatch_ahead=self.dispatch_ahead, placement=self.placement)
        self.last_result = res
        res.raise_if_failed()
        for g in self.groups.values():
            if hasattr(g, "check"):
                g.check()
        loss = 0.0
        for k in self.loss_ids:
            loss += float(self.host_tensor(k, (1,), "fp32")[0])
        return loss

    def sync_to_host(self) -> int:
        """Copy every device-resident persistent object back into the host store (its host bytes go stale
        while it lives on the device between steps).  Call before reading weights from the store, e.g. to
        checkpoint.  Returns the bytes copied."""
        held = self.session.resident()
        if not held:
            return 0
        n = 0
        if self.device is None:
            import ctypes
            for oid, (ptr, size) in held.items():
                ctypes.memmove(self.store.buffer(oid).ptr, ptr, size)
                n += size
            return n
        import torch
        from ..runtime.interop import torch_view
        from ..runtime.executable import Buffer
        self.backend.synchronize()
        for oid, (ptr, size) in held.items():
            src = torch_view(Buffer(ptr, size, "fast", oid), (size,), "uint8", 0, self.device)
            torch_view(self.store.buffer(oid), (size,), "uint8", 0, None).copy_(src)
            n += size
        torch.cuda.synchronize(self.device)
        return n

    def close(self):
        self.backend.synchronize()
        self.session.drop_resident()
        for g in self.groups.values():
            if hasattr(g, "close"):
                g.close()
        from ..runtime.interop import invalidate_views
        invalidate_views()
        self.store.close()


def synthetic_rounds(cfg, rounds: int, tokens_per_round: int, vocab: int, seed: int = 0, step: int = 0, pin: bool = False):
    """Uniform random token ids with next-token targets (the data of every benchmark config)."""
    import torch
    g = torch.Generator().manual_seed(seed * 1000003 + step)
    out = []
    for _ in range(rounds):
        ids = torch.randint(0, vocab, (tokens_per_round + 1,), generator=g, dtype=torch.int64).to(torch.int32)
        tk, tg = ids[:-1].clone(), ids[1:].clone()
        if pin and torch.cuda.is_available():
            tk, tg = tk.pin_memory(), tg.pin_memory()
        out.append((tk, tg))
    return out


def run_engine(family: str, cfg, steps: int, *, budget_gib=None, device=0, hyper=None, seed=0, data_seed=0,
               verbose=True, **kw) -> RunResult:
    tr = Trainer(family, cfg, budget_gib=budget_gib, device=device, hyper=hyper, seed=seed, **kw)
    res = RunResult(tokens_per_step=tr.T * tr.rounds, meta={"family": family, "preset": getattr(cfg, "name", ""),
                                                            "plan_makespan_us": tr.planned.makespan_us,
                                                            "peak_fast_bytes": tr.planned.peak_fast_bytes})
    vocab = getattr(cfg, "vocab_size")
    try:
        for s in range(steps):
            data = synthetic_rounds(cfg, tr.rounds, tr.T, vocab, data_seed, s)
            t0 = time.time()
            loss = tr.step(data)
            dt = time.time() - t0
            res.losses.append(loss)
            res.step_wall_s.append(dt)
            if verbose:
                print(f"step {s + 1:4d} loss {loss:.4f} {res.tokens_per_step / dt:,.0f} tok/s", flush=True)
    finally:
        tr.close()
    return res
