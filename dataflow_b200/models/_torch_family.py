"""Families whose blocks are written once, as a differentiable torch function.

A family gives, per *kind* of layer, its weight fields and ``block_fn(dims, kind, x, w, seg, layer) -> (y, aux)``
in plain torch.  From that this module derives everything the framework needs: packed layouts per kind, the lowering
(several kinds of layers in one program), forward and backward executables, seeded initial values, and the pure-torch
twin.  The backward executable re-runs the block function on the saved input under autograd and takes the
vector-Jacobian products (nothing but the block input is kept between forward and backward, so no recompute tasks
exist for these families); ``aux`` is an auxiliary loss whose gradient is injected there (router balance, indexer KL).

This is the *reference-form lane* of the newer architectures (multi-head latent attention, sparse attention with a
learned indexer, gated delta-rule linear attention): they lower, plan, run on the engine on either backend and train
against their twins; hand-written sm_100a kernels for their inner ops can replace pieces of ``block_fn`` one at a time.
Reference role: the per-family ``blocks.py`` / ``model.py`` pairs of ``src/dataflow_training/model_families/{dsv3,dsv32,
qwen35,qwen35moe}/``, whose forms (``blocks/modules/mla_forms.py``, ``dsa_forms.py``, ``blocks/ops.py:509-623``) these
block functions restate.
"""
from __future__ import annotations

from ..blocks.init_policy import set_init_layer

import dataclasses
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Sequence

from ..blocks.base_blocks import OptimizerStep, _Base, common_executables
from ..blocks.layouts import DTypePolicy, Field, PackedLayout, grad_layout, opt_state_layout, weight_layout
from ..lowering.shaped_program import (LayerKindSpec, LooseCosts, ShapedConfig, ShapedHardware, build_shaped_program, optimizer_cost_seed,
                                       resolve_hardware)
from .families import ModelFamily, register_family


@dataclass(frozen=True)
class TorchDims:
    """What the shared executables (embedding, head + loss, optimizer) need, plus the family's own numbers in ``x``."""
    n_layers: int
    d: int
    vocab: int
    T: int
    seq_len: int
    head_chunk: int
    eps: float = 1e-6
    theta: float = 10000.0
    x: Any = None                      # the family's config (dims the block function reads)
    kinds: tuple[str, ...] = ()        # kind of every layer


@dataclass(frozen=True)
class TorchFamilySpec:
    name: str
    config_type: type
    presets: Mapping[str, Callable[[], Any]]
    layer_kinds: Callable[[Any], Sequence[str]]                        # cfg -> kind of every layer
    kind_fields: Callable[[Any, str], Sequence[Field]]                  # (cfg, kind) -> weight fields
    block_fn: Callable[..., Any]                                        # (cfg, kind, x, w, seg, layer) -> (y, aux | None)
    kind_flops: Callable[[Any, str, int], tuple[float, float]]          # (cfg, kind, tokens) -> (matmul, attention) forward FLOPs
    doc: str = ""
    # cross-layer sharing: a *leader* layer's block function returns a third value, a dict of tensors that is stored in
    # its context object ``A`` (fields from ``ctx_fields``); a *follower* (``leader_of(cfg, layer)`` names its leader)
    # gets that dict as the ``shared`` argument of its block function, forward and backward
    ctx_fields: Callable[[Any, int], Sequence[Field]] | None = None     # (cfg, tokens) -> fields of A
    leader_of: Callable[[Any, int], int | None] | None = None
    # backward-time accumulation inside a group: a follower's block function may return, under the key ``"_deposit"`` of
    # its third value, a dict of tensors (fields from ``accum_fields``); the followers' BACKWARD tasks sum them into the
    # group's accumulator object ``G_{step}_{round}_{leader}`` (created by the first backward of the group to run,
    # mutated by the others), and the leader's backward passes the sums to its block function as ``accum`` together with
    # ``group_size`` (members of the group, the leader included)
    accum_fields: Callable[[Any, int], Sequence[Field]] | None = None   # (cfg, tokens) -> fields of G
    # expert parallelism (``cfg.ep`` > 1): these fields carry the expert axis first and hold this rank's E / ep experts;
    # the block function then receives the group as ``ep`` and routes through ``_forms.moe_mlp_ep``.  Everything else is
    # replicated and fed different data per rank: its gradients are summed over the group in front of the optimizer
    ep_fields: tuple[str, ...] = ()


CTX = PackedLayout((Field("stamp", (4,), "fp32"),))


@dataclass(frozen=True)
class MultiKindLayouts:
    dims: Any
    policy: DTypePolicy
    by_kind: Mapping[str, tuple[PackedLayout, PackedLayout, PackedLayout]]
    embed_w: PackedLayout
    embed_dw: PackedLayout
    embed_o: PackedLayout
    head_w: PackedLayout
    head_dw: PackedLayout
    head_o: PackedLayout
    ctx: PackedLayout = CTX
    extra: Mapping[str, PackedLayout] = field(default_factory=dict)

    def of_layer(self, layer: int):
        return self.by_kind[self.dims.kinds[int(layer)]]

    @property
    def block_w(self):
        return self.of_layer(0)[0]

    @property
    def block_dw(self):
        return self.of_layer(0)[1]

    @property
    def block_o(self):
        return self.of_layer(0)[2]

    def layout_of(self, oid: str):
        fixed = {"W_embed": self.embed_w, "O_embed": self.embed_o, "W_head": self.head_w, "O_head": self.head_o}
        if oid in fixed:
            return fixed[oid]
        if oid.startswith("dW_embed"):
            return self.embed_dw
        if oid.startswith("dW_head"):
            return self.head_dw
        tail = oid.rsplit("_", 1)[-1]
        if tail.isdigit() and int(tail) < len(self.dims.kinds):
            if oid.startswith("dW_"):
                return self.of_layer(int(tail))[1]
            if oid.startswith("W_"):
                return self.of_layer(int(tail))[0]
            if oid.startswith("O_"):
                return self.of_layer(int(tail))[2]
        if oid.startswith("A_"):
            return self.ctx
        if oid.startswith("G_"):
            return self.extra.get("accum")
        return None

    def object_layouts(self, program):
        out = {}
        for oid in program.object_sizes():
            lay = self.layout_of(oid)
            if lay is not None:
                out[oid] = lay
        return out


def embed_fields(d: TorchDims):
    return (Field("wte", (d.vocab, d.d), "bf16", "embedding", "normal"),)


def head_fields(d: TorchDims):
    return (Field("final_norm", (d.d,), "bf16", "vector", "ones"), Field("w_head", (d.d, d.vocab), "bf16", "matrix", "normal"))


def _segments_bounds(seg):
    cu = seg.cu_seqlens
    return [int(v) for v in (cu.tolist() if hasattr(cu, "tolist") else cu)]


# ------------------------------------------------------------------------------------------------- executables
class _TorchBlock(_Base):
    spec: TorchFamilySpec = None

    def weights(self, buf, layer):
        return self.views(buf, self.lay.of_layer(layer)[0])

    def compute_dtype(self):
        import torch
        return torch.float32 if self.device is None else torch.bfloat16

    def shared_from_leader(self, ctx, layer, n):
        spec = self.spec
        if spec.leader_of is None:
            return None
        leader = spec.leader_of(self.dims.x, layer)
        if leader is None:
            return None
        r = int(ctx.task.block_params.get("round", 0))
        for b in ctx.inputs:
            if b.object_id.startswith("A_") and b.object_id.endswith(f"_{r}_{leader}"):
                return {k: v[:n] for k, v in self.views(b, self.lay.ctx).items() if k != "stamp"}
        raise RuntimeError(f"task {ctx.task.id}: the context of leader layer {leader} is not among the inputs")

    def followers_of(self, layer):
        spec, d = self.spec, self.dims
        if spec.leader_of is None:
            return []
        return [i for i in range(d.n_layers) if spec.leader_of(d.x, i) == layer]

    def call(self, ctx, x, w, layer, grad: bool, **extra):
        import torch
        d = self.dims
        seg = self.segments(ctx)
        cdt = self.compute_dtype()
        xin = x.to(cdt)
        wl = {k: v.to(cdt) for k, v in w.items()}
        if grad:
            xin = xin.detach().requires_grad_(True)
            wl = {k: v.detach().requires_grad_(True) for k, v in wl.items()}
        shared = self.shared_from_leader(ctx, layer, x.shape[0])
        if int(getattr(d.x, "ep", 1) or 1) > 1:
            grp = ctx.groups.get(ctx.task.comm_groups.get("ep", "ep"))
            if grp is None:
                raise RuntimeError(f"task {ctx.task.id} needs the group 'ep' (pass groups={{'ep': ...}})")
            if x.shape[0] != d.T:
                raise ValueError("expert-parallel blocks need full rounds (the peers exchange exactly T rows with each rank)")
            extra = dict(extra, ep=grp)
        with torch.set_grad_enabled(grad):
            res = self.spec.block_fn(d.x, d.kinds[layer], xin, wl, seg, layer, **({"shared": shared} if shared is not None else {}), **extra)
        self.emitted = res[2] if len(res) > 2 else None
        return xin, wl, res[0], res[1]


class TorchBlockFwd(_TorchBlock):
    """(x, W) -> (y, A): A is a stamp; the backward re-runs the block from x."""

    def run(self, ctx):
        d = self.dims
        layer = int(ctx.task.block_params["layer"])
        n = self.segments(ctx).n_tokens
        x = self.tview(ctx.inputs[0], (d.T, d.d))[:n]
        y = self.tview(ctx.outputs[0], (d.T, d.d))[:n]
        _, _, out, _ = self.call(ctx, x, self.weights(ctx.inputs[1], layer), layer, False)
        y.copy_(out.to(y.dtype))
        a = self.views(ctx.outputs[1], self.lay.ctx)
        a["stamp"].zero_()
        for k, v in (self.emitted or {}).items():
            if not k.startswith("_"):
                a[k][:n].copy_(v)


class TorchBlockBwd(_TorchBlock):
    """(dy, A, x, W[, dW]) -> (dx[, dW]) by autograd through the block function."""

    def run(self, ctx):
        import torch
        d = self.dims
        layer = int(ctx.task.block_params["layer"])
        n = self.segments(ctx).n_tokens
        dy = self.tview(ctx.inputs[0], (d.T, d.d))[:n]
        x = self.tview(ctx.inputs[2], (d.T, d.d))[:n]
        dx = self.tview(ctx.outputs[0], (d.T, d.d))[:n]
        acc = not self.creating(ctx, "dW_")
        g = self.views(self.by_id(ctx, "dW_"), self.lay.of_layer(layer)[1])
        extra = {}
        gbuf = self.by_id(ctx, "G_")
        if gbuf is not None and self.spec.leader_of(d.x, layer) is None:      # the leader consumes the group's sums
            extra = {"accum": {k: v[:n] for k, v in self.views(gbuf, self.lay.extra["accum"]).items()},
                     "group_size": 1 + len(self.followers_of(layer))}
        xin, wl, y, aux = self.call(ctx, x, self.weights(ctx.inputs[3], layer), layer, True, **extra)
        if gbuf is not None and not extra:                                     # a follower adds its share
            dep = (self.emitted or {}).get("_deposit") or {}
            create = self.creating(ctx, "G_")
            for k, v in self.views(gbuf, self.lay.extra["accum"]).items():
                if create:
                    v.zero_()
                if k in dep:
                    v[:n].add_(dep[k].detach().to(v.dtype))
        total = (y * dy.to(y.dtype)).sum()
        if aux is not None:
            # the auxiliary loss enters every round with the weight the main loss has: 1 / (rows of the whole step)
            total = total + aux * (float(n) / float(ctx.run_args.get("valid_rows", n)))
        names = [k for k in wl if k in g]
        grads = torch.autograd.grad(total, [xin] + [wl[k] for k in names], allow_unused=True)
        dx.copy_(grads[0].to(dx.dtype))
        for k, gv in zip(names, grads[1:]):
            if gv is None:
                if not acc:
                    g[k].zero_()
                continue
            if acc:
                g[k].add_(gv.to(g[k].dtype))
            else:
                g[k].copy_(gv.to(g[k].dtype))


class KindOptimizerStep(OptimizerStep):
    def layouts_for(self, ctx):
        if ctx.task.block_params.get("target", "block") == "block" and "layer" in ctx.task.block_params:
            return self.lay.of_layer(int(ctx.task.block_params["layer"]))
        return super().layouts_for(ctx)


class _KindGradSum:
    """Block optimizer under expert parallelism: the gradients of the replicated fields of the task's layer (all but the
    expert stacks) are summed over the job first."""

    def __init__(self, inner, lay, skip):
        self.inner, self.lay, self.skip = inner, lay, tuple(skip)

    def __getattr__(self, name):
        return getattr(self.__dict__["inner"], name)        # layout helpers and device of the wrapped executable

    def _summed(self, ctx):
        from .tp_mlp.blocks import ReplicatedGradSum
        gl = self.lay.of_layer(int(ctx.task.block_params.get("layer", 0)))[1]
        return ReplicatedGradSum(self.inner, gl, None, "ep", skip=self.skip)

    def launch(self, ctx):
        self._summed(ctx).launch(ctx)

    def run(self, ctx):
        self._summed(ctx).run(ctx)


# ------------------------------------------------------------------------------------------------- twin
def make_twin(spec: TorchFamilySpec, cfg):
    import torch

    class Twin(torch.nn.Module):
        def __init__(self):
            super().__init__()
            d = derive(spec, cfg)
            self.d = d
            self.wte = torch.nn.Parameter(torch.zeros(d.vocab, d.d))
            self.final_norm = torch.nn.Parameter(torch.ones(d.d))
            self.w_head = torch.nn.Parameter(torch.zeros(d.d, d.vocab))
            self.layers = torch.nn.ModuleList()
            for i, kind in enumerate(d.kinds):
                m = torch.nn.Module()
                for f in spec.kind_fields(cfg, kind):
                    m.register_parameter(f.name, torch.nn.Parameter(torch.zeros(tuple(f.shape))))
                self.layers.append(m)

        def run_layers(self, tokens, n, seg, sums, collect):
            d = self.d
            x = self.wte[tokens[:n]]
            aux_total = 0.0
            emitted = {}
            for i, m in enumerate(self.layers):
                w = dict(m.named_parameters())
                leader = spec.leader_of(cfg, i) if spec.leader_of else None
                kw = {"shared": emitted[leader]} if leader is not None else {}
                if leader is None and i in sums:
                    kw.update(accum=sums[i], group_size=1 + sum(1 for j in range(d.n_layers) if spec.leader_of(cfg, j) == i))
                res = spec.block_fn(cfg, d.kinds[i], x, w, seg, i, **kw)
                x, aux = res[0], res[1]
                if len(res) > 2 and res[2]:
                    emitted[i] = res[2]
                    dep = res[2].get("_deposit")
                    if collect is not None and dep and leader is not None:
                        tgt = collect.setdefault(leader, {})
                        for k, v in dep.items():
                            tgt[k] = tgt[k] + v if k in tgt else v.clone()
                if aux is not None:
                    aux_total = aux_total + aux
            return x, aux_total

        def loss(self, tokens, targets, bounds, total_rows=None):
            from ..data.segments import make_segments
            d = self.d
            tokens, targets = torch.as_tensor(tokens).long(), torch.as_tensor(targets).long()
            n = int(bounds[-1])
            seg = make_segments(list(bounds), None)
            sums = {}
            if spec.accum_fields is not None:
                # what the followers deposit is a detached function of the forward values: collect it in a first pass
                with torch.no_grad():
                    self.run_layers(tokens, n, seg, {}, sums)
            x, aux_total = self.run_layers(tokens, n, seg, sums, None)
            xn = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + d.eps) * self.final_norm
            logits = xn @ self.w_head
            tg = targets[:n]
            valid = tg >= 0
            nll = torch.nn.functional.cross_entropy(logits[valid], tg[valid], reduction="sum")
            rows = float(total_rows) if total_rows else float(valid.sum())
            self.last_aux = aux_total
            main = nll / rows
            if isinstance(aux_total, float):
                return main
            term = aux_total * (n / rows)
            return main + (term - term.detach())          # the auxiliary loss steers gradients; the reported loss is the CE

    return Twin()


def bridge(spec: TorchFamilySpec, cfg, views_of):
    d = derive(spec, cfg)
    lay = layouts(spec, d, cfg.policy() if hasattr(cfg, "policy") else None, getattr(cfg, "optimizer", "adamw"))
    sd = {"wte": views_of("W_embed", lay.embed_w)["wte"].float().clone()}
    hv = views_of("W_head", lay.head_w)
    sd["final_norm"], sd["w_head"] = hv["final_norm"].float().clone(), hv["w_head"].float().clone()
    for i in range(d.n_layers):
        for name, t in views_of(f"W_{i}", lay.of_layer(i)[0]).items():
            sd[f"layers.{i}.{name}"] = t.float().clone()
    return sd


# ------------------------------------------------------------------------------------------------- derivations
def derive(spec: TorchFamilySpec, cfg) -> TorchDims:
    T = int(cfg.seq_len) * int(cfg.batch)
    return TorchDims(int(cfg.n_layers), int(cfg.d_model), int(cfg.vocab_size), T, int(cfg.seq_len),
                     min(int(getattr(cfg, "head_chunk_tokens", 2048)), T), float(getattr(cfg, "rms_eps", 1e-6)),
                     float(getattr(cfg, "rope_theta", 10000.0)), cfg, tuple(spec.layer_kinds(cfg)))


def layouts(spec: TorchFamilySpec, d: TorchDims, policy=None, optimizer: str = "adamw") -> MultiKindLayouts:
    policy = policy or DTypePolicy.named("bf16")
    rule = lambda f: optimizer  # noqa: E731
    by_kind = {}
    for kind in dict.fromkeys(d.kinds):
        f = tuple(spec.kind_fields(d.x, kind))
        by_kind[kind] = (weight_layout(f, policy), grad_layout(f, policy), opt_state_layout(f, policy, rule_of=rule))
    ef, hf = embed_fields(d), head_fields(d)
    ctx = CTX if spec.ctx_fields is None else PackedLayout(tuple(CTX.fields) + tuple(spec.ctx_fields(d.x, d.T)))
    extra = {} if spec.accum_fields is None else {"accum": PackedLayout(tuple(spec.accum_fields(d.x, d.T)))}
    return MultiKindLayouts(d, policy, by_kind, weight_layout(ef, policy), grad_layout(ef, policy), opt_state_layout(ef, policy, rule_of=rule),
                            weight_layout(hf, policy), grad_layout(hf, policy), opt_state_layout(hf, policy, rule_of=rule), ctx, extra)


def _subop(name, flops=0.0, nbytes=0.0, eff="matmul"):
    return {"name": name, "flops": float(flops), "memory_bytes": float(nbytes), "efficiency": eff, "dtype": "bf16"}


def lower(spec: TorchFamilySpec, cfg, recompute_levels=None, hw: ShapedHardware | None = None, block_params=None, comm_groups=None,
          zero=None, resident_params: bool = False):
    hw = hw or resolve_hardware("b200")
    d = derive(spec, cfg)
    lay = layouts(spec, d, cfg.policy() if hasattr(cfg, "policy") else None, getattr(cfg, "optimizer", "adamw"))
    kinds = {}
    for kind, (wl, gl, ol) in lay.by_kind.items():
        mm, at = spec.kind_flops(cfg, kind, d.T)
        ew = 12.0 * d.T * d.d * 2
        fwd = hw.matmul_us(mm) + hw.attn_us(at) + hw.mem_us(ew)
        # the backward re-runs the forward, then differentiates it
        bwd = fwd + hw.matmul_us(2 * mm) + hw.attn_us(2.5 * at, True) + hw.mem_us(2.5 * ew)
        fs = (_subop("gemms", mm), _subop("attention", at, eff="attention"), _subop("elementwise", nbytes=ew, eff="memory"))
        bs = (_subop("gemms", 3 * mm), _subop("attention", 3.5 * at, eff="attention_bwd"), _subop("elementwise", nbytes=3.5 * ew, eff="memory"))
        ws = int(d.T * d.d * 2 * 24)
        kinds[kind] = LayerKindSpec(kind, wl.size_bytes, gl.size_bytes, ol.size_bytes, lay.ctx.size_bytes, fwd, bwd, fwd,
                                    optimizer_cost_seed(hw, wl.size_bytes, gl.size_bytes, ol.size_bytes, getattr(cfg, "optimizer", "adamw")),
                                    fs, bs, fs, (_subop("optimizer", nbytes=2 * wl.size_bytes + gl.size_bytes + 2 * ol.size_bytes, eff="memory"),),
                                    ws, 2 * ws, 0)
    head_gemm = 2.0 * d.T * d.d * d.vocab
    loose = LooseCosts(hw.mem_us(2.0 * d.T * d.d * 2) + 5, hw.mem_us(4.0 * d.T * d.d * 2) + 30,
                       hw.matmul_us(3 * head_gemm) + hw.mem_us(3.0 * d.T * d.vocab * 2), 2.0,
                       (_subop("head_gemms", 3 * head_gemm), _subop("ce", nbytes=3.0 * d.T * d.vocab * 2, eff="memory")),
                       d.head_chunk * d.vocab * 2 + d.head_chunk * d.d * 4 + (1 << 20))
    sc = ShapedConfig(cfg.name, d.n_layers, d.T, int(cfg.grad_accum_rounds), d.d, 2, getattr(cfg, "optimizer_placement", "interleaved"))
    total_mm = sum(spec.kind_flops(cfg, k, 1)[0] + spec.kind_flops(cfg, k, 1)[1] for k in d.kinds)
    prog = build_shaped_program(
        sc, kinds, list(d.kinds),
        embed_w_bytes=lay.embed_w.size_bytes, embed_dw_bytes=lay.embed_dw.size_bytes, embed_o_bytes=lay.embed_o.size_bytes,
        head_w_bytes=lay.head_w.size_bytes, head_dw_bytes=lay.head_dw.size_bytes, head_o_bytes=lay.head_o.size_bytes,
        loose=loose, hw=hw, recompute_levels=None, block_params=block_params,
        comm_groups=({"ep": "ep", **dict(comm_groups or {})} if int(getattr(cfg, "ep", 1) or 1) > 1 else comm_groups), zero=zero,
        resident_params=resident_params,
        metadata={"family": spec.name, "preset": cfg.name, "flops_per_token": 3.0 * (total_mm + 2.0 * d.d * d.vocab),
                  "seq_len": cfg.seq_len, "batch": cfg.batch, "block_lane": "autograd", "ep": int(getattr(cfg, "ep", 1) or 1)})
    return share_leader_contexts(spec, cfg, prog, lay.extra["accum"].size_bytes if "accum" in lay.extra else 0)


def share_leader_contexts(spec: TorchFamilySpec, cfg, prog, accum_bytes: int = 0):
    """Lowering post-pass: forward and backward tasks of a follower layer also read the context object of their leader
    (same step, same round), which keeps it alive until the last follower's backward has run.  With ``accum_bytes``
    every group that has followers also gets its accumulator ``G_{step}_{round}_{leader}``: the backward of the group's
    last layer (the first to run) creates it, the other followers' backwards mutate it, the leader's backward reads it."""
    if spec.leader_of is None:
        return prog
    from ..core.program import OutputSpec
    n_layers = int(cfg.n_layers)
    last_member = {}
    for i in range(n_layers):
        lead = spec.leader_of(cfg, i)
        if lead is not None:
            last_member[lead] = i
    tasks = []
    for t in prog.tasks:
        layer, key = t.block_params.get("layer") if t.block_params else None, t.compute_block_key or ""
        if layer is None or not key.endswith(("_fwd", "_bwd")):
            tasks.append(t)
            continue
        layer = int(layer)
        leader = spec.leader_of(cfg, layer)
        own = next(o for o in (list(t.inputs) + [x.id for x in t.outputs]) if o.startswith("A_"))
        stem = own.rsplit("_", 1)[0]
        if leader is None:
            if accum_bytes and key.endswith("_bwd") and layer in last_member:
                t = dataclasses.replace(t, inputs=tuple(t.inputs) + ("G" + stem[1:] + f"_{layer}",))
            tasks.append(t)
            continue
        t = dataclasses.replace(t, inputs=tuple(t.inputs) + (stem + f"_{leader}",))
        if accum_bytes and key.endswith("_bwd"):
            gid = "G" + stem[1:] + f"_{leader}"
            if layer == last_member[leader]:
                t = dataclasses.replace(t, outputs=tuple(t.outputs) + (OutputSpec(gid, int(accum_bytes)),))
            else:
                t = dataclasses.replace(t, inputs=tuple(t.inputs) + (gid,), mutates=tuple(t.mutates) + (gid,))
        tasks.append(t)
    return dataclasses.replace(prog, tasks=tuple(tasks))


def initial_values(spec: TorchFamilySpec, program, cfg, views_of, seed: int = 0, layouts_=None, rank: int = 0) -> None:
    """Seeded initial values.  Under expert parallelism every rank draws the FULL expert stacks from the generator (so the
    same seed gives the same model at every world size) and keeps the experts it owns (``rank``)."""
    import torch
    from .llama3.model import init_field
    d = derive(spec, cfg)
    lay = layouts_ or layouts(spec, d, cfg.policy() if hasattr(cfg, "policy") else None, getattr(cfg, "optimizer", "adamw"))
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    ep = int(getattr(cfg, "ep", 1) or 1)
    ids = {o.id for o in program.initial_objects}
    for oid in ["W_embed"] + [f"W_{i}" for i in range(d.n_layers)] + ["W_head"]:
        if oid not in ids:
            continue
        set_init_layer(oid)
        wl = lay.layout_of(oid)
        wv = views_of(oid, wl)
        for f in wl.fields:
            if ep > 1 and f.name in spec.ep_fields:
                full = torch.empty((f.shape[0] * ep,) + tuple(f.shape[1:]), dtype=torch.float32)
                init_field(full, f, gen, d.n_layers)
                wv[f.name].copy_(full[rank * f.shape[0]:(rank + 1) * f.shape[0]])
            else:
                init_field(wv[f.name], f, gen, d.n_layers)
        oname = "O" + oid[1:]
        if oname in ids:
            ov = views_of(oname, lay.layout_of(oname))
            for name, t in ov.items():
                if name.endswith(".master"):
                    t.copy_(wv[name[:-7]].float())
                else:
                    t.zero_()


def build_resolver(spec: TorchFamilySpec, dims, hyper, kernels, device, layouts_=None, policy=None):
    hyper = dict(hyper or {})
    lay = layouts_ or layouts(spec, dims, policy or DTypePolicy.from_dict(hyper.get("dtype_policy", "bf16")), hyper.get("optimizer", "adamw"))
    table = common_executables(dims, lay, kernels, device, hyper)
    table["optimizer_block"] = KindOptimizerStep(dims, lay, kernels, device, hyper)
    fwd, bwd = TorchBlockFwd(dims, lay, kernels, device, hyper), TorchBlockBwd(dims, lay, kernels, device, hyper)
    fwd.spec = bwd.spec = spec
    for kind in dict.fromkeys(dims.kinds):
        table[f"{kind}_fwd"], table[f"{kind}_bwd"] = fwd, bwd
    if int(getattr(dims.x, "ep", 1) or 1) > 1:
        from .tp_mlp.blocks import ReplicatedGradSum
        table["optimizer_block"] = _KindGradSum(table["optimizer_block"], lay, spec.ep_fields)
        table["optimizer_embed"] = ReplicatedGradSum(table["optimizer_embed"], lay.embed_dw, None, "ep")
        table["optimizer_head"] = ReplicatedGradSum(table["optimizer_head"], lay.head_dw, None, "ep")

    def resolver(task):
        try:
            return table[task.compute_block_key]
        except KeyError:
            raise KeyError(f"{spec.name}: no executable for compute key {task.compute_block_key!r} (task {task.id})") from None
    resolver.table = table
    return resolver


def register_torch_family(spec: TorchFamilySpec) -> ModelFamily:
    return register_family(ModelFamily(
        name=spec.name, config_type=spec.config_type, derive_dims=lambda cfg: derive(spec, cfg),
        lower=lambda cfg, **kw: lower(spec, cfg, **kw),
        initial_values=lambda program, cfg, views_of, seed=0, layouts=None, rank=0: initial_values(spec, program, cfg, views_of, seed, layouts,
                                                                                                   rank),
        build_resolver=lambda dims, hyper, kernels, device, layouts=None, policy=None: build_resolver(spec, dims, hyper, kernels, device, layouts, policy),
        family_layouts=lambda dims, policy=None, optimizer="adamw": layouts(spec, dims, policy, optimizer),
        presets=dict(spec.presets), twin=lambda cfg: make_twin(spec, cfg), bridge=lambda cfg, views_of: bridge(spec, cfg, views_of),
        block_kinds=tuple(dict.fromkeys(k for p in spec.presets.values() for k in spec.layer_kinds(p()))), flops_per_token=None))
