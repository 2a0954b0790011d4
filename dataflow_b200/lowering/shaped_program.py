"""Chain grammar: (layer kinds, training geometry) → bare Dataflow Program for ONE optimizer step.

Per grad-accumulation round ``r``::

    prologue_round  embed_fwd  L x {kind}_fwd  head_loss  L x [ {kind}_recompute ] {kind}_bwd (reverse)  embed_bwd

with one ``optimizer_*`` task per layer (+ embed, head) placed right after the
last mutation of that layer's gradient in the last round ("interleaved") or
after everything ("tail").  Round 0 *creates* ``dW`` objects (task outputs), later
rounds *mutate* them.  Object and task ids follow the reference's naming
grammar so tools and checkpoints interoperate
(``src/dataflow_training/lowering/shaped_program.py:354-785``, README naming table).
Costs are roofline seeds from ``ShapedHardware`` and are replaced by measured
task profiles before planning when available.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Mapping, Sequence

from ..core import (ObjectSpec, OutputSpec, Program, RecomputeOption, RecomputeRewrite, TaskSpec)


# --------------------------------------------------------------------------- hardware
@dataclass(frozen=True)
class ShapedHardware:
    name: str
    peak_tflops: float                 # dense bf16
    matmul_eff: float = 0.75
    attn_fwd_eff: float = 0.45
    attn_bwd_eff: float = 0.35
    hbm_gbs: float = 3000.0
    mem_eff: float = 0.85
    h2d_gbs: float = 50.0
    d2h_gbs: float = 50.0
    scale_up_gbs: float = 0.0          # per-direction NVLink bandwidth per GPU
    fast_gib: float = 80.0
    peak_tflops_fp8: float = 0.0
    host_gbs: float = 0.0              # host-memory bandwidth per direction shared by all GPUs of a node (0 = unknown)
    link_gbs: float = 0.0              # what one GPU's host link does alone (set where h2d / d2h were lowered to a share)

    def shared(self, ranks_per_node: int) -> "ShapedHardware":
        """The preset as one of ``ranks_per_node`` GPUs sees it: the copy lanes of all GPUs of a node end in the
        same host memory, so each gets at most its share of the host bandwidth."""
        if ranks_per_node <= 1 or not self.host_gbs:
            return self
        share = self.host_gbs / ranks_per_node
        return replace(self, h2d_gbs=min(self.h2d_gbs, share), d2h_gbs=min(self.d2h_gbs, share), link_gbs=self.link_gbs or self.h2d_gbs)

    def matmul_us(self, flops: float, dtype: str = "bf16") -> float:
        peak = self.peak_tflops_fp8 if dtype.startswith("fp8") and self.peak_tflops_fp8 else self.peak_tflops
        return flops / (peak * 1e12 * self.matmul_eff) * 1e6

    def attn_us(self, flops: float, backward: bool = False) -> float:
        eff = self.attn_bwd_eff if backward else self.attn_fwd_eff
        return flops / (self.peak_tflops * 1e12 * eff) * 1e6

    def mem_us(self, nbytes: float) -> float:
        return nbytes / (self.hbm_gbs * 1e9 * self.mem_eff) * 1e6

    def comm_us(self, nbytes: float) -> float:
        return nbytes / (max(self.scale_up_gbs, 1e-9) * 1e9) * 1e6


HW_PRESETS: dict[str, ShapedHardware] = {
    "b200": ShapedHardware("b200", 1669.0, 0.80, 0.45, 0.35, 6524.0, 0.90, 52.0, 52.0, 770.0, 180.0, 3300.0, 160.0),
    "h100": ShapedHardware("h100", 989.0, 0.72, 0.55, 0.45, 3350.0, 0.85, 52.0, 50.0, 450.0, 80.0, 1979.0),
    "rtx 5090": ShapedHardware("rtx 5090", 209.0, 0.90, 0.6, 0.5, 1792.0, 0.85, 25.0, 25.0, 0.0, 32.0),
    "rtx 3090": ShapedHardware("rtx 3090", 71.0, 0.85, 0.6, 0.5, 936.0, 0.85, 16.5, 18.7, 0.0, 24.0),
    "cpu": ShapedHardware("cpu", 1.0, 0.5, 0.5, 0.5, 100.0, 0.8, 20.0, 20.0, 0.0, 64.0),
}


def resolve_hardware(name: str | None = None) -> ShapedHardware:
    """Preset by (sub)name; ``None`` picks the current CUDA device, or ``cpu``."""
    if name is None:
        try:
            import torch
            name = torch.cuda.get_device_name(0).lower() if torch.cuda.is_available() else "cpu"
        except Exception:
            name = "cpu"
    key = name.lower()
    for k, hw in HW_PRESETS.items():
        if k in key or key in k:
            return hw
    raise KeyError(f"no hardware preset matches {name!r}; known: {sorted(HW_PRESETS)}")


# --------------------------------------------------------------------------- kind specs
@dataclass(frozen=True)
class LooseCosts:
    """Cost seeds of the non-layer tasks (µs) and their sub-op breakdowns."""
    embed_fwd_us: float = 10.0
    embed_bwd_us: float = 20.0
    head_loss_us: float = 100.0
    prologue_us: float = 1.0
    head_subops: tuple = ()
    head_workspace: int = 0


@dataclass(frozen=True)
class LayerKindSpec:
    """Everything the grammar needs to know about one kind of layer."""
    kind: str
    w_bytes: int
    dw_bytes: int
    o_bytes: int
    ctx_bytes: int                        # saved context A (level 0), for ``tokens`` of one round
    fwd_us: float
    bwd_us: float
    recompute_us: float
    opt_us: float
    fwd_subops: tuple = ()
    bwd_subops: tuple = ()
    recompute_subops: tuple = ()
    opt_subops: tuple = ()
    workspace_fwd: int = 0
    workspace_bwd: int = 0
    workspace_opt: int = 0
    aux_bytes: int = 0                    # persistent per-layer counters (Aux_i)
    aux_temp_bytes: int = 0               # per-round never-recomputed metadata (AuxTemp)
    recompute_levels: tuple[tuple[int, int, float], ...] = ()   # (level, saved_bytes, recompute_us)


OPT_TRAFFIC = {"adamw": 1.0, "sgd": 0.4, "sgdm": 0.6, "muon": 1.2, "frozen": 0.0}


def optimizer_cost_seed(hw: ShapedHardware, w_bytes: int, dw_bytes: int, o_bytes: int, rule: str = "adamw") -> float:
    """Memory-bound: read W, dW, O; write W, O."""
    return hw.mem_us((2 * w_bytes + dw_bytes + 2 * o_bytes) * OPT_TRAFFIC.get(rule, 1.0)) + 5.0


@dataclass(frozen=True)
class ShapedConfig:
    """Geometry shared by every family's lowering."""
    name: str
    n_layers: int
    tokens_per_round: int
    grad_accum_rounds: int
    d_model: int
    act_dtype_bytes: int = 2
    optimizer_placement: str = "interleaved"      # interleaved | tail
    tied_embeddings: bool = False
    steps: int = 1


def _meta(subops, extra: Mapping[str, Any] | None = None) -> dict:
    m: dict[str, Any] = {}
    if subops:
        m["cost_subops"] = [dict(s) for s in subops]
    if extra:
        m.update(extra)
    return m


def build_shaped_program(cfg: ShapedConfig, kinds: Mapping[str, LayerKindSpec], layer_kinds: Sequence[str], *,
                         embed_w_bytes: int, embed_dw_bytes: int, embed_o_bytes: int,
                         head_w_bytes: int, head_dw_bytes: int, head_o_bytes: int,
                         loose: LooseCosts, hw: ShapedHardware,
                         recompute_levels: Mapping[int, int] | None = None,
                         block_params: Mapping[str, Any] | None = None,
                         comm_groups: Mapping[str, str] | None = None,
                         metadata: Mapping[str, Any] | None = None,
                         opt_embed_us: float | None = None, opt_head_us: float | None = None,
                         zero: Mapping[str, Any] | None = None,
                         resident_params: bool = False) -> Program:
    """Emit the bare program.  ``recompute_levels[i] > 0`` (all rounds) or
    ``recompute_levels[(round, i)] > 0`` (one round) makes layer ``i`` save a reduced context and
    inserts a ``{kind}_recompute`` task in front of its backward.  ``resident_params`` starts and ends every
    whole weight object on the fast tier: a session that keeps final-fast objects between runs then carries
    the parameters from step to step with no transfer (the planner may still evict them inside a step)."""
    L = cfg.n_layers
    assert len(layer_kinds) == L
    levels = dict(recompute_levels or {})
    s = 0
    T = cfg.tokens_per_round
    x_bytes = T * cfg.d_model * cfg.act_dtype_bytes
    tok_bytes = T * 4
    bp = dict(block_params or {})
    cg = dict(comm_groups or {})
    # ZeRO data parallelism: stage 3 keeps only this rank's flat slice of every weight object
    # (``Ws_*``) and of its optimizer state persistent; the full ``W_*`` is a per-step temp made by a
    # ``param_gather`` task in front of its first use.  Stage 1 keeps ``W_*`` whole and persistent and
    # shards the optimizer state only.
    zstage = int(zero.get("stage", 0)) if zero else 0
    zworld = int(zero.get("world", 1)) if zero else 1
    zfactor = float(zero.get("opt_bytes_per_param_byte", 6.0)) if zero else 0.0
    # Re-gathering (FSDP) mode of stage 3: a block's full weights are gathered in front of EVERY use and freed after
    # it, and every backward's gradient is reduce-scattered straight into this rank's fp32 slice, so neither full
    # weights nor full gradients stay resident; the optimizer then runs locally on the slice.  NVLink carries
    # 2 x rounds gathers + rounds reduce-scatters per layer instead of PCIe carrying evicted weights.
    regather = bool(zero.get("regather")) if zero else False
    # With ``comm_async`` the re-gathers and reduce-scatters run on the group's communication stream: a gather is
    # issued one layer ahead of its consumer (which waits for it on-stream), a reduce-scatter is joined one layer
    # later (``grad_rs_join``), so NVLink traffic overlaps the neighbouring layer's compute.
    comm_async = bool(zero.get("comm_async", True)) if zero else False
    zfactor_blocks = float(zero.get("block_opt_bytes_per_param_byte", zfactor)) if zero else 0.0

    def zslice(nbytes: int) -> int:
        per = (nbytes + zworld - 1) // zworld
        return (per + 255) // 256 * 256

    def zo(nbytes: int, solo_o: int, block: bool = False) -> int:
        return int(zslice(nbytes) * (zfactor_blocks if block and regather else zfactor)) if zstage else solo_o

    if zstage:
        bp["shard"] = {"stage": zstage, "rank": int(zero.get("rank", 0)), "world": zworld}
        cg.setdefault("dp", zero.get("group", "dp"))
    gathered: dict[str, int] = {}        # W object id -> full byte size (stage 3)
    init: list[ObjectSpec] = []
    resident_ids: set[str] = set()

    def param_objects(name: str, w_bytes: int, o_bytes: int) -> None:
        wid, oid = f"W_{name}", f"O_{name}"
        is_block = name.isdigit()
        if zstage == 3:
            # a re-gathered block keeps its slice on the device from step to step (it is small)
            init.append(ObjectSpec(f"Ws_{name}", zslice(w_bytes), "fast" if regather and is_block and resident_params else "backing",
                                   "parameter", persistent=True))
            if regather and is_block and resident_params:
                resident_ids.add(f"Ws_{name}")
            gathered[wid] = w_bytes
        else:
            init.append(ObjectSpec(wid, w_bytes, "fast" if resident_params else "backing", "parameter", persistent=True))
            if resident_params:
                resident_ids.add(wid)
        ob = zo(w_bytes, o_bytes, is_block)
        if ob:
            init.append(ObjectSpec(oid, ob, "backing", "optimizer_state", persistent=True))

    param_objects("embed", embed_w_bytes, embed_o_bytes)
    for i in range(L):
        k = kinds[layer_kinds[i]]
        param_objects(str(i), k.w_bytes, k.o_bytes)
        if k.aux_bytes:
            init.append(ObjectSpec(f"Aux_{i}", k.aux_bytes, "backing", "other", persistent=True))
    if head_w_bytes:
        # tied: the head object only carries what is not shared with the embedding (final norm)
        param_objects("head", head_w_bytes, head_o_bytes)
    for r in range(cfg.grad_accum_rounds):
        init.append(ObjectSpec(f"tokens_{s}_{r}", tok_bytes, "backing", "input"))
        init.append(ObjectSpec(f"targets_{s}_{r}", tok_bytes, "backing", "input"))

    tasks: list[TaskSpec] = []
    rewrites: list[RecomputeRewrite] = []
    finals: dict[str, str] = {o.id: ("fast" if o.id in resident_ids else "backing") for o in init if o.persistent}
    R = cfg.grad_accum_rounds
    last = R - 1
    opt_tasks_tail: list[TaskSpec] = []

    def gather_task(wid: str, params, out_id: str | None = None, tag: str = "") -> None:
        """Stage 3: materialise the full weight object from the ranks' slices before its first use (or, when
        re-gathering, before this use: ``out_id`` names the temporary)."""
        if wid not in gathered:
            return
        nbytes = gathered[wid]
        us = hw.comm_us(nbytes * (zworld - 1) / zworld) + hw.mem_us(2 * nbytes) + 10.0
        if tag and comm_async:
            us = 15.0           # issued on the communication stream one layer ahead: only the launch is on the chain
        tasks.append(TaskSpec(f"param_gather_{s}_{wid[2:]}{tag}", inputs=("Ws_" + wid[2:],),
                              outputs=(OutputSpec(out_id or wid, nbytes, "fast", "parameter"),),
                              runtime_us=us,
                              group="comm", compute_block_key="param_gather", block_params={**bp, **params},
                              comm_groups=cg, metadata=_meta(({"name": "all_gather", "memory_bytes": float(nbytes),
                                                               "efficiency": "scale_up"},))))

    def opt_task(tid: str, key: str, w: str, dw: str, o: str | None, us: float, subops, ws: int, params) -> TaskSpec:
        if zstage == 3:
            w = "Ws_" + w[2:]
        if zstage and o is None:
            o = "O_" + w.split("_", 1)[1]
        if zstage:
            us = us / zworld + hw.comm_us(float(sizes_of[dw]) * (zworld - 1) / zworld) + 20.0
        ins = (w, dw) + ((o,) if o else ())
        return TaskSpec(tid, inputs=ins, mutates=(w,) + ((o,) if o else ()), runtime_us=us, workspace_bytes=ws,
                        group="optimizer", compute_block_key=key, block_params={**bp, **params},
                        comm_groups=cg, metadata=_meta(subops))

    def place_opt(t: TaskSpec):
        (tasks if cfg.optimizer_placement == "interleaved" else opt_tasks_tail).append(t)

    pending_join = None

    def emit_join(i: int, dw: str, gacc: str, k) -> None:
        """One layer after its reduce-scatter was issued: wait for it (the full gradient is freed here) and, in
        the last round, step the optimizer on the slice."""
        if comm_async:
            tasks.append(TaskSpec(f"grad_rs_join_{s}_{cur_round[0]}_{i}", inputs=(dw, gacc), runtime_us=5.0, group="comm",
                                  compute_block_key="grad_rs_join", block_params={**bp, "layer": i, "round": cur_round[0]},
                                  comm_groups=cg))
        if cur_round[0] == last:
            t = opt_task(f"optimizer_{s}_{i}", "optimizer_block", f"W_{i}", gacc, f"O_{i}",
                         k.opt_us, k.opt_subops, k.workspace_opt, {"step": s, "layer": i, "kind": k.kind, "local": True})
            place_opt(replace(t, runtime_us=k.opt_us / zworld + 10.0))

    cur_round = [0]
    sizes_of: dict[str, int] = {f"dW_embed_{s}": embed_dw_bytes, f"dW_head_{s}": head_dw_bytes}
    for i in range(L):
        sizes_of[f"dW_{s}_{i}"] = kinds[layer_kinds[i]].dw_bytes
    for r in range(R):
        create = r == 0
        cur_round[0] = r
        if create:
            gather_task("W_embed", {"target": "embed"})
        tasks.append(TaskSpec(f"prologue_round_{s}_{r}", outputs=(OutputSpec(f"current_round_{s}_{r}", 4, "fast", "other"),),
                              runtime_us=loose.prologue_us, group="prologue", compute_block_key="prologue_round",
                              block_params={**bp, "round": r}))
        tasks.append(TaskSpec(f"embed_fwd_{s}_{r}", inputs=(f"tokens_{s}_{r}", "W_embed", f"current_round_{s}_{r}"),
                              outputs=(OutputSpec(f"y_embed_{s}_{r}", x_bytes, "fast", "activation"),),
                              runtime_us=loose.embed_fwd_us, group="fwd", compute_block_key="embed_fwd",
                              block_params={**bp, "round": r}))
        prev = f"y_embed_{s}_{r}"
        for i in range(L):
            k = kinds[layer_kinds[i]]
            lvl = levels.get((r, i), levels.get(i, 0))
            ctx_bytes = k.ctx_bytes
            if lvl:
                ctx_bytes = next(sb for (lv, sb, _) in k.recompute_levels if lv == lvl)
            outs = [OutputSpec(f"y_{s}_{r}_{i}", x_bytes, "fast", "activation")]
            if ctx_bytes:
                outs.append(OutputSpec(f"A_{s}_{r}_{i}" if not lvl else f"Ap_{s}_{r}_{i}", ctx_bytes, "fast", "activation"))
            if k.aux_temp_bytes:
                outs.append(OutputSpec(f"AuxTemp_{s}_{r}_{i}", k.aux_temp_bytes, "fast", "other"))
            w_f = f"W_{i}"
            if regather and zstage == 3:
                w_f = f"Wg_{s}_{r}_{i}f"
                ahead = [0, 1] if i == 0 else [i + 1]
                for j in ahead:
                    if j < L:
                        gather_task(f"W_{j}", {"target": "block", "layer": j}, f"Wg_{s}_{r}_{j}f", f"_{r}f")
            elif create:
                gather_task(f"W_{i}", {"target": "block", "layer": i})
            ins = (prev, w_f) + ((f"Aux_{i}",) if k.aux_bytes else ())
            tasks.append(TaskSpec(f"block_fwd_{s}_{r}_{i}", inputs=ins, outputs=tuple(outs),
                                  mutates=(f"Aux_{i}",) if k.aux_bytes else (),
                                  runtime_us=k.fwd_us, workspace_bytes=k.workspace_fwd, group="fwd",
                                  compute_block_key=f"{k.kind}_fwd",
                                  block_params={**bp, "layer": i, "round": r, "recompute_level": lvl},
                                  comm_groups=cg, metadata=_meta(k.fwd_subops)))
            if create and k.recompute_levels:
                rewrites.append(RecomputeRewrite(
                    f"A_{s}_{r}_{i}", f"block_fwd_{s}_{r}_{i}", f"block_recompute_{s}_{r}_{i}",
                    (RecomputeOption(0, k.ctx_bytes, 0.0, "save"),) +
                    tuple(RecomputeOption(lv, sb, us, f"level{lv}") for lv, sb, us in k.recompute_levels),
                    f"{k.kind}_fwd", f"{k.kind}_recompute", f"layer{i}"))
            prev = f"y_{s}_{r}_{i}"
        # head + loss
        if regather and zstage == 3 and L:
            gather_task(f"W_{L - 1}", {"target": "block", "layer": L - 1}, f"Wg_{s}_{r}_{L - 1}b", f"_{r}b")
        if create:
            gather_task("W_head", {"target": "head"})
        head_in = [prev, f"targets_{s}_{r}", "W_head"] + (["W_embed"] if cfg.tied_embeddings else [])
        head_out = [OutputSpec(f"dy_{s}_{r}_{L - 1}" if L else f"dy_embed_{s}_{r}", x_bytes, "fast", "activation"),
                    OutputSpec(f"loss_{s}_{r}", 4, "backing", "output")]
        head_mut: tuple[str, ...] = ()
        head_dw = f"dW_head_{s}"
        tied_dw = f"dW_embed_{s}"
        if create:
            head_out.append(OutputSpec(head_dw, head_dw_bytes, "fast", "gradient"))
            if cfg.tied_embeddings:
                head_out.append(OutputSpec(tied_dw, embed_dw_bytes, "fast", "gradient"))
        else:
            head_in.append(head_dw)
            head_mut = (head_dw,)
            if cfg.tied_embeddings:
                head_in.append(tied_dw)
                head_mut = (head_dw, tied_dw)
        tasks.append(TaskSpec(f"head_loss_{s}_{r}", inputs=tuple(head_in), outputs=tuple(head_out), mutates=head_mut,
                              runtime_us=loose.head_loss_us, workspace_bytes=loose.head_workspace, group="head",
                              compute_block_key="head_loss", block_params={**bp, "round": r},
                              comm_groups=cg, metadata=_meta(loose.head_subops)))
        finals[f"loss_{s}_{r}"] = "backing"
        if r == last and head_dw_bytes:
            place_opt(opt_task(f"optimizer_head_{s}", "optimizer_head", "W_head", head_dw,
                               "O_head" if (head_o_bytes or zstage) else None,
                               opt_head_us if opt_head_us is not None else optimizer_cost_seed(hw, head_w_bytes, head_dw_bytes, head_o_bytes),
                               (), 0, {"step": s, "target": "head"}))
        # backward
        for i in reversed(range(L)):
            k = kinds[layer_kinds[i]]
            lvl = levels.get((r, i), levels.get(i, 0))
            x_in = f"y_{s}_{r}_{i - 1}" if i > 0 else f"y_embed_{s}_{r}"
            dy = f"dy_{s}_{r}_{i}"
            dx = f"dy_{s}_{r}_{i - 1}" if i > 0 else f"dy_embed_{s}_{r}"
            a_obj = f"A_{s}_{r}_{i}"
            aux_t = (f"AuxTemp_{s}_{r}_{i}",) if k.aux_temp_bytes else ()
            w_b = f"W_{i}"
            fsdp_block = regather and zstage == 3 and k.dw_bytes
            if regather and zstage == 3:
                w_b = f"Wg_{s}_{r}_{i}b"
                if i - 1 >= 0:
                    gather_task(f"W_{i - 1}", {"target": "block", "layer": i - 1}, f"Wg_{s}_{r}_{i - 1}b", f"_{r}b")
            if lvl:
                rus = next(us for (lv, _, us) in k.recompute_levels if lv == lvl)
                saved = next(sb for (lv, sb, _) in k.recompute_levels if lv == lvl)
                rin = (x_in, w_b) + ((f"Ap_{s}_{r}_{i}",) if saved else ()) + aux_t
                tasks.append(TaskSpec(f"block_recompute_{s}_{r}_{i}", inputs=rin,
                                      outputs=(OutputSpec(a_obj, k.ctx_bytes, "fast", "activation"),),
                                      runtime_us=rus, workspace_bytes=k.workspace_fwd, group="recompute",
                                      compute_block_key=f"{k.kind}_recompute",
                                      block_params={**bp, "layer": i, "round": r, "recompute_level": lvl},
                                      comm_groups=cg, metadata=_meta(k.recompute_subops)))
            ins = [dy, a_obj, x_in, w_b] + list(aux_t)
            outs = [OutputSpec(dx, x_bytes, "fast", "activation")]
            mut: tuple[str, ...] = ()
            dw = f"dW_{s}_{r}_{i}" if fsdp_block else f"dW_{s}_{i}"
            if k.dw_bytes:
                if create or fsdp_block:
                    outs.append(OutputSpec(dw, k.dw_bytes, "fast", "gradient"))
                else:
                    ins.append(dw)
                    mut = (dw,)
            tasks.append(TaskSpec(f"block_bwd_{s}_{r}_{i}", inputs=tuple(ins), outputs=tuple(outs), mutates=mut,
                                  runtime_us=k.bwd_us, workspace_bytes=k.workspace_bwd, group="bwd",
                                  compute_block_key=f"{k.kind}_bwd", block_params={**bp, "layer": i, "round": r},
                                  comm_groups=cg, metadata=_meta(k.bwd_subops)))
            if fsdp_block:
                # reduce-scatter this round's gradient into the rank's fp32 slice; the full gradient dies at the join
                gacc = f"G_{s}_{i}"
                gbytes = 2 * zslice(k.dw_bytes)
                rs_us = hw.comm_us(k.dw_bytes * (zworld - 1) / zworld) + hw.mem_us(k.dw_bytes + gbytes) + 10.0
                tasks.append(TaskSpec(f"grad_rs_{s}_{r}_{i}", inputs=(dw,) + (() if create else (gacc,)),
                                      outputs=(OutputSpec(gacc, gbytes, "fast", "gradient"),) if create else (),
                                      mutates=() if create else (gacc,),
                                      runtime_us=15.0 if comm_async else rs_us,
                                      group="comm", compute_block_key="grad_rs",
                                      block_params={**bp, "layer": i, "round": r, "target": "block", "first": create},
                                      comm_groups=cg, metadata=_meta(({"name": "reduce_scatter", "memory_bytes": float(k.dw_bytes),
                                                                       "efficiency": "scale_up"},))))
                sizes_of[gacc] = gbytes
                if pending_join is not None:
                    emit_join(*pending_join)
                pending_join = (i, dw, gacc, k)
            elif r == last and k.dw_bytes:
                place_opt(opt_task(f"optimizer_{s}_{i}", "optimizer_block", f"W_{i}", dw, f"O_{i}" if (k.o_bytes or zstage) else None,
                                   k.opt_us, k.opt_subops, k.workspace_opt, {"step": s, "layer": i, "kind": k.kind}))
        # embedding backward
        ein = [f"dy_embed_{s}_{r}", f"tokens_{s}_{r}"]
        eout: tuple[OutputSpec, ...] = ()
        emut: tuple[str, ...] = ()
        if create and not cfg.tied_embeddings:
            eout = (OutputSpec(tied_dw, embed_dw_bytes, "fast", "gradient"),)
        else:
            ein.append(tied_dw)
            emut = (tied_dw,)
        tasks.append(TaskSpec(f"embed_bwd_{s}_{r}", inputs=tuple(ein), outputs=eout, mutates=emut,
                              runtime_us=loose.embed_bwd_us, group="bwd", compute_block_key="embed_bwd",
                              block_params={**bp, "round": r}))
        if pending_join is not None:
            emit_join(*pending_join)
            pending_join = None
        if r == last:
            place_opt(opt_task(f"optimizer_embed_{s}", "optimizer_embed", "W_embed", tied_dw,
                               "O_embed" if (embed_o_bytes or zstage) else None,
                               opt_embed_us if opt_embed_us is not None else optimizer_cost_seed(hw, embed_w_bytes, embed_dw_bytes, embed_o_bytes),
                               (), 0, {"step": s, "target": "embed"}))
    tasks.extend(opt_tasks_tail)
    if zstage:
        metadata = {**dict(metadata or {}), "zero": {"stage": zstage, "world": zworld, "rank": int(zero.get("rank", 0)),
                                                     "regather": regather},
                    "zero_full_bytes": dict(gathered)}
    md = {"tokens_per_step": T * R, "tokens_per_round": T, "grad_accum_rounds": R, "n_layers": L,
          "hardware": hw.name, **dict(metadata or {})}
    return Program(cfg.name, tuple(init), tuple(tasks), finals, None, None,
                   int(hw.h2d_gbs * 1e3), int(hw.d2h_gbs * 1e3), tuple(rewrites), md)
