"""Analytic training workloads: a model described by dimensions becomes a hardware-free ``WorkloadProgram``.

No tensors are touched: every layer is a module of the workload library (``modules.py``) traced on shape-only tensors
(``tracing.py``), whose ops (``ops.py``) record forward and backward FLOPs, bytes, saved activations and parameter counts;
``TrainingBuilder`` schedules the traces into forward / head / backward / recompute / optimizer tasks for a number of
gradient-accumulation rounds.  The result is priced on any ``HardwareSpec`` (``schema.realize_workload``) and planned
by any policy — the "what would this model do on that box" path that needs no GPU.
Reference role: ``src/dataflow_sim/workloads/dataflow_builder/__init__.py:65-463`` (dtype policies, training and
parallelism configs, symbolic tracing), ``workloads/training_builder.py:61-286`` (task scheduling, interleaved or tail
optimizer), ``workloads/modules/*.py`` and ``workloads/ops/**`` (per-module FLOP / byte formulas, expert parallelism
priced on the scale-up fabric).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace

from .schema import SubOp, WorkloadCost, WorkloadObject, WorkloadOutput, WorkloadProgram, WorkloadTask

DTYPE_BYTES = {"fp32": 4, "tf32": 4, "bf16": 2, "fp16": 2, "fp8": 1, "fp8_e4m3": 1, "fp8_e5m2": 1, "fp4": 0.5}


@dataclass(frozen=True)
class DTypePolicy:
    param: str = "bf16"
    grad: str = "bf16"
    activation: str = "bf16"
    compute: str = "bf16"
    master: str | None = "fp32"
    moments: str = "fp32"

    def __post_init__(self):
        for name in ("param", "grad", "activation", "compute", "moments"):
            if getattr(self, name) not in DTYPE_BYTES:
                raise ValueError(f"dtype policy: {name} = {getattr(self, name)!r} is not one of {sorted(DTYPE_BYTES)}")
        if self.master is not None and self.master not in DTYPE_BYTES:
            raise ValueError(f"dtype policy: master = {self.master!r} is not one of {sorted(DTYPE_BYTES)} (or None)")

    def state_bytes_per_param(self, optimizer: str) -> float:
        n_moments = {"adamw": 2, "muon": 1, "sgdm": 1, "sgd": 0, "frozen": 0}[optimizer]
        return (DTYPE_BYTES[self.master] if self.master else 0) + n_moments * DTYPE_BYTES[self.moments]


@dataclass(frozen=True)
class ParallelismConfig:
    dp: int = 1
    tp: int = 1
    ep_group_size: int = 1
    zero_stage: int = 0

    def __post_init__(self):
        for name in ("dp", "tp", "ep_group_size"):
            if int(getattr(self, name)) < 1:
                raise ValueError(f"parallel layout: {name} = {getattr(self, name)} must be at least 1")
        if self.zero_stage not in (0, 1, 2, 3):
            raise ValueError(f"parallel layout: zero_stage = {self.zero_stage} must be 0, 1, 2 or 3")


@dataclass(frozen=True)
class TrainingConfig:
    seq_len: int = 4096
    tokens_per_round: int = 16384
    rounds: int = 1
    optimizer: str = "adamw"
    optimizer_placement: str = "interleaved"        # interleaved | tail
    recompute: str = "none"                         # none | selective | full
    dtypes: DTypePolicy = field(default_factory=DTypePolicy)
    parallel: ParallelismConfig = field(default_factory=ParallelismConfig)

    def __post_init__(self):
        if int(self.seq_len) < 1 or int(self.tokens_per_round) < 1 or int(self.rounds) < 1:
            raise ValueError(f"training shape: seq_len = {self.seq_len}, tokens_per_round = {self.tokens_per_round}, rounds = {self.rounds} "
                             f"must all be at least 1")
        if self.seq_len > self.tokens_per_round:
            raise ValueError(f"training shape: a round of {self.tokens_per_round} tokens cannot hold a sequence of {self.seq_len}")
        if self.recompute not in ("none", "selective", "full"):
            raise ValueError(f"recompute = {self.recompute!r} must be none, selective or full")
        if self.optimizer_placement not in ("interleaved", "tail"):
            raise ValueError(f"optimizer_placement = {self.optimizer_placement!r} must be interleaved or tail")


@dataclass(frozen=True)
class AttnSpec:
    kind: str = "dense"             # dense | mla | dsa | linear | mamba | none
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    window: int = 0                 # sliding window (0: full causal)
    q_lora: int = 0                 # MLA
    kv_lora: int = 0
    rope_dim: int = 0
    v_head_dim: int = 0
    index_heads: int = 0            # DSA indexer
    index_dim: int = 0
    index_topk: int = 0
    state_dim: int = 0              # linear attention / mamba state per head


@dataclass(frozen=True)
class MlpSpec:
    kind: str = "swiglu"            # swiglu | relu2 | gelu | moe | none
    d_ff: int = 0
    n_experts: int = 0
    top_k: int = 0
    d_expert: int = 0
    n_shared: int = 0
    expert_act: str = "swiglu"      # swiglu | relu2


@dataclass(frozen=True)
class LayerSpec:
    attn: AttnSpec
    mlp: MlpSpec


@dataclass(frozen=True)
class ModelSpec:
    name: str
    d_model: int
    vocab: int
    layers: tuple
    tied_embeddings: bool = False

    @property
    def n_layers(self) -> int:
        return len(self.layers)


# ------------------------------------------------------------------------------------------- the scheduler
class TrainingBuilder:
    """Schedules one optimizer step of ``model`` under ``cfg`` into a ``WorkloadProgram``."""

    def __init__(self, model: ModelSpec, cfg: TrainingConfig):
        self.m, self.cfg = model, cfg
        self.act_b = DTYPE_BYTES[cfg.dtypes.activation]
        self.par_b = DTYPE_BYTES[cfg.dtypes.param]
        self.grad_b = DTYPE_BYTES[cfg.dtypes.grad]
        self._traces: dict = {}

    # -- costs
    def _mm(self, name: str, flops: float, bytes_: float = 0.0) -> SubOp:
        return SubOp(name=name, kind="matmul", flops=flops, dtype=self.cfg.dtypes.compute, bytes=bytes_)

    def trace(self, layer: LayerSpec):
        """The recorded trace of one layer's block under this configuration (cached per distinct layer spec)."""
        from .modules import block_from_spec
        from .tracing import TraceContext, trace_block
        got = self._traces.get(layer)
        if got is None:
            cfg = self.cfg
            ctx = TraceContext(cfg.tokens_per_round, cfg.seq_len, act_dtype=cfg.dtypes.activation, param_dtype=cfg.dtypes.param,
                               compute_dtype=cfg.dtypes.compute, grad_dtype=cfg.dtypes.grad, tp=cfg.parallel.tp,
                               ep=cfg.parallel.ep_group_size, dp=cfg.parallel.dp)
            got = self._traces[layer] = trace_block(block_from_spec(layer, self.m.d_model), ctx, self.m.d_model)
        return got

    def _layer_cost(self, layer: LayerSpec, backward: bool) -> tuple[WorkloadCost, dict]:
        tr = self.trace(layer)
        info = {"params": tr.total_params, "local_params": tr.local_params, "active_params": tr.active_params,
                "saved_bytes": int(tr.saved_bytes()), "saved_bytes_selective": int(tr.saved_bytes(selective=True))}
        return WorkloadCost(ops=list(tr.bwd if backward else tr.fwd)), info

    # -- program
    def build(self) -> WorkloadProgram:
        cfg, mdl = self.cfg, self.m
        d, T = mdl.d_model, cfg.tokens_per_round
        dp = cfg.parallel.dp
        objects, tasks, final = [], [], {}
        opt_b = cfg.dtypes.state_bytes_per_param(cfg.optimizer)
        shard = dp if cfg.parallel.zero_stage >= 1 else 1
        infos = []
        for i, layer in enumerate(mdl.layers):
            _, info = self._layer_cost(layer, False)
            infos.append(info)
            wb = int(info["local_params"] * self.par_b / (dp if cfg.parallel.zero_stage >= 3 else 1))
            objects.append(WorkloadObject(id=f"W_{i}", bytes=wb, type="parameter"))
            final[f"W_{i}"] = "backing"
            if opt_b:
                objects.append(WorkloadObject(id=f"O_{i}", bytes=int(info["local_params"] * opt_b / shard), type="optimizer_state"))
                final[f"O_{i}"] = "backing"
        emb = mdl.vocab * d
        head_params = 0 if mdl.tied_embeddings else emb
        objects.append(WorkloadObject(id="W_embed", bytes=int(emb * self.par_b), type="parameter"))
        final["W_embed"] = "backing"
        if head_params:
            objects.append(WorkloadObject(id="W_head", bytes=int(head_params * self.par_b), type="parameter"))
            final["W_head"] = "backing"
        if opt_b:
            objects.append(WorkloadObject(id="O_embed", bytes=int((emb + head_params) * opt_b / shard), type="optimizer_state"))
            final["O_embed"] = "backing"
        head_w = "W_head" if head_params else "W_embed"
        x_bytes = int(T * d * self.act_b)
        L = mdl.n_layers
        recompute = cfg.recompute

        def opt_task(i: int) -> WorkloadTask:
            p = infos[i]["local_params"] / shard
            ops = [SubOp(name="optimizer", kind="memory", bytes=p * (opt_b * 2 + self.par_b + self.grad_b))]
            if cfg.optimizer == "muon":
                ops.append(self._mm("newton_schulz", 5 * 3 * 2.0 * p * d))
            if dp > 1:
                ops.append(SubOp(name="grad_reduce", kind="scale_up", bytes=infos[i]["local_params"] * self.grad_b * (dp - 1) / dp *
                                 (1 if cfg.parallel.zero_stage else 2)))
            ins = [f"W_{i}", f"dW_{i}"] + ([f"O_{i}"] if opt_b else [])
            return WorkloadTask(id=f"opt_{i}", inputs=ins, mutates=[f"W_{i}"] + ([f"O_{i}"] if opt_b else []),
                                cost=WorkloadCost(ops=ops), phase="optimizer")

        for r in range(cfg.rounds):
            tasks.append(WorkloadTask(id=f"embed_{r}", inputs=["W_embed"], outputs=[WorkloadOutput(id=f"X_{r}_0", bytes=x_bytes, type="activation")],
                                      cost=WorkloadCost(ops=[SubOp(name="embed", kind="memory", bytes=2.0 * x_bytes)]), phase="fwd", tokens=T))
            for i, layer in enumerate(mdl.layers):
                cost, info = self._layer_cost(layer, False)
                # full recompute keeps the block input only; selective drops what element-wise work rebuilds
                saved = x_bytes if recompute == "full" else int(info["saved_bytes_selective" if recompute == "selective" else "saved_bytes"])
                tasks.append(WorkloadTask(id=f"fwd_{r}_{i}", inputs=[f"X_{r}_{i}", f"W_{i}"],
                                          outputs=[WorkloadOutput(id=f"A_{r}_{i}", bytes=saved, type="activation"),
                                                   WorkloadOutput(id=f"X_{r}_{i + 1}", bytes=x_bytes, type="activation")],
                                          cost=cost, workspace_bytes=int(info["saved_bytes"]), phase="fwd", tokens=T))
            head_flops = 2.0 * T * d * mdl.vocab
            tasks.append(WorkloadTask(id=f"head_{r}", inputs=[f"X_{r}_{L}", head_w] + (["dW_head"] if r else []),
                                      outputs=[WorkloadOutput(id=f"dX_{r}_{L}", bytes=x_bytes, type="activation")] +
                                      ([] if r else [WorkloadOutput(id="dW_head", bytes=int((head_params or emb) * self.grad_b), type="gradient")]),
                                      mutates=["dW_head"] if r else [],
                                      cost=WorkloadCost(ops=[self._mm("head_fwd_bwd", 3.0 * head_flops),
                                                             SubOp(name="loss", kind="memory", bytes=4.0 * T * min(mdl.vocab, 8192) * 4)]),
                                      workspace_bytes=int(T * min(mdl.vocab, 8192) * 4), phase="head", tokens=T))
            for i in reversed(range(L)):
                layer = mdl.layers[i]
                bcost, info = self._layer_cost(layer, True)
                act_in = f"A_{r}_{i}"
                if recompute != "none":
                    tr = self.trace(layer)
                    rc = WorkloadCost(ops=list(tr.fwd if recompute == "full" else tr.recompute_cheap))
                    tasks.append(WorkloadTask(id=f"recompute_{r}_{i}", inputs=[f"A_{r}_{i}", f"W_{i}"],
                                              outputs=[WorkloadOutput(id=f"R_{r}_{i}", bytes=int(info["saved_bytes"]), type="activation")],
                                              cost=rc, phase="recompute", tokens=T))
                    act_in = f"R_{r}_{i}"
                first = r == 0
                ins = [f"dX_{r}_{i + 1}", act_in, f"W_{i}"] + ([] if first else [f"dW_{i}"])
                outs = [WorkloadOutput(id=f"dX_{r}_{i}", bytes=x_bytes, type="activation")]
                if first:
                    outs.append(WorkloadOutput(id=f"dW_{i}", bytes=int(info["local_params"] * self.grad_b), type="gradient"))
                tasks.append(WorkloadTask(id=f"bwd_{r}_{i}", inputs=ins, outputs=outs, mutates=[] if first else [f"dW_{i}"],
                                          cost=bcost, workspace_bytes=int(info["saved_bytes"]), phase="bwd", tokens=T))
                if r == cfg.rounds - 1 and cfg.optimizer_placement == "interleaved" and cfg.optimizer != "frozen":
                    tasks.append(opt_task(i))
            tasks.append(WorkloadTask(id=f"embed_bwd_{r}", inputs=[f"dX_{r}_0"] + (["dW_embed"] if r else []),
                                      outputs=[] if r else [WorkloadOutput(id="dW_embed", bytes=int(emb * self.grad_b), type="gradient")],
                                      mutates=["dW_embed"] if r else [],
                                      cost=WorkloadCost(ops=[SubOp(name="embed_bwd", kind="memory", bytes=3.0 * x_bytes)]), phase="bwd"))
        if cfg.optimizer != "frozen":
            if cfg.optimizer_placement == "tail":
                tasks.extend(opt_task(i) for i in reversed(range(L)))
            ins = ["W_embed", "dW_embed", "dW_head"] + (["W_head"] if head_params else []) + (["O_embed"] if opt_b else [])
            tasks.append(WorkloadTask(id="opt_embed", inputs=ins, mutates=["W_embed"] + (["W_head"] if head_params else []) + (["O_embed"] if opt_b else []),
                                      cost=WorkloadCost(ops=[SubOp(name="optimizer", kind="memory",
                                                                   bytes=(emb + head_params) / shard * (opt_b * 2 + self.par_b + self.grad_b))]),
                                      phase="optimizer"))
        total_params = sum(i["params"] for i in infos) + emb + head_params
        active = sum(i["active_params"] for i in infos) + emb + head_params
        md = {"model": mdl.name, "tokens_per_step": T * cfg.rounds, "seq_len": cfg.seq_len, "rounds": cfg.rounds,
              "total_params": int(total_params), "active_params": int(active), "optimizer": cfg.optimizer,
              "recompute": recompute, "parallel": asdict(cfg.parallel)}
        return WorkloadProgram(name=f"{mdl.name}-train", objects=objects, tasks=tasks, final_locations=final, metadata=md)


def trace_training_model(model: ModelSpec, cfg: TrainingConfig) -> WorkloadProgram:
    tp, ep = cfg.parallel.tp, cfg.parallel.ep_group_size
    for i, layer in enumerate(model.layers):
        a, m = layer.attn, layer.mlp
        if tp > 1:
            # a tensor-parallel layout cuts heads and hidden columns into equal parts: say which dimension does not divide
            # (instead of failing on a shape deep inside the traced block)
            for what, n in (("attention heads", getattr(a, "n_heads", tp)), ("key/value heads", getattr(a, "n_kv_heads", tp)),
                            ("MLP hidden size", getattr(m, "d_ff", tp))):
                if a.kind == "none" and "heads" in what:
                    continue
                if n and int(n) % tp and not (what == "key/value heads" and int(n) < tp):
                    raise ValueError(f"layer {i}: {what} = {n} is not divisible by tp = {tp}")
        if ep > 1 and m.kind == "moe" and int(getattr(m, "n_experts", ep)) % ep:
            raise ValueError(f"layer {i}: {m.n_experts} experts are not divisible by an expert-parallel group of {ep}")
    try:
        return TrainingBuilder(model, cfg).build()
    except AssertionError as e:
        raise ValueError(f"the model's shapes do not fit this layout (tp = {tp}, ep = {ep}): {e}") from None


# ------------------------------------------------------------------------------------------- model library
def _uniform(n: int, attn: AttnSpec, mlp: MlpSpec) -> tuple:
    return tuple(LayerSpec(attn, mlp) for _ in range(n))


def _hybrid(n: int, full: AttnSpec, lin: AttnSpec, mlp: MlpSpec, every: int = 4) -> tuple:
    return tuple(LayerSpec(full if (i + 1) % every == 0 else lin, mlp) for i in range(n))


def _dense_then(n: int, n_dense: int, attn: AttnSpec, dense: MlpSpec, moe: MlpSpec) -> tuple:
    return tuple(LayerSpec(attn, dense if i < n_dense else moe) for i in range(n))


_MLA = AttnSpec("mla", 128, 128, 128, q_lora=1536, kv_lora=512, rope_dim=64, v_head_dim=128)
_DSA = replace(_MLA, kind="dsa", index_heads=64, index_dim=128, index_topk=2048)
_GDN = AttnSpec("linear", 32, 16, 128, state_dim=128)

MODEL_LIBRARY: dict[str, ModelSpec] = {
    "llama3_8b": ModelSpec("llama3_8b", 4096, 128256, _uniform(32, AttnSpec("dense", 32, 8, 128), MlpSpec("swiglu", 14336))),
    "llama3_70b": ModelSpec("llama3_70b", 8192, 128256, _uniform(80, AttnSpec("dense", 64, 8, 128), MlpSpec("swiglu", 28672))),
    "qwen3_8b": ModelSpec("qwen3_8b", 4096, 151936, _uniform(36, AttnSpec("dense", 32, 8, 128), MlpSpec("swiglu", 12288))),
    "qwen3_moe_30b_a3b": ModelSpec("qwen3_moe_30b_a3b", 2048, 151936,
                                   _uniform(48, AttnSpec("dense", 32, 4, 128), MlpSpec("moe", 0, 128, 8, 768))),
    "qwen3_hybrid_dense": ModelSpec("qwen3_hybrid_dense", 4096, 151936,
                                    _hybrid(36, AttnSpec("dense", 32, 8, 128), _GDN, MlpSpec("swiglu", 12288))),
    "qwen3_hybrid_moe": ModelSpec("qwen3_hybrid_moe", 2048, 151936,
                                  _hybrid(48, AttnSpec("dense", 16, 2, 256), _GDN, MlpSpec("moe", 0, 512, 10, 512, 1))),
    "olmoe_1b_7b": ModelSpec("olmoe_1b_7b", 2048, 50304, _uniform(16, AttnSpec("dense", 16, 16, 128), MlpSpec("moe", 0, 64, 8, 1024))),
    "deepseek_v3": ModelSpec("deepseek_v3", 7168, 129280, _dense_then(61, 3, _MLA, MlpSpec("swiglu", 18432), MlpSpec("moe", 0, 256, 8, 2048, 1))),
    "deepseek_v3_2": ModelSpec("deepseek_v3_2", 7168, 129280, _dense_then(61, 3, _DSA, MlpSpec("swiglu", 18432), MlpSpec("moe", 0, 256, 8, 2048, 1))),
    "glm5": ModelSpec("glm5", 5120, 151552, _dense_then(92, 3, AttnSpec("dense", 96, 8, 128), MlpSpec("swiglu", 12288), MlpSpec("moe", 0, 160, 8, 1536, 1))),
    "glm5_2": ModelSpec("glm5_2", 6144, 154880, _dense_then(78, 3, replace(_DSA, n_heads=64, n_kv_heads=64, q_lora=2048), MlpSpec("swiglu", 12288),
                                                             MlpSpec("moe", 0, 256, 8, 2048, 1))),
    "kimi_k2": ModelSpec("kimi_k2", 7168, 163840, _dense_then(61, 1, replace(_MLA, n_heads=64, n_kv_heads=64), MlpSpec("swiglu", 18432),
                                                             MlpSpec("moe", 0, 384, 8, 2048, 1))),
    "gpt_oss_120b": ModelSpec("gpt_oss_120b", 2880, 201088,
                              tuple(LayerSpec(AttnSpec("dense", 64, 8, 64, window=128 if i % 2 == 0 else 0), MlpSpec("moe", 0, 128, 4, 2880))
                                    for i in range(36))),
    "nemotron_h_8b": ModelSpec("nemotron_h_8b", 4096, 131072,
                               tuple(LayerSpec(AttnSpec("dense", 32, 8, 128), MlpSpec("none")) if i % 13 == 6 else
                                     LayerSpec(AttnSpec("mamba", 128, 8, 64, state_dim=128), MlpSpec("none")) if i % 2 == 0 else
                                     LayerSpec(AttnSpec("none"), MlpSpec("relu2", 21504)) for i in range(52))),
}


def get_model(name: str) -> ModelSpec:
    if name not in MODEL_LIBRARY:
        raise KeyError(f"unknown model {name!r}; known: {sorted(MODEL_LIBRARY)}")
    return MODEL_LIBRARY[name]
