"""Symbolic tracing of one block: modules are called on shape-only tensors and every op they run records what it costs.

A ``TraceContext`` carries the training geometry of one round (tokens ``T``, sequence length ``S``, dtypes, the parallel
layout) and collects, while a module's ``forward`` runs,

    forward sub-ops          hardware-free cost terms (tensor FLOPs of a dtype, bytes through device memory, bytes over the
                             scale-up fabric) in execution order
    backward sub-ops         what the same op costs in the backward pass (data gradient and weight gradient for a matmul,
                             2.5x the forward FLOPs for attention, one more pass over the operands for element-wise ops),
                             kept in reverse order
    saved tensors            what the backward needs from the forward, with a flag for tensors that are cheap to rebuild
                             (outputs of element-wise ops and norms: selective recompute drops exactly these)
    parameters               element counts: total, held by this rank (tensor / expert sharding), touched per token (mixture
                             of experts)

``trace_block`` returns the collected ``BlockTrace``; the training builder turns traces into tasks.  Shapes are the LOCAL
shapes of one rank: a tensor-parallel layout divides head and hidden dimensions before ops see them.
Reference role: ``src/dataflow_sim/workloads/dataflow_builder/__init__.py`` (``TraceContext`` / ``DataflowModule``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable

from .schema import SubOp

DTYPE_BYTES = {"fp32": 4, "tf32": 4, "bf16": 2, "fp16": 2, "fp8": 1, "fp8_e4m3": 1, "fp8_e5m2": 1, "fp4": 0.5, "int32": 4, "int8": 1, "bits": 0.125}


@dataclass(frozen=True)
class Sym:
    """A tensor that has a name, a shape and a dtype, and no values."""
    name: str
    shape: tuple
    dtype: str = "bf16"

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    @property
    def nbytes(self) -> float:
        return self.numel * DTYPE_BYTES[self.dtype]

    def like(self, name: str, shape: tuple | None = None, dtype: str | None = None) -> "Sym":
        return Sym(name, tuple(shape) if shape is not None else self.shape, dtype or self.dtype)


@dataclass(frozen=True)
class Saved:
    name: str
    bytes: float
    cheap: bool = False           # rebuilt by re-running element-wise work: dropped under selective recompute
    module: str = ""


@dataclass(frozen=True)
class ParamInfo:
    name: str
    numel: int                    # of the whole model
    local: float                  # held by this rank
    active: float                 # touched per token (of the whole model)
    kind: str = "matrix"          # matrix | vector | embedding | experts


@dataclass
class BlockTrace:
    fwd: list[SubOp] = field(default_factory=list)
    bwd: list[SubOp] = field(default_factory=list)
    recompute_cheap: list[SubOp] = field(default_factory=list)      # forward ops that rebuild the cheap saved tensors
    saved: list[Saved] = field(default_factory=list)
    params: list[ParamInfo] = field(default_factory=list)
    workspace_bytes: float = 0.0

    @property
    def total_params(self) -> int:
        return int(sum(p.numel for p in self.params))

    @property
    def local_params(self) -> float:
        return float(sum(p.local for p in self.params))

    @property
    def active_params(self) -> float:
        return float(sum(p.active for p in self.params))

    def saved_bytes(self, selective: bool = False) -> float:
        return float(sum(s.bytes for s in self.saved if not (selective and s.cheap)))

    def flops(self, phase: str = "fwd") -> float:
        return float(sum(op.flops for op in (self.fwd if phase == "fwd" else self.bwd)))


class TraceContext:
    def __init__(self, tokens: int, seq_len: int, *, act_dtype: str = "bf16", param_dtype: str = "bf16", compute_dtype: str = "bf16",
                 grad_dtype: str = "bf16", tp: int = 1, ep: int = 1, dp: int = 1):
        self.T, self.S = int(tokens), int(seq_len)
        self.act_dtype, self.param_dtype, self.compute_dtype, self.grad_dtype = act_dtype, param_dtype, compute_dtype, grad_dtype
        self.tp, self.ep, self.dp = int(tp), int(ep), int(dp)
        self.trace = BlockTrace()
        self._scope: list[str] = []
        self.cheap_names: set[str] = set()          # tensors an element-wise op or a norm produced: rebuilt, not kept, under selective recompute

    # -- naming
    def scope(self, name: str):
        ctx = self

        class _S:
            def __enter__(self_inner):
                ctx._scope.append(name)

            def __exit__(self_inner, *exc):
                ctx._scope.pop()
                return False
        return _S()

    def path(self, name: str = "") -> str:
        return ".".join(self._scope + ([name] if name else []))

    # -- tensors and parameters
    def tensor(self, name: str, shape: Iterable[int], dtype: str | None = None) -> Sym:
        return Sym(self.path(name), tuple(int(s) for s in shape), dtype or self.act_dtype)

    def param(self, name: str, shape: Iterable[int], *, shard: str | None = None, active: float = 1.0, kind: str = "matrix",
              dtype: str | None = None) -> Sym:
        """Register a parameter by its GLOBAL shape; returns the tensor this rank holds (``shard``: ``"tp"`` divides the last
        dimension over the tensor-parallel ranks (column parallel), ``"tp_rows"`` the first (row parallel), ``"ep"`` the leading
        expert dimension over the expert-parallel ranks).
        ``active``: share of the parameter a token touches (``top_k / n_experts`` for routed experts)."""
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        div = self.tp if shard in ("tp", "tp_rows") else (self.ep if shard == "ep" else 1)
        self.trace.params.append(ParamInfo(self.path(name), n, n / div, n * active, kind))
        local = shape
        if shard == "ep":
            local = (max(shape[0] // self.ep, 1),) + shape[1:]
        elif shard == "tp":
            local = shape[:-1] + (max(shape[-1] // self.tp, 1),)
        elif shard == "tp_rows":
            local = (max(shape[0] // self.tp, 1),) + shape[1:]
        return Sym(self.path(name), local, dtype or self.param_dtype)

    # -- recording
    def emit(self, name: str, kind: str, *, flops: float = 0.0, bytes: float = 0.0, dtype: str | None = None, phase: str = "fwd",
             efficiency: float | None = None, cheap: bool = False) -> None:
        op = SubOp(name=self.path(name), kind=kind, flops=float(flops), bytes=float(bytes), dtype=dtype or self.compute_dtype,
                   efficiency=efficiency)
        if phase == "fwd":
            self.trace.fwd.append(op)
            if cheap:
                self.trace.recompute_cheap.append(op)
                self.cheap_names.add(op.name)
        else:
            self.trace.bwd.insert(0, op)               # the backward runs the ops in reverse

    def save(self, t: Sym, cheap: bool = False) -> None:
        self.trace.saved.append(Saved(t.name, t.nbytes, cheap, self.path()))

    def workspace(self, nbytes: float) -> None:
        self.trace.workspace_bytes = max(self.trace.workspace_bytes, float(nbytes))


class DataflowModule:
    """A module of the workload library: ``forward(ctx, x)`` runs ops of ``ops.py`` on symbolic tensors."""
    name = "module"

    def forward(self, ctx: TraceContext, x: Sym) -> Sym:        # pragma: no cover - interface
        raise NotImplementedError

    def __call__(self, ctx: TraceContext, x: Sym) -> Sym:
        with ctx.scope(self.name):
            return self.forward(ctx, x)


def trace_block(module: DataflowModule, ctx: TraceContext, d_model: int) -> BlockTrace:
    """Run ``module`` on a (tokens, d_model) residual-stream tensor and return what was recorded."""
    x = ctx.tensor("x", (ctx.T, d_model))
    y = module(ctx, x)
    if y.shape != x.shape:
        raise ValueError(f"block {module.name!r} maps {x.shape} to {y.shape}: a block must keep the residual stream's shape")
    return ctx.trace
