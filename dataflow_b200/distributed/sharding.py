"""Who holds which bytes: regions of packed objects assigned to ranks.

* ZeRO: a packed object is one flat byte range cut into ``world`` equal 256-byte aligned slices (the last rank
  takes the tail) — ``zero_slices``; eligibility of the flat fused path — ``rs_eligible``.
* Tensor parallel: column shards (``w_qkv`` by KV-head groups, ``w13`` by d_ff) and row shards (``wo``, ``w2``) —
  ``tp_attn_shards``, ``tp_mlp_shards``; replicated fields (norm gains) are owned by every rank.
* Expert parallel: whole experts per rank — ``expert_shards``.

``ShardPlan.validate`` checks that every element of every field is owned (replicated or by exactly one rank).
Role parity: reference ``src/dataflow_training/distributed/sharding.py:39-652``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Mapping, Sequence

FIELD_ALIGN = 256


@dataclass(frozen=True)
class Region:
    """Rows ``[row_lo, row_hi)`` x columns ``[col_lo, col_hi)`` of one 2-D field (vectors use one row)."""
    field: str
    row_lo: int
    row_hi: int
    col_lo: int
    col_hi: int

    @property
    def numel(self) -> int:
        return max(self.row_hi - self.row_lo, 0) * max(self.col_hi - self.col_lo, 0)


@dataclass(frozen=True)
class Assignment:
    region: Region
    owner: int | None              # None = replicated on every rank of the axis


@dataclass
class ShardPlan:
    world: int
    shapes: dict[str, tuple[int, int]]
    assignments: list[Assignment] = field(default_factory=list)

    def owned_regions(self, rank: int) -> list[Region]:
        return [a.region for a in self.assignments if a.owner in (None, rank)]

    def owned_ranges(self, rank: int, fieldname: str) -> list[Region]:
        return [r for r in self.owned_regions(rank) if r.field == fieldname]

    def replicated(self, fieldname: str) -> bool:
        return any(a.owner is None and a.region.field == fieldname for a in self.assignments)

    def local_shape(self, rank: int, fieldname: str) -> tuple[int, int]:
        regs = self.owned_ranges(rank, fieldname)
        if not regs:
            return (0, 0)
        rows = sorted({(r.row_lo, r.row_hi) for r in regs})
        cols = sorted({(r.col_lo, r.col_hi) for r in regs})
        return (sum(b - a for a, b in rows), sum(b - a for a, b in cols))

    @property
    def equal_shards(self) -> bool:
        sizes = [sum(r.numel for r in self.owned_regions(k)) for k in range(self.world)]
        return len(set(sizes)) == 1

    def validate(self) -> "ShardPlan":
        for name, (rows, cols) in self.shapes.items():
            regs = [a for a in self.assignments if a.region.field == name]
            if not regs:
                raise ValueError(f"field {name!r} is assigned to nobody")
            if any(a.owner is None for a in regs):
                if len(regs) != 1 or regs[0].region.numel != rows * cols:
                    raise ValueError(f"field {name!r}: a replicated field must be one whole region")
                continue
            covered = sum(a.region.numel for a in regs)
            if covered != rows * cols:
                raise ValueError(f"field {name!r}: regions cover {covered} of {rows * cols} elements")
            for i, a in enumerate(regs):
                if not 0 <= a.owner < self.world:
                    raise ValueError(f"field {name!r}: owner {a.owner} outside the {self.world}-rank axis")
                for b in regs[i + 1:]:
                    ra, rb = a.region, b.region
                    if ra.row_lo < rb.row_hi and rb.row_lo < ra.row_hi and ra.col_lo < rb.col_hi and rb.col_lo < ra.col_hi:
                        raise ValueError(f"field {name!r}: regions of ranks {a.owner} and {b.owner} overlap")
        return self


def _split(n: int, world: int) -> list[tuple[int, int]]:
    if n % world:
        raise ValueError(f"{n} does not divide over {world} ranks")
    k = n // world
    return [(r * k, (r + 1) * k) for r in range(world)]


def _whole(name, shape) -> Assignment:
    return Assignment(Region(name, 0, shape[0], 0, shape[1]), None)


def tp_mlp_shards(d_model: int, d_ff: int, world: int, fused_w13: bool = True) -> ShardPlan:
    """``w13`` (d, 2F) column-sharded so each rank holds matching gate and up columns; ``w2`` (F, d) row-sharded."""
    shapes = {"w13" if fused_w13 else "w1": (d_model, 2 * d_ff if fused_w13 else d_ff), "w2": (d_ff, d_model), "norm2": (1, d_model)}
    if not fused_w13:
        shapes["w3"] = (d_model, d_ff)
    plan = ShardPlan(world, shapes)
    for r, (a, b) in enumerate(_split(d_ff, world)):
        if fused_w13:
            plan.assignments.append(Assignment(Region("w13", 0, d_model, a, b), r))                    # gate columns
            plan.assignments.append(Assignment(Region("w13", 0, d_model, d_ff + a, d_ff + b), r))      # up columns
        else:
            plan.assignments.append(Assignment(Region("w1", 0, d_model, a, b), r))
            plan.assignments.append(Assignment(Region("w3", 0, d_model, a, b), r))
        plan.assignments.append(Assignment(Region("w2", a, b, 0, d_model), r))
    plan.assignments.append(_whole("norm2", shapes["norm2"]))
    return plan.validate()


def tp_attn_shards(d_model: int, n_heads: int, n_kv_heads: int, head_dim: int, world: int) -> ShardPlan:
    """Fused ``w_qkv`` (d, (hq + 2 hkv) hd) column-sharded by KV-head group (a rank keeps whole GQA groups);
    ``wo`` (hq hd, d) row-sharded by the same query heads."""
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} KV heads do not divide over {world} ranks (GQA groups stay whole)")
    q, kv = n_heads * head_dim, n_kv_heads * head_dim
    shapes = {"w_qkv": (d_model, q + 2 * kv), "wo": (q, d_model), "norm1": (1, d_model)}
    plan = ShardPlan(world, shapes)
    for r in range(world):
        qa, qb = _split(q, world)[r]
        ka, kb = _split(kv, world)[r]
        plan.assignments += [Assignment(Region("w_qkv", 0, d_model, qa, qb), r),
                             Assignment(Region("w_qkv", 0, d_model, q + ka, q + kb), r),
                             Assignment(Region("w_qkv", 0, d_model, q + kv + ka, q + kv + kb), r),
                             Assignment(Region("wo", qa, qb, 0, d_model), r)]
    plan.assignments.append(_whole("norm1", shapes["norm1"]))
    return plan.validate()


def expert_shards(n_experts: int, world: int, expert_fields: Mapping[str, tuple[int, int]]) -> ShardPlan:
    """Whole experts per rank: fields are stacked (E * rows, cols); rank r owns experts [r E/w, (r+1) E/w)."""
    shapes = {k: (n_experts * v[0], v[1]) for k, v in expert_fields.items()}
    plan = ShardPlan(world, shapes)
    for r, (a, b) in enumerate(_split(n_experts, world)):
        for k, (rows, cols) in expert_fields.items():
            plan.assignments.append(Assignment(Region(k, a * rows, b * rows, 0, cols), r))
    return plan.validate()


def local_experts(n_experts: int, world: int, rank: int) -> range:
    a, b = _split(n_experts, world)[rank]
    return range(a, b)


# ---------------------------------------------------------------- ZeRO flat slices
def slice_bytes(total: int, world: int) -> int:
    per = (int(total) + world - 1) // world
    return (per + FIELD_ALIGN - 1) // FIELD_ALIGN * FIELD_ALIGN


def zero_slices(total: int, world: int) -> list[tuple[int, int]]:
    """``[(offset, length)]`` per rank: equal aligned slices, the last ranks take what is left (possibly nothing)."""
    per = slice_bytes(total, world)
    out = []
    for r in range(world):
        lo = min(per * r, total)
        out.append((lo, min(per * (r + 1), total) - lo))
    return out


def rs_eligible(param_dtypes: Iterable[str], grad_dtypes: Iterable[str], rules: Iterable[str]) -> bool:
    """The flat fused reduce-scatter + AdamW path needs one optimizer rule (adamw), one dtype, param dtype == grad dtype."""
    p, g, r = set(param_dtypes), set(grad_dtypes), set(rules)
    return r == {"adamw"} and len(p) == 1 and p == g
