"""The op library of the workload tracer: what every op of a transformer block costs, forward and backward, as
hardware-free terms (``tracing.TraceContext.emit``).  An op takes symbolic tensors, returns symbolic tensors, records its
forward cost, the cost of its backward, and the tensors its backward needs.

Conventions
    rows are tokens of one round (``ctx.T``); a sequence has ``ctx.S`` tokens; causal attention does half of the square
    a matmul's forward is ``2 M N K`` FLOPs and streams its three operands once; its backward is the data gradient and the
        weight gradient, ``2 M N K`` each
    attention's backward is 2.5x its forward FLOPs (two of the five products are recomputed from the saved statistics)
    an element-wise op reads its inputs and writes its outputs once; its backward reads the incoming gradient and what it
        saved, and writes the outgoing gradient
    collectives move ``bytes * (n - 1) / n`` over the scale-up fabric per rank
Reference role: ``src/dataflow_sim/workloads/ops/{forward,backward,optimizer}/*.py``.
"""
from __future__ import annotations

from .tracing import DTYPE_BYTES, Sym, TraceContext


def _saved_once(ctx: TraceContext, t: Sym, cheap: bool = False) -> None:
    """Save ``t`` for the backward once; a tensor that an element-wise op or a norm produced is marked cheap to rebuild."""
    if not any(s.name == t.name for s in ctx.trace.saved):
        ctx.save(t, cheap or t.name in ctx.cheap_names)


# ------------------------------------------------------------------------------------------------ matmuls
def linear(ctx: TraceContext, x: Sym, w: Sym, name: str, *, input_cheap: bool = False, out_dtype: str | None = None) -> Sym:
    """y (rows, N) = x (rows, K) @ w (K, N): forward, and data + weight gradients in the backward.  Saves ``x``."""
    rows, k = x.shape[0], x.shape[-1]
    assert w.shape[0] == k, f"{name}: x {x.shape} @ w {w.shape}"
    n = w.shape[1]
    y = ctx.tensor(name, (rows, n), out_dtype)
    flops = 2.0 * rows * k * n
    gb = DTYPE_BYTES[ctx.grad_dtype]
    ctx.emit(name, "matmul", flops=flops, bytes=x.nbytes + w.nbytes + y.nbytes)
    ctx.emit(name + ".dgrad", "matmul", flops=flops, bytes=y.nbytes + w.nbytes + x.nbytes, phase="bwd")
    ctx.emit(name + ".wgrad", "matmul", flops=flops, bytes=x.nbytes + y.nbytes + w.numel * gb, phase="bwd")
    _saved_once(ctx, x, input_cheap)
    return y


def grouped_linear(ctx: TraceContext, xp: Sym, w: Sym, name: str, *, input_cheap: bool = False) -> Sym:
    """Rows of expert e times ``w[e]``: xp (rows, K), w (experts held here, K, N).  Every held expert's weight is streamed."""
    rows, k = xp.shape
    assert w.shape[1] == k, f"{name}: xp {xp.shape} x w {w.shape}"
    n = w.shape[2]
    y = ctx.tensor(name, (rows, n))
    flops = 2.0 * rows * k * n
    gb = DTYPE_BYTES[ctx.grad_dtype]
    ctx.emit(name, "matmul", flops=flops, bytes=xp.nbytes + w.nbytes + y.nbytes)
    ctx.emit(name + ".dgrad", "matmul", flops=flops, bytes=y.nbytes + w.nbytes + xp.nbytes, phase="bwd")
    ctx.emit(name + ".wgrad", "matmul", flops=flops, bytes=xp.nbytes + y.nbytes + w.numel * gb, phase="bwd")
    _saved_once(ctx, xp, input_cheap)
    return y


# ------------------------------------------------------------------------------------------------ norms and element-wise
def rmsnorm(ctx: TraceContext, x: Sym, name: str, *, bias: bool = False, width: int | None = None) -> Sym:
    """RMSNorm (``bias``: LayerNorm) over the last dimension; saves the input and one statistic per row."""
    d = width or x.shape[-1]
    ctx.param(name + ".w", (d,), kind="vector")
    if bias:
        ctx.param(name + ".b", (d,), kind="vector")
    y = x.like(ctx.path(name))
    stats = Sym(ctx.path(name + ".rstd"), (x.numel // x.shape[-1], 2 if bias else 1), "fp32")
    ctx.emit(name, "memory", bytes=x.nbytes + y.nbytes + stats.nbytes, cheap=True)
    ctx.emit(name + ".bwd", "memory", bytes=3.0 * x.nbytes + stats.nbytes, phase="bwd")
    _saved_once(ctx, x)
    _saved_once(ctx, stats)
    return Sym(y.name, y.shape, y.dtype)


def rope(ctx: TraceContext, x: Sym, name: str) -> Sym:
    ctx.emit(name, "memory", bytes=2.0 * x.nbytes)          # in place on the projection's output: nothing to rebuild it from
    ctx.emit(name + ".bwd", "memory", bytes=2.0 * x.nbytes, phase="bwd")
    return x.like(ctx.path(name))


def gated_activation(ctx: TraceContext, h: Sym, name: str, *, gated: bool = True) -> Sym:
    """SwiGLU on a packed [gate | up] projection (``gated``), or a plain activation (GELU, squared ReLU) otherwise.  The
    output is the next matmul's input: cheap to rebuild from ``h``."""
    out = ctx.tensor(name, (h.shape[0], h.shape[1] // 2 if gated else h.shape[1]))
    ctx.emit(name, "memory", bytes=h.nbytes + out.nbytes, cheap=True)
    ctx.emit(name + ".bwd", "memory", bytes=out.nbytes + 2.0 * h.nbytes, phase="bwd")
    _saved_once(ctx, h)
    return out


def residual_add(ctx: TraceContext, x: Sym, y: Sym, name: str, *, fused: bool = True) -> Sym:
    """``fused``: the add rides the producing matmul's epilogue and costs nothing of its own."""
    if not fused:
        ctx.emit(name, "memory", bytes=3.0 * x.nbytes)
    return x.like(ctx.path(name))


def causal_conv(ctx: TraceContext, x: Sym, width: int, name: str) -> Sym:
    """Depthwise causal convolution along tokens + SiLU."""
    ctx.param(name + ".w", (x.shape[-1], width), kind="vector")
    y = x.like(ctx.path(name))
    ctx.emit(name, "memory", bytes=2.0 * x.nbytes, cheap=True)
    ctx.emit(name + ".bwd", "memory", bytes=3.0 * x.nbytes, phase="bwd")
    _saved_once(ctx, x)
    return y


# ------------------------------------------------------------------------------------------------ attention
def attention(ctx: TraceContext, q: Sym, k: Sym, v: Sym, name: str, *, window: int = 0) -> Sym:
    """Causal (optionally sliding-window) softmax attention with grouped heads.  q (T, Hq, D), k / v (T, Hkv, D / Dv)."""
    t, hq, d = q.shape
    dv = v.shape[-1]
    span = min(window, ctx.S) if window else ctx.S
    causal = 1.0 if (window and window < ctx.S) else 0.5
    flops = 2.0 * t * span * hq * (d + dv) * causal
    out = ctx.tensor(name, (t, hq, dv))
    lse = Sym(ctx.path(name + ".lse"), (hq, t), "fp32")
    io = q.nbytes + k.nbytes + v.nbytes + out.nbytes
    ctx.emit(name, "attention", flops=flops, bytes=io)
    ctx.emit(name + ".bwd", "attention", flops=2.5 * flops, bytes=2.0 * io + lse.nbytes, phase="bwd")
    for t_ in (q, k, v, out, lse):
        _saved_once(ctx, t_)
    return out


def lightning_indexer(ctx: TraceContext, qi: Sym, ki: Sym, topk: int, name: str) -> Sym:
    """Index scores (ReLU-weighted sum over a few small heads, one shared key) over the causal prefix and the top-k row
    selection.  The (heads, queries, keys) intermediate never exists; the (queries, keys) scores do, in blocks."""
    t, hi, di = qi.shape
    flops = 2.0 * t * ctx.S * hi * di * 0.5
    scores_bytes = t * ctx.S * 0.5 * 4.0
    sel = Sym(ctx.path(name + ".sel"), (t, min(topk, ctx.S)), "int32")
    ctx.emit(name + ".scores", "attention", flops=flops, bytes=qi.nbytes + ki.nbytes + scores_bytes)
    ctx.emit(name + ".topk", "memory", bytes=4.0 * scores_bytes + sel.nbytes)
    # the indexer's own objective in the backward: scores at the selection, their gradient into q, k and the head weights
    kk = sel.shape[1]
    ctx.emit(name + ".kl_bwd", "attention", flops=3.0 * 2.0 * t * kk * hi * di, bytes=qi.nbytes + t * kk * di * DTYPE_BYTES[ki.dtype], phase="bwd")
    _saved_once(ctx, qi)
    _saved_once(ctx, ki)
    _saved_once(ctx, sel)
    return sel


def sparse_latent_attention(ctx: TraceContext, q_abs: Sym, latent: Sym, sel: Sym, v_width: int, name: str) -> Sym:
    """Attention of every query over its selected keys in the latent (absorbed) form: q_abs (T, H, c + r), one gathered
    (kk, c + r) block per query shared by all heads, values = the first ``v_width`` latent columns."""
    t, h, c = q_abs.shape
    kk = sel.shape[1]
    flops = 2.0 * t * kk * h * (c + v_width)
    gathered = t * kk * c * DTYPE_BYTES[latent.dtype]
    out = ctx.tensor(name, (t, h, v_width))
    ctx.emit(name, "attention", flops=flops, bytes=q_abs.nbytes + gathered + out.nbytes)
    ctx.emit(name + ".bwd", "attention", flops=2.5 * flops, bytes=2.0 * (q_abs.nbytes + gathered + out.nbytes), phase="bwd")
    for t_ in (q_abs, latent, out):
        _saved_once(ctx, t_)
    return out


def gated_delta_rule(ctx: TraceContext, q: Sym, k: Sym, v: Sym, name: str, *, chunk: int = 64) -> Sym:
    """Chunk-parallel gated delta rule (linear attention with a (Dk, Dv) state per head): per token and head the state
    update and read are 2 Dk Dv each, the intra-chunk products 2 C (Dk + Dv), the triangular solve C^2 / 2 per chunk row."""
    t, h, dk = q.shape
    dv = v.shape[-1]
    flops = t * h * (4.0 * dk * dv + 2.0 * chunk * (dk + dv) + chunk * chunk * 0.5)
    out = ctx.tensor(name, (t, h, dv))
    io = q.nbytes + k.nbytes + v.nbytes + out.nbytes
    ctx.emit(name, "matmul", flops=flops, bytes=io, efficiency=0.35)
    ctx.emit(name + ".bwd", "matmul", flops=2.5 * flops, bytes=2.0 * io, phase="bwd", efficiency=0.35)
    for t_ in (q, k, v, out):
        _saved_once(ctx, t_)
    return out


def mamba2_scan(ctx: TraceContext, x: Sym, b: Sym, c: Sym, name: str, *, chunk: int = 128) -> Sym:
    """Selective state-space scan in its chunked (SSD) form: x (T, H, P), b / c (T, G, N)."""
    t, h, p = x.shape
    n = b.shape[-1]
    flops = t * h * (6.0 * p * n + 2.0 * chunk * (p + n))
    out = x.like(ctx.path(name))
    io = x.nbytes + b.nbytes + c.nbytes + out.nbytes
    ctx.emit(name, "matmul", flops=flops, bytes=io, efficiency=0.35)
    ctx.emit(name + ".bwd", "matmul", flops=2.5 * flops, bytes=2.0 * io, phase="bwd", efficiency=0.35)
    for t_ in (x, b, c):
        _saved_once(ctx, t_)
    return out


# ------------------------------------------------------------------------------------------------ mixture of experts
def router(ctx: TraceContext, x: Sym, n_experts: int, top_k: int, name: str) -> Sym:
    w = ctx.param(name + ".w", (x.shape[-1], n_experts))
    logits = linear(ctx, x, w, name + ".logits", out_dtype="fp32")
    sel = Sym(ctx.path(name + ".route"), (x.shape[0], top_k, 2), "fp32")
    ctx.emit(name + ".topk", "memory", bytes=logits.nbytes + sel.nbytes, cheap=True)
    ctx.emit(name + ".bwd", "memory", bytes=2.0 * logits.nbytes + sel.nbytes, phase="bwd")
    _saved_once(ctx, logits)
    _saved_once(ctx, sel)
    return sel


def moe_dispatch(ctx: TraceContext, x: Sym, top_k: int, name: str) -> Sym:
    """Token rows to the expert-major layout (``top_k`` rows per token); over the fabric when experts are split."""
    rows = x.shape[0] * top_k
    xp = ctx.tensor(name, (rows, x.shape[-1]))
    ctx.emit(name, "memory", bytes=x.nbytes + xp.nbytes)
    ctx.emit(name + ".bwd", "memory", bytes=x.nbytes + xp.nbytes, phase="bwd")
    if ctx.ep > 1:
        moved = xp.nbytes * (ctx.ep - 1) / ctx.ep
        ctx.emit(name + ".a2a", "scale_up", bytes=moved)
        ctx.emit(name + ".a2a.bwd", "scale_up", bytes=moved, phase="bwd")
    return xp


def moe_combine(ctx: TraceContext, yp: Sym, tokens: int, top_k: int, name: str) -> Sym:
    y = ctx.tensor(name, (tokens, yp.shape[-1]))
    ctx.emit(name, "memory", bytes=yp.nbytes + y.nbytes)
    ctx.emit(name + ".bwd", "memory", bytes=2.0 * yp.nbytes + y.nbytes, phase="bwd")
    if ctx.ep > 1:
        moved = yp.nbytes * (ctx.ep - 1) / ctx.ep
        ctx.emit(name + ".a2a", "scale_up", bytes=moved)
        ctx.emit(name + ".a2a.bwd", "scale_up", bytes=moved, phase="bwd")
    _saved_once(ctx, yp)
    return y


# ------------------------------------------------------------------------------------------------ collectives
def all_gather_rows(ctx: TraceContext, x: Sym, name: str) -> Sym:
    """Sequence parallelism: every rank holds ``rows / tp``; the gather in front of a column-parallel matmul (the matching
    reduce-scatter of the gradient in the backward)."""
    if ctx.tp > 1:
        moved = x.nbytes * (ctx.tp - 1) / ctx.tp
        ctx.emit(name, "scale_up", bytes=moved)
        ctx.emit(name + ".bwd", "scale_up", bytes=moved, phase="bwd")
    return x


def reduce_scatter_rows(ctx: TraceContext, x: Sym, name: str) -> Sym:
    if ctx.tp > 1:
        moved = x.nbytes * (ctx.tp - 1) / ctx.tp
        ctx.emit(name, "scale_up", bytes=moved)
        ctx.emit(name + ".bwd", "scale_up", bytes=moved, phase="bwd")
    return x


# ------------------------------------------------------------------------------------------------ embedding, head, optimizer
def embedding_cost(tokens: int, d_model: int, act_bytes: float) -> tuple[float, float]:
    """(forward bytes, backward bytes): a gather of rows, and a sorted scatter-add of their gradients."""
    x = tokens * d_model * act_bytes
    return 2.0 * x, 3.0 * x


def head_loss_flops(tokens: int, d_model: int, vocab: int) -> float:
    """Chunked output projection + cross entropy with its backward in one task: forward, data gradient, weight gradient."""
    return 3.0 * 2.0 * tokens * d_model * vocab


def optimizer_bytes(local_params: float, state_bytes_per_param: float, param_bytes: float, grad_bytes: float) -> float:
    """Read the gradient and the parameter, read and write the state, write the parameter."""
    return local_params * (2.0 * state_bytes_per_param + 2.0 * param_bytes + grad_bytes)


def newton_schulz_flops(rows: int, cols: int, steps: int = 5) -> float:
    """Muon's orthogonalisation of one (rows, cols) matrix: three products per step on the smaller side."""
    small, large = min(rows, cols), max(rows, cols)
    return steps * (2.0 * small * small * large * 2 + 2.0 * small * small * small)
