"""Parity checks through the daemon: read what the engine produced as host copies fetched by the client.

``gradcheck`` looks at the engine's objects in the memory of its own process.  A daemon keeps its memory to itself; what a
client can do is ``get_object``, which returns the bytes of an object the store holds on the host.  These helpers run a
family's step through a client and compare with the family's pure-torch twin using nothing but such fetches, so the check
exercises the same path a user's process has: registration with a resolver spec, object upload, ``run``, ``fetch``.

    with_backing_retention   a program copy whose listed objects must end in backing memory, so the store has them after a run
    fetch_host_tensor        one object as a flat host tensor
    fetch_views              one object split into its layout's named tensors (copies; nothing aliases daemon memory)
    client_model_step        one SGD step (lr 1: the update IS the gradient) through the client against ``loss.backward()``
                             of the twin from the same initial bytes; returns ``gradcheck.CheckReport``

Reference role: ``src/dataflow_training/testing/client_parity.py`` (``with_backing_retention``, ``fetch_host_tensor``,
``client_model_step`` :207).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .gradcheck import CheckReport, cos_sim, rel_l2


def with_backing_retention(program, ids):
    """``program`` with every id of ``ids`` pinned to backing memory in ``final_locations``."""
    return dataclasses.replace(program, final_locations={**dict(program.final_locations), **{oid: "backing" for oid in ids}})


def fetch_host_tensor(client, oid: str, dtype: str = "fp32"):
    import torch
    from ..runtime.interop import _dtypes
    raw = client.get_object(oid)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(_dtypes()[dtype])


def fetch_views(client, oid: str, layout) -> dict:
    """name -> tensor for every field of ``layout``, cut from one fetch of the object."""
    import torch
    from ..runtime.interop import _ITEMSIZE, _dtypes
    raw = torch.frombuffer(bytearray(client.get_object(oid)), dtype=torch.uint8)
    offs = layout.offsets()
    out = {}
    for f in layout.fields:
        n = 1
        for s in f.shape:
            n *= int(s)
        nbytes = n * _ITEMSIZE[f.dtype]
        if offs[f.name] + nbytes > raw.numel():
            raise ValueError(f"{oid!r} has {raw.numel()} bytes, field {f.name!r} ends at {offs[f.name] + nbytes}")
        out[f.name] = raw[offs[f.name]:offs[f.name] + nbytes].view(_dtypes()[f.dtype]).reshape(tuple(int(s) for s in f.shape))
    return out


def client_model_step(client, family: str, *, preset: str = "tiny", overrides: Mapping[str, Any] | None = None, policy: str = "fp32",
                      seed: int = 3, tol: float = 2e-2, shape: str = "uniform") -> CheckReport:
    """Initialise through the daemon, read the initial weights back, run one plain-SGD step through ``client.run``, read the
    weights again; the difference is the engine's gradient, compared per tensor with the twin's autograd gradient."""
    import torch
    from ..lowering.planning import plan_program
    from ..models.families import build_init_program, resolve_family
    from ..register import canonical_spec
    from ..run.driver import synthetic_rounds
    from .family_gate import ragged_bounds
    fam = resolve_family(family)
    cfg = dataclasses.replace(fam.presets[preset](), dtype_policy=policy, optimizer="sgd", **dict(overrides or {}))
    hyper = {"optimizer": "sgd", "lr": 1.0, "weight_decay": 0.0, "momentum": 0.0, "schedule": {"kind": "constant", "peak_lr": 1.0}}
    spec = canonical_spec(family, cfg, hyper, seed=seed)
    dims = fam.derive_dims(cfg)
    layouts = fam.family_layouts(dims, cfg.policy() if hasattr(cfg, "policy") else None, "sgd")
    prog = plan_program(fam.lower(cfg), None).program
    persistent = [o.id for o in prog.initial_objects if o.persistent]
    prog = with_backing_retention(prog, persistent)
    init = build_init_program(prog)
    made = set()
    for o in list(init.initial_objects) + list(prog.initial_objects):
        if o.id not in made:
            client.create_object(o.id, o.size_bytes, replace=True)
            made.add(o.id)
    reg = client.register_program(init, spec)
    try:
        out = client.run(reg["prog_id"])
        if out["state"] != "done":
            raise RuntimeError(f"initialisation through the daemon ended {out['state']}: {out.get('error')}")
    finally:
        client.unregister_program(reg["prog_id"])

    def views_of(oid, layout):
        return fetch_views(client, oid, layout)

    before = {k: v.clone() for k, v in fam.bridge(cfg, views_of).items()}
    twin = fam.twin(cfg)
    twin.load_state_dict(before)
    R, T = cfg.grad_accum_rounds, cfg.tokens_per_round
    data = synthetic_rounds(cfg, R, T, 64, 11, 0)
    bounds = {r: (ragged_bounds(T, cfg.seq_len, r) if shape == "ragged" else list(range(0, T + 1, cfg.seq_len))) for r in range(R)}
    twin.zero_grad()
    loss_twin = 0.0
    for r, (tk, tg) in enumerate(data):
        loss = twin.loss(tk, tg, bounds[r], total_rows=T * R)
        loss.backward()
        loss_twin += float(loss.detach())
    reg = client.register_program(prog, spec)
    try:
        args: dict[str, Any] = {"step": 1, "valid_rows": T * R}
        if shape == "ragged":
            args["seq_lens"] = {str(r): b for r, b in bounds.items()}
        for r, (tk, tg) in enumerate(data):
            client.put_object(f"tokens_0_{r}", tk.numpy().tobytes())
            client.put_object(f"targets_0_{r}", tg.numpy().tobytes())
        out = client.run(reg["prog_id"], args=args, fetch=[f"loss_0_{r}" for r in range(R)])
        if out["state"] != "done":
            raise RuntimeError(f"the step through the daemon ended {out['state']}: {out.get('error')}")
        loss_engine = float(sum(out["fetched"].values()))
        after = fam.bridge(cfg, views_of)
    finally:
        client.unregister_program(reg["prog_id"])
    rep = CheckReport(family, loss_engine, loss_twin, tol=tol)
    grads = {k: p.grad for k, p in twin.named_parameters()}
    for k, w0 in before.items():
        if k not in grads:
            continue
        g_ref = grads[k] if grads[k] is not None else torch.zeros_like(w0)
        g_eng = w0.float() - after[k].float()
        rep.grad_rel_l2[k] = rel_l2(g_eng, g_ref)
        rep.grad_cos[k] = cos_sim(g_eng, g_ref)
        rep.grad_norm[k] = float(g_ref.float().norm())
    return rep
