"""Fleet mode: one ``dataflowd`` daemon per rank, driven in lock step by this conductor process.

The in-process launcher (``run/conductor.py`` over ``torch.distributed.run``) is what the fused peer-memory kernels need;
fleet mode is the service's own training path, the shape the reference trains in: the conductor

    launches one daemon per rank            (``distributed.daemons.launch`` -> ``tools/train/daemonize.py``)
    connects an ``EngineClient`` to each    (unix sockets on this box)
    links the daemons into a star           (``peer_connect`` from the coordinator, rank 0)
    creates the peer group                  (``create_peer_group``: the attachment barrier; NCCL on GPUs, the peer plane's
                                             host lane on CPU daemons)
    per rank: creates the persistent objects, runs the init program, registers the planned training program
    per step: uploads every rank's rounds, starts one ``run`` per rank on its own thread, joins, sums the losses
    shuts the daemons down.

State lives in the daemons' stores, not in the conductor.  Ranks are replicas (mode ``co``): every optimizer task first sums
its gradient object over the peer group (``register.py`` wraps the optimizer executables when the resolver spec says so), so
replicas stay bitwise equal.  Role parity: reference ``src/dataflow_training/run/conductor.py:146-452`` and
``run/loop.py:115-436``.
"""
from __future__ import annotations

import dataclasses
import os
import socket
import tempfile
import time
from typing import Any, Callable

from ..distributed import daemons
from ..distributed.ranks import RankState, StepRun
from ..distributed.topology import HostSpec, Member
from .driver import RunResult


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _upload_rounds(state: RankState, packed, first_round: int) -> tuple[dict[int, list[int]], int]:
    """This rank's rounds of a packed step into its daemon's store; returns (sequence bounds per round, bytes)."""
    seq_lens, nbytes = {}, 0
    for r in range(state.rounds):
        rd = packed.rounds[first_round + r]
        state.client.put_object(f"tokens_0_{r}", rd.tokens.tobytes())
        state.client.put_object(f"targets_0_{r}", rd.targets.tobytes())
        nbytes += rd.tokens.nbytes + rd.targets.nbytes
        b = list(rd.bounds)
        if rd.content < len(rd.tokens):
            b.append(len(rd.tokens))          # the tail rides as one masked segment
        seq_lens[r] = b
    return seq_lens, nbytes


def check_fleet_versions(statuses: dict[str, dict], local_rev: str, local_env: str) -> None:
    """Refuse a mixed fleet: every daemon must run the conductor's code (digest of the package's sources) and the conductor's
    framework / CUDA versions.  Skewed code gives structurally mismatched collectives (a hang, or garbage that is summed
    silently); skewed versions make replicas drift.  Role parity: reference ``src/dataflow_training/run/conductor.py:78-142``."""
    for name, st in statuses.items():
        rev, env = st.get("code_rev"), st.get("env")
        if rev != local_rev:
            raise RuntimeError(f"fleet version skew: {name} runs code {rev} but the conductor runs {local_rev} — bring every host to the "
                               f"same revision before a fleet run")
        if env != local_env:
            raise RuntimeError(f"fleet environment skew: {name} runs [{env}] but the conductor runs [{local_env}]")


def run_fleet(spec, log: Callable[[str], None] = print) -> RunResult:
    """Train ``spec`` (a ``conductor.RunSpec`` with ``world`` ranks, replicas) through one daemon per rank on this box."""
    from ..data.pipeline import pipeline_from_args
    from ..lowering.planning import plan_program
    from ..models.families import build_init_program, resolve_family
    from ..register import canonical_spec
    from ..service.client import EngineClient
    from .rank_main import build_cfg
    from .recipe import Recipe

    if spec.parallel not in ("co", "dp"):
        raise ValueError(f"fleet mode runs replicas (--parallel co); {spec.parallel!r} needs the in-process launcher")
    family, cfg = build_cfg(spec)
    fam = resolve_family(family)
    world = int(spec.world)
    recipe = Recipe(**{"total_steps": spec.steps, **spec.recipe})
    hyper = recipe.hyper()
    cpu = spec.device is None
    host = HostSpec(name="local")
    root = tempfile.mkdtemp(prefix="dataflow_fleet_")
    members = [Member("local", 0 if cpu else (spec.devices[r] if spec.devices else r)) for r in range(world)]
    names = [f"rank{r}" for r in range(world)]
    ports = [_free_port() for _ in range(world)]
    # one plan for every rank (replicas run the same program); planned here, on the conductor
    program = plan_program(fam.lower(cfg), None if spec.budget_gib is None else int(spec.budget_gib * 2 ** 30)).program
    rspec = canonical_spec(family, cfg, hyper, seed=spec.seed)
    if world > 1:
        rspec["dp"] = {"mode": "co", "group": "dp"}
    # profile window (--prof-dir with --profile-start-before-step / --profile-stop-after-step): NVTX ranges on in every daemon,
    # each wrapped in the timeline profiler when this machine has one; without one the window still switches the ranges
    window = None
    profiler = None
    if getattr(spec, "prof_dir", None) and int(getattr(spec, "profile_start_before_step", 0) or 0) > 0:
        window = (int(spec.profile_start_before_step), int(spec.profile_stop_after_step or spec.profile_start_before_step))
        os.makedirs(spec.prof_dir, exist_ok=True)
        profiler = daemons.timeline_profiler(host)
        log(f"[fleet] profile window steps {window[0]}..{window[1]}: " + (f"timelines by {profiler}" if profiler else
            "no timeline profiler on this machine; NVTX ranges only"))
    states: list[RankState] = []
    paths = []
    clients: list[Any] = []
    store_gib = max(sum(o.size_bytes for o in program.initial_objects) * 2 / 2 ** 30 + 0.1, 0.2)
    try:
        for r in range(world):
            # every daemon gets its own runtime files: several ranks share a host (and, on CPU, a "device")
            wrap = None
            if window is not None and profiler is not None:
                # the capture window is opened and closed through the daemons' profiler-control verb (below)
                wrap = daemons.timeline_command(profiler, os.path.join(spec.prof_dir, f"timeline_rank{r}"))
            p = daemons.launch(host, members[r], backing_gib=spec.backing_budget_gib or store_gib, kernels=spec.kernels,
                               peer_name=names[r], peer_listen=f"127.0.0.1:{ports[r]}", root=root, tag=f"r{r}",
                               device="cpu" if cpu else str(members[r].device), wrap=wrap,
                               env={"DATAFLOW_NVTX": "1"} if window is not None else None)
            paths.append(p)
            clients.append(EngineClient(p["socket"], f"fleet-rank{r}", timeout=600.0))
            log(f"[fleet] rank {r} up ({'cpu' if cpu else 'cuda:' + str(members[r].device)}, socket {p['socket']})")
        from .. import code_revision, environment_line
        check_fleet_versions({names[r]: c.engine_status() for r, c in enumerate(clients)}, code_revision(), environment_line())
        log(f"[fleet] version handshake ok ({code_revision()}, {environment_line()})")
        if world > 1:
            for r in range(1, world):
                clients[0].peer_connect(names[r], f"127.0.0.1:{ports[r]}")
            g = clients[0].create_peer_group("dp", names, backend="auto", timeout=120.0)
            log(f"[fleet] peer group dp ready: {g['members']} on the {g['backend']} lane")
        R = int(program.metadata.get("grad_accum_rounds", cfg.grad_accum_rounds))
        T = int(program.metadata.get("tokens_per_round", getattr(cfg, "tokens_per_round", 0)))
        loss_ids = sorted(o.id for t in program.tasks for o in t.outputs if o.location == "backing" and o.id.startswith("loss_"))
        init = build_init_program(program)
        for r, c in enumerate(clients):
            for o in init.initial_objects:
                c.create_object(o.id, o.size_bytes)
            ireg = c.register_program(init, rspec)
            c.run(ireg["prog_id"])
            c.unregister_program(ireg["prog_id"])
            reg = c.register_program(program, rspec)
            states.append(RankState(r, c, reg["prog_id"], rounds=R, tokens_per_round=T, loss_ids=loss_ids))
        wide = dataclasses.replace(cfg, grad_accum_rounds=R * world)
        stepper = pipeline_from_args(wide, spec.data, policy=spec.packing_policy, allow_round_split=spec.allow_round_split)(None)
        res = RunResult(tokens_per_step=T * R * world, meta={"family": family, "world": world, "launcher": "fleet",
                                                            "lane": "nccl" if not cpu and world > 1 else "hostmem"})
        try:
            for s in range(spec.steps):
                packed = stepper.next_step()
                if packed is None:
                    log(f"data source exhausted after {s} steps")
                    break
                if window is not None and s + 1 == window[0]:
                    for c in clients:
                        c.profiler_control("start")
                t0 = time.perf_counter()
                jobs = []
                for st in states:
                    seq_lens, _ = _upload_rounds(st, packed, st.rank * R)
                    jobs.append(StepRun(st, s + 1, max(packed.valid_rows, 1), seq_lens))
                for j in jobs:
                    j.start()
                for j in jobs:
                    j.join()
                for j in jobs:
                    if j.error is not None:
                        raise j.error
                loss = float(sum(j.loss for j in jobs))        # every rank holds its share of the step's mean loss
                dt = time.perf_counter() - t0
                res.losses.append(loss)
                res.step_wall_s.append(dt)
                log(f"step {s + 1:5d}  loss {loss:.4f}  {packed.content_tokens / dt:,.0f} tok/s")
                if window is not None and s + 1 == window[1]:
                    for c in clients:
                        c.profiler_control("stop")
        finally:
            if hasattr(stepper, "close"):
                stepper.close()
        if spec.out:
            res.save(spec.out)
        return res
    finally:
        for c in clients:
            try:
                c.shutdown()
            except Exception:       # noqa: BLE001
                pass
            try:
                c.close()
            except Exception:       # noqa: BLE001
                pass
        for r, p in enumerate(paths):
            if not daemons.wait_exit(host, members[r], root, timeout=20.0, tag=f"r{r}"):
                daemons.kill(host, members[r], root, tag=f"r{r}")
