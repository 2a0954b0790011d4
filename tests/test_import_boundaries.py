"""Layering rules of the package, enforced.

Engine side: ``core`` (the IR), ``runtime`` (the executor), ``service`` (the daemon), ``checkpoint`` (the record layer).
Planner: ``sim``.  Workload side: everything else (``ops``, ``blocks``, ``models``, ``lowering``, ``distributed``, ``data``,
``run``, ``parallel``, ``testing``).

Run-time checks use a fresh interpreter each, so an earlier import cannot mask a transitive leak:
- ``core`` drags in nothing heavy (no torch, no numpy, no simulator);
- ``runtime`` never imports torch or the simulator (tensors are reached lazily through ``runtime.interop``);
- ``blocks`` does not pull in the simulator.

Static checks scan every import statement with ``ast`` (a mention in a docstring is naturally fine):
- R1: no engine-side module imports a workload package: the engine never sees model vocabulary;
- R2: workload modules reach the engine only through its public surfaces;
- R3: the simulator is imported at module top level only where planning lives (``lowering``, ``run``, the planner's own
  package and the bridge in ``core.convert`` is lazy): everywhere else it is a lazy in-function import, so a deployment
  that only executes planned programs does not need it.
Parity: reference ``tests/test_import_boundaries.py`` (R1-R4 of ``docs/architecture.md``).
"""
import ast
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "dataflow_b200"
ENGINE = ("core", "runtime", "service", "checkpoint")
WORKLOAD = ("ops", "blocks", "models", "lowering", "distributed", "data", "run", "parallel", "testing")
# what the workload may import from the engine side
ENGINE_SURFACES = (
    "dataflow_b200.core", "dataflow_b200.runtime", "dataflow_b200.checkpoint", "dataflow_b200.service",
    "dataflow_b200.service.client", "dataflow_b200.service.registry", "dataflow_b200.service.wire",
    "dataflow_b200.service.server",
    "dataflow_b200.service.snapshots",      # the snapshot file format (dataflow-snapshot/v1) is a documented schema
)
SIM_TOP_LEVEL_OK = ("lowering", "run", "sim")


def fresh_modules(statement: str) -> set[str]:
    """Modules that ``statement`` adds to a fresh interpreter (what the interpreter's own start-up hooks load is not
    the statement's doing)."""
    code = f"import sys\nbefore = set(sys.modules)\n{statement}\nprint('\\n'.join(sorted(set(sys.modules) - before)))"
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return set(r.stdout.split())


def imports_of(path: Path, top_level_only: bool = False):
    """(absolute module name, line) for every import statement of ``path``; relative imports are resolved."""
    tree = ast.parse(path.read_text())
    pkg_parts = list(path.relative_to(ROOT).with_suffix("").parts)
    if pkg_parts[-1] == "__init__":
        pkg_parts = pkg_parts[:-1]
    else:
        pkg_parts = pkg_parts[:-1]
    nodes = tree.body if top_level_only else list(ast.walk(tree))
    out = []
    for n in nodes:
        if isinstance(n, ast.Import):
            out += [(a.name, n.lineno) for a in n.names]
        elif isinstance(n, ast.ImportFrom):
            if n.level:
                base = pkg_parts[:len(pkg_parts) - (n.level - 1)]
                mod = ".".join(base + ([n.module] if n.module else []))
                # ``from . import x`` / ``from .. import y``: the names are submodules
                if not n.module:
                    out += [(mod + "." + a.name, n.lineno) for a in n.names]
                    continue
            else:
                mod = n.module or ""
            out.append((mod, n.lineno))
    return out


def side_of(module: str) -> str | None:
    parts = module.split(".")
    if parts[0] != "dataflow_b200" or len(parts) < 2:
        return None
    return parts[1]


def py_files(sub: str):
    return sorted((PKG / sub).rglob("*.py"))


def test_core_is_dependency_free():
    mods = fresh_modules("import dataflow_b200.core")
    heavy = {m for m in mods if m.split(".")[0] in ("torch", "numpy", "jax", "cuda")} | {m for m in mods if m.startswith("dataflow_b200.sim")}
    assert not heavy, sorted(heavy)[:10]


def test_runtime_never_imports_torch_or_the_simulator():
    mods = fresh_modules("import dataflow_b200.runtime")
    bad = {m for m in mods if m.split(".")[0] in ("torch", "jax")} | {m for m in mods if m.startswith("dataflow_b200.sim")}
    assert not bad, sorted(bad)[:10]


def test_blocks_never_import_the_simulator():
    mods = fresh_modules("import dataflow_b200.blocks")
    assert not {m for m in mods if m.startswith("dataflow_b200.sim")}


def test_engine_never_imports_the_workload():
    leaks = []
    for sub in ENGINE:
        for f in py_files(sub):
            for mod, line in imports_of(f):
                if side_of(mod) in WORKLOAD:
                    leaks.append(f"{f.relative_to(ROOT)}:{line} imports {mod}")
    assert not leaks, "\n".join(leaks)


def test_workload_uses_engine_public_surfaces_only():
    leaks = []
    for sub in WORKLOAD:
        for f in py_files(sub):
            for mod, line in imports_of(f):
                if side_of(mod) not in ENGINE:
                    continue
                ok = mod in ENGINE_SURFACES or mod.startswith(("dataflow_b200.core.", "dataflow_b200.runtime.", "dataflow_b200.checkpoint."))
                if not ok:
                    leaks.append(f"{f.relative_to(ROOT)}:{line} imports {mod}")
    assert not leaks, "\n".join(leaks)


def test_simulator_is_required_only_where_planning_lives():
    leaks = []
    for sub in ENGINE + WORKLOAD:
        if sub in SIM_TOP_LEVEL_OK:
            continue
        for f in py_files(sub):
            for mod, line in imports_of(f, top_level_only=True):
                if side_of(mod) == "sim":
                    leaks.append(f"{f.relative_to(ROOT)}:{line} imports {mod} at module top level")
    assert not leaks, "\n".join(leaks)
