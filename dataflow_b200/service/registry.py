"""Resolver registry of the service: ``kind`` → builder of a task resolver.  A registered program
carries a ``resolver_spec`` (JSON); the daemon looks only at ``spec["kind"]`` and caches the built
resolver by the spec's canonical JSON.  Includes the debug ``JitterResolver`` (random extra busy time
per task: proves results are event-driven, not timing-driven).  Parity: reference
``src/dataflow/service/registry.py:27-117``."""
from __future__ import annotations

import random
from typing import Any, Callable, Mapping

from ..core.jsonio import canonical_json
from ..runtime.executable import SyntheticExecutable
from .wire import ServiceError

_BUILDERS: dict[str, Callable[[Mapping[str, Any], Any], Callable]] = {}
_CACHE: dict[str, Callable] = {}


def register_program_resolver(kind: str, build: Callable[[Mapping[str, Any], Any], Callable]) -> None:
    """``build(spec, env) -> resolver(task) -> Executable``; ``env`` carries device / kernel set."""
    _BUILDERS[kind] = build
    for k in [k for k in _CACHE if f'"kind":"{kind}"' in k]:
        del _CACHE[k]


def list_resolvers() -> list[str]:
    return sorted(_BUILDERS)


def lookup_resolver(spec: Mapping[str, Any] | None, env=None):
    if not spec:
        return None
    kind = spec.get("kind")
    if kind not in _BUILDERS:
        raise ServiceError("BAD_REQUEST", f"no resolver registered for kind {kind!r}; known: {list_resolvers()}")
    key = canonical_json(dict(spec)) + f"|{getattr(env, 'device', None)}|{getattr(env, 'kernel_set', None)}"
    r = _CACHE.get(key)
    if r is None:
        r = _CACHE[key] = _BUILDERS[kind](spec, env)
    return r


class JitterExecutable:
    """Synthetic task whose busy time is its planned runtime times a random factor."""

    def __init__(self, rng: random.Random, spread: float):
        self.rng, self.spread = rng, spread

    def launch(self, ctx) -> None:
        f = 1.0 + self.rng.uniform(-self.spread, self.spread)
        ctx.backend.busy(0, float(ctx.task.runtime_us) * max(f, 0.0))


class JitterResolver:
    def __init__(self, seed: int = 0, spread: float = 0.5):
        self.rng = random.Random(seed)
        self.spread = spread

    def __call__(self, task):
        return JitterExecutable(self.rng, self.spread)


register_program_resolver("synthetic", lambda spec, env: (lambda task: SyntheticExecutable()))
register_program_resolver("jitter", lambda spec, env: JitterResolver(int(spec.get("seed", 0)), float(spec.get("spread", 0.5))))
