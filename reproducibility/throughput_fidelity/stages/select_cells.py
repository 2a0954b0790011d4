"""Which predicted cells are worth a measurement.  A cell is a (optimizer, sequence length, tokens per round, rounds,
budget) point.  Infeasible cells are out.  From the rest at most ``target`` are taken so that the budget axis and the
regimes the planner can be in are all represented: cells are grouped by geometry, each group ordered by budget, and the
picks go round-robin over the groups taking from each the lowest budget, the highest, then the ones that split the largest
remaining gap in predicted link occupancy (so compute-bound, link-bound and recompute-heavy plans all get measured)."""
from __future__ import annotations


def select_cells(pred: list[dict], target: int) -> list[int]:
    ok = [i for i, r in enumerate(pred) if r.get("s_step")]
    if len(ok) <= target:
        return ok
    groups: dict[tuple, list[int]] = {}
    for i in ok:
        r = pred[i]
        groups.setdefault((r.get("opt"), r["seq"], r["t_round"], r["rounds"]), []).append(i)
    for g in groups.values():
        g.sort(key=lambda i: (pred[i]["budget"] is None, pred[i]["budget"] or 0.0))
    picked: list[int] = []
    taken: dict[tuple, list[int]] = {k: [] for k in groups}

    def next_of(key) -> int | None:
        g, t = groups[key], taken[key]
        rest = [i for i in g if i not in t]
        if not rest:
            return None
        if not t:
            return rest[0]
        if len(t) == 1:
            return rest[-1]
        # the unmeasured cell farthest (in predicted link occupancy) from everything measured in this group
        far = lambda i: min(abs(pred[i].get("link_pct", 0.0) - pred[j].get("link_pct", 0.0)) for j in t)  # noqa: E731
        return max(rest, key=far)

    while len(picked) < target:
        progressed = False
        for key in groups:
            if len(picked) >= target:
                break
            i = next_of(key)
            if i is not None:
                taken[key].append(i)
                picked.append(i)
                progressed = True
        if not progressed:
            break
    return sorted(picked)
