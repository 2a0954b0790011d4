"""The simulator's HTTP routes and the panel data behind its page."""
import pytest

from chains import train_chain
from dataflow_b200.sim import run
from dataflow_b200.sim.app import views
from dataflow_b200.sim.policies import get_all_policies

fastapi = pytest.importorskip("fastapi")


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from dataflow_b200.sim.app.api import create_app
    return TestClient(create_app())


BODY = {"model": "llama3_8b", "training": {"rounds": 2, "tokens_per_round": 8192}, "hardware": "B200", "fast_memory_gib": 60}


def test_residency_spans_add_up_to_the_simulators_ledger():
    planned = get_all_policies()["max_reduce"](train_chain(L=6, rounds=2), 3000)
    log = run(planned, snapshots=True)
    spans = views.residency_spans(planned, log)
    sizes = planned.sizes()
    # at every event the bytes of the objects whose spans cover that instant are what the ledger says (sampled just after)
    times = sorted({ev.t for ev in log.events})
    ledger = {}
    for ev in log.events:
        ledger[ev.t] = ev.fast_bytes                    # the last event at a time wins
    for t in times[:-1]:
        held = sum(sizes[o] for o, ivs in spans.items() if any(a <= t < b for a, b in ivs))
        assert held == ledger[t], t
    at = views.resident_at(planned, log, times[len(times) // 2])
    assert at["fast_bytes"] == ledger[times[len(times) // 2]] and at["objects"][0]["bytes"] >= at["objects"][-1]["bytes"]


def test_memory_by_type_stays_under_the_capacity_and_names_the_types():
    planned = get_all_policies()["min_grow"](train_chain(L=6, rounds=2), 3000)
    log = run(planned, snapshots=True)
    m = views.memory_by_type(planned, log, points=64)
    assert len(m["t_us"]) == 64 and set(m["types"]) >= {"weight", "activation"}
    total = [sum(m["bytes"][n][k] for n in m["types"]) for k in range(64)]
    assert max(total) <= 3000 and max(total) > 0 and m["capacity_bytes"] == 3000


def test_plan_table_and_reference_rows():
    planned = get_all_policies()["lookahead"](train_chain(L=4, rounds=1), 2500)
    log = run(planned)
    rows = views.plan_table(planned, log)
    assert [r["task"] for r in rows] == [t.id for t in planned.tasks] and rows[0]["start_us"] == 0.0
    assert sum(len(r["prefetches"]) for r in rows) == len([iv for iv in log.task_intervals if iv.track == "from_slow"])
    refs = views.reference_rows(planned)
    assert [r["first_touch_us"] for r in refs] == sorted(r["first_touch_us"] for r in refs)
    assert {r["object"] for r in refs} == set(planned.sizes())
    st = views.stall_rows(planned, log)
    assert st["stall_us"] == pytest.approx(sum(log.stalls.values())) and set(st["lanes"]) == {"from_slow", "to_slow"}


def test_simulate_returns_the_requested_panels(client):
    r = client.post("/api/simulate", json={**BODY, "policy": "pressurefit",
                                           "panels": ["plan", "memory_by_type", "residency", "stalls", "references", "candidates"]})
    assert r.status_code == 200, r.text
    j = r.json()
    assert {"plan", "memory_by_type", "residency", "stalls", "references", "candidates", "summary", "timeline"} <= set(j)
    assert j["candidates"]["planner"] == "pressurefit" and j["candidates"]["candidate_count"] == len(j["candidates"]["candidates"])
    assert j["summary"]["compute_pct_by_kind"]["matmul"] > 50 and len(j["summary"]["top_ops"]) == 10
    assert len(j["plan"]) == len([iv for iv in j["timeline"] if iv["track"] == "compute"])
    assert all(s[0] <= s[1] for o in j["residency"] for s in o["spans"])
    # a planner without a search record answers null; an unknown panel is refused
    r2 = client.post("/api/simulate", json={**BODY, "policy": "max_reduce", "panels": ["candidates"], "timeline": False})
    assert r2.status_code == 200 and r2.json()["candidates"] is None
    assert client.post("/api/simulate", json={**BODY, "panels": ["nope"]}).status_code == 422


def test_compare_and_sweep_routes(client):
    r = client.post("/api/compare", json={**BODY, "policies": ["max_reduce", "min_grow", "all_resident", "sliding_window"]})
    assert r.status_code == 200, r.text
    j = r.json()
    rows = {x["policy"]: x for x in j["rows"]}
    assert not rows["all_resident"]["ok"] and "Planning" in rows["all_resident"]["error"]        # 60 GiB does not hold everything
    assert rows["max_reduce"]["ok"] and rows["max_reduce"]["x_lower_bound"] >= 1.0
    assert j["best"] in ("max_reduce", "min_grow") and rows[j["best"]]["makespan_us"] <= rows["sliding_window"]["makespan_us"]
    assert client.post("/api/compare", json={**BODY, "policies": ["nope"]}).status_code == 404
    s = client.post("/api/sweep", json={**BODY, "policy": "max_reduce", "budgets_gib": [8, 40, 80, 160]})
    assert s.status_code == 200, s.text
    pts = s.json()["rows"]
    assert [p["budget_gib"] for p in pts] == [8, 40, 80, 160] and not pts[0]["ok"] and pts[-1]["ok"]
    good = [p["tokens_per_s"] for p in pts if p["ok"]]
    assert good == sorted(good)                          # more memory never makes the plan slower
    assert client.post("/api/sweep", json=BODY).status_code == 422


def test_validate_route_reports_by_stage(client):
    from dataclasses import replace
    from dataflow_b200.sim import TransferTrigger
    good = get_all_policies()["max_reduce"](train_chain(L=4, rounds=1), 3000)
    r = client.post("/api/validate", json={"chain": good.to_dict()})
    assert r.status_code == 200 and r.json()["valid"] and all(s["ran"] and not s["problems"] for s in r.json()["stages"])
    tasks = list(good.tasks)
    k, keeps = next((i, o) for i, t in enumerate(tasks) for o in t.inputs
                    if o not in t.releases_after and all(x.obj_id != o for x in t.offload_after))
    tasks[k] = replace(tasks[k], prefetch_after=tasks[k].prefetch_after + [TransferTrigger(keeps)])    # it is still resident
    bad = client.post("/api/validate", json={"chain": replace(good, tasks=tasks).to_dict()}).json()
    assert not bad["valid"]
    stages = {s["stage"]: s for s in bad["stages"]}
    assert not stages["ids"]["problems"] and stages["transfers"]["problems"][0]["rule"] == "prefetch-already-resident"
    assert stages["transfers"]["problems"][0]["meaning"] and not stages["lifetimes"]["ran"]
    # as a planner's input the same chain is refused for another reason: it already carries a plan (ids and capacity pass)
    assert client.post("/api/validate", json={"chain": good.bare().to_dict(), "planning_input": True}).json()["valid"]
    assert client.post("/api/validate", json={"chain": {"tasks": [{"id": "a"}]}}).status_code == 422


def test_the_page_has_every_panel_and_calls_only_routes_that_exist(client):
    import re
    page = client.get("/").text
    for panel in ("summary", "timeline", "memory", "bytype", "phases", "kinds", "topops", "subops", "plan", "stalls", "candidates",
                  "references", "scrub", "comparison", "sweepplot", "measuredplot"):
        assert f'id="{panel}"' in page, panel
    routes = {r.path for r in client.app.routes}
    for path in set(re.findall(r'"(/api/[a-z/]+)"', page)):
        assert path in routes, path
    # every element the script looks up by id exists in the markup
    for ident in set(re.findall(r'\$\("([A-Za-z_]+)"\)', page)):
        assert f'id="{ident}"' in page, ident
    assert page.count("<script>") == 1
    script = page[page.index("<script>") + 8:page.index("</script>")]
    assert _js_structure_errors(script) == []


def _js_structure_errors(src: str) -> list[str]:
    """Brackets, quotes and template literals of a script balance (no JavaScript engine here: this catches what a typo
    breaks most often).  Regular-expression literals are recognised after ``(``, ``,``, ``=``, ``:`` and ``.replace(``."""
    errs, stack = [], []
    pairs = {")": "(", "]": "[", "}": "{"}
    i, n, line = 0, len(src), 1
    prev = ""                                            # the last significant character outside strings
    while i < n:
        c = src[i]
        if c == "\n":
            line += 1
        top = stack[-1] if stack else ""
        if top == "`":                                    # inside a template literal
            if c == "\\":
                i += 2
                continue
            if c == "`":
                stack.pop()
            elif c == "$" and i + 1 < n and src[i + 1] == "{":
                stack.append("${")
                i += 2
                continue
            i += 1
            continue
        if c in "\"'":
            j = i + 1
            while j < n and src[j] != c:
                if src[j] == "\n":
                    errs.append(f"line {line}: string runs over the end of the line")
                    break
                j += 2 if src[j] == "\\" else 1
            i, prev = j + 1, c
            continue
        if c == "/" and i + 1 < n and src[i + 1] == "/":
            while i < n and src[i] != "\n":
                i += 1
            continue
        if c == "/" and prev in "(,=:" :                 # a regular-expression literal
            j = i + 1
            in_class = False
            while j < n and (src[j] != "/" or in_class):
                if src[j] == "\\":
                    j += 1
                elif src[j] == "[":
                    in_class = True
                elif src[j] == "]":
                    in_class = False
                j += 1
            i, prev = j + 1, "/"
            continue
        if c == "`":
            stack.append("`")
        elif c in "([{":
            stack.append(c)
        elif c in ")]}":
            if c == "}" and top == "${":
                stack.pop()
            elif not stack or stack[-1] != pairs[c]:
                errs.append(f"line {line}: {c!r} closes {top!r}")
                return errs
            else:
                stack.pop()
        if not c.isspace():
            prev = c
        i += 1
    if stack:
        errs.append(f"unclosed {stack}")
    return errs


def test_the_structure_check_sees_a_broken_script():
    assert _js_structure_errors("const f = x => { return `a${x.map(y => `(${y})`).join(\",\")}`; };") == []
    assert _js_structure_errors("const f = x => { return `a${x}; };") != []
    assert _js_structure_errors("f(a, [b, c);") != []
    assert _js_structure_errors("s.replace(/[&<>]/g, c => c)") == []


def test_hardware_overrides_change_the_prediction(client):
    base = client.post("/api/simulate", json={**BODY, "policy": "max_reduce", "timeline": False}).json()["summary"]
    slow = client.post("/api/simulate", json={**BODY, "policy": "max_reduce", "timeline": False, "hardware_overrides": {"from_slow_gbs": 10, "to_slow_gbs": 10}})
    assert slow.status_code == 200 and slow.json()["summary"]["makespan_us"] > base["makespan_us"] * 1.5      # a fifth of the host link
    eff = client.post("/api/simulate", json={**BODY, "policy": "max_reduce", "timeline": False, "hardware_overrides": {"matmul_efficiency": 0.4}}).json()["summary"]
    assert eff["compute_us_by_kind"]["matmul"] > base["compute_us_by_kind"]["matmul"] * 1.5
    assert client.post("/api/simulate", json={**BODY, "hardware_overrides": {"warp_drive": 9}}).status_code == 422


def test_nonsense_inputs_are_refused_with_a_reason_never_a_server_error():
    from fastapi.testclient import TestClient
    from dataflow_b200.sim.app.api import create_app
    c = TestClient(create_app(), raise_server_exceptions=False)
    base = {"model": "llama3_8b", "hardware": "B200", "fast_memory_gib": 60, "policy": "max_reduce", "timeline": False}
    cases = {"rounds": {"training": {"rounds": 0}}, "tokens_per_round": {"training": {"tokens_per_round": 0}},
             "seq_len": {"training": {"seq_len": -4096}}, "cannot hold a sequence": {"training": {"seq_len": 65536, "tokens_per_round": 4096}},
             "dp": {"training": {"parallel": {"dp": 0}}}, "not divisible by tp": {"training": {"parallel": {"tp": 3}}},
             "zero_stage": {"training": {"parallel": {"dp": 8, "zero_stage": 9}}}, "recompute": {"training": {"recompute": "sometimes"}},
             "dtype policy": {"training": {"dtypes": {"compute": "fp3"}}}, "is negative": {"hardware_overrides": {"matmul_efficiency": -1}},
             "negative-size": {"fast_memory_gib": -3}, "bandwidth": {"hardware_overrides": {"from_slow_gbs": 0, "to_slow_gbs": 0}}}
    for needle, over in cases.items():
        r = c.post("/api/simulate", json={**base, **over})
        assert r.status_code in (404, 422), (needle, r.status_code, r.text[:200])
        assert needle in str(r.json()["detail"]), (needle, r.json()["detail"])
    # what is merely unusual still runs: one sequence per round, a budget larger than the device
    assert c.post("/api/simulate", json={**base, "training": {"seq_len": 4096, "tokens_per_round": 4096}}).status_code == 200
    assert c.post("/api/simulate", json={**base, "fast_memory_gib": 1e6}).status_code == 200
