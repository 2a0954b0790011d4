"""The layout registry (keyed, validated field tables with pinned digests) and parameter initialisation as data."""
import dataclasses
import json
import os
from pathlib import Path

import pytest
import torch

from dataflow_b200.blocks.init_policy import InitPolicy, InitRule, build_init_policy, register_init_rule
from dataflow_b200.blocks.layout_registry import describe, layouts_digest, registered_layouts, validate
from dataflow_b200.models.families import all_families, resolve_family

FIXTURE = Path(__file__).parent / "fixtures" / "layout_digests.json"


def test_every_family_registers_well_formed_layouts():
    for name, fam in sorted(all_families().items()):
        reg = registered_layouts(fam, fam.presets["tiny"]())
        assert f"{name}/embed" in reg and f"{name}/head" in reg and len(reg) >= 3
        for e in reg.values():
            assert validate(e) == [], e.key
        roots = sorted(r for e in reg.values() for r in e.roots)
        assert len(roots) == len(set(roots))                      # every weight object is backed by exactly one entry


def test_kinds_group_layers_and_fields_are_addressable():
    fam = resolve_family("glm52")
    reg = registered_layouts(fam, fam.presets["tiny"]())
    kinds = {e.kind for e in reg.values()} - {"embed", "head"}
    assert kinds == {"gdl", "gdf", "gml", "gmf"}                 # dense / moe x leader / follower
    lead, follow = reg["glm52/gml"], reg["glm52/gmf"]
    assert lead.field("wi_q")[4] > 0
    with pytest.raises(KeyError):
        follow.field("wi_q")                                      # followers carry no indexer
    name, shape, dtype, off, size, role, init = lead.field("w_router")
    assert off % 256 == 0 and size == shape[0] * shape[1] * 2 and dtype == "bf16"


def test_layout_digests_are_pinned():
    from dataflow_b200.models.families import _BUILTIN                 # plugins registered by other tests are not pinned
    now = {name: layouts_digest(fam, fam.presets["tiny"]()) for name, fam in sorted(all_families().items()) if name in _BUILTIN}
    if os.environ.get("DATAFLOW_REGEN_HASHES"):
        FIXTURE.write_text(json.dumps(now, indent=1, sort_keys=True) + "\n")
    pinned = json.loads(FIXTURE.read_text())
    assert now == pinned, "weight layouts changed: regenerate the fixture (DATAFLOW_REGEN_HASHES=1) if that is intended"
    assert describe("llama3", resolve_family("llama3").presets["tiny"]())["llama3/block"]["fields"][0][0] == "attn_norm"


def _weights(hyper=None, seed=3):
    from dataflow_b200.run.driver import Trainer
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper={"lr": 1e-3, **(hyper or {})}, seed=seed)
    tr.sync_to_host()
    sd = {k: v.clone() for k, v in fam.bridge(cfg, tr.views_of).items()}
    tr.close()
    return sd


def test_default_policy_is_the_layouts_own_tags_and_rules_override_by_name_and_layer():
    base = _weights()
    again = _weights({"init_policy": None})
    assert all(torch.equal(base[k], again[k]) for k in base)                       # no policy = the tags, byte for byte
    spec = {"default": {"rule": "normal", "args": {"std": 0.1}},
            "overrides": [["*_norm", {"rule": "constant", "args": {"value": 1.0}}],
                          ["w2", {"rule": "scaled_normal", "args": {"std": 0.02, "divide_by": 4.0}}]],
            "layer_overrides": [[[1], {"default": {"rule": "constant", "args": {"value": 0.25}}}]]}
    got = _weights({"init_policy": spec})
    assert torch.all(got["layers.0.attn_norm"] == 1.0) and torch.all(got["final_norm"] == 1.0)
    assert float(got["layers.0.w_qkv"].std()) == pytest.approx(0.1, rel=0.05)
    assert float(got["layers.0.w2"].std()) == pytest.approx(0.005, rel=0.05)
    assert torch.all(got["layers.1.w_qkv"] == 0.25) and torch.all(got["layers.1.attn_norm"] == 0.25)    # layer 1: its sub-policy, entirely
    assert float(got["wte"].std()) == pytest.approx(0.1, rel=0.05)
    assert build_init_policy(spec).to_dict()["layer_overrides"][0][0] == [1]


def test_init_rules_are_a_registry_of_names():
    register_init_rule("ramp", lambda scale=1.0: (lambda n, gen: torch.arange(n, dtype=torch.float32) * scale))
    pol = InitPolicy(overrides=(("final_norm", InitRule("ramp", {"scale": 2.0})),))
    got = _weights({"init_policy": pol})
    assert got["final_norm"][:3].tolist() == [0.0, 2.0, 4.0]
    with pytest.raises(KeyError, match="unknown init rule"):
        InitRule("nope").build()
