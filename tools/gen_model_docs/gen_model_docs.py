"""Generate the model reference pages: one Markdown file per family (presets, packed weight fields, the stage list of a
block, the task grammar of one step, the ops it uses) plus an index.

    python tools/gen_model_docs/gen_model_docs.py --out docs/models

Reference role: ``tools/gen_model_docs/gen_model_docs.py`` and ``gen_model_page.py``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import _cli  # noqa: E402,F401


def family_page(name: str) -> str:
    from dataflow_b200.models.families import resolve_family
    fam = resolve_family(name)
    preset = "tiny" if "tiny" in fam.presets else sorted(fam.presets)[0]
    cfg = fam.presets[preset]()
    dims = fam.derive_dims(cfg)
    lay = fam.family_layouts(dims)
    prog = fam.lower(cfg)
    out = [f"# {name}", "", f"Presets: {', '.join(f'`{p}`' for p in sorted(fam.presets))}", "", f"## Packed block weights (`{preset}`)", "",
           "| field | shape | dtype | kind |", "|---|---|---|---|"]
    out += [f"| {f.name} | {tuple(f.shape)} | {f.dtype} | {f.kind} |" for f in lay.block_w.fields]
    out += ["", "## Saved context of one block", "", "| field | shape | dtype |", "|---|---|---|"]
    out += [f"| {f.name} | {tuple(f.shape)} | {f.dtype} |" for f in lay.ctx.fields]
    keys = []
    for t in prog.tasks:
        if t.compute_block_key not in keys:
            keys.append(t.compute_block_key)
    out += ["", "## Task grammar of one step", "", "Compute keys in first-use order: " + ", ".join(f"`{k}`" for k in keys), "",
            f"{len(prog.tasks)} tasks for {cfg.grad_accum_rounds} round(s) of {cfg.n_layers} layers; objects: "
            + ", ".join(sorted({o.split('_')[0] for o in prog.object_sizes()})), ""]
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--out", default="docs/models")
    a = ap.parse_args(argv)
    from dataflow_b200.models.families import all_families
    os.makedirs(a.out, exist_ok=True)
    names = sorted(all_families())
    for n in names:
        open(os.path.join(a.out, f"{n}.md"), "w").write(family_page(n))
    open(os.path.join(a.out, "index.md"), "w").write("# Model families\n\n" + "\n".join(f"- [{n}]({n}.md)" for n in names) + "\n")
    print(f"wrote {len(names) + 1} pages to {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
