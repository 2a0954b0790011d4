"""List every registered family with its presets and headline dimensions.

    python tools/gen_model_docs/list_models.py [--json]

Reference role: ``tools/gen_model_docs/list_models.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from _cli import table  # noqa: E402


def model_rows():
    from dataflow_b200.models.families import all_families
    rows = []
    for name, fam in sorted(all_families().items()):
        for preset, make in sorted(fam.presets.items()):
            cfg = make()
            lay = fam.family_layouts(fam.derive_dims(cfg))
            n_params = (lay.block_w.size_bytes * cfg.n_layers + lay.embed_w.size_bytes + lay.head_w.size_bytes) // 2
            rows.append({"family": name, "preset": preset, "layers": cfg.n_layers, "d_model": cfg.d_model, "vocab": getattr(cfg, "vocab_size", None),
                         "seq_len": cfg.seq_len, "experts": getattr(cfg, "n_experts", 0) or None, "params_m": n_params / 1e6})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rows = model_rows()
    if a.json:
        print(json.dumps(rows, indent=1))
    else:
        print(table(rows, [("family", "{}"), ("preset", "{}"), ("layers", "{}"), ("d_model", "{}"), ("vocab", "{}"), ("seq_len", "{}"),
                           ("experts", "{}"), ("params_m", "{:.1f}")]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
