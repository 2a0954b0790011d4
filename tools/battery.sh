#!/usr/bin/env bash
# Cross-box validation battery: copy the tree to a remote host and run the CPU suite, the GPU suite (when the host has
# a GPU), the structural gates and a short bench there.
#   tools/battery.sh <remote-host> <remote-path>        # over ssh + rsync
#   tools/battery.sh local                              # the same battery on this machine
# Role of the reference's tools/battery.sh.
set -euo pipefail
run_battery='
set -e
python -c "import __graft_entry__ as g; g.build()"
python -m pytest tests -x -q -m "not gpu"
if python -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  python -m pytest tests -x -q -m gpu
  python bench.py --steps 3 --warmup 3
fi
python tools/verify/sweep_ladder3.py
python tools/verify/pressure_correctness.py --budgets 0.03,0.02
python tools/bench/pressurefit_exact_oracle.py --chains 5 --tasks 6
python tools/bench/planner_quality_gate.py --quick --check
python bench.py --plan-only
'
if [ "${1:-}" = "local" ]; then
  cd "$(dirname "$0")/.." && bash -c "$run_battery"
  exit 0
fi
host="${1:?remote host}"; path="${2:?remote path}"
rsync -a --delete --exclude .git --exclude _work "$(dirname "$0")/../" "$host:$path/"
ssh "$host" "cd '$path' && bash -c '$run_battery'"
