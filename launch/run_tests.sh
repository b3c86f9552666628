#!/usr/bin/env bash
# Test sweeps.  `launch/run_tests.sh cpu` needs no GPU (gloo ranks); `gpu` needs >= 1 B200 (multi-GPU cases skip themselves).
set -euo pipefail
cd "$(dirname "$0")/.."
case "${1:-cpu}" in
  cpu) python -m pytest tests -x -q -m "not gpu" ;;
  gpu) python -c "import __graft_entry__ as g; g.build()" && NCCL_NVLS_ENABLE=0 python -m pytest tests -x -q -m gpu ;;
  all) "$0" cpu && "$0" gpu ;;
  *) echo "usage: $0 [cpu|gpu|all]" >&2; exit 2 ;;
esac
