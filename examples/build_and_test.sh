#!/usr/bin/env bash
# Builds the native library for sm_100a in-tree and runs the test tiers.
# usage: build_and_test.sh [cpu|gpu|all]      (default: cpu; gpu needs at least one B200)
set -euo pipefail
cd "$(dirname "$0")/.."
TIER=${1:-cpu}
python -c "import __graft_entry__ as g; g.build()"
case "$TIER" in
  cpu) python -m pytest tests -x -q -m "not gpu" ;;
  gpu) python -m pytest tests -x -q -m gpu ;;
  all) python -m pytest tests -x -q -m "not gpu" && python -m pytest tests -x -q -m gpu ;;
  *) echo "unknown tier: $TIER" >&2; exit 2 ;;
esac
