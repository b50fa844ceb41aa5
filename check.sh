#!/bin/bash
# Static checks (reference check.sh: flake8 + mypy + formatting).  Tools that are not installed are skipped.
set -u
cd "$(dirname "$0")"
rc=0
python -m compileall -q pippy_b200 examples tests bench.py __graft_entry__.py || rc=1
if python -c "import flake8" 2>/dev/null; then python -m flake8 --max-line-length 120 pippy_b200 || rc=1; fi
if python -c "import black" 2>/dev/null; then python -m black --check -l 120 pippy_b200 tests examples || rc=1; fi
python - <<'PY' || rc=1
# every CUDA source must compile for sm_100a
import __graft_entry__ as g
g.build()
PY
exit $rc
