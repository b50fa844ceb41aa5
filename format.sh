#!/bin/bash
# Formats the Python sources in place (reference format.sh drives ufmt / black the same way).
cd "$(dirname "$0")"
if python -c "import black" 2>/dev/null; then python -m black -l 120 pippy_b200 tests examples bench.py; else echo "black is not installed"; fi
