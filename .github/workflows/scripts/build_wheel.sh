#!/bin/bash
# Builds dist/fastfold_b200-*.whl with the native library inside (setup.py compiles it before packaging).
set -euo pipefail
python3 -m venv /opt/venv
/opt/venv/bin/pip install --upgrade pip wheel setuptools
/opt/venv/bin/pip install torch --index-url https://download.pytorch.org/whl/cu128
/opt/venv/bin/pip install numpy einops scipy
/opt/venv/bin/python setup.py bdist_wheel
ls -l dist/
