#!/bin/bash
# usage: scripts/download_pdb_mmcif.sh <DOWNLOAD_DIR>   (one data set; see download_one.sh)
set -euo pipefail
if [[ $# -ne 1 ]]; then echo "usage: $0 <DOWNLOAD_DIR>" >&2; exit 1; fi
"$(cd "$(dirname "$0")" && pwd)/download_one.sh" pdb_mmcif "$1"
