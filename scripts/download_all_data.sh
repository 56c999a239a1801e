#!/bin/bash
# Downloads the genetic databases and model parameters the data pipeline and inference.py can use
# (role of the reference's scripts/download_*.sh).  Usage: scripts/download_all_data.sh <DOWNLOAD_DIR> [full_dbs|reduced_dbs]
set -euo pipefail
if [[ $# -lt 1 ]]; then echo "usage: $0 <DOWNLOAD_DIR> [full_dbs|reduced_dbs]" >&2; exit 1; fi
command -v aria2c >/dev/null || { echo "aria2c is required (apt install aria2)" >&2; exit 1; }
ROOT="$1"; MODE="${2:-full_dbs}"
case "$MODE" in full_dbs|reduced_dbs) ;; *) echo "download mode must be full_dbs or reduced_dbs" >&2; exit 1;; esac
HERE="$(cd "$(dirname "$0")" && pwd)"
"$HERE/download_one.sh" params      "$ROOT"
if [[ "$MODE" == reduced_dbs ]]; then "$HERE/download_one.sh" small_bfd "$ROOT"; else "$HERE/download_one.sh" bfd "$ROOT"; fi
for db in mgnify pdb70 pdb_mmcif uniref30 uniref90 uniprot pdb_seqres; do "$HERE/download_one.sh" "$db" "$ROOT"; done
echo "All data downloaded under $ROOT"
