"""Recording stand-ins for the alignment tools (jackhmmer, hhblits, hhsearch, hmmbuild, hmmsearch, kalign): shell scripts
that append their command line to the file named by ``$RECORD`` (when set) and write minimal, well-formed output files
where the wrappers expect them.  ``STANDIN_QUERY`` sets the sequence the fake alignments are built around."""
import os
import stat

SCRIPT = r"""#!/bin/bash
if [ -n "$RECORD" ]; then echo "$(basename "$0") $*" >> "$RECORD"; fi
q=${STANDIN_QUERY:-ACDEFGHIKL}
args=("$@")
prev=${args[$((${#args[@]}-2))]}
fasta=""
for a in "$@"; do case "$a" in *.fasta|*.fa) if [ -z "$fasta" ] && [ -f "$a" ]; then fasta="$a"; fi ;; esac; done
if [ -n "$fasta" ]; then s=$(grep -v '^>' "$fasta" | tr -d '\n'); if [ -n "$s" ] && [ ${#s} -lt 400 ]; then q=$s; fi; fi
rf=$(printf 'x%.0s' $(seq 1 ${#q}))
case "$(basename "$0")" in
  hmmbuild) printf 'HMMER3/f [stand-in]\n//\n' > "$prev" ;;
esac
while [ $# -gt 0 ]; do
  case "$1" in
    -A) printf '# STOCKHOLM 1.0\n\nquery %s\nhit1  %s\n#=GC RF %s\n//\n' "$q" "${q:0:${#q}-1}A" "$rf" > "$2" ;;
    --tblout) printf '# target\nhit1 - query - 1e-5 10 0\n' > "$2" ;;
    -oa3m) printf '>query\n%s\n>hit1\n%s\n' "$q" "${q:0:${#q}-1}A" > "$2" ;;
    -o) if [ "$2" != "/dev/null" ]; then
          case "$(basename "$0")" in
            kalign) printf '>a\nACDEFGHIKL\n>b\nACDE-GHIKL\n' > "$2" ;;
            *) printf 'Query         query\nMatch_columns %d\n\n' ${#q} > "$2" ;;
          esac
        fi ;;
  esac
  shift
done
"""

TOOLS = ("jackhmmer", "hhblits", "hhsearch", "hmmbuild", "hmmsearch", "kalign")


def make_tool_standins(directory):
    """Writes one executable per tool into ``directory``; returns ``{tool name: path}``."""
    os.makedirs(directory, exist_ok=True)
    out = {}
    for name in TOOLS:
        path = os.path.join(str(directory), name)
        with open(path, "w") as fh:
            fh.write(SCRIPT)
        os.chmod(path, os.stat(path).st_mode | stat.S_IEXEC)
        out[name] = path
    return out
