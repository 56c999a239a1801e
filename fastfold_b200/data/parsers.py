"""Parsers for the text formats of the alignment tools: FASTA, A3M, Stockholm, HHR (role of fastfold/data/parsers.py)."""
import collections
import dataclasses
import re
import string
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

DeletionMatrix = Sequence[Sequence[int]]


@dataclasses.dataclass(frozen=True)
class TemplateHit:
    index: int
    name: str
    aligned_cols: int
    sum_probs: Optional[float]
    query: str
    hit_sequence: str
    indices_query: List[int]
    indices_hit: List[int]


def parse_fasta(fasta_string: str) -> Tuple[List[str], List[str]]:
    sequences, descriptions = [], []
    idx = -1
    for line in fasta_string.splitlines():
        line = line.strip()
        if line.startswith(">"):
            idx += 1
            descriptions.append(line[1:])
            sequences.append("")
        elif line and idx >= 0:
            sequences[idx] += line
    return sequences, descriptions


def parse_a3m(a3m_string: str) -> Tuple[List[str], DeletionMatrix, List[str]]:
    """Aligned sequences (lower-case insertions removed), per-position deletion counts, descriptions."""
    sequences, descriptions = parse_fasta(a3m_string)
    deletion_matrix = []
    for seq in sequences:
        vec, count = [], 0
        for ch in seq:
            if ch.islower():
                count += 1
            else:
                vec.append(count)
                count = 0
        deletion_matrix.append(vec)
    table = str.maketrans("", "", string.ascii_lowercase)
    return [s.translate(table) for s in sequences], deletion_matrix, descriptions


def parse_stockholm(stockholm_string: str) -> Tuple[List[str], DeletionMatrix, List[str]]:
    name_to_seq = collections.OrderedDict()
    for line in stockholm_string.splitlines():
        line = line.strip()
        if not line or line.startswith(("#", "//")):
            continue
        name, seq = line.split()
        name_to_seq[name] = name_to_seq.get(name, "") + seq
    msa, deletion_matrix = [], []
    query, keep = "", []
    for i, seq in enumerate(name_to_seq.values()):
        if i == 0:
            query = seq
            keep = [j for j, r in enumerate(query) if r != "-"]
        msa.append("".join(seq[j] for j in keep))
        vec, count = [], 0
        for s, q in zip(seq, query):
            if s != "-" or q != "-":
                if q == "-":
                    count += 1
                else:
                    vec.append(count)
                    count = 0
        deletion_matrix.append(vec)
    return msa, deletion_matrix, list(name_to_seq.keys())


def convert_stockholm_to_a3m(stockholm_format: str, max_sequences: Optional[int] = None) -> str:
    msa, _, names = parse_stockholm(stockholm_format)
    if max_sequences:
        msa, names = msa[:max_sequences], names[:max_sequences]
    return "\n".join(">%s\n%s" % (n, s) for n, s in zip(names, msa)) + "\n"


def deduplicate_stockholm_msa(stockholm_msa: str) -> str:
    seen, keep = set(), set()
    for line in stockholm_msa.splitlines():
        if line.strip() and not line.startswith(("#", "//")):
            name, seq = line.split()
            if seq not in seen:
                seen.add(seq)
                keep.add(name)
    out = []
    for line in stockholm_msa.splitlines():
        if not line.strip() or line.startswith("//") or line.startswith("# STOCKHOLM"):
            out.append(line)
        elif line.startswith("#"):
            parts = line.split()
            if len(parts) > 1 and (parts[1] in keep or parts[0] == "#=GC"):
                out.append(line)
        elif line.split()[0] in keep:
            out.append(line)
    return "\n".join(out) + "\n"


def _iter_hhr_hits(lines):
    starts = [i for i, l in enumerate(lines) if l.startswith("No ")]
    for a, b in zip(starts, starts[1:] + [len(lines)]):
        yield lines[a:b]


def parse_hhr(hhr_string: str) -> Sequence[TemplateHit]:
    """Hits of an HH-suite result file with the aligned residue indices of query and template."""
    hits = []
    for block in _iter_hhr_hits(hhr_string.splitlines()):
        number = int(block[0].split()[-1])
        name = block[1][1:]
        m = re.search(r"Aligned_cols=(\d+).*Sum_probs=([0-9.]+)", block[2])
        aligned_cols, sum_probs = (int(m.group(1)), float(m.group(2))) if m else (0, None)
        query, hit, iq, ih = "", "", [], []
        for line in block[3:]:
            if line.startswith("Q ") and not line.startswith(("Q ss_", "Q Consensus")):
                parts = line.split()
                qstart, qseq = int(parts[2]) - 1, parts[3]
                query += qseq
                pos = qstart
                for ch in qseq:
                    iq.append(-1 if ch == "-" else pos)
                    pos += ch != "-"
            elif line.startswith("T ") and not line.startswith(("T ss_", "T Consensus")):
                parts = line.split()
                tstart, tseq = int(parts[2]) - 1, parts[3]
                hit += tseq
                pos = tstart
                for ch in tseq:
                    ih.append(-1 if ch == "-" else pos)
                    pos += ch != "-"
        hits.append(TemplateHit(number, name, aligned_cols, sum_probs, query, hit, iq, ih))
    return hits
