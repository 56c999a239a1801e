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


def _stockholm_line_kept(line: str, names) -> bool:
    """Which lines of a Stockholm file survive when only the sequences in ``names`` are kept: blank lines, the header, the
    terminator and the reference annotation always; ``#=GS`` descriptions and alignment rows of kept sequences; no other
    markup."""
    text = line.strip()
    if not text or text == "//" or line.startswith("# STOCKHOLM") or line.startswith("#=GC RF"):
        return True
    if line.startswith("#=GS"):
        return line.split(maxsplit=2)[1] in names
    if line.startswith("#"):
        return False
    return line.partition(" ")[0] in names


def deduplicate_stockholm_msa(stockholm_msa: str) -> str:
    """Keeps the first of every set of sequences that are equal once the columns the query (first sequence) has a gap in
    are ignored; rows are joined over the blocks of the file first (fastfold/data/parsers.py:354-386)."""
    rows: Dict[str, str] = {}
    for line in stockholm_msa.splitlines():
        if line.strip() and not line.startswith(("#", "//")):
            name, part = line.split()
            rows[name] = rows.get(name, "") + part
    if not rows:
        return stockholm_msa
    query = next(iter(rows.values()))
    match_cols = [i for i, ch in enumerate(query) if ch != "-"]
    seen, keep = set(), set()
    for name, row in rows.items():
        key = "".join(row[i] for i in match_cols if i < len(row))
        if key not in seen:
            seen.add(key)
            keep.add(name)
    return "\n".join(ln for ln in stockholm_msa.splitlines() if _stockholm_line_kept(ln, keep)) + "\n"


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


# ---------------------------------------------------------------------------
# Stockholm utilities used by the alignment runner (fastfold/data/parsers.py:186-330)
# ---------------------------------------------------------------------------
def _keep_stockholm_lines(lines: Iterable[str], names: set) -> str:
    """Header, per-file annotations and every line that belongs to one of ``names``."""
    out = []
    for line in lines:
        s = line.strip()
        if not s or s.startswith("//") or s.startswith("# STOCKHOLM"):
            continue
        if s.startswith("#=GS") or s.startswith("#=GR"):
            if s.split()[1] in names:
                out.append(line.rstrip("\n"))
        elif s.startswith("#"):
            out.append(line.rstrip("\n"))          # #=GF / #=GC apply to the whole alignment
        elif s.split()[0] in names:
            out.append(line.rstrip("\n"))
    return "# STOCKHOLM 1.0\n" + "\n".join(out) + "\n//\n"


def truncate_stockholm_msa(stockholm_msa_path: str, max_sequences: int) -> str:
    """The first ``max_sequences`` sequences of a (possibly huge) Stockholm file, read in two streaming passes."""
    names = set()
    with open(stockholm_msa_path) as f:
        for line in f:
            s = line.strip()
            if s and not s.startswith(("#", "//")):
                names.add(s.split()[0])
                if len(names) >= max_sequences:
                    break
    with open(stockholm_msa_path) as f:
        return _keep_stockholm_lines(f, names)


def remove_empty_columns_from_stockholm_msa(stockholm_msa: str) -> str:
    """Drops the columns in which every sequence has a gap.  A file is processed chunk by chunk, a chunk being the alignment
    rows up to and including their ``#=GC RF`` line, which is trimmed with them; a chunk left without columns becomes empty
    lines (fastfold/data/parsers.py:314-351)."""
    lines = stockholm_msa.splitlines()
    out = list(lines)
    chunk = []                                   # indices of the alignment rows collected since the last annotation line
    for i, line in enumerate(lines):
        if line.startswith("#=GC RF"):
            width = len(line.rpartition(" ")[2])
            datas = [lines[j].rpartition(" ")[2] for j in chunk]
            keep = [c for c in range(width) if any(d[c] != "-" for d in datas)]
            for j in chunk + [i]:
                head, _, data = lines[j].rpartition(" ")
                out[j] = (head + " " + "".join(data[c] for c in keep)) if keep else ""
            chunk = []
        elif line.strip() and not line.startswith(("#", "//")):
            chunk.append(i)
    return "\n".join(out)


def convert_stockholm_to_a3m(stockholm_format: str, max_sequences: Optional[int] = None, remove_first_row_gaps: bool = True) -> str:
    """Stockholm -> A3M: columns that are gaps in the query become lower-case insertions in the other rows."""
    descriptions, sequences = {}, collections.OrderedDict()
    for line in stockholm_format.splitlines():
        s = line.strip()
        if not s or s.startswith("//"):
            continue
        if s.startswith("#=GS"):
            parts = s.split(maxsplit=3)
            if len(parts) == 4 and parts[2] == "DE":
                descriptions[parts[1]] = parts[3]
            continue
        if s.startswith("#"):
            continue
        name, seq = s.split()
        if name not in sequences:
            if max_sequences and len(sequences) >= max_sequences:
                continue
            sequences[name] = ""
        sequences[name] += seq
    if not sequences:
        return ""
    query = next(iter(sequences.values()))
    out = []
    for name, seq in sequences.items():
        if remove_first_row_gaps:
            chars = []
            for q, c in zip(query, seq):
                if q != "-":
                    chars.append(c)
                elif c != "-":
                    chars.append(c.lower())
            seq = "".join(chars)
        else:
            seq = seq.replace(".", "")
        out.append(">%s %s\n%s" % (name, descriptions.get(name, ""), seq))
    return "\n".join(out) + "\n"


def parse_e_values_from_tblout(tblout: str) -> Dict[str, float]:
    e_values = {"query": 0.0}
    for line in tblout.splitlines():
        if line and not line.startswith("#"):
            f = line.split()
            e_values[f[0]] = float(f[4])
    return e_values


def _hmmsearch_description(desc: str):
    """``<pdb>_<chain>/<start>-<end> mol:protein length:<n>  <text>`` -> (name, start, end, length)."""
    m = re.match(r"^([a-zA-Z\d]{4}_[a-zA-Z0-9.]+)/(\d+)-(\d+).*?length:(\d+)", desc.strip())
    if not m:
        raise ValueError("Could not parse hmmsearch description %r" % desc)
    return m.group(1), int(m.group(2)), int(m.group(3)), int(m.group(4))


def parse_hmmsearch_a3m(query_sequence: str, a3m_string: str, skip_first: bool = True) -> Sequence[TemplateHit]:
    """Template hits from an hmmsearch alignment converted to A3M (multimer template search)."""
    seqs, descs = parse_fasta(a3m_string)
    pairs = list(zip(seqs, descs))[1 if skip_first else 0:]
    iq = [-1 if ch == "-" else i for i, ch in enumerate(query_sequence)]
    hits = []
    for i, (seq, desc) in enumerate(pairs, 1):
        if "mol:protein" not in desc:
            continue
        name, start, _, _ = _hmmsearch_description(desc)
        aligned = sum(1 for ch in seq if ch.isupper())
        ih, pos = [], start - 1
        for ch in seq:
            if ch == "-":
                ih.append(-1)
            else:
                ih.append(pos)
                pos += 1
        upper = seq.upper()
        # insertions relative to the query (lower case) have no query column: drop them from the pairing
        cols = [k for k, ch in enumerate(seq) if not ch.islower()]
        hits.append(TemplateHit(i, name, aligned, None, query_sequence, "".join(upper[k] for k in cols), iq, [ih[k] for k in cols]))
    return hits


def parse_hmmsearch_sto(output_string: str, input_sequence: str) -> Sequence[TemplateHit]:
    """Template hits straight from hmmsearch's Stockholm output: converted to A3M with the query row's gaps kept (the hit
    rows are aligned to the query as searched), every row a candidate."""
    a3m = convert_stockholm_to_a3m(output_string, remove_first_row_gaps=False)
    return parse_hmmsearch_a3m(query_sequence=input_sequence, a3m_string=a3m, skip_first=False)


@dataclasses.dataclass(frozen=True)
class HitMetadata:
    """The fields of an hmmsearch hit description ``<pdb>_<chain>/<start>-<end> mol:protein length:<n>  <text>``."""
    pdb_id: str
    chain: str
    start: int
    end: int
    length: int
    text: str


def parse_hmmsearch_description(description: str) -> HitMetadata:
    m = re.match(r"^>?([a-zA-Z\d]{4})_([a-zA-Z0-9.]+)/(\d+)-(\d+).*?length:(\d+) *(.*)$", description.strip())
    if not m:
        raise ValueError("Could not parse hmmsearch description %r" % description)
    return HitMetadata(pdb_id=m.group(1), chain=m.group(2), start=int(m.group(3)), end=int(m.group(4)), length=int(m.group(5)), text=m.group(6))


@dataclasses.dataclass(frozen=True)
class Msa:
    """A parsed alignment file: rows, per-row deletion counts and row descriptions, all of the same length."""
    sequences: Sequence[str]
    deletion_matrix: DeletionMatrix
    descriptions: Sequence[str]

    def __post_init__(self):
        if not (len(self.sequences) == len(self.deletion_matrix) == len(self.descriptions)):
            raise ValueError("All fields of an MSA must have the same length")

    def __len__(self):
        return len(self.sequences)

    def truncate(self, max_seqs: int) -> "Msa":
        return Msa(self.sequences[:max_seqs], self.deletion_matrix[:max_seqs], self.descriptions[:max_seqs])

    @classmethod
    def from_a3m(cls, a3m_string: str) -> "Msa":
        return cls(*parse_a3m(a3m_string))

    @classmethod
    def from_stockholm(cls, stockholm_string: str) -> "Msa":
        return cls(*parse_stockholm(stockholm_string))

