#!/bin/bash
# Downloads and unpacks ONE data set: scripts/download_one.sh <name> <DOWNLOAD_DIR>
# names: params bfd small_bfd mgnify pdb70 pdb_mmcif uniref30 uniref90 uniprot pdb_seqres
set -euo pipefail
NAME="$1"; ROOT="$2"
fetch() { mkdir -p "$2"; aria2c "$1" --dir="$2"; }
case "$NAME" in
  params)
    D="$ROOT/params"; fetch "https://storage.googleapis.com/alphafold/alphafold_params_2022-12-06.tar" "$D"
    tar --extract --verbose --file="$D/alphafold_params_2022-12-06.tar" --directory="$D" --preserve-permissions; rm "$D/alphafold_params_2022-12-06.tar";;
  bfd)
    D="$ROOT/bfd"; F="bfd_metaclust_clu_complete_id30_c90_final_seq.sorted_opt.tar.gz"
    fetch "https://storage.googleapis.com/alphafold-databases/casp14_versions/$F" "$D"; tar -xvzf "$D/$F" -C "$D"; rm "$D/$F";;
  small_bfd)
    D="$ROOT/small_bfd"; fetch "https://storage.googleapis.com/alphafold-databases/reduced_dbs/bfd-first_non_consensus_sequences.fasta.gz" "$D"
    gunzip "$D/bfd-first_non_consensus_sequences.fasta.gz";;
  mgnify)
    D="$ROOT/mgnify"; fetch "https://storage.googleapis.com/alphafold-databases/v2.3/mgy_clusters_2022_05.fa.gz" "$D"; gunzip "$D/mgy_clusters_2022_05.fa.gz";;
  pdb70)
    D="$ROOT/pdb70"; fetch "http://wwwuser.gwdg.de/~compbiol/data/hhsuite/databases/hhsuite_dbs/old-releases/pdb70_from_mmcif_200401.tar.gz" "$D"
    tar -xvzf "$D/pdb70_from_mmcif_200401.tar.gz" -C "$D"; rm "$D/pdb70_from_mmcif_200401.tar.gz";;
  pdb_mmcif)
    D="$ROOT/pdb_mmcif"; mkdir -p "$D/raw" "$D/mmcif_files"
    rsync --recursive --links --perms --times --compress --info=progress2 --delete --port=33444 rsync.rcsb.org::ftp_data/structures/divided/mmCIF/ "$D/raw"
    find "$D/raw/" -type f -iname "*.gz" -exec gunzip {} +
    find "$D/raw" -type f -name "*.cif" -exec mv {} "$D/mmcif_files" \;
    rm -r "$D/raw"; aria2c "ftp://ftp.wwpdb.org/pub/pdb/data/status/obsolete.dat" --dir="$D";;
  uniref30)
    D="$ROOT/uniref30"; fetch "https://storage.googleapis.com/alphafold-databases/v2.3/UniRef30_2021_03.tar.gz" "$D"
    tar -xvzf "$D/UniRef30_2021_03.tar.gz" -C "$D"; rm "$D/UniRef30_2021_03.tar.gz";;
  uniref90)
    D="$ROOT/uniref90"; fetch "ftp://ftp.uniprot.org/pub/databases/uniprot/uniref/uniref90/uniref90.fasta.gz" "$D"; gunzip "$D/uniref90.fasta.gz";;
  uniprot)
    D="$ROOT/uniprot"
    fetch "ftp://ftp.ebi.ac.uk/pub/databases/uniprot/current_release/knowledgebase/complete/uniprot_trembl.fasta.gz" "$D"
    fetch "ftp://ftp.ebi.ac.uk/pub/databases/uniprot/current_release/knowledgebase/complete/uniprot_sprot.fasta.gz" "$D"
    gunzip "$D/uniprot_trembl.fasta.gz" "$D/uniprot_sprot.fasta.gz"; cat "$D/uniprot_sprot.fasta" >> "$D/uniprot_trembl.fasta"
    mv "$D/uniprot_trembl.fasta" "$D/uniprot.fasta"; rm "$D/uniprot_sprot.fasta";;
  pdb_seqres)
    D="$ROOT/pdb_seqres"; fetch "ftp://ftp.wwpdb.org/pub/pdb/derived_data/pdb_seqres.txt" "$D";;
  *) echo "unknown data set $NAME" >&2; exit 1;;
esac
