# add '--gpus [N]' to run Dynamic Axial Parallelism over N GPUs
# add '--enable_workflow' to run the alignment tools as a parallel workflow
# add '--use_precomputed_alignments [path_to_alignments]' to skip the alignment tools
# add '--chunk_size [N]' to bound the peak memory of long sequences
# add '--inplace' to update activations in place (long sequences)

python inference.py target.fasta data/pdb_mmcif/mmcif_files \
    --output_dir ./outputs \
    --gpus 2 \
    --uniref90_database_path data/uniref90/uniref90.fasta \
    --mgnify_database_path data/mgnify/mgy_clusters_2022_05.fa \
    --pdb70_database_path data/pdb70/pdb70 \
    --uniref30_database_path data/uniref30/UniRef30_2021_03 \
    --bfd_database_path data/bfd/bfd_metaclust_clu_complete_id30_c90_final_seq.sorted_opt \
    --jackhmmer_binary_path `which jackhmmer` \
    --hhblits_binary_path `which hhblits` \
    --hhsearch_binary_path `which hhsearch` \
    --kalign_binary_path `which kalign` \
    --param_path data/params/params_model_1.npz \
    --model_name model_1 \
    --enable_workflow \
    --inplace
