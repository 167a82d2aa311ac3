#!/bin/bash
# Tokenised arrow (or jsonl) shards of a corpus -> one .bin/.idx store per file.
#   launch/convert_data.sh <tokenizer> <input-path> <output-path> <subset> [<subset> ...]
# The files of every subset are divided among JOBS processes. On one machine the jobs run side by side (JOBS defaults to
# the number of cores / 4); under a SLURM array every task converts its own share:
#   sbatch --array=0-63 --cpus-per-task=4 --wrap "launch/convert_data.sh T raw tmp cc wiki"
set -euo pipefail
TOKENIZER=$1; INPUT=$2; OUTPUT=$3; shift 3
export TOKENIZERS_PARALLELISM=false
run() {  # <jobs> <job index> <subsets...>
    local jobs=$1 index=$2; shift 2
    python -m lm_engine.cli.preprocess_data convert-tree --tokenizer "$TOKENIZER" --input-path "$INPUT" --output-path "$OUTPUT" \
        --data-subsets "$@" --jobs "$jobs" --job-index "$index" --workers "${WORKERS:-1}"
}
if [ -n "${SLURM_ARRAY_TASK_ID:-}" ]; then
    run "${SLURM_ARRAY_TASK_COUNT}" "$((SLURM_ARRAY_TASK_ID - ${SLURM_ARRAY_TASK_MIN:-0}))" "$@"
else
    JOBS=${JOBS:-$(( ($(nproc) + 3) / 4 ))}
    pids=()
    for ((index = 0; index < JOBS; index++)); do
        run "$JOBS" "$index" "$@" &
        pids+=($!)
    done
    status=0
    for pid in "${pids[@]}"; do wait "$pid" || status=1; done
    exit $status
fi
