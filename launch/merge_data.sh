#!/bin/bash
# The per-file stores written by launch/convert_data.sh -> a few large stores per subset (MAX_FILE_SIZE in GB, default 100),
# with <output-path>/files.json recording what went where.
#   launch/merge_data.sh <input-path> <output-path> <subset> [<subset> ...]
set -euo pipefail
INPUT=$1; OUTPUT=$2; shift 2
exec python -m lm_engine.cli.preprocess_data merge-tree --input-path "$INPUT" --output-path "$OUTPUT" --data-subsets "$@" \
    --max-file-size "${MAX_FILE_SIZE:-100}"
