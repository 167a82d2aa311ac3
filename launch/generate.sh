#!/bin/bash
# launch/generate.sh <config.yml>   (single GPU)
exec python -m lm_engine.generate --config "$1"
