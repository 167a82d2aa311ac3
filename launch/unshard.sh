#!/bin/bash
# launch/unshard.sh <config.yml>   (single process; reads the sharded checkpoint, writes safetensors)
exec python -m lm_engine.unshard --config "$1"
