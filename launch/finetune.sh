#!/bin/bash
# launch/finetune.sh <config.yml>
exec "$(dirname "$0")/common.sh" lm_engine.finetune "$1"
