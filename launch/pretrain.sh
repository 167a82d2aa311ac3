#!/bin/bash
# launch/pretrain.sh <config.yml>
exec "$(dirname "$0")/common.sh" lm_engine.pretrain "$1"
