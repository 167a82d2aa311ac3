#!/bin/bash
# launch/distill.sh <config.yml>
exec "$(dirname "$0")/common.sh" lm_engine.distill "$1"
