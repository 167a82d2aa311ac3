"""Distillation entry point: the pretraining driver in distillation mode (parity: lm_engine/distill.py:5-10)."""

from .enums import Mode
from .pretrain import main

if __name__ == "__main__":
    main(Mode.distillation)
