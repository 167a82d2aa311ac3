"""Distillation entry point: the pretraining driver with a teacher model beside the student
(parity: lm_engine/distill.py:5-10).

    torchrun ... -m lm_engine.distill --config configs/distillation.yml
"""

from . import pretrain
from .enums import Mode


def main() -> None:
    """Console-script form of ``python -m lm_engine.distill``."""
    pretrain.main(Mode.distillation)


if __name__ == "__main__":
    main()
