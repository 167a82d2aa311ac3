"""Every example config under ``configs/`` parses into the argument tree of its entry point."""

import glob
import os

import pytest

from lm_engine.arguments import args_from_dict
from lm_engine.enums import Mode
from lm_engine.utils import load_yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODES = {"unshard.yml": Mode.unsharding, "generation.yml": Mode.inference, "distillation.yml": Mode.distillation}


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "configs", "**", "*.yml"), recursive=True)))
def test_example_config_parses(path):
    args = args_from_dict(MODES.get(os.path.basename(path), Mode.training), load_yaml(path))
    if hasattr(args, "model_args") and getattr(args.model_args, "pretrained_config", None):
        config = args.model_args.pretrained_config
        assert len(config["sequence_mixer_blocks"]) == len(config["mlp_blocks"]) == config["num_layers"]
