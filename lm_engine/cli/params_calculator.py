"""Count the parameters (total and active per token) and the training FLOPs of a model described by a config, without
allocating it."""

import json
from argparse import ArgumentParser

import torch
from transformers import AutoConfig, AutoModelForCausalLM

from .. import hf_models  # noqa: F401
from ..train_utils import get_model_tflops


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--config", required=True, help="directory or config.json of the model")
    parser.add_argument("--batch-size", type=int, default=1)
    parser.add_argument("--sequence-length", type=int, default=4096)
    args = parser.parse_args()

    config = AutoConfig.from_pretrained(args.config)
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(config)
    total = sum(p.numel() for p in model.parameters())
    active = total
    for module in model.modules():
        if hasattr(module, "get_num_active_parameters"):
            active -= sum(p.numel() for p in module.parameters()) - module.get_num_active_parameters()
    print(json.dumps({"total_parameters": total, "active_parameters": active,
                      "tflop_per_step": get_model_tflops(config, args.batch_size, args.sequence_length, None, None)}, indent=2))


if __name__ == "__main__":
    main()
