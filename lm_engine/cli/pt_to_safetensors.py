"""Re-save a checkpoint stored as a full ``torch.save`` state dict (``pytorch_model*.bin``) as sharded safetensors."""

from argparse import ArgumentParser

import torch
from transformers import AutoModelForCausalLM, AutoTokenizer

from .. import hf_models  # noqa: F401


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--model", required=True)
    parser.add_argument("--save-path", required=True)
    parser.add_argument("--dtype", default="bfloat16")
    args = parser.parse_args()
    model = AutoModelForCausalLM.from_pretrained(args.model, dtype=getattr(torch, args.dtype))
    model.save_pretrained(args.save_path, safe_serialization=True)
    try:
        AutoTokenizer.from_pretrained(args.model).save_pretrained(args.save_path, legacy_format=False)
    except Exception:
        pass  # checkpoints without tokenizer files


if __name__ == "__main__":
    main()
