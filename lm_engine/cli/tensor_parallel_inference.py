"""Generate with a model split over the GPUs of one node (launch with torchrun; world size = tensor-parallel size).

Every rank reads only its slices of the unsharded safetensors checkpoint."""

from argparse import ArgumentParser

import torch
from transformers import AutoTokenizer

from ..hf_models.models.tensor_parallel import GPTBaseForCausalLM_TP
from ..utils import ProcessGroupManager, init_distributed


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--model", required=True)
    parser.add_argument("--prompt", nargs="+", required=True)
    parser.add_argument("--max-new-tokens", type=int, default=50)
    parser.add_argument("--dtype", default="bfloat16")
    args = parser.parse_args()

    import os

    init_distributed(tensor_parallel_world_size=int(os.environ.get("WORLD_SIZE", 1)))
    model = GPTBaseForCausalLM_TP.from_pretrained(args.model, dtype=getattr(torch, args.dtype)).eval()
    device = next(model.parameters()).device
    tokenizer = AutoTokenizer.from_pretrained(args.model)
    tokenizer.padding_side = "left"
    if tokenizer.pad_token_id is None:
        tokenizer.pad_token = tokenizer.eos_token
    batch = tokenizer(args.prompt, return_tensors="pt", padding=True).to(device)
    out = model.generate(batch["input_ids"], attention_mask=batch["attention_mask"], max_new_tokens=args.max_new_tokens)
    if ProcessGroupManager.get_global_rank() == 0:
        for prompt, ids in zip(args.prompt, out):
            print(f"--- {prompt!r}\n{tokenizer.decode(ids[batch['input_ids'].shape[1]:], skip_special_tokens=True)}")
    ProcessGroupManager.destroy_process_groups()


if __name__ == "__main__":
    main()
