"""Generate continuations for prompts with a saved model on one device."""

from argparse import ArgumentParser

import torch
from transformers import AutoModelForCausalLM, AutoTokenizer

from .. import hf_models  # noqa: F401  (registers the model classes with transformers)


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--model", required=True)
    parser.add_argument("--prompt", nargs="+", required=True)
    parser.add_argument("--max-new-tokens", type=int, default=50)
    parser.add_argument("--dtype", default="bfloat16")
    parser.add_argument("--sample", action="store_true")
    args = parser.parse_args()

    device = "cuda" if torch.cuda.is_available() else "cpu"
    tokenizer = AutoTokenizer.from_pretrained(args.model)
    tokenizer.padding_side = "left"
    if tokenizer.pad_token_id is None:
        tokenizer.pad_token = tokenizer.eos_token
    model = AutoModelForCausalLM.from_pretrained(args.model, dtype=getattr(torch, args.dtype)).to(device).eval()
    batch = tokenizer(args.prompt, return_tensors="pt", padding=True).to(device)
    out = model.generate(batch["input_ids"], attention_mask=batch["attention_mask"], max_new_tokens=args.max_new_tokens, do_sample=args.sample)
    for prompt, ids in zip(args.prompt, out):
        print(f"--- {prompt!r}\n{tokenizer.decode(ids[batch['input_ids'].shape[1]:], skip_special_tokens=True)}")


if __name__ == "__main__":
    main()
