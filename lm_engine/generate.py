"""``python -m lm_engine.generate --config cfg.yml``: batched generation over the test split of the configured
datasets; writes ``output-{data_name}.jsonl`` with ``generated_text`` and ``num_generated_tokens`` per example
(parity: lm_engine/generate.py:18-135)."""

from __future__ import annotations

import json
import os

import torch

from .arguments import InferenceArgs, get_args
from .checkpointing import load_checkpoint_for_inference
from .data.base import BaseDataset
from .data.finetuning import get_datasets_list
from .data.utils import collate_fn
from .enums import DatasetSplit, Mode
from .kernels import enable_kernels
from .model_wrapper import ModelWrapper
from .pretrain import set_seed
from .utils import ProgressBar, setup_tf32, string_to_torch_dtype


def generate(args: InferenceArgs, model: ModelWrapper, datasets_list: list[BaseDataset], mode: Mode) -> None:
    gp = args.generation_parameters
    generate_kwargs = {k: v for k, v in dict(do_sample=gp.do_sample, max_new_tokens=gp.max_new_tokens,
                                             temperature=gp.temperature, top_k=gp.top_k, top_p=gp.top_p).items() if v is not None}
    os.makedirs(args.output_dir, exist_ok=True)
    device = next(model.parameters()).device
    bar = ProgressBar(0, sum(len(d) for d in datasets_list))
    for dataset in datasets_list:
        path = os.path.join(args.output_dir, f"output-{dataset.data_name}.jsonl")
        with open(path, "w") as handle:
            batch: list[dict] = []

            def flush() -> None:
                if not batch:
                    return
                collated = collate_fn(batch, mode=mode, loss_mask=None, eos_token_id=model.eos_token_id,
                                      is_encoder_decoder=model.is_encoder_decoder, use_padding_free_transformer=False, device=device)
                texts, counts = model.generate(collated, generate_kwargs)
                for text, count in zip(texts, counts):
                    handle.write(json.dumps({"generated_text": text, "num_generated_tokens": count}) + "\n")
                bar.update(len(batch))
                batch.clear()

            for index in range(len(dataset)):
                batch.append(dataset[index])
                if len(batch) == gp.batch_size:
                    flush()
            flush()


def main(argv: list[str] | None = None) -> None:
    mode = Mode.inference
    setup_tf32()
    args: InferenceArgs = get_args(mode, argv)
    if torch.cuda.is_available():
        torch.cuda.set_device(0)
    set_seed(args.random_args.seed)
    with enable_kernels(args.kernel_args.kernels):
        if args.load_args is None:
            model = ModelWrapper(mode=mode, model_name=args.model_args.model_name, pretrained_config=args.model_args.pretrained_config,
                                 model_class=args.model_args.model_class, dtype=string_to_torch_dtype(args.mixed_precision_args.dtype),
                                 efficient_initialization=False, use_padding_free_transformer=False,
                                 trust_remote_code=args.model_args.trust_remote_code, tokenizer_name=args.tokenizer_args.tokenizer_name)
        else:
            model, _, _ = load_checkpoint_for_inference(args, mode)
        if torch.cuda.is_available():
            model = model.to(torch.device("cuda", 0))
        model.eval()
        datasets_list, _ = get_datasets_list(args.datasets, DatasetSplit.test, mode, model.tokenizer, model.is_encoder_decoder)
        generate(args, model, datasets_list, mode)


if __name__ == "__main__":
    main()
