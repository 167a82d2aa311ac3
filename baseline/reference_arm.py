"""Reference arm of the benchmark: the unmodified reference package installed under ``baseline/_ref``, driven through
its own public API (``get_model_container`` -> ``wrap_model_container_for_distributed_training`` (FSDP2) ->
``get_optimizer_container`` -> ``train_step_without_pipeline_parallel``), same metric and model config as the native
arm. Nothing of this repository's package is imported here.

Two things outside of the reference's files are adjusted so that it can start on this image, both recorded in the
printed JSON under ``reference_notes``:
  * transformers 5.x builds config subclasses that have no ``__init__`` of their own as dataclasses, which skips the
    reference's ``CommonConfig.__init__``; the subclasses are pointed back at it (the behaviour under the
    transformers versions the reference was written for);
  * its optional kernel packages (cute-kernels, torchao, ...) are not installed, so it runs with ``flash_attention_2``
    and its own eager fallbacks, which is how the reference itself degrades.
On one GPU the full model does not fit next to FSDP2's fp32 states and eager activations, so block gradient
checkpointing (a reference option) is switched on there and reported.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import traceback


# torch_compile setting that was faster when both were timed on a B200, by number of GPUs (see the benchmark notes):
# 1 GPU: 12,658 tok/s compiled vs 12,504 eager; 2 GPUs: 33,479 vs 30,220 (4 and 8 follow the 2-GPU result). Sizes without
# an entry run eager. If the compiled variant raises, the run starts over eager (see run_reference).
REFERENCE_COMPILE_FASTER = {1: True, 2: True, 4: True, 8: True}


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}


def run_reference(cli, spec: dict, repo_root: str):
    ref_root = os.path.join(repo_root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "lm_engine")):
        return _unavailable("baseline/_ref is missing: the reference has not been installed (pip install --no-index --target baseline/_ref of the reference tree)")
    # make sure `import lm_engine` resolves to the reference, never to this repository's package
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.abspath(repo_root)]
    sys.path.insert(0, ref_root)
    try:
        return _run(cli, spec, repo_root)
    except Exception as error:  # report instead of crashing the driver
        rank = int(os.environ.get("RANK", 0))
        if rank == 0:
            traceback.print_exc()
        choice = getattr(cli, "reference_compile", "auto")
        if choice == "auto" and REFERENCE_COMPILE_FASTER.get(cli.gpus, False) and os.environ.get("BENCH_REFERENCE_RETRY") != "1":
            # the compiled variant failed on this machine: every rank starts over, eager, in a fresh process image
            # (rendezvous on another port, rank 0 hosting the store, so nothing of the failed attempt is reused)
            env = dict(os.environ, BENCH_REFERENCE_RETRY="1")
            if "MASTER_PORT" in env:
                env["MASTER_PORT"] = str(int(env["MASTER_PORT"]) + 7)
            for key in ("TORCHELASTIC_RUN_ID", "TORCHELASTIC_USE_AGENT_STORE"):
                env.pop(key, None)
            argv = [a for a in sys.argv if a not in ("--reference-compile", "auto", "on")]
            sys.stdout.flush()
            sys.stderr.flush()
            os.execve(sys.executable, [sys.executable] + argv + ["--reference-compile", "off"], env)
        if rank == 0:
            return _unavailable(f"{type(error).__name__}: {error}")
        return None


def _run(cli, spec: dict, repo_root: str):
    import torch
    import torch.distributed as dist

    import lm_engine  # the reference

    assert os.path.abspath(lm_engine.__file__).startswith(os.path.abspath(os.path.join(repo_root, "baseline", "_ref")))
    notes = []

    from lm_engine.hf_models import config as ref_config_module

    original_init = ref_config_module.CommonConfig.__init__

    def common_init(self, *args, **kwargs):
        original_init(self, *args, **kwargs)
        # transformers 5.x rewrites `rope_scaling=None` into a {"rope_type": "default", ...} dict; the reference tests
        # `config.rope_scaling is None` to decide between plain RoPE and YaRN, so put the None back.
        rope = self.__dict__.get("rope_parameters")
        if isinstance(rope, dict) and "factor" not in rope:
            self.__dict__["rope_parameters"] = None

    import lm_engine.hf_models as ref_models

    patched = []
    for name in ("GPTBaseConfig", "PaLMConfig", "LadderResidualConfig"):
        cls = getattr(ref_models, name, None)
        if cls is not None:
            cls.__init__ = common_init
            patched.append(name)
    if patched:
        notes.append("transformers 5.x compatibility: " + ", ".join(patched) + ".__init__ routed to CommonConfig.__init__; "
                     "rope_scaling=None restored after transformers' rope normalisation; model._no_split_modules converted back to a list")

    from lm_engine.arguments import TrainingArgs
    from lm_engine.distributed import wrap_model_container_for_distributed_training
    from lm_engine.enums import Mode
    from lm_engine.hf_models import disable_generation_cache
    from lm_engine.kernels import enable_kernels
    from lm_engine.model_wrapper import get_model_container
    from lm_engine.optimization import get_optimizer_container, get_scheduler_container
    from lm_engine.pretrain import train_step_without_pipeline_parallel
    from lm_engine.train_utils import get_model_tflops
    from lm_engine.utils import ProcessGroupManager, StepTracker, init_distributed, set_logger
    from contextlib import nullcontext

    set_logger("WARNING")
    for key, value in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29517"), ("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(key, value)  # single-process launch without torchrun
    world = int(os.environ.get("WORLD_SIZE", 1))
    assert world == cli.gpus, f"--gpus {cli.gpus} but WORLD_SIZE={world}"
    layers = cli.layers or spec["num_layers"]
    ga = cli.gradient_accumulation_steps or spec["gradient_accumulation_steps"]
    mb, seq = spec["micro_batch_size"], spec["sequence_length"]

    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=spec["num_attention_heads"],
                num_key_value_heads=spec["num_key_value_heads"], add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=spec["intermediate_size"], add_bias=False)
    if "num_experts" in spec:  # the reference's MoE: FSDP over the expert bank, eager per-expert loop (its scattermoe kernel is absent)
        mlp = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=spec["intermediate_size"], add_bias=False,
                   num_experts=spec["num_experts"], num_experts_per_tok=spec["num_experts_per_tok"])
    pretrained_config = dict(
        router_aux_loss_coef=spec.get("router_aux_loss_coef", 0.001),
        model_type="gpt_base", vocab_size=spec["vocab_size"], hidden_size=spec["hidden_size"], num_layers=layers,
        max_position_embeddings=seq, position_embedding_type="rope", rope_theta=spec["rope_theta"],
        normalization_function="rmsnorm", layer_norm_epsilon=1e-5, initializer_range=0.02, tie_word_embeddings=False,
        bos_token_id=0, eos_token_id=1, pad_token_id=2,
        sequence_mixer_blocks=[dict(attn) for _ in range(layers)], mlp_blocks=[dict(mlp) for _ in range(layers)])

    # The reference insists on a tokenizer even for pretraining on token ids; there is no network, so a four-token
    # stub (bos/eos/pad/unk with the ids of the model config) is written locally. It is never used to tokenize.
    tokenizer_dir = os.path.join(tempfile.gettempdir(), f"bench-ref-tokenizer-{os.environ.get('RANK', '0')}")
    if not os.path.exists(os.path.join(tokenizer_dir, "tokenizer.json")):
        from tokenizers import Tokenizer
        from tokenizers.models import WordLevel
        from tokenizers.pre_tokenizers import Whitespace
        from transformers import PreTrainedTokenizerFast

        tok = Tokenizer(WordLevel({"<bos>": 0, "<eos>": 1, "<pad>": 2, "<unk>": 3}, unk_token="<unk>"))
        tok.pre_tokenizer = Whitespace()
        PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<bos>", eos_token="<eos>", pad_token="<pad>",
                                unk_token="<unk>").save_pretrained(tokenizer_dir)
    notes.append("stub 4-token tokenizer created locally (the reference requires tokenizer_args.tokenizer_name)")

    checkpointing = world == 1 and cli.layers is None and "num_experts" not in spec  # the 8B dense model does not fit one GPU otherwise
    # `torch_compile` is a stock option of the reference (distributed_args.torch_compile wraps every model in
    # torch.compile). REFERENCE_COMPILE_DEFAULT records which setting was faster when both were timed on a B200.
    choice = getattr(cli, "reference_compile", "auto")
    compile_on = REFERENCE_COMPILE_FASTER.get(cli.gpus, False) if choice == "auto" else choice == "on"
    distributed_args = dict(stage=3, fsdp_algorithm=2, communication_dtype="fp32", torch_compile=compile_on)
    if os.environ.get("BENCH_REFERENCE_RETRY") == "1":
        notes.append("distributed_args.torch_compile=False: the compiled variant raised an exception on this machine, the run was repeated eager")
    else:
        notes.append(f"distributed_args.torch_compile={compile_on} ({'chosen with --reference-compile' if choice != 'auto' else 'the faster setting as measured'})")
    if checkpointing:
        distributed_args["gradient_checkpointing_method"] = "block"
        notes.append("block gradient checkpointing enabled (1 GPU: fp32 FSDP2 states + eager activations exceed 180 GB otherwise)")
    config = dict(
        datasets=[dict(class_name="MegatronDataset", data_name="Megatron", class_args=dict(sequence_length=seq))],
        model_args=dict(model_class="AutoModelForCausalLM", pretrained_config=pretrained_config,
                        use_padding_free_transformer=True, efficient_initialization=True),
        tokenizer_args=dict(tokenizer_name=tokenizer_dir),
        tuning_args=dict(tuning_method="pretraining"),
        save_args=dict(save_path=os.path.join(tempfile.gettempdir(), "bench-ref-unused"), save_interval=10**9),
        training_parameters=dict(num_training_steps=10**6, micro_batch_size=mb, gradient_accumulation_steps=ga,
                                 eval_during_training=False, gradient_clipping=1.0),
        optimizer_args=dict(class_name="TorchAdamW", class_args=dict(lr=3e-4, weight_decay=0.1, betas=[0.9, 0.95], eps=1e-10)),
        lr_scheduler_args=dict(lr_decay_style="cosine", num_warmup_steps=10, lr_decay_factor=0.1),
        mixed_precision_args=dict(dtype="bf16"),
        distributed_args=distributed_args,
        kernel_args=dict(kernels=["flash_attention_2"]),
        logging_args=dict(log_interval=10**9),
    )
    args = TrainingArgs(**config)

    d = args.distributed_args
    init_distributed(
        tensor_parallel_world_size=d.tensor_parallel_world_size,
        pipeline_parallel_world_size=d.pipeline_parallel_world_size,
        data_parallel_replication_world_size=d.zero_topology.data_parallel_replication_world_size,
        data_parallel_sharding_world_size=d.zero_topology.data_parallel_sharding_world_size,
        zero_stage=d.stage, timeout_minutes=d.timeout_minutes, use_async_tensor_parallel=d.use_async_tensor_parallel)
    rank = ProcessGroupManager.get_global_rank()
    device = torch.device("cuda", torch.cuda.current_device())
    StepTracker(micro_batch_size=mb, gradient_accumulation_steps=ga)
    torch.manual_seed(1234)

    with enable_kernels(args.kernel_args.kernels):
        container = get_model_container(args, Mode.training)
        for wrapper in container:
            # transformers 5.x turns `_no_split_modules` into a set; the reference concatenates and indexes it as a list
            if isinstance(getattr(wrapper.model, "_no_split_modules", None), (set, frozenset)):
                wrapper.model._no_split_modules = sorted(wrapper.model._no_split_modules)
        container, schedule = wrap_model_container_for_distributed_training(args, container)
        optimizers = get_optimizer_container(
            optimizer_class_name=args.optimizer_args.class_name, optimizer_class_args=args.optimizer_args.class_args,
            model_container=container, params_group_method=args.optimizer_args.params_group_method,
            use_optimizer_with_backward_hook=False)
        schedulers = get_scheduler_container(
            model_container=container, optimizer_container=optimizers, num_warmup_steps=10, num_constant_steps=0,
            num_decay_steps=None, num_training_steps=10**6, lr_decay_style=args.lr_scheduler_args.lr_decay_style,
            lr_decay_factor=0.1, extra_lr_scheduler_args={}, use_optimizer_with_backward_hook=False)
        container.train()

        gen = torch.Generator().manual_seed(1234 + rank)
        n_device = ga * (cli.warmup + cli.steps)
        n_host = 0 if cli.skip_e2e else ga * cli.steps
        pool_device = [torch.randint(0, spec["vocab_size"], (mb, seq + 1), generator=gen, dtype=torch.long).to(device) for _ in range(n_device)]
        pool = [torch.randint(0, spec["vocab_size"], (mb, seq + 1), generator=gen, dtype=torch.long).pin_memory() for _ in range(n_host)]

        class Feed:
            def __init__(self, tensors):
                self.tensors, self.i = tensors, 0

            def __iter__(self):
                return self

            def __next__(self):
                t = self.tensors[self.i % len(self.tensors)]
                self.i += 1
                return {"text": t}

        multiplier = 1.0 / (mb * seq)

        def step(feed):
            return train_step_without_pipeline_parallel(
                model_container=container, optimizer_container=optimizers, lr_scheduler_container=schedulers,
                train_dataloader=feed, gradient_clipping=1.0, forward_context=nullcontext, backward_context=nullcontext,
                sync_every_gradient_accumulation_step=False, lm_loss_multiplier=multiplier)

        def timed(feed, read_back):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            last = None
            for _ in range(cli.steps):
                metrics = step(feed)
                if read_back:
                    last = float(metrics["loss"])
            end.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item(), last

        with disable_generation_cache():
            feed_device = Feed(pool_device)
            for _ in range(cli.warmup):
                metrics = step(feed_device)
            loss_after_warmup = float(metrics["loss"])
            ms, _ = timed(feed_device, False)
            e2e = None
            if not cli.skip_e2e:
                ms_e2e, last_loss = timed(Feed(pool), True)
                e2e = {"value": cli.steps * ga * mb * seq * world / (ms_e2e / 1e3), "unit": "tokens/s",
                       "ms_per_step": ms_e2e / cli.steps, "h2d_bytes_per_step": ga * mb * (seq + 1) * 8,
                       "d2h_bytes_per_step": 4, "last_loss": last_loss}

    ms_per_step = ms / cli.steps
    tokens_per_step = ga * mb * seq * world
    tflops = get_model_tflops(container[0].config, ga * mb * world, seq, None, {}) / world / (ms_per_step / 1e3)
    result = {
        "impl": "reference", "metric": ("pretraining tokens/s (40-expert top-8 MoE, expert parallel)" if "num_experts" in spec else
                                        "pretraining tokens/s (8B dense, ZeRO-3 sharded data parallel)"),
        "value": tokens_per_step / (ms_per_step / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": cli.steps,
        "warmup": cli.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
        "config": {"model": spec["name"] + ("" if cli.layers is None else f"-DEBUG-{cli.layers}-layers"),
                   "global_batch": ga * mb * world, "seq_len": seq, "micro_batch_per_gpu": mb, "gradient_accumulation_steps": ga,
                   "parallelism": f"fsdp{world} (FSDP2 fully_shard, stage 3, fp32 reduce)",
                   "kernels": ["flash_attention_2"], "gradient_checkpointing": "block" if checkpointing else None,
                   "torch_compile": compile_on},
        "tflops_per_gpu_useful": tflops, "loss_after_warmup": loss_after_warmup,
        "peak_memory_gib": torch.cuda.max_memory_allocated() / 2**30, "reference_notes": notes,
    }
    if e2e is not None:
        result["e2e"] = e2e
    try:
        ProcessGroupManager.destroy_process_groups()
    except Exception:
        pass
    return result if rank == 0 else None
