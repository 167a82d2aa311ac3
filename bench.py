"""Headline benchmark: pretraining throughput (tokens/s, whole job) of the 8B dense decoder with sharded (ZeRO-3)
data parallelism, bf16 compute with fp32 master weights and AdamW, sequence length 4096, micro-batch 2 per GPU and
16 gradient-accumulation micro-steps per optimizer step (global batch 32 sequences per GPU: 256 on 8 GPUs).

    python bench.py --gpus N --steps K --warmup W                 # this engine
    python bench.py --impl reference --gpus N --steps K --warmup W   # the unmodified reference from baseline/_ref

For N > 1 launch through ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...``.
Rank 0 prints one JSON line. Data is synthetic (uniform random tokens), weights are randomly initialised.

Two regions are timed, each over exactly K optimizer steps with a barrier + device synchronise on both sides and
CUDA events on the launching stream, maximum over ranks:
  * ``value``: inputs already resident on the device, nothing read back;
  * ``e2e`` : every micro-step copies its token batch from pinned host memory and every step reads the loss back.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO_ROOT = os.path.dirname(os.path.abspath(__file__))

DENSE_8B = dict(
    name="dense-8b-gpt_base",
    vocab_size=128256, hidden_size=4096, num_layers=32, num_attention_heads=32, num_key_value_heads=8,
    intermediate_size=14336, rope_theta=500000, sequence_length=4096, micro_batch_size=2, gradient_accumulation_steps=16,
)

# scattered-MoE decoder, 40 experts top-8; experts spread over the GPUs (expert parallel = world size)
MOE_40E = dict(
    name="moe-40e-top8-gpt_base",
    vocab_size=49152, hidden_size=1536, num_layers=32, num_attention_heads=24, num_key_value_heads=8,
    intermediate_size=512, num_experts=40, num_experts_per_tok=8, router_aux_loss_coef=0.01, rope_theta=10000,
    sequence_length=4096, micro_batch_size=4, gradient_accumulation_steps=4,
)
SPECS = {"dense": DENSE_8B, "moe": MOE_40E}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="native", choices=["native", "reference"])
    p.add_argument("--config", type=str, default="dense", choices=sorted(SPECS), help="dense: 8B dense FSDP (headline); moe: 40-expert top-8 MoE")
    p.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (the result is then not the headline config)")
    p.add_argument("--gradient-accumulation-steps", type=int, default=None, help="debug only")
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--no-moe", action="store_true", help="dense run only: skip the second record (40-expert MoE)")
    p.add_argument("--moe-steps", type=int, default=None, help="timed steps of the MoE record (default: max(3, steps // 4))")
    p.add_argument("--reference-compile", type=str, default="auto", choices=["auto", "on", "off"],
                   help="reference arm: its own distributed_args.torch_compile option (auto = the faster one as measured on a B200)")
    p.add_argument("--expert-capacity-factor", type=float, default=None,
                   help="MoE with expert parallelism: static row buffers of this multiple of a rank's balanced share instead of the "
                        "default exact (dropless) sizing; dropped entries are counted and reported")
    p.add_argument("--tensor-parallel", type=int, default=1,
                   help="tensor-parallel size with sequence parallelism; the other GPUs form the sharded data-parallel group (not the headline mode)")
    p.add_argument("--fp8", type=str, default=None, choices=["tensorwise", "mxfp8"], help="run the linear layers in fp8 with this recipe (not the headline mode)")
    p.add_argument("--sequence-length", type=int, default=None, help="override the sequence length (not the headline config)")
    p.add_argument("--micro-batch-size", type=int, default=None, help="override the micro-batch size (not the headline config)")
    p.add_argument("--pipeline-parallel", type=int, default=1,
                   help="pipeline stages (1F1B, one stage per pipeline rank); the other GPUs form the sharded data-parallel group (not the headline mode)")
    p.add_argument("--sharded-parameters", action="store_true",
                   help="distributed_args.keep_parameters_gathered=false: blocks are gathered and released one by one (not the headline mode)")
    p.add_argument("--budget-output", type=str, default=None,
                   help="after the timed regions run one more step with per-site device timers and write the per-kernel time budget there (JSON)")
    p.add_argument("--child-output", type=str, default=None, help=argparse.SUPPRESS)
    return p.parse_args()


def model_config(spec: dict, layers: int | None) -> dict:
    n = layers or spec["num_layers"]
    attn = dict(sequence_mixer_type="softmax_attention", num_attention_heads=spec["num_attention_heads"],
                num_key_value_heads=spec["num_key_value_heads"], add_bias=False)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=spec["intermediate_size"], add_bias=False)
    if "num_experts" in spec:
        mlp = dict(mlp_type="MoE", activation_function="swiglu", intermediate_size=spec["intermediate_size"], add_bias=False,
                   num_experts=spec["num_experts"], num_experts_per_tok=spec["num_experts_per_tok"])
    return dict(
        router_aux_loss_coef=spec.get("router_aux_loss_coef", 0.001),
        model_type="gpt_base", vocab_size=spec["vocab_size"], hidden_size=spec["hidden_size"], num_layers=n,
        max_position_embeddings=spec["sequence_length"], position_embedding_type="rope", rope_theta=spec["rope_theta"],
        normalization_function="rmsnorm", layer_norm_epsilon=1e-5, initializer_range=0.02, tie_word_embeddings=False,
        bos_token_id=0, eos_token_id=1, pad_token_id=2,
        sequence_mixer_blocks=[dict(attn) for _ in range(n)], mlp_blocks=[dict(mlp) for _ in range(n)],
    )


def training_config(spec: dict, layers: int | None, ga: int, steps: int, kernels: list[str], extra_distributed: dict | None = None) -> dict:
    distributed = dict(stage=3, communication_dtype="fp32")
    distributed.update(extra_distributed or {})
    return dict(
        datasets=[dict(class_name="SyntheticDataset", data_name="synthetic",
                       class_args=dict(sequence_length=spec["sequence_length"], seed=1234, vocab_size=spec["vocab_size"]))],
        model_args=dict(model_class="AutoModelForCausalLM", pretrained_config=model_config(spec, layers),
                        use_padding_free_transformer=True, efficient_initialization=True),
        tuning_args=dict(tuning_method="pretraining"),
        save_args=dict(save_path=os.path.join(tempfile.gettempdir(), "bench-unused"), save_interval=10**9),
        training_parameters=dict(num_training_steps=steps, micro_batch_size=spec["micro_batch_size"],
                                 gradient_accumulation_steps=ga, eval_during_training=False, gradient_clipping=1.0),
        optimizer_args=dict(class_name="TorchAdamW", class_args=dict(lr=3e-4, weight_decay=0.1, betas=[0.9, 0.95], eps=1e-10)),
        lr_scheduler_args=dict(lr_decay_style="cosine", num_warmup_steps=10, lr_decay_factor=0.1),
        mixed_precision_args=dict(dtype="bf16"),
        distributed_args=distributed,
        kernel_args=dict(kernels=kernels),
        logging_args=dict(log_interval=10**9),
    )


# ----------------------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region is being timed."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        with open(self.path) as handle:
            for line in handle:
                cells = [c.strip() for c in line.split(",")]
                if len(cells) < 9:
                    continue
                try:
                    clocks.append(float(cells[1]))
                    max_clock = float(cells[2])
                except ValueError:
                    continue
                for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), cells[5:9]):
                    if cell.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock, "reasons": sorted(reasons),
                "samples": len(clocks)}


def measured_peak_tflops() -> tuple[float, str]:
    path = os.path.join(REPO_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return float(json.load(handle)["bf16_tflops_sustained"]), "measured (sustained cuBLAS bf16)"
    return 1400.0, "fallback"


# ----------------------------------------------------------------------------------------------------------------------
def run_native(cli) -> dict:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REPO_ROOT)
    from lm_engine import ops
    from lm_engine.arguments import args_from_dict
    from lm_engine.distributed import wrap_model_container_for_distributed_training
    from lm_engine.enums import Kernel, Mode
    from lm_engine.kernels import enable_kernels
    from lm_engine.model_wrapper import get_model_container
    from lm_engine.optimization import get_optimizer_container, get_scheduler_container
    from lm_engine.pretrain import set_seed, train_step_without_pipeline_parallel
    from lm_engine.train_utils import get_model_tflops
    from lm_engine.utils import ProcessGroupManager, StepTracker, init_distributed, set_logger

    set_logger("WARNING")
    ops.require_native()
    # an op that would leave the sm_100a kernels for a PyTorch path raises instead (the pipeline-parallel exploration mode
    # only counts such sites and reports them)
    ops.set_strict(cli.pipeline_parallel == 1 and cli.tensor_parallel == 1 and cli.fp8 is None)
    spec = dict(SPECS[cli.config])
    if cli.sequence_length:
        spec["sequence_length"] = cli.sequence_length
    if cli.micro_batch_size:
        spec["micro_batch_size"] = cli.micro_batch_size
    moe = "num_experts" in spec
    ga = cli.gradient_accumulation_steps or spec["gradient_accumulation_steps"]
    kernels = [k.value for k in Kernel if k != Kernel.ladder_residual_overlapped_layer]
    expert_parallel = cli.gpus if moe and cli.gpus > 1 and spec["num_experts"] % cli.gpus == 0 else 1
    # expert row buffers are sized exactly for the fullest rank of every layer (no capacity factor: nothing can be dropped)
    capacity = cli.expert_capacity_factor
    extra = {"expert_parallel_world_size": expert_parallel, "expert_capacity_factor": capacity} if expert_parallel > 1 else {}
    if cli.sharded_parameters:
        extra["keep_parameters_gathered"] = False
    tp_size = cli.tensor_parallel
    if tp_size > 1:
        extra.update(tensor_parallel_world_size=tp_size, sequence_parallel=True)
    pp = cli.pipeline_parallel
    if pp > 1:
        extra.update(pipeline_parallel_world_size=pp, num_pipeline_stages=pp, pipeline_parallel_schedule="1F1B")
    config_dict = training_config(spec, cli.layers, ga, cli.steps + cli.warmup, kernels, extra)
    if cli.fp8:
        config_dict["mixed_precision_args"] = dict(dtype="fp8", fp8_recipe=cli.fp8)
    args = args_from_dict(Mode.training, config_dict)

    init_distributed(zero_stage=3, expert_parallel_world_size=expert_parallel, pipeline_parallel_world_size=pp,
                     tensor_parallel_world_size=tp_size)
    world = ProcessGroupManager.get_world_size()
    assert world == cli.gpus, f"--gpus {cli.gpus} but WORLD_SIZE={world}"
    rank = ProcessGroupManager.get_global_rank()
    device = ProcessGroupManager.get_device()
    StepTracker(spec["micro_batch_size"], ga)
    set_seed(1234)

    with enable_kernels(args.kernel_args.kernels):
        container = get_model_container(args, Mode.training)
        container, pipeline_schedule = wrap_model_container_for_distributed_training(args, container)
        optimizers = get_optimizer_container("TorchAdamW", args.optimizer_args.class_args, container)
        schedulers = get_scheduler_container(container, optimizers, 10, 0, None, 10**6, args.lr_scheduler_args.lr_decay_style, 0.1, {})
        container.train()

        mb, seq = spec["micro_batch_size"], spec["sequence_length"]
        multiplier = 1.0 / (mb * seq)
        # all pipeline ranks of one data-parallel replica read the same tokens
        gen = torch.Generator().manual_seed(1234 + (rank if pp * tp_size == 1 else ProcessGroupManager.get_data_parallel_rank()))
        # a fresh micro-batch for every micro-step of every step (nothing is seen twice)
        n_device = ga * (cli.warmup + cli.steps)
        n_host = 0 if cli.skip_e2e else ga * cli.steps
        pool_device = [torch.randint(0, spec["vocab_size"], (mb, seq + 1), generator=gen, dtype=torch.long).to(device) for _ in range(n_device)]
        pool = [torch.randint(0, spec["vocab_size"], (mb, seq + 1), generator=gen, dtype=torch.long).pin_memory() for _ in range(n_host)]

        class Feed:
            def __init__(self, tensors):
                self.tensors, self.i = tensors, 0

            def __next__(self):
                t = self.tensors[self.i % len(self.tensors)]
                self.i += 1
                return {"text": t}

        def step(feed):
            if pipeline_schedule is not None:
                from lm_engine.pretrain import train_step_with_pipeline_parallel

                return train_step_with_pipeline_parallel(container, pipeline_schedule, optimizers, schedulers, feed, 1.0, seq)
            return train_step_without_pipeline_parallel(container, optimizers, schedulers, feed, 1.0, lm_loss_multiplier=multiplier)

        def loss_of(metrics):  # only the last pipeline stage has one
            return float(metrics["loss"]) if "loss" in list(metrics.keys()) else None

        def timed(feed, read_back: bool):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            launches0 = ops.launch_count()
            sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
            if sampler:
                sampler.start()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            last = None
            walls = []
            wall0 = time.perf_counter()
            for _ in range(cli.steps):
                metrics = step(feed)
                if read_back:
                    last = loss_of(metrics)  # device -> host read of the step result
                    wall1 = time.perf_counter()  # the read-back has synchronised: this is the step's wall time
                    walls.append(round((wall1 - wall0) * 1e3, 1))
                    wall0 = wall1
            end.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ms = start.elapsed_time(end)
            clocks = sampler.stop() if sampler else None
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item(), ops.launch_count() - launches0, clocks, (last, walls) if read_back else last

        feed_device = Feed(pool_device)
        for _ in range(cli.warmup):
            metrics = step(feed_device)
        loss_after_warmup = loss_of(metrics)
        ops.check_status()

        ms, launches, clocks, _ = timed(feed_device, read_back=False)
        e2e = None
        if not cli.skip_e2e:
            ms_e2e, _, _, (last_loss, step_walls) = timed(Feed(pool), read_back=True)
            tokens = cli.steps * ga * mb * seq * (world // (pp * tp_size))
            e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / cli.steps,
                   "h2d_bytes_per_step": ga * mb * (seq + 1) * 8, "d2h_bytes_per_step": 4, "last_loss": last_loss,
                   "wall_ms_of_each_step": step_walls}
        ops.check_status()

        if cli.budget_output is not None:
            # one extra, untimed-for-the-headline step with CUDA events around every launch site of the block schedule,
            # the loss and the optimizer tail; the sites are sequential on one stream, so their sum is the step
            from lm_engine.ops import timeline

            torch.cuda.synchronize()
            timeline.enable_timing(True)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            step(feed_device)
            t1.record()
            sites = timeline.report()
            timeline.enable_timing(False)
            if rank == 0:
                with open(cli.budget_output, "w") as handle:
                    json.dump({"step_ms": t0.elapsed_time(t1), "n_gpus": world, "config": spec["name"], "sites": sites}, handle, indent=1)

    tokens_per_step = ga * mb * seq * (world // (pp * tp_size))
    ms_per_step = ms / cli.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    tflops_model = get_model_tflops(container[0].config, ga * mb * (world // (pp * tp_size)), seq)
    peak, peak_src = measured_peak_tflops()
    tflops_per_gpu = tflops_model / world / (ms_per_step / 1e3)
    result = {
        "impl": "native", "metric": ("pretraining tokens/s (40-expert top-8 MoE, expert parallel)" if moe else
                                     "pretraining tokens/s (8B dense, ZeRO-3 sharded data parallel)"), "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": cli.steps, "warmup": cli.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cli.fp8 is None else f"fp8 ({cli.fp8}) linears, bf16 elsewhere", "data": "synthetic uniform-random tokens, random-init weights",
        "config": {"model": spec["name"] + ("" if cli.layers is None else f"-DEBUG-{cli.layers}-layers"),
                   "global_batch": ga * mb * (world // (pp * tp_size)), "seq_len": seq, "micro_batch_per_gpu": mb, "gradient_accumulation_steps": ga,
                   "parallelism": (f"ep{expert_parallel} x " if moe else "") + (f"pp{pp} (1F1B, {ga} micro-batches) x " if pp > 1 else "") +
                   (f"tp{tp_size} (sequence parallel) x " if tp_size > 1 else "") +
                   f"fsdp{world // (pp * tp_size)} (ZeRO-3 sharded fp32 master/AdamW/gradients; " +
                   ("blocks gathered and released one by one)" if cli.sharded_parameters else "gathered bf16 weights kept for the step)"),
                   "optimizer": "AdamW fp32 master", "l2": "working set per step >> 126 MB L2 (inputs larger than L2)",
                   "kernels": kernels, "gradient_checkpointing": None},
        "tflops_per_gpu": tflops_per_gpu, "mfu": tflops_per_gpu / peak, "mfu_peak": f"{peak} TFLOP/s {peak_src}",
        "clocks": clocks, "gpu_launches": launches, "pytorch_fallbacks": sum(ops.fallback_counts().values()), "loss_after_warmup": loss_after_warmup,
        "peak_memory_gib": torch.cuda.max_memory_allocated() / 2**30,
        # the driver's view (includes the symmetric-memory arenas, which the tensor allocator does not see)
        "device_memory_used_gib": (torch.cuda.mem_get_info()[1] - torch.cuda.mem_get_info()[0]) / 2**30,
    }
    if expert_parallel > 1:
        from lm_engine.parallel.expert_parallel import dropped_entries

        dropped = torch.tensor([dropped_entries(device)], dtype=torch.int64, device=device)
        torch.distributed.all_reduce(dropped)
        result["config"]["expert_capacity_factor"] = capacity
        result["config"]["expert_entries_dropped"] = int(dropped.item())
    if e2e is not None:
        result["e2e"] = e2e
    ProcessGroupManager.destroy_process_groups()
    return result if rank == 0 else None


def moe_record(cli) -> dict | None:
    """Second record of the default run: the 40-expert top-8 MoE config, measured by a child process of every rank (same
    launch environment, rendezvous on the next port) after this process has released the GPU. Returns rank 0's record."""
    import gc

    import torch

    gc.collect()
    torch.cuda.empty_cache()
    rank = int(os.environ.get("RANK", 0))
    env = dict(os.environ)
    if "MASTER_PORT" in env:
        env["MASTER_PORT"] = str(int(env["MASTER_PORT"]) + 1)
    # the children rendezvous among themselves: rank 0's child hosts the store instead of looking for the launcher's
    for key in ("TORCHELASTIC_RUN_ID", "TORCHELASTIC_USE_AGENT_STORE"):
        env.pop(key, None)
    out_path = os.path.join(tempfile.gettempdir(), f"bench-moe-{os.getpid()}-{rank}.json")
    steps = cli.moe_steps or max(3, cli.steps // 4)
    # six warm-up steps for both arms: with dropless exact sizing the row buffers grow to the largest need seen so far, and
    # they have to have stopped growing before the timed steps (a step that grows them costs about twice a normal one)
    cmd = [sys.executable, os.path.abspath(__file__), "--config", "moe", "--gpus", str(cli.gpus), "--steps", str(steps), "--warmup", "6",
           "--impl", cli.impl, "--reference-compile", "off", "--child-output", out_path]
    if cli.skip_e2e:
        cmd.append("--skip-e2e")
    done = subprocess.run(cmd, env=env, stdout=subprocess.DEVNULL if rank else None)
    record = None
    if rank == 0:
        if done.returncode == 0 and os.path.exists(out_path):
            with open(out_path) as handle:
                record = json.load(handle)
            os.unlink(out_path)
        else:
            record = {"unavailable": f"the MoE run exited with code {done.returncode}"}
    return record


def main() -> None:
    cli = parse_args()
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    if cli.impl == "reference":
        from baseline.reference_arm import run_reference

        result = run_reference(cli, SPECS[cli.config], REPO_ROOT)
    else:
        result = run_native(cli)
    headline = (cli.config == "dense" and cli.layers is None and cli.gradient_accumulation_steps is None and not cli.sharded_parameters
                and cli.pipeline_parallel == 1 and cli.tensor_parallel == 1 and cli.fp8 is None and cli.sequence_length is None
                and cli.micro_batch_size is None)
    if headline and not cli.no_moe and cli.child_output is None:
        # the metric names both models: the MoE record rides along under "moe"; the headline `value` stays the dense one
        moe = moe_record(cli)
        if result is not None and moe is not None:
            keep = ("value", "unit", "ms_per_step", "steps", "warmup", "config", "e2e", "tflops_per_gpu", "mfu", "gpu_launches",
                    "loss_after_warmup", "peak_memory_gib", "clocks", "metric", "unavailable", "reference_notes")
            result["moe"] = {k: moe[k] for k in keep if k in moe}
    if result is not None:
        if cli.child_output is not None:
            with open(cli.child_output, "w") as handle:
                json.dump(result, handle)
        else:
            print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
