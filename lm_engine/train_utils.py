"""Helpers shared by the training drivers: metric reduction, logging, profiler, and the model FLOP count.

Parity: lm_engine/train_utils.py:17-212. ``get_model_tflops`` follows the reference's accounting exactly so that the
logged TFLOP/s and MFU are comparable: a linear layer costs 2mkn forward and twice that backward (one more forward
when its block is recomputed), attention costs ``2 b s (s + 1) h`` forward and 2.5x that backward, MoE layers
multiply the MLP cost by ``top_k``, gated activations by 1.5, plus the vocabulary projection.
"""

from __future__ import annotations

import logging
from contextlib import nullcontext

import torch
import torch.distributed as dist

from .enums import GradientCheckpointingMethod
from .hf_models import is_custom_model
from .hf_models.layers.activations import is_glu
from .utils import ExperimentsTracker, MetricsTrackingDict, ProcessGroupManager, log_metrics


def all_reduce_metrics_tracker(metrics_tracker: MetricsTrackingDict) -> MetricsTrackingDict:
    """Average every metric over the data parallel group with ONE collective (sum + divide: gloo has no AVG)."""
    keys = sorted(metrics_tracker.keys())
    if not keys:
        return metrics_tracker
    device = ProcessGroupManager.get_device() if ProcessGroupManager.is_initialized() else torch.device("cpu")
    values = torch.stack([torch.as_tensor(metrics_tracker[k], dtype=torch.float32, device=device).reshape(()) for k in keys])
    if ProcessGroupManager.is_initialized() and ProcessGroupManager.get_data_parallel_world_size() > 1:
        dist.all_reduce(values, op=dist.ReduceOp.SUM, group=ProcessGroupManager.get_data_parallel_group())
        values = values / ProcessGroupManager.get_data_parallel_world_size()
    values = values.tolist()
    for k, v in zip(keys, values):
        metrics_tracker[k] = v
    return metrics_tracker


def track_metrics(global_step: int, experiments_tracker: ExperimentsTracker | None, metrics_tracker: MetricsTrackingDict,
                  context: str) -> None:
    values = metrics_tracker.get_dict()
    if experiments_tracker is not None:
        experiments_tracker.track(values, step=global_step, context=context)
    parts = [f"step = {global_step}"]
    for key in sorted(values):
        value = values[key]
        text = f"{value:.4e}" if key == "learning_rate" else f"{value:.4f}" if isinstance(value, float) else str(value)
        parts.append(f"{context}-{key} = {text}")
    log_metrics(logging.INFO, ", ".join(parts))


def get_torch_profiler(torch_profiler_trace_path: str | None):
    """One traced step (after 5 idle + 5 warm-up steps) on global rank 0; other ranks effectively never trace."""
    if torch_profiler_trace_path is None:
        return nullcontext()
    wait = 5 if ProcessGroupManager.get_global_rank() == 0 else 150000
    return torch.profiler.profile(
        activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
        schedule=torch.profiler.schedule(wait=wait, warmup=5, active=1, repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(torch_profiler_trace_path),
        record_shapes=True,
    )


def _linear_flops(m: float, k: float, n: float, recompute: bool = False) -> float:
    forward = 2 * m * k * n
    return forward * (4 if recompute else 3)


def _attention_flops(b: int, s: int, h: int) -> float:
    forward = 2 * b * s * (s + 1) * h
    return forward * 3.5


def get_model_tflops(config, batch_size: int, sequence_length: int,
                     gradient_checkpointing_method: GradientCheckpointingMethod | None = None,
                     gradient_checkpointing_args: dict | None = None) -> float:
    """Model TFLOP for one pass (forward + backward) over ``batch_size`` sequences of ``sequence_length`` tokens."""
    if not is_custom_model(config.model_type):
        return 0
    gradient_checkpointing_args = gradient_checkpointing_args or {}
    b, s, h, v = batch_size, sequence_length, config.hidden_size, config.vocab_size
    checkpointed = (gradient_checkpointing_args.get("num_blocks", config.num_layers)
                    if gradient_checkpointing_method == GradientCheckpointingMethod.block else 0)
    total = 0.0
    for i in range(config.num_layers):
        mixer = config.sequence_mixer_blocks[i]
        kind = mixer.sequence_mixer_type
        rc = i < checkpointed
        if kind == "causal_convolution":
            f = _linear_flops(b * s, h, mixer.in_channels, rc)
            f += _linear_flops(b * s, mixer.in_channels, mixer.out_channels, rc) / mixer.num_groups
            f += _linear_flops(b * s, mixer.out_channels, h, rc)
        elif kind in ("softmax_attention", "stickbreaking_attention"):
            f = _linear_flops(b * s, h, h * (1 + 2 * mixer.num_key_value_heads / mixer.num_attention_heads), rc)
            f += _linear_flops(b * s, h, h, rc)
            f += _attention_flops(b, s, h)
        elif kind == "multihead_latent_attention":
            f = 2 * _linear_flops(b * s, h, mixer.query_compression_size + 2 * mixer.key_value_compression_size, rc)
            f += _linear_flops(b * s, h, h, rc)
            f += _attention_flops(b, s, h)
        elif kind == "mamba2":
            f = 2 * (4 * b * s * h * mixer.intermediate_size + 4 * b * s * mixer.intermediate_size * mixer.state_size)
        elif kind in ("rnn", "gru"):
            gates = 3 if kind == "gru" else 1
            head_dim = mixer.state_size / mixer.num_heads
            f = _linear_flops(b * s, h, gates * mixer.state_size) + _linear_flops(b * s, mixer.state_size, h)
            f += gates * s * mixer.num_heads * (_linear_flops(b, head_dim, head_dim) + b * head_dim)
        else:
            raise NotImplementedError(f"unexpected sequence_mixer_type ({kind})")
        total += f

        mlp = config.mlp_blocks[i]
        f = 2 * _linear_flops(b * s, h, mlp.intermediate_size, rc)
        if mlp.mlp_type == "MoE":
            f *= mlp.num_experts_per_tok
        if is_glu(mlp.activation_function):
            f *= 1.5
        total += f
    total += _linear_flops(b * s, h, v)
    return total / 1e12


def check_device_health() -> None:
    """Stop the run if a kernel reported a bounded wait that ran out, a peer barrier that a rank never reached, or a
    violated assumption of a fused op since the last check.

    Every device-side wait of this library is bounded: on expiry a kernel records a status code and returns, so the
    step goes on with partial data. The training loops call this where they synchronise with the device anyway (after
    reading the logged loss, and always before a checkpoint is written) so that such a step is never trained on further
    or saved. Costs one small device-to-host read per status word; does nothing on CPU."""
    if not torch.cuda.is_available():
        return
    from . import ops
    from .parallel.symmetric import check_all_peer_groups

    ops.check_status()
    check_all_peer_groups()
