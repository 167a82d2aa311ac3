"""Pipeline parallelism: stage placement, schedules and the training step.

The reference wraps every local stage in ``torch.distributed.pipelining.PipelineStage`` and runs a stock schedule
(lm_engine/distributed.py:358-424, lm_engine/pretrain.py:46-140 there). Here the schedule is an explicit list of
actions per rank and the transfers are point-to-point sends of the stage boundary tensors:

* stage ``s`` of ``S`` lives on pipeline rank ``s % P`` (looped placement, ``S / P`` stages per rank);
* an action is ``(F | B, stage, micro-batch)``; ``GPipe`` runs every forward, then every backward; ``1F1B`` (one
  stage per rank) warms up with ``P - rank - 1`` forwards and then alternates one forward with one backward, which
  bounds the live activations by the pipeline depth; ``Interleaved1F1B`` does the same over the virtual stages of a
  rank in Megatron-LM's order (micro-batches a multiple of ``P``);
* a boundary transfer carries the hidden states and the running auxiliary loss forward, and their gradients backward.
  Every (source, destination, direction) triple has its own process group, so transfers of one triple are matched
  in program order and different triples cannot block one another (NCCL serialises the operations of a communicator);
* all pipeline ranks of one data-parallel replica read the same batch; the first stage uses the tokens, the last stage
  the labels, every stage the packing metadata.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..hf_models.loss import is_aux_loss_zero
from ..utils import MetricsTrackingDict, ProcessGroupManager, StepTracker, divide_if_divisible

FORWARD, BACKWARD = "F", "B"


# ----------------------------------------------------------------------------------------------------------------------
# schedules (pure functions of sizes: tested on CPU without process groups)
def _gpipe(rank: int, world: int, local_stages: list[int], microbatches: int) -> list[tuple[str, int, int]]:
    forward = [(FORWARD, s, m) for s in local_stages for m in range(microbatches)]
    backward = [(BACKWARD, s, m) for s in reversed(local_stages) for m in range(microbatches)]
    return forward + backward


def _one_f_one_b(rank: int, world: int, local_stages: list[int], microbatches: int) -> list[tuple[str, int, int]]:
    assert len(local_stages) == 1, "1F1B places one stage on every pipeline rank; use Interleaved1F1B for more"
    stage = local_stages[0]
    warmup = min(world - rank - 1, microbatches)
    actions = [(FORWARD, stage, m) for m in range(warmup)]
    f, b = warmup, 0
    while f < microbatches:
        actions.append((FORWARD, stage, f))
        actions.append((BACKWARD, stage, b))
        f, b = f + 1, b + 1
    actions += [(BACKWARD, stage, m) for m in range(b, microbatches)]
    return actions


def _interleaved(rank: int, world: int, local_stages: list[int], microbatches: int) -> list[tuple[str, int, int]]:
    chunks = len(local_stages)
    if chunks == 1:
        return _one_f_one_b(rank, world, local_stages, microbatches)
    divide_if_divisible(microbatches, world, "Interleaved1F1B needs the micro-batch count to be a multiple of the pipeline size")
    total = microbatches * chunks

    def unit(k: int, forward: bool) -> tuple[int, int]:
        chunk = (k // world) % chunks
        if not forward:
            chunk = chunks - 1 - chunk
        micro = (k // (world * chunks)) * world + k % world
        return local_stages[chunk], micro

    warmup = min((world - rank - 1) * 2 + (chunks - 1) * world, total)
    actions = [(FORWARD, *unit(k, True)) for k in range(warmup)]
    f, b = warmup, 0
    while f < total:
        actions.append((FORWARD, *unit(f, True)))
        actions.append((BACKWARD, *unit(b, False)))
        f, b = f + 1, b + 1
    actions += [(BACKWARD, *unit(k, False)) for k in range(b, total)]
    return actions


_SCHEDULES = {"GPipe": _gpipe, "1F1B": _one_f_one_b, "Interleaved1F1B": _interleaved, "LoopedBFS": _gpipe}


def build_actions(schedule: str, rank: int, world: int, num_stages: int, microbatches: int) -> list[tuple[str, int, int]]:
    if schedule not in _SCHEDULES:
        raise ValueError(f"unexpected pipeline_parallel_schedule ({schedule}); known: {sorted(_SCHEDULES)}")
    per_rank = divide_if_divisible(num_stages, world, "number of stages must be a multiple of the pipeline size")
    local = [rank + i * world for i in range(per_rank)]
    return _SCHEDULES[schedule](rank, world, local, microbatches)


# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class PipelineSchedule:
    name: str
    num_stages: int
    microbatches: int
    rank: int
    world: int
    actions: list[tuple[str, int, int]]
    stage_to_wrapper: dict[int, object]
    groups: dict[tuple[int, int, str], dist.ProcessGroup | None] = field(default_factory=dict)
    global_rank_of: list[int] = field(default_factory=list)  # pipeline rank -> global rank (same dp/tp coordinates)

    def owner(self, stage: int) -> int:
        return stage % self.world


def _pipeline_peers() -> list[int]:
    return dist.get_process_group_ranks(ProcessGroupManager.get_pipeline_parallel_group())


def build_pipeline_schedule(args, model_container) -> PipelineSchedule:
    d = args.distributed_args
    world = ProcessGroupManager.get_pipeline_parallel_world_size()
    rank = ProcessGroupManager.get_pipeline_parallel_rank()
    microbatches = args.training_parameters.gradient_accumulation_steps
    actions = build_actions(d.pipeline_parallel_schedule, rank, world, d.num_pipeline_stages, microbatches)
    wrappers = {w.pipeline_stage_id: w for w in model_container}
    schedule = PipelineSchedule(d.pipeline_parallel_schedule, d.num_pipeline_stages, microbatches, rank, world, actions, wrappers,
                                global_rank_of=_pipeline_peers())
    schedule.groups = _make_transfer_groups(world)
    return schedule


def _make_transfer_groups(world: int) -> dict:
    """One group per (source, destination, direction) between neighbouring pipeline ranks of THIS pipeline group.
    ``new_group`` is collective over the whole job, so every rank creates the groups of every pipeline group."""
    if world == 1:
        return {}
    mine = tuple(_pipeline_peers())
    gathered: list = [None] * dist.get_world_size()
    dist.all_gather_object(gathered, mine)
    out = {}
    nccl = torch.cuda.is_available() and "nccl" in str(dist.get_backend())
    for peers in sorted(set(gathered)):
        for src in range(world):
            dst = (src + 1) % world
            for direction in (FORWARD, BACKWARD):
                a, b = (src, dst) if direction == FORWARD else (dst, src)
                group = dist.new_group([peers[a], peers[b]]) if nccl and peers[a] != peers[b] else None
                if peers == mine:
                    out[(a, b, direction)] = group
    if nccl:
        _connect_transfer_groups(out, mine)
    return out


def _connect_transfer_groups(groups: dict, peers: tuple[int, ...]) -> None:
    """One tiny blocking transfer over every group this rank belongs to, in one global order of the keys. The first
    point-to-point operation on a group creates its communicator, which blocks the host until the peer joins: done
    here, where both ends walk the same list, instead of inside the schedule, where one end may be a whole forward and
    backward pass away from its matching call (the pipeline ranks' action lists are not symmetric)."""
    me = dist.get_rank()
    token = torch.zeros(1, device=torch.device("cuda", torch.cuda.current_device()))
    for (a, b, direction) in sorted(groups):
        group = groups[(a, b, direction)]
        if group is None:
            continue
        if peers[a] == me:
            dist.send(token, dst=peers[b], group=group)
        elif peers[b] == me:
            dist.recv(token, src=peers[a], group=group)
    torch.cuda.synchronize()


class _Mailbox:
    """Point-to-point transfers of one training step.

    What crosses a stage boundary (hidden states + the running auxiliary loss, or their gradients) travels as ONE
    message: the scalar is appended to the flattened hidden states as raw fp32 bits. Receives are posted ahead of
    time (``prefetch``) so that a transfer runs under the compute of the action before the one that consumes it;
    ``recv`` only waits. Sends are asynchronous and are waited for at the end of the step.
    """

    def __init__(self, schedule: PipelineSchedule) -> None:
        self.schedule = schedule
        self.pending = []
        self.local: dict[tuple, list[torch.Tensor]] = {}
        self.posted: dict[tuple, tuple] = {}

    @staticmethod
    def _tail(dtype: torch.dtype) -> int:
        return 4 // torch.empty((), dtype=dtype).element_size() if dtype != torch.float64 else 1

    @classmethod
    def _pack(cls, hidden: torch.Tensor, scalar: torch.Tensor) -> torch.Tensor:
        tail = cls._tail(hidden.dtype)
        flat = torch.empty(hidden.numel() + tail, device=hidden.device, dtype=hidden.dtype)
        flat[: hidden.numel()].copy_(hidden.detach().reshape(-1))
        if hidden.dtype == torch.float64:
            flat[-1] = scalar.detach().double()
        else:
            flat[hidden.numel() :].view(torch.float32).copy_(scalar.detach().float().reshape(1))
        return flat

    @classmethod
    def _unpack(cls, flat: torch.Tensor, like: torch.Tensor) -> list[torch.Tensor]:
        hidden = flat[: like.numel()].view(like.shape)
        if like.dtype == torch.float64:
            scalar = flat[-1].float()
        else:
            scalar = flat[like.numel() :].view(torch.float32).reshape(())
        return [hidden, scalar]

    def _route(self, src_stage: int, dst_stage: int, micro: int, direction: str):
        s = self.schedule
        src, dst = s.owner(src_stage), s.owner(dst_stage)
        tag = (dst_stage * s.microbatches + micro) * 2 + (0 if direction == FORWARD else 1)
        return src, dst, s.groups.get((src, dst, direction)), tag

    def send(self, tensors: list[torch.Tensor], src_stage: int, dst_stage: int, micro: int, direction: str) -> None:
        src, dst, group, tag = self._route(src_stage, dst_stage, micro, direction)
        if src == dst:
            self.local[(dst_stage, micro, direction)] = [t.detach() for t in tensors]
            return
        flat = self._pack(tensors[0], tensors[1])
        self.pending.append((dist.isend(flat, dst=self.schedule.global_rank_of[dst], group=group, tag=tag), flat))

    def prefetch(self, like: torch.Tensor, src_stage: int, dst_stage: int, micro: int, direction: str) -> None:
        """Post the receive for ``(dst_stage, micro, direction)`` now; ``like`` gives shape and dtype of the hidden states."""
        key = (dst_stage, micro, direction)
        src, dst, group, tag = self._route(src_stage, dst_stage, micro, direction)
        if src == dst or key in self.posted:
            return
        flat = torch.empty(like.numel() + self._tail(like.dtype), device=like.device, dtype=like.dtype)
        work = dist.irecv(flat, src=self.schedule.global_rank_of[src], group=group, tag=tag)
        self.posted[key] = (work, flat, like)

    def recv(self, like: list[torch.Tensor], src_stage: int, dst_stage: int, micro: int, direction: str) -> list[torch.Tensor]:
        key = (dst_stage, micro, direction)
        src, dst, _, _ = self._route(src_stage, dst_stage, micro, direction)
        if src == dst:
            return self.local.pop(key)
        self.prefetch(like[0], src_stage, dst_stage, micro, direction)
        work, flat, hidden_like = self.posted.pop(key)
        work.wait()
        return self._unpack(flat, hidden_like)

    def finish(self) -> None:
        for work, _ in self.pending:
            work.wait()
        self.pending.clear()
        assert not self.posted, "a posted pipeline receive was never consumed"


# ----------------------------------------------------------------------------------------------------------------------
def _boundary_like(wrapper, inputs: dict) -> list[torch.Tensor]:
    """Shapes of what crosses a stage boundary: hidden states (token-sharded under sequence parallelism) + aux loss."""
    model = wrapper.model
    hidden = model.config.hidden_size
    device = next(model.parameters()).device
    dtype = next(model.parameters()).dtype
    ids = inputs["input_ids"]
    tp = ProcessGroupManager.get_tensor_parallel_world_size() if wrapper.sequence_parallel else 1
    if ids.dim() == 1:
        shape = (ids.shape[0] // tp, hidden)
    else:
        shape = (ids.shape[0], ids.shape[1] // tp, hidden)
    return [torch.empty(shape, device=device, dtype=dtype), torch.empty((), device=device, dtype=torch.float32)]


def run_stage(wrapper, inputs: dict, labels, boundary_input, lm_loss_multiplier: float = 1):
    """Forward of one stage. First stage: tokens in; later stages: ``boundary_input = (hidden_states, aux_loss)``.
    Returns ``(hidden_states, aux_loss)`` or, on the last stage, the loss dictionary."""
    kwargs = {k: v for k, v in inputs.items() if k != "labels"}
    if not wrapper.is_first_stage:
        kwargs.pop("input_ids", None)
        kwargs["pipeline_parallel_input"] = boundary_input
    output = wrapper.model(**kwargs, return_dict=True)
    if not wrapper.is_last_stage:
        return output
    return wrapper.get_loss(output, labels, lm_loss_multiplier=lm_loss_multiplier)


def pipeline_train_step(model_container, schedule: PipelineSchedule, optimizer_container, lr_scheduler_container, train_dataloader,
                        gradient_clipping, sequence_length: int | None = None, lm_loss_multiplier: float | None = None) -> MetricsTrackingDict:
    """One optimizer step under pipeline parallelism. The last stage's loss is a sum over tokens scaled by
    ``lm_loss_multiplier``; when it is not given it is ``1 / (micro_batch_size * sequence_length)``, the normalisation
    of the step without pipeline parallelism (parity: lm_engine/distributed.py:398 of the reference)."""
    from ..data import get_next_batch

    if lm_loss_multiplier is None:
        mbs = next(iter(schedule.stage_to_wrapper.values())).micro_batch_size
        lm_loss_multiplier = 1.0 if sequence_length is None else 1.0 / (mbs * sequence_length)

    # the loader yields either all micro-batches of the step at once or one micro-batch per item
    micro_batch_size = next(iter(schedule.stage_to_wrapper.values())).micro_batch_size
    micro_batches: list = []
    while len(micro_batches) < schedule.microbatches:
        batch = get_next_batch(train_dataloader)
        if isinstance(batch, dict):
            batch = batch["text"]
        if batch is None:  # ranks that receive their tokens by tensor-parallel broadcast
            micro_batches.append(None)
        else:
            micro_batches.extend(batch.split(micro_batch_size, dim=0))
    assert len(micro_batches) == schedule.microbatches, "the loader's batch is not a whole number of micro-batches"

    mailbox = _Mailbox(schedule)
    prepared: dict[tuple[int, int], tuple] = {}
    live: dict[tuple[int, int], tuple] = {}  # (stage, micro) -> (boundary inputs that need gradients, outputs)
    metrics = MetricsTrackingDict({})
    last = schedule.num_stages - 1

    def prepare(stage: int, micro: int):
        key = (stage, micro)
        if key not in prepared:
            wrapper = schedule.stage_to_wrapper[stage]
            inputs = wrapper._prepare_model_inputs({"text": micro_batches[micro]})
            labels = inputs.pop("labels")
            prepared[key] = (inputs, labels)
        return prepared[key]

    def post_receive(index: int) -> None:
        # the receive of action `index` is posted while the action before it computes
        if index >= len(schedule.actions):
            return
        kind, stage, micro = schedule.actions[index]
        wrapper = schedule.stage_to_wrapper[stage]
        if kind == FORWARD and stage > 0:
            inputs, _ = prepare(stage, micro)
            mailbox.prefetch(_boundary_like(wrapper, inputs)[0], stage - 1, stage, micro, FORWARD)
        elif kind == BACKWARD and stage < last and (stage, micro) in prepared:
            inputs, _ = prepared[(stage, micro)]
            mailbox.prefetch(_boundary_like(wrapper, inputs)[0], stage + 1, stage, micro, BACKWARD)

    post_receive(0)
    for index, (kind, stage, micro) in enumerate(schedule.actions):
        post_receive(index + 1)
        wrapper = schedule.stage_to_wrapper[stage]
        if kind == FORWARD:
            inputs, labels = prepare(stage, micro)
            boundary = None
            if stage > 0:
                hidden, aux = mailbox.recv(_boundary_like(wrapper, inputs), stage - 1, stage, micro, FORWARD)
                boundary = (hidden.requires_grad_(True), aux.clone().requires_grad_(True))
            output = run_stage(wrapper, inputs, labels, boundary, lm_loss_multiplier)
            if stage < last:
                hidden_out, aux_out = output
                mailbox.send([hidden_out, aux_out.float()], stage, stage + 1, micro, FORWARD)
                live[(stage, micro)] = (boundary, (hidden_out, aux_out))
            else:
                live[(stage, micro)] = (boundary, output["loss"])
                with torch.inference_mode():
                    metrics = metrics + {k: v.detach().float() if isinstance(v, torch.Tensor) else v for k, v in output.items()}
        else:
            boundary, output = live.pop((stage, micro))
            if stage == last:
                (output / schedule.microbatches).backward()
            else:
                hidden_out, aux_out = output
                g_hidden, g_aux = mailbox.recv([hidden_out, aux_out.float()], stage + 1, stage, micro, BACKWARD)
                roots, grads = [hidden_out], [g_hidden]
                if aux_out.requires_grad:
                    roots.append(aux_out)
                    grads.append(g_aux.to(aux_out.dtype))
                torch.autograd.backward(roots, grads)
            if stage > 0:
                hidden_in, aux_in = boundary
                g_aux_in = aux_in.grad if aux_in.grad is not None else torch.zeros_like(aux_in)
                mailbox.send([hidden_in.grad, g_aux_in], stage, stage - 1, micro, BACKWARD)
            wrapper._lm_engine.fold_autograd_grads()
            prepared.pop((stage, micro), None)
    mailbox.finish()

    # one global gradient norm over all stages, then every stage steps
    engines = [w._lm_engine for w in model_container]
    total = None
    for engine in engines:
        engine.reduce_gradients()
        part = engine.grad_norm_sq()
        total = part.clone() if total is None else total + part
    if schedule.world > 1:
        dist.all_reduce(total, group=ProcessGroupManager.get_pipeline_parallel_group())
    grad_norm = None
    for engine, optimizer, scheduler in zip(engines, optimizer_container, lr_scheduler_container):
        grad_norm = engine.optimizer_step(optimizer, scheduler, gradient_clipping, precomputed_norm_sq=total)

    with torch.inference_mode():
        if len(metrics.keys()) > 0:
            metrics = metrics / schedule.microbatches
        metrics["grad_norm"] = grad_norm.reshape(()).clone()
    return metrics
