"""Wrapper for next-token pretraining on fixed-length samples of ``sequence_length + 1`` tokens.

Parity: lm_engine/model_wrapper/pretraining.py:24-315. ``input_ids = tokens[:, :-1]``, ``labels = tokens[:, 1:]``;
the loss is the SUM of token cross entropies times ``lm_loss_multiplier`` plus ``router_aux_loss_coef * aux_loss``.
With the padding-free transformer the micro-batch is flattened; documents are either the fixed-length samples
(pre-built ``cu_seqlens`` / ``position_ids``) or, with ``reset_attention_mask``, the spans between EOS tokens.
"""

from __future__ import annotations

import torch

from ..enums import Kernel, Mode
from ..hf_models import get_autoregressive_language_modeling_loss, is_aux_loss_zero
from ..kernels import is_kernel_allowed
from ..utils import MetricsTrackingDict, ProcessGroupManager, StepTracker
from .base import ModelWrapper


class ModelWrapperForPretraining(ModelWrapper):
    def __init__(self, *args, micro_batch_size: int, sequence_length: int, reset_attention_mask: bool = False,
                 reset_position_ids: bool = False, **kwargs) -> None:
        self.micro_batch_size = micro_batch_size
        self.sequence_length = sequence_length
        self.reset_attention_mask = reset_attention_mask
        self.reset_position_ids = reset_position_ids
        self._extra_metrics = MetricsTrackingDict({})
        self._packed_cache: dict = {}
        super().__init__(*args, **kwargs)
        if self.is_pipeline_parallel_enabled and self.tie_word_embeddings:
            raise NotImplementedError("tied embeddings are not supported with pipeline parallel")

    # ------------------------------------------------------------------ inputs
    def _fixed_packing(self, device) -> tuple[torch.Tensor, torch.Tensor]:
        key = (str(device), self.micro_batch_size, self.sequence_length)
        if key not in self._packed_cache:
            mb, seq = self.micro_batch_size, self.sequence_length
            cu = torch.arange(0, mb * seq + 1, seq, dtype=torch.int32, device=device)
            pos = torch.arange(seq, dtype=torch.int32, device=device).repeat(mb)
            self._packed_cache[key] = (cu, pos)
        return self._packed_cache[key]

    def _prepare_model_inputs(self, batch: dict) -> dict:
        tokens = batch["text"]
        device = next(self.model.parameters()).device
        if ProcessGroupManager.is_tensor_parallel_enabled():
            from .utils import broadcast_tensor_parallel_input

            tokens = broadcast_tensor_parallel_input(tokens, (self.micro_batch_size, self.sequence_length + 1))
        else:
            tokens = tokens.to(device, non_blocking=True)
        input_ids = tokens[:, :-1]
        labels = tokens[:, 1:]
        out = {}
        if self.use_padding_free_transformer:
            mb, seq = input_ids.shape
            input_ids = input_ids.reshape(-1)
            labels = labels.reshape(-1)
            if self.reset_attention_mask:
                eos_positions = torch.where(input_ids == self.eos_token_id)[0]
                ends = eos_positions + 1
                sample_ends = torch.arange(seq, mb * seq + 1, seq, device=input_ids.device)
                bounds = torch.unique(torch.cat([ends.new_zeros(1), ends, sample_ends]))
                cu_seqlens = bounds.to(torch.int32)
                lengths = cu_seqlens[1:] - cu_seqlens[:-1]
                max_seqlen = int(lengths.max().item())
                if self.reset_position_ids:
                    starts = torch.repeat_interleave(cu_seqlens[:-1].long(), lengths.long())
                    position_ids = torch.arange(mb * seq, device=input_ids.device) - starts
                else:
                    position_ids = torch.arange(seq, device=input_ids.device).repeat(mb)
            else:
                cu_seqlens, position_ids = self._fixed_packing(input_ids.device)
                max_seqlen = seq
            out.update(cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, position_ids=position_ids)
        out.update(input_ids=input_ids.contiguous(), labels=labels.contiguous())
        if ProcessGroupManager.is_tensor_parallel_enabled():
            out["output_parallel_lm_logits"] = True
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, batch: dict | torch.Tensor, aux_loss_from_pipeline_parallel=0, lm_loss_multiplier: float = 1) -> dict:
        if isinstance(batch, torch.Tensor):
            batch = {"text": batch}
        inputs = self._prepare_model_inputs(batch)
        labels = inputs.pop("labels")
        if self.is_pipeline_parallel_enabled:
            return self._forward_pipeline_stage(inputs, labels, batch.get("pipeline_parallel_input"), lm_loss_multiplier)
        output = self.model(**inputs, return_dict=True)
        return self.get_loss(output, labels, lm_loss_multiplier=lm_loss_multiplier)

    def get_loss(self, model_outputs, labels: torch.Tensor, lm_loss_multiplier: float = 1) -> dict:
        # under tensor parallelism the LM head is vocabulary-parallel: its logits go to the vocabulary-parallel loss
        fused = (is_kernel_allowed(Kernel.fused_linear_cross_entropy_cute) and self.is_custom_model
                 and not ProcessGroupManager.is_tensor_parallel_enabled())
        hint = None
        if fused and self.training and torch.is_grad_enabled():
            ga = StepTracker.get_gradient_accumulation_steps() or 1
            hint = lm_loss_multiplier / ga
        m_width = getattr(self.config, "m_width", None)
        lm_loss = get_autoregressive_language_modeling_loss(
            lm_logits=None if fused else model_outputs.logits,
            labels=labels,
            hidden_states=self._hidden_for_fused(model_outputs, m_width) if fused else None,
            vocab_weight=self.model.get_output_embeddings().weight if fused else None,
            cu_seqlens=None,
            use_padding_free_transformer=self.use_padding_free_transformer,
            reduction="sum",
            shift_logits_and_labels=False,
            tensor_parallel_enabled=ProcessGroupManager.is_tensor_parallel_enabled(),
            grad_scale_hint=hint,
        )
        lm_loss = lm_loss * lm_loss_multiplier
        aux_loss = getattr(model_outputs, "aux_loss", 0)
        if is_aux_loss_zero(aux_loss):
            return {"loss": lm_loss, "lm_loss": lm_loss}
        loss = lm_loss + self.router_aux_loss_coef * aux_loss
        return {"loss": loss, "lm_loss": lm_loss, "aux_loss": aux_loss}

    @staticmethod
    def _hidden_for_fused(model_outputs, m_width):
        # the model already divided the hidden states by m_width when no labels were passed to it
        return model_outputs.last_hidden_state

    def _forward_pipeline_stage(self, inputs: dict, labels, boundary_input, lm_loss_multiplier: float = 1):
        """``boundary_input``: ``(hidden_states, aux_loss)`` from the previous stage (``None`` on the first stage)."""
        from ..parallel.pipeline import run_stage

        return run_stage(self, inputs, labels, boundary_input, lm_loss_multiplier)

    def get_extra_metrics(self) -> MetricsTrackingDict:
        return self._extra_metrics

    def reset_extra_metrics(self) -> None:
        self._extra_metrics = MetricsTrackingDict({})
