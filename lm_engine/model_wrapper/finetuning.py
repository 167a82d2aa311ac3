"""Wrapper for supervised finetuning on collated batches (parity: lm_engine/model_wrapper/finetuning.py:18-120).

The loss is the SUM of token cross entropies (labels shifted inside; with packed inputs the last token of every
document is masked) times ``lm_loss_multiplier``; the driver sets the multiplier to one over the number of target
tokens of the whole accumulation window.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..communication import Communication
from ..enums import Kernel
from ..hf_models import get_autoregressive_language_modeling_loss, is_aux_loss_zero
from ..kernels import is_kernel_allowed
from ..utils import ProcessGroupManager
from .base import ModelWrapper


class ModelWrapperForFinetuning(ModelWrapper):
    def forward(self, batch: dict, lm_loss_multiplier: float = 1) -> dict:
        if ProcessGroupManager.is_tensor_parallel_enabled():
            batch = self._broadcast_inputs_for_tensor_parallel(batch)
        else:
            device = next(self.model.parameters()).device
            batch = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        labels = batch.pop("labels")
        output = self.model(**batch, return_dict=True)
        return self.get_loss(output, labels, cu_seqlens=batch.get("cu_seqlens"), lm_loss_multiplier=lm_loss_multiplier)

    def get_loss(self, model_outputs, labels: torch.Tensor, cu_seqlens: torch.Tensor | None, lm_loss_multiplier: float = 1) -> dict:
        fused = is_kernel_allowed(Kernel.fused_linear_cross_entropy_cute) and self.is_custom_model
        lm_loss = get_autoregressive_language_modeling_loss(
            lm_logits=None if fused else model_outputs.logits,
            labels=labels,
            hidden_states=model_outputs.last_hidden_state if fused else None,
            vocab_weight=self.model.get_output_embeddings().weight if fused else None,
            cu_seqlens=cu_seqlens,
            use_padding_free_transformer=self.use_padding_free_transformer,
            reduction="sum",
            shift_logits_and_labels=True,
            tensor_parallel_enabled=ProcessGroupManager.is_tensor_parallel_enabled(),
        )
        lm_loss = lm_loss * lm_loss_multiplier
        aux_loss = getattr(model_outputs, "aux_loss", 0)
        if is_aux_loss_zero(aux_loss):
            return {"loss": lm_loss, "lm_loss": lm_loss}
        loss = lm_loss + self.router_aux_loss_coef * aux_loss
        return {"loss": loss, "lm_loss": lm_loss, "aux_loss": aux_loss}

    def _broadcast_inputs_for_tensor_parallel(self, batch: dict | None) -> dict:
        """Only tp-rank 0 has a batch: broadcast its keys / shapes / dtypes, then every tensor."""
        device = ProcessGroupManager.get_device()
        group = ProcessGroupManager.get_tensor_parallel_group()
        src = ProcessGroupManager.get_tensor_parallel_first_rank()
        first = ProcessGroupManager.is_tensor_parallel_first_rank()
        meta = None
        if first:
            meta = {k: (tuple(v.shape), v.dtype) if isinstance(v, torch.Tensor) else ("py", v) for k, v in batch.items()}
        meta = Communication.broadcast_object(meta, src=src, group=group)
        out = {}
        for key, info in meta.items():
            if info[0] == "py":
                out[key] = info[1]
                continue
            shape, dtype = info
            tensor = batch[key].to(device) if first else torch.empty(shape, dtype=dtype, device=device)
            dist.broadcast(tensor, src=src, group=group)
            out[key] = tensor
        return out
