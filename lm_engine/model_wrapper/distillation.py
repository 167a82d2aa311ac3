"""Wrapper for knowledge distillation during pretraining (parity: lm_engine/model_wrapper/distillation.py:27-197).

``loss = CE(student) + kl_divergence_weight * KL`` with forward (teacher || student) or backward KL evaluated on fp32
log-probabilities with ``batchmean`` reduction. The teacher is loaded from ``teacher_args.model_name``, frozen, always
in eval mode and excluded from checkpoints.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..enums import Kernel, KLDivergenceMethod, Mode
from ..hf_models import get_autoregressive_language_modeling_loss, is_aux_loss_zero
from ..kernels import is_kernel_allowed
from ..utils import ProcessGroupManager
from .pretraining import ModelWrapperForPretraining


class ModelWrapperForDistillation(ModelWrapperForPretraining):
    def __init__(self, *args, teacher_model_name: str | None, teacher_model_class, teacher_model_dtype: torch.dtype,
                 kl_divergence_method: KLDivergenceMethod, kl_divergence_weight: float = 1, **kwargs) -> None:
        self.teacher_model_name = teacher_model_name
        self.teacher_model_class = teacher_model_class
        self.teacher_model_dtype = teacher_model_dtype
        self.kl_divergence_method = kl_divergence_method
        self.kl_divergence_weight = kl_divergence_weight
        super().__init__(*args, **kwargs)
        if ProcessGroupManager.is_tensor_parallel_enabled() or self.is_pipeline_parallel_enabled:
            raise NotImplementedError("distillation does not support tensor or pipeline parallelism")
        if is_kernel_allowed(Kernel.fused_linear_cross_entropy_cute):
            raise ValueError("distillation needs the student logits: disable fused_linear_cross_entropy_cute")

    def _setup_model(self) -> None:
        super()._setup_model()
        kwargs = {"torch_dtype": self.teacher_model_dtype}
        if self.use_padding_free_transformer:
            kwargs["use_padding_free_transformer"] = True
        self.teacher_model = self.teacher_model_class.from_pretrained(self.teacher_model_name, **kwargs)
        self.teacher_model.eval()
        for p in self.teacher_model.parameters():
            p.requires_grad_(False)

    def has_teacher_model(self) -> bool:
        return True

    def train(self, mode: bool = True):
        super().train(mode)
        self.teacher_model.eval()  # the teacher never leaves eval mode
        return self

    def forward(self, batch: dict | torch.Tensor, aux_loss_from_pipeline_parallel=0, lm_loss_multiplier: float = 1) -> dict:
        if isinstance(batch, torch.Tensor):
            batch = {"text": batch}
        inputs = self._prepare_model_inputs(batch)
        labels = inputs.pop("labels")
        student = self.model(**inputs, return_dict=True)
        with torch.inference_mode():
            teacher_logits = self.teacher_model(**inputs, return_dict=True).logits
        teacher_logits = teacher_logits.clone()
        return self.get_loss(student, labels, teacher_logits, lm_loss_multiplier)

    def get_loss(self, model_outputs, labels: torch.Tensor, teacher_logits: torch.Tensor | None = None,
                 lm_loss_multiplier: float = 1) -> dict:
        student_logits = model_outputs.logits
        lm_loss = get_autoregressive_language_modeling_loss(
            lm_logits=student_logits, labels=labels, use_padding_free_transformer=self.use_padding_free_transformer,
            reduction="sum", shift_logits_and_labels=False) * lm_loss_multiplier
        s = F.log_softmax(student_logits.float().reshape(-1, student_logits.shape[-1]), dim=-1)
        t = F.log_softmax(teacher_logits.float().reshape(-1, teacher_logits.shape[-1]), dim=-1)
        if self.kl_divergence_method == KLDivergenceMethod.forward:
            kl = F.kl_div(s, t, reduction="batchmean", log_target=True)  # KL(teacher || student)
        elif self.kl_divergence_method == KLDivergenceMethod.backward:
            kl = F.kl_div(t, s, reduction="batchmean", log_target=True)  # KL(student || teacher)
        else:
            raise ValueError(f"unexpected kl_divergence_method ({self.kl_divergence_method})")
        loss = lm_loss + self.kl_divergence_weight * kl
        out = {"loss": loss, "lm_loss": lm_loss, "kl_divergence": kl}
        aux_loss = getattr(model_outputs, "aux_loss", 0)
        if not is_aux_loss_zero(aux_loss):
            out["loss"] = loss + self.router_aux_loss_coef * aux_loss
            out["aux_loss"] = aux_loss
        return out
