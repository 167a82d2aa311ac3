"""Model wrapper: resolves config / tokenizer / model from the argument tree and owns generation and export.

Parity: lm_engine/model_wrapper/base.py:17-276. Training builds the model on the meta device whenever the sharded
engine will own the parameters (nothing is allocated twice); inference loads directly in the target dtype.
"""

from __future__ import annotations

import logging

import torch
import torch.nn as nn
from transformers import AutoConfig, AutoTokenizer

from ..enums import Kernel, Mode
from ..hf_models import get_model_parallel_class, is_custom_model
from ..kernels import is_kernel_allowed
from ..utils import ProcessGroupManager, SafeTensorsWeightsManager, log_rank_0, string_to_torch_dtype


class ModelWrapper(nn.Module):
    def __init__(
        self,
        mode: Mode,
        model_name: str | None,
        pretrained_config: dict | None,
        model_class,
        dtype: torch.dtype,
        efficient_initialization: bool,
        use_padding_free_transformer: bool,
        sequence_parallel: bool = False,
        num_pipeline_stages: int = 1,
        pipeline_stage_id: int = 0,
        trust_remote_code: bool = False,
        tokenizer_name: str | None = None,
        additional_special_tokens: list[str] | None = None,
        keep_in_fp32: bool = True,
    ) -> None:
        super().__init__()
        self.mode = mode
        self.model_name = model_name
        self.pretrained_config = pretrained_config
        self.model_class = model_class
        self.efficient_initialization = efficient_initialization
        self.dtype = dtype
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.tokenizer_name = model_name if tokenizer_name is None else tokenizer_name
        self.trust_remote_code = trust_remote_code
        self.keep_in_fp32 = keep_in_fp32

        self.num_pipeline_stages = num_pipeline_stages
        self.pipeline_stage_id = pipeline_stage_id
        self.is_pipeline_parallel_enabled = num_pipeline_stages > 1
        self.is_first_stage = pipeline_stage_id == 0
        self.is_last_stage = pipeline_stage_id == num_pipeline_stages - 1

        self._setup_config()
        self.is_custom_model = is_custom_model(self.config.model_type)
        self.tp_world_size = ProcessGroupManager.get_tensor_parallel_world_size()
        self.model_parallel = self.tp_world_size > 1 or self.is_pipeline_parallel_enabled
        if self.model_parallel:
            self.model_class = get_model_parallel_class(self.config.model_type)
        if self.use_padding_free_transformer and not self.is_custom_model:
            raise ValueError("the padding-free transformer is only available for the model types of this package")

        total, active = self.calculate_num_parameters()
        log_rank_0(logging.INFO, f"total parameters in the model = {total:,}")
        log_rank_0(logging.INFO, f"active parameters in the model = {active:,}")

        self._setup_tokenizer()
        self._setup_model()
        if self.mode == Mode.training and additional_special_tokens:
            self._add_special_tokens(additional_special_tokens)

    # ------------------------------------------------------------------ setup
    def _setup_config(self) -> None:
        if self.model_name is None:
            self.config = AutoConfig.for_model(**self.pretrained_config)
        else:
            self.config = AutoConfig.from_pretrained(self.model_name, trust_remote_code=self.trust_remote_code)
        self.tie_word_embeddings = getattr(self.config, "tie_word_embeddings", False)
        self.is_encoder_decoder = getattr(self.config, "is_encoder_decoder", False)
        self.router_aux_loss_coef = getattr(self.config, "router_aux_loss_coef", None)
        log_rank_0(logging.INFO, str(self.config))

    def _setup_tokenizer(self) -> None:
        if self.tokenizer_name is None:
            self.tokenizer = None
            self.eos_token_id = getattr(self.config, "eos_token_id", None)
            log_rank_0(logging.WARN, "no tokenizer is loaded since neither tokenizer_name nor model_name is given")
        else:
            self.tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_name)
            self.eos_token_id = self.tokenizer.eos_token_id

    def _model_kwargs(self) -> dict:
        kwargs = {}
        if self.is_custom_model:
            if self.use_padding_free_transformer:
                kwargs["use_padding_free_transformer"] = True
            if self.model_parallel:
                kwargs["sequence_parallel"] = self.sequence_parallel
                if self.is_pipeline_parallel_enabled:
                    kwargs["num_pipeline_stages"] = self.num_pipeline_stages
                    kwargs["pipeline_stage_id"] = self.pipeline_stage_id
        else:
            kwargs["attn_implementation"] = "flash_attention_2" if is_kernel_allowed(Kernel.flash_attention_2) else "sdpa"
        if self.trust_remote_code:
            kwargs["trust_remote_code"] = True
        return kwargs

    def _build_from_config(self, **kwargs) -> nn.Module:
        if self.model_parallel or hasattr(self.model_class, "_from_config") and not hasattr(self.model_class, "from_config"):
            return self.model_class._from_config(self.config, **kwargs)
        return self.model_class.from_config(self.config, **kwargs)

    def _setup_model(self) -> None:
        kwargs = self._model_kwargs()
        training = self.mode == Mode.training
        if self.model_name is None:
            if training and self.is_custom_model:
                # parameters are materialised unit by unit by the sharded engine
                with torch.device("meta"):
                    self.model = self._build_from_config(**kwargs)
                self._initialised_on_meta = True
            else:
                if not training:
                    kwargs["torch_dtype"] = self.dtype
                self.model = self._build_from_config(**kwargs)
                self._initialised_on_meta = False
        else:
            self._initialised_on_meta = False
            if not training or not self.keep_in_fp32:
                kwargs["torch_dtype"] = self.dtype
            if self.model_parallel:
                self.model = self.model_class.from_pretrained(self.model_name, **kwargs)
            else:
                self.model = self.model_class.from_pretrained(self.model_name, **kwargs)

    def _add_special_tokens(self, tokens: list[str]) -> None:
        original = len(self.tokenizer)
        self.tokenizer.add_special_tokens({"additional_special_tokens": tokens})
        if len(self.tokenizer) != original:
            self.model.resize_token_embeddings(len(self.tokenizer))

    # ------------------------------------------------------------------ API
    def has_teacher_model(self) -> bool:
        return False

    def calculate_num_parameters(self) -> tuple[int, int]:
        """(total, active) parameter counts from a meta-device instance; MoE layers count only ``top_k`` experts."""
        from ..hf_models.layers.mlp import MoE

        with torch.device("meta"):
            if self.config.model_type in ("gpt_base", "gpt_crosslayer", "palm", "ladder_residual", "desync_residual"):
                from transformers import AutoModelForCausalLM

                model = AutoModelForCausalLM.from_config(self.config)
            else:
                model = self.model_class.from_config(self.config)
            total = sum(p.numel() for p in model.parameters())
            active = total
            for module in model.modules():
                if isinstance(module, MoE):
                    active -= sum(p.numel() for p in module.parameters())
                    active += module.get_num_active_parameters()
        return total, active

    @torch.no_grad()
    def generate(self, batch: dict, generate_kwargs: dict) -> tuple[list[str], list[int]]:
        if self.is_encoder_decoder:
            raise NotImplementedError("generation for encoder-decoder models is not implemented")
        device = next(self.model.parameters()).device
        inputs = {k: torch.as_tensor(v, device=device) for k, v in batch.items() if k in ("input_ids", "attention_mask")}
        generated = self.model.generate(**inputs, **generate_kwargs, eos_token_id=self.eos_token_id)
        sequences = generated if isinstance(generated, torch.Tensor) else generated.sequences
        new_tokens = sequences[:, inputs["input_ids"].shape[1]:]
        counts = ((new_tokens != self.eos_token_id).sum(dim=-1)).tolist() if self.eos_token_id is not None else [new_tokens.shape[1]] * len(new_tokens)
        texts = self.tokenizer.batch_decode(new_tokens, skip_special_tokens=True) if self.tokenizer is not None else [str(r.tolist()) for r in new_tokens]
        return texts, counts

    def save_pretrained(self, save_path: str, state_dict: dict | None = None) -> None:
        if self.tokenizer is not None:
            self.tokenizer.save_pretrained(save_path, legacy_format=False)
        if state_dict is None:
            engine = getattr(self.model, "_lm_engine", None) or getattr(self, "_lm_engine", None)
            if engine is not None:
                state_dict = {k[len("model."):] if k.startswith("model.") else k: v for k, v in engine.full_state_dict().items()}
            else:
                state_dict = self.model.state_dict()
        else:
            state_dict = {k[len("model."):] if k.startswith("model.") else k: v for k, v in state_dict.items()}
        model = getattr(self, "model", None)
        if model is not None and not getattr(self.config, "architectures", None):
            # what transformers' own save_pretrained records; the unsharded weights are those of the single-device class
            self.config.architectures = [type(model).__name__.removesuffix("_TP")]
        self.config.save_pretrained(save_path)
        SafeTensorsWeightsManager.save_state_dict(state_dict, save_path)
