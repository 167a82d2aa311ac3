from .gpt_base import GPTBaseForCausalLM, GPTBaseModel
