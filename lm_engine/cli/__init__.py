"""Command line utilities around the public API (``python -m lm_engine.cli.<name> --help``).

Parity: the reference's ``tools/`` examples (tools/{export_to_hf,import_from_hf,inference,params_calculator,
pt_to_safetensors,tensor_parallel_inference}.py and tools/data/*.py), as argument-driven modules instead of scripts
with paths to edit.
"""
