from __future__ import annotations

import torch.nn as nn


def get_module_class_from_name(model: nn.Module, name: str) -> type[nn.Module] | None:
    """Depth-first search for the class of the first sub-module whose class name is ``name``."""
    for module in model.modules():
        if type(module).__name__ == name:
            return type(module)
    return None
