"""B200-native LM training engine with the public surface of IBM's LM Engine (``lm_engine``)."""

from .utils import SafeTensorsWeightsManager

__all__ = ["SafeTensorsWeightsManager"]
