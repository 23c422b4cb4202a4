from nanonemo_b200.models.config import ModelConfig
from nanonemo_b200.models.model import NanoNemo

__all__ = ["ModelConfig", "NanoNemo"]
