from .model import LayerCall, Model
from . import llama  # registers LlamaForCausalLM
from . import zukotar  # registers Zukotar
from . import livovik  # registers Livovik
from . import bazulorn  # registers Bazulorn
from . import purozen  # registers Purozen

__all__ = ["LayerCall", "Model", "llama", "zukotar", "livovik", "bazulorn", "purozen"]
