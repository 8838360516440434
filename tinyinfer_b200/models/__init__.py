from .decoder import DecoderModel
from .gulisun import GulisunForCausalLM
from .qwen3 import Qwen3ForCausalLM
from .ravutar import RavutarForCausalLM
from .sinulix import SinulixForCausalLM

__all__ = ["DecoderModel", "GulisunForCausalLM", "Qwen3ForCausalLM", "RavutarForCausalLM", "SinulixForCausalLM"]
