from .decoder import DecoderModel, StreamDecoderModel
from .fezozen import FezozenForCausalLM
from .gulisun import GulisunForCausalLM
from .qwen3 import Qwen3ForCausalLM
from .ravutar import RavutarForCausalLM
from .sinulix import SinulixForCausalLM

__all__ = ["DecoderModel", "StreamDecoderModel", "FezozenForCausalLM", "GulisunForCausalLM", "Qwen3ForCausalLM", "RavutarForCausalLM", "SinulixForCausalLM"]
