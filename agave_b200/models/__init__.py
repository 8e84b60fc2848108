from .decoder import DecoderModel, decoder_param_specs
from . import gemma3 as _gemma3      # registers the architecture

__all__ = ["DecoderModel", "decoder_param_specs"]
