from .decoder import DecoderModel, LayerCall

__all__ = ["DecoderModel", "LayerCall"]
