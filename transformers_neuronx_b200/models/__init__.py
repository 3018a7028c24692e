from .decoder import DecoderModel
