from .base import Architecture
from .decoder import DecoderModel, build_model, model_parameter_specs
