from .config import ModelConfig, from_hf_dict, load_config, preset  # noqa: F401
from .decoder import DecoderModel, ForwardBatch, TPInfo, random_init  # noqa: F401
