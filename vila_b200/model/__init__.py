"""vila_b200.model — mirrors the names callers import from `llava.model`."""
from .configuration import (LlavaConfig, Qwen2Config, SiglipVisionConfig, nvila_8b,
                            nvila_8b_dynamic_s2, nvila_lite_3b, nvila_video_8b, tiny_test_config)
from .llava_llama import (BasicImageEncoder, BasicVideoEncoder, LlavaLlamaModel, SyntheticTokenizer,
                          TSPVideoEncoder)
from .ludazen import LudazenConfig, LudazenForCausalLM, LudazenLayerConfig
from .lufatar import LufatarConfig, LufatarForCausalLM, LufatarLayerConfig
from .modeling_vila import VILAForCausalLM
from .moronex import MoronexConfig, MoronexForCausalLM, MoronexLayerConfig
from .nusovik import NusovikConfig, NusovikForCausalLM, NusovikLayerConfig
from .projector import MultimodalProjector
from .registry import LANGUAGE_MODELS, language_model_architecture, load_language_model
from .qwen2 import GraphDecoder, MegaDecoder, PagedKVCache, Qwen2ForCausalLM
from .vision import SiglipVisionModel, SiglipVisionTower

__all__ = [n for n in dir() if not n.startswith("_")]
