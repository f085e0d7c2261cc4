"""Model families (reference: lib/core/nn/{gpt,llama,moe_transformer,...}.dart, lib/core/nn/vision/*.dart)."""
from .gpt import GPT, GPTConfig
from .llama import Llama, LlamaConfig, LlamaBlock
from .moe_lm import MoELanguageModel, MoEBlock
from .vit import (ViTBackbone, ViTClassifier, ViTFaceEmbedding, ViTObjectDetector, VisionEncoder, patchify,
                  vit_cls_feature, vitClsFeature)
