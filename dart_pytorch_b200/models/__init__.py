"""Model families (reference: lib/core/nn/{gpt,llama,moe_transformer,...}.dart, lib/core/nn/vision/*.dart)."""
from .gpt import GPT, GPTConfig
from .llama import Llama, LlamaConfig, LlamaBlock
from .moe_lm import MoELanguageModel, MoEBlock
from .vit import (ViTBackbone, ViTClassifier, ViTFaceEmbedding, ViTObjectDetector, VisionEncoder, patchify,
                  vit_cls_feature, vitClsFeature)
from .seq_models import TransformerLM, AFTAttention, AFTBlock, AFTLanguageModel, EncoderDecoderTransformer
from .neox import (GPTJConfig, GPTJBlock, GPTJModel, PythiaConfig, PythiaBlock, PythiaModel, CausalLMMixin,
                   compute_rotary_dim)
from .bert import BertConfig, BertEmbeddings, BertLayer, BertModel
from .modalities import (TextTransformer, AudioTransformer, VideoTransformer, MultiModalClassifier,
                         MultiModalEncoder, MultiModalGenerator, MultiModalLM, mean_rows, meanRows)
from .sentence import (PoolingMode, TokenEncoder, SentenceEncoder, CrossEncoder, Similarity, SemanticSearchHit,
                       SentenceLosses, pool_tokens, poolTokens, l2_normalize_row, l2NormalizeRow)
from .muzero_lm import (MuZeroLM, MuZeroRepresentation, MuZeroDynamics, MuZeroPrediction, MuZeroUnroll)
from .vision_language import CLIPVisionConfig, CLIPVisionModel, LlamaVision
from .lc0 import (Lc0Net, Lc0Reader, Lc0Input, Lc0Weights, Lc0ConvBlock, Lc0SEUnit, Lc0Residual, Lc0Output, START_FEN,
                  startFen)
