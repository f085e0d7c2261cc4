"""Neural-network building blocks (reference: lib/core/nn/*.dart)."""
from .module import Module, make_param
from .layers import (Linear, LayerNorm, RMSNorm, Embedding, Dropout, SinusoidalPositionalEncoding,
                     LearnedPositionalEmbedding, SwiGluFfn, VisionProjector, causal_mask, activation_name)
from .attention import RopeCache, MHACache, EncoderCache, MultiHeadAttention, MultiHeadCrossAttention
from .transformer import (Activation, TransformerBlock, TransformerEncoder, TransformerDecoderBlock,
                          TransformerDecoder)

causalMask = causal_mask
from .moe import (Expert, MoEFeedForward, GateFunction, BiasUpdateRule, ExpertActivation, ExpertVariant)
from .conv import Conv2d, im2col
