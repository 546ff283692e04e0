from .config import AttentionType, MLPType, NormType, TransformerConfig
from .modules import (MLP, CausalSelfAttention, PrecomputeFreqsCis, TransformerChunk, TransformerFirstStage,
                      TransformerLastStage, TransformerLayer, TransformerModel)
