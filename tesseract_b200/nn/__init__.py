from .modules import (BatchNorm1d, BatchNorm2d, CrossEntropyLoss, DiTBlock, Embedding, FeedForward, LayerNorm, Linear,
                      Module, ModuleList, MultiHeadAttention, ReLU, RMSNorm, RotaryEmbedding, Sequential, Sigmoid,
                      Tanh, TransformerBlock)

__all__ = ["BatchNorm1d", "BatchNorm2d", "CrossEntropyLoss", "DiTBlock", "Embedding", "FeedForward", "LayerNorm",
           "Linear", "Module", "ModuleList", "MultiHeadAttention", "ReLU", "RMSNorm", "RotaryEmbedding",
           "Sequential", "Sigmoid", "Tanh", "TransformerBlock"]
