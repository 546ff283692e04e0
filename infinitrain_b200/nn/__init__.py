from . import functional, init
from .layers import (CrossEntropyLoss, Embedding, LayerNorm, Linear, ModuleDict, ModuleList, NewGELU, RMSNorm,
                     Sequential, Sigmoid, SwiGLU)
from .module import CloneableModule, Module

function = functional
