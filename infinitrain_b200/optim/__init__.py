from .optimizer import SGD, Adam, AdamW, Optimizer, OptimizerCreator
