from .gpt import GPT2ModelPipe, SequentialWrapper, cross_entropy
from .utils import (get_params_for_weight_decay_optimization, mark_norms_for_sequence_parallel_grad_sync)
from .embeddings import SoftEmbedding

__all__ = ["GPT2ModelPipe", "SequentialWrapper", "SoftEmbedding", "cross_entropy",
           "get_params_for_weight_decay_optimization", "mark_norms_for_sequence_parallel_grad_sync"]
