"""B200 (sm_100a) implementations of MegaFold's fused Pairformer operators.

Public names follow the reference: ``TritonEvoformer`` / ``EvoformerAttention``,
``LayernormLinear`` / ``LayernormLinearFunction``, ``FusedTransition`` / ``FusedSwiGLU``.
Everything runs in hand-written CUDA behind a C ABI (include/megafold_b200.h); there is no CPU
or library fallback.
"""
from .evoattention import EvoformerAttention, TritonEvoformer, evo_attention_backward, evo_attention_forward
from .fused_layernorm_linear import (LayernormLinear, LayernormLinearFunction, layernorm_linear_backward,
                                     layernorm_linear_forward)
from .fused_transition import (FusedSwiGLU, FusedSwiGLUFunction, FusedTransition, TransitionFunction,
                               transition_backward, transition_forward)
from .host_pipeline import evoformer_fwd_bwd_host
from .pairformer_block import PairformerBlock
from .sharded import AllReduceGradient, row_shard, sharded_evoformer

__all__ = [
    "EvoformerAttention", "TritonEvoformer", "evo_attention_forward", "evo_attention_backward",
    "LayernormLinear", "LayernormLinearFunction", "FusedSwiGLU", "FusedSwiGLUFunction", "FusedTransition",
    "TransitionFunction", "layernorm_linear_forward", "layernorm_linear_backward", "transition_forward",
    "transition_backward", "AllReduceGradient", "row_shard", "sharded_evoformer", "evoformer_fwd_bwd_host", "PairformerBlock",
]
