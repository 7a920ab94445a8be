"""B200-native (sm_100a) Forgetting Attention: a drop-in for
``forgetting_transformer.forgetting_attention`` and the FoX-Pro fused
RMSNorm + output gate, backed by hand-written CUDA kernels behind a C ABI."""
from .norm_gate import FusedGroupNormGated, GroupNorm, RMSNorm, group_norm, group_norm_gated, rms_norm  # noqa: F401
from .ops import (ForgettingAttention, acp_threshold_from_data, acp_threshold_from_qk_norm,  # noqa: F401
                  forgetting_attention, forgetting_attention_from_gate_logits, seq_start_from_attention_mask)
from .glu import swiglu, swiglu_linear, swiglu_linear_packed  # noqa: F401
from .token_shift import TokenShift, token_shift  # noqa: F401
from .block import FoxMLP, FoxProAttentionLayer, FoxProBlock, ShiftLinear  # noqa: F401
from .cache import FgateCache  # noqa: F401
from .ops import make_graphed  # noqa: F401
from ._lib import FoxError, check_status  # noqa: F401
from .cross_entropy import CrossEntropyLossFunction, FusedCrossEntropyLoss, cross_entropy_loss  # noqa: F401

__all__ = ["forgetting_attention", "forgetting_attention_from_gate_logits", "ForgettingAttention", "FusedGroupNormGated", "group_norm_gated", "GroupNorm",
           "group_norm", "RMSNorm", "rms_norm", "TokenShift", "token_shift", "acp_threshold_from_qk_norm",
           "acp_threshold_from_data", "seq_start_from_attention_mask", "FoxProBlock", "FoxProAttentionLayer", "FoxMLP",
           "ShiftLinear", "FgateCache", "make_graphed", "swiglu", "swiglu_linear", "swiglu_linear_packed", "check_status", "FoxError", "cross_entropy_loss",
           "CrossEntropyLossFunction", "FusedCrossEntropyLoss"]
