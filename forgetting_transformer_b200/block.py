"""The FoX-Pro block (attention layer + SwiGLU MLP) composed from this package's operators.

Mirrors the data flow of upstream's ``ForgettingAttentionLayer`` / ``ForgettingTransformerMLP`` /
``ForgettingTransformerBlock`` (modeling_forgetting_transformer.py:98-430, 467-516, 519-622) in the "Pro"
configuration: output gate + output norm, per-head QK-norm, data-dependent K and V token shift, full forget
gate, no rotary embedding; training path and, with an ``FgateCache``, the prefill / generation path.  The matrix products are ``nn.Linear`` / ``F.linear`` (cuBLAS);
everything between them is a kernel of this library:

    x -> RMSNorm -> q_proj, ShiftLinear(k), ShiftLinear(v), fgate_proj, ogate_proj
      -> per-head RMSNorm(q), RMSNorm(k) -> forgetting_attention(log sigmoid(fgate))
      -> per-head RMSNorm * sigmoid(ogate) -> o_proj -> (+ residual, RMSNorm with prenorm) -> SwiGLU MLP -> +
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .norm_gate import FusedGroupNormGated, GroupNorm, RMSNorm
from .ops import (acp_threshold_from_qk_norm, forgetting_attention, forgetting_attention_from_gate_logits,
                  seq_start_from_attention_mask)
from .glu import swiglu_linear_packed
from .token_shift import token_shift

__all__ = ["ShiftLinear", "FoxProAttentionLayer", "FoxMLP", "FoxProBlock"]


class ShiftLinear(nn.Module):
    """Linear projection followed by the data-dependent token shift (upstream lines 44-95): a sequence goes
    through the token-shift kernel, a single generated token is mixed with the cached projection of the token
    before it.  ``shift_state`` (B, output_dim), when given, is overwritten with the last token's projection."""

    def __init__(self, input_dim: int, output_dim: int, num_heads: int, bias: bool = False, shift_bias: bool = False):
        super().__init__()
        assert output_dim % num_heads == 0
        self.num_heads = num_heads
        self.linear = nn.Linear(input_dim, output_dim, bias=bias)
        self.shift_proj = nn.Linear(input_dim, num_heads, bias=shift_bias)

    def forward(self, x: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                shift_state: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, T, _ = x.shape
        out = self.linear(x)
        alpha = torch.sigmoid(self.shift_proj(x).float())
        out_per_head = out.view(B, T, self.num_heads, -1)
        if T > 1:
            if attention_mask is not None:
                out_per_head = torch.where(attention_mask[:, :, None, None].bool(), out_per_head, 0.0)
            result = token_shift(out_per_head, alpha, 1.0 - alpha)
        else:
            assert shift_state is not None, "a single token needs the projection of the token before it"
            prev = shift_state.view(B, 1, self.num_heads, -1)
            a = alpha[..., None]
            result = a * prev.float() + (1.0 - a) * out_per_head.float()      # fp32, as upstream's weight_sum
        if shift_state is not None:
            shift_state.copy_(out[:, -1, :])
        return result.to(out.dtype).reshape(B, T, -1)


class FoxProAttentionLayer(nn.Module):

    def __init__(self, hidden_size: int, num_heads: int, norm_eps: float = 1e-6, qk_norm: bool = True,
                 use_k_shift: bool = True, use_v_shift: bool = True, fgate_bias: float = 0.0,
                 log_pruning_tolerance: Optional[float] = None, initializer_range: float = 0.02):
        super().__init__()
        assert hidden_size % num_heads == 0
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, hidden_size // num_heads
        self.q_proj = nn.Linear(hidden_size, hidden_size, bias=False)
        self.k_proj = (ShiftLinear(hidden_size, hidden_size, num_heads) if use_k_shift
                       else nn.Linear(hidden_size, hidden_size, bias=False))
        self.v_proj = (ShiftLinear(hidden_size, hidden_size, num_heads) if use_v_shift
                       else nn.Linear(hidden_size, hidden_size, bias=False))
        self.use_k_shift, self.use_v_shift = use_k_shift, use_v_shift
        self.o_proj = nn.Linear(hidden_size, hidden_size, bias=False)
        self.fgate_proj = nn.Linear(hidden_size, num_heads, bias=True)
        self.ogate_proj = nn.Linear(hidden_size, hidden_size, bias=False)
        self.output_norm = FusedGroupNormGated(num_groups=num_heads, hidden_size=hidden_size, eps=norm_eps,
                                               activation="sigmoid", is_rms_norm=True)
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm = GroupNorm(num_groups=num_heads, hidden_size=hidden_size, is_rms_norm=True)
            self.k_norm = GroupNorm(num_groups=num_heads, hidden_size=hidden_size, is_rms_norm=True)
        self.log_pruning_tolerance = log_pruning_tolerance
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, mean=0.0, std=initializer_range)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        with torch.no_grad():
            self.fgate_proj.bias.fill_(fgate_bias)

    def init_shift_state(self, batch_size: int) -> dict:
        """Zero K / V shift states of one sequence batch (upstream's ``init_shift_state``): the projection of
        the token before the first one."""
        w = self.q_proj.weight
        z = lambda: torch.zeros(batch_size, self.hidden_size, dtype=w.dtype, device=w.device)
        return {"key_shift": z(), "value_shift": z()}

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                past_key_values=None, layer_idx: int = 0) -> torch.Tensor:
        """With ``past_key_values`` (an ``FgateCache`` whose shift states were registered with
        ``update_shift_cache``) the layer appends its keys, values and log gates to the cache and attends over
        the whole history (upstream lines 296-362); a single new token takes the split-KV generation kernels."""
        dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else hidden_states.dtype
        hidden_states = hidden_states.to(dtype)
        B, T, _ = hidden_states.shape
        H, D = self.num_heads, self.head_dim
        k_state = v_state = None
        if past_key_values is not None:
            k_state = past_key_values.key_shift_cache[layer_idx]
            v_state = past_key_values.value_shift_cache[layer_idx]
        step_mask = attention_mask
        if attention_mask is not None and attention_mask.shape[1] != T:
            step_mask = attention_mask[:, -T:]          # the mask covers the history, the shift only this call
        q = self.q_proj(hidden_states)
        k = self.k_proj(hidden_states, step_mask, k_state) if self.use_k_shift else self.k_proj(hidden_states)
        v = self.v_proj(hidden_states, step_mask, v_state) if self.use_v_shift else self.v_proj(hidden_states)
        if self.qk_norm:
            q = self.q_norm(q).to(q.dtype)
            k = self.k_norm(k).to(k.dtype)
        fgate_logit = self.fgate_proj(hidden_states).transpose(1, 2)               # (B, H, T) view
        q, k, v = [t.view(B, T, H, D).transpose(1, 2) for t in (q, k, v)]          # head-first views
        log_fgate = None
        if past_key_values is not None:     # the cache holds log gates: form them here
            log_fgate = F.logsigmoid(fgate_logit.float())
            k, v, log_fgate = past_key_values.update(k, v, log_fgate, layer_idx)
        N = k.shape[2]
        thr = None
        if self.log_pruning_tolerance is not None:
            assert self.qk_norm, "the closed-form threshold needs QK-norm"
            thr = acp_threshold_from_qk_norm(self.q_norm.weight, self.k_norm.weight, H, D, N,
                                             self.log_pruning_tolerance)
        seq_start = None
        if attention_mask is not None:
            assert attention_mask.shape == (B, N), ((B, N), tuple(attention_mask.shape))
            seq_start = seq_start_from_attention_mask(attention_mask)
        if log_fgate is None:               # training path: log sigmoid folded into the operator's prefix sums
            o = forgetting_attention_from_gate_logits(q, k, v, fgate_logit, head_first=True, seq_start=seq_start,
                                                      sm_scale=1 / math.sqrt(D), adaptive_threshold=thr)
        else:
            o = forgetting_attention(q, k, v, log_fgate, head_first=True, seq_start=seq_start,
                                     sm_scale=1 / math.sqrt(D), adaptive_threshold=thr)
        o = o.transpose(1, 2).reshape(B, T, self.hidden_size)
        o = self.output_norm(o, self.ogate_proj(hidden_states))
        return self.o_proj(o)


class FoxMLP(nn.Module):
    """SwiGLU MLP (upstream lines 467-516): down_proj(silu(gate) * y) with [gate, y] = gate_proj(x)."""

    def __init__(self, hidden_size: int, intermediate_size: int, initializer_range: float = 0.02):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size * 2, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        for m in (self.gate_proj, self.down_proj):
            nn.init.normal_(m.weight, mean=0.0, std=initializer_range)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return swiglu_linear_packed(self.gate_proj(x), self.down_proj.weight, self.down_proj.bias)


class FoxProBlock(nn.Module):
    """attn_norm -> attention -> (residual add + mlp_norm, prenorm) -> MLP -> residual add (upstream lines 552-622)."""

    def __init__(self, hidden_size: int = 1536, num_heads: int = 24, intermediate_size: int = 4096,
                 norm_eps: float = 1e-6, fgate_bias: float = 0.0, log_pruning_tolerance: Optional[float] = None):
        super().__init__()
        self.attn_norm = RMSNorm(hidden_size, eps=norm_eps)
        self.attn = FoxProAttentionLayer(hidden_size, num_heads, norm_eps=norm_eps, fgate_bias=fgate_bias,
                                         log_pruning_tolerance=log_pruning_tolerance)
        self.mlp_norm = RMSNorm(hidden_size, eps=norm_eps)
        self.mlp = FoxMLP(hidden_size, intermediate_size)

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                past_key_values=None, layer_idx: int = 0) -> torch.Tensor:
        """hidden_states (B, T, hidden) in fp16/bf16 (the residual stream is kept in that dtype here)."""
        residual = hidden_states
        hidden_states = self.attn(self.attn_norm(hidden_states), attention_mask, past_key_values, layer_idx)
        hidden_states, residual = self.mlp_norm(hidden_states, residual, True)
        return residual + self.mlp(hidden_states)
