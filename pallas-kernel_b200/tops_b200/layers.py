"""`GatedLinearAttention`: the one in-tree caller of the GLA ops in the reference
(`tops/layers/gla.py:72-345`), as a torch.nn.Module on the kernels of this package.

Same constructor arguments, projections and control flow: q/k/v (and the low-rank gate) projections,
optional causal depthwise short convolutions (`tops/modules/convolution.py`), the gate
`log_sigmoid(gk) / gate_logit_normalizer` (`gla_gate`), `fused_recurrent_gla` for sequences of at most
64 tokens and the configured mode otherwise (chunk_size 16 as upstream), the fused RMS-norm + swish gate
on the output (`FusedRMSNormGated`) or the plain RMS norm followed by the gate activation, and the output
projection.  The linear projections and the short convolution are torch's own (they are outside the path
this package replaces); everything between them runs on this package's kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .ops.gate import gla_gate
from .ops.gla import chunk_gla, fused_chunk_gla, fused_recurrent_gla
from .ops.norm import FusedRMSNormGated

# "gelu" is the tanh approximation: the reference's table holds jax.nn.gelu, whose default is approximate=True
# (tops/layers/gla.py:25-32)
ACT2FN = {"swish": F.silu, "silu": F.silu, "gelu": lambda x: F.gelu(x, approximate="tanh"), "relu": F.relu,
          "sigmoid": torch.sigmoid, "tanh": torch.tanh}


class RMSNorm(nn.Module):
    """x * rsqrt(mean(x^2) + eps) * weight in fp32 (`tops/modules/layernorm.py`)."""

    def __init__(self, hidden_size, elementwise_affine=True, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size)) if elementwise_affine else None

    def forward(self, x):
        y = x.float()
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * self.weight.float()
        return y.to(x.dtype)


class ShortConvolution(nn.Module):
    """Causal depthwise 1-D convolution with optional SiLU (`tops/modules/convolution.py:6-178`).
    `cache` holds the last `kernel_size` inputs per sequence as `[N, W, D]`."""

    def __init__(self, hidden_size, kernel_size, bias=False, activation="silu"):
        super().__init__()
        self.hidden_size, self.kernel_size, self.activation = hidden_size, kernel_size, activation
        self.conv = nn.Conv1d(hidden_size, hidden_size, kernel_size, groups=hidden_size, bias=bias)

    def _conv(self, x):   # [B,T,D] with W-1 zeros (or cached inputs) already in front
        y = self.conv(x.transpose(1, 2)).transpose(1, 2)
        return F.silu(y) if self.activation in ("silu", "swish") else y

    def forward(self, x, cache=None, output_final_state=False, cu_seqlens=None):
        W = self.kernel_size
        if cu_seqlens is not None:
            assert x.shape[0] == 1, "cu_seqlens requires B=1"
            assert cache is None, "packed sequences start from an empty cache"
            cu = [int(c) for c in cu_seqlens]
            segs = [self._conv(F.pad(x[:, a:b], (0, 0, W - 1, 0))) for a, b in zip(cu[:-1], cu[1:])]
            state = None
            if output_final_state:
                state = torch.stack([F.pad(x[0, a:b], (0, 0, W, 0))[-W:] for a, b in zip(cu[:-1], cu[1:])])
            return torch.cat(segs, 1), state
        front = x.new_zeros(x.shape[0], W - 1, x.shape[2]) if cache is None else cache[:, 1:].to(x.dtype)
        full = torch.cat([front, x], 1)
        state = None
        if output_final_state:
            state = F.pad(full, (0, 0, max(0, W - full.shape[1]), 0))[:, -W:]
        return self._conv(full), state


class Cache(list):
    """Per-layer recurrent state (and convolution state), the duck type the layer expects of `past_key_values`."""

    def update(self, recurrent_state=None, conv_state=None, layer_idx=0, offset=0):
        while len(self) <= layer_idx:
            self.append(None)
        self[layer_idx] = {"recurrent_state": recurrent_state, "conv_state": conv_state}
        return self[layer_idx]


class GatedLinearAttention(nn.Module):
    def __init__(self, mode="chunk", hidden_size=1024, expand_k=0.5, expand_v=1.0, num_heads=4, num_kv_heads=None,
                 feature_map=None, use_short_conv=False, conv_size=4, conv_bias=False, use_output_gate=True,
                 gate_fn="swish", elementwise_affine=True, norm_eps=1e-5, gate_logit_normalizer=16,
                 gate_low_rank_dim=16, clamp_min=None, fuse_norm=True, layer_idx=None):
        super().__init__()
        self.mode, self.hidden_size, self.num_heads = mode, hidden_size, num_heads
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.num_kv_groups = self.num_heads // self.num_kv_heads
        self.feature_map_fn = ACT2FN[feature_map] if feature_map is not None else None
        self.use_short_conv, self.use_output_gate = use_short_conv, use_output_gate
        self.key_dim, self.value_dim = int(hidden_size * expand_k), int(hidden_size * expand_v)
        self.key_dim_per_group = self.key_dim // self.num_kv_groups
        self.value_dim_per_group = self.value_dim // self.num_kv_groups
        self.clamp_min, self.layer_idx = clamp_min, layer_idx
        assert mode in ["chunk", "fused_recurrent", "fused_chunk"], f"Not supported mode `{mode}`."
        assert self.key_dim % num_heads == 0, f"key dim must be divisible by num_heads of {num_heads}"
        assert self.value_dim % num_heads == 0, f"value dim must be divisible by num_heads of {num_heads}"
        self.head_k_dim, self.head_v_dim = self.key_dim // num_heads, self.value_dim // num_heads
        self.q_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, self.key_dim_per_group, bias=False)
        self.v_proj = nn.Linear(hidden_size, self.value_dim_per_group, bias=False)
        if use_output_gate:
            self.g_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, "silu")
            self.k_conv1d = ShortConvolution(self.key_dim_per_group, conv_size, conv_bias, "silu")
            self.v_conv1d = ShortConvolution(self.value_dim_per_group, conv_size, conv_bias, "silu")
        self.gk_proj = nn.Sequential(nn.Linear(hidden_size, gate_low_rank_dim, bias=False),
                                     nn.Linear(gate_low_rank_dim, self.key_dim_per_group, bias=True))
        self.o_proj = nn.Linear(self.value_dim, hidden_size, bias=False)
        if gate_fn == "swish" and fuse_norm and use_output_gate:
            self.g_norm_swish_gate = FusedRMSNormGated(self.head_v_dim, elementwise_affine, norm_eps)
            self.fuse_norm_and_gate = True
        else:
            self.fuse_norm_and_gate = False
            self.g_norm = RMSNorm(self.head_v_dim, elementwise_affine, norm_eps)
            self.gate_fn_act = ACT2FN[gate_fn]
        self.gate_logit_normalizer = gate_logit_normalizer

    def _heads(self, x, head_dim, groups):
        x = x.reshape(*x.shape[:-1], -1, head_dim)
        return x if groups == 1 else x.repeat_interleave(groups, dim=-2)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False,
                output_attentions=False, **kwargs):
        if attention_mask is not None:
            assert attention_mask.ndim == 2, "Expected attention_mask as a 0-1 matrix with shape [batch_size, seq_len]."
        q_len = hidden_states.shape[1]
        mode = "fused_recurrent" if q_len <= 64 else self.mode
        last_state = None
        if past_key_values is not None and self.layer_idx is not None and len(past_key_values) > self.layer_idx:
            last_state = past_key_values[self.layer_idx]
        cu_seqlens = kwargs.get("cu_seqlens")
        conv_states = None
        if self.use_short_conv:
            cq = ck = cv = None
            if last_state is not None and last_state["conv_state"] is not None:
                cq, ck, cv = last_state["conv_state"]
            q, cq = self.q_conv1d(self.q_proj(hidden_states), cq, use_cache, cu_seqlens)
            k, ck = self.k_conv1d(self.k_proj(hidden_states), ck, use_cache, cu_seqlens)
            v, cv = self.v_conv1d(self.v_proj(hidden_states), cv, use_cache, cu_seqlens)
            conv_states = (cq, ck, cv)
        else:
            q, k, v = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
        gk = self.gk_proj(hidden_states)
        q = self._heads(q, self.head_k_dim, 1)
        k = self._heads(k, self.head_k_dim, self.num_kv_groups)
        gk = self._heads(gk, self.head_k_dim, self.num_kv_groups)
        v = self._heads(v, self.head_v_dim, self.num_kv_groups)
        gk = gla_gate(gk.contiguous(), self.gate_logit_normalizer, self.clamp_min)
        if self.feature_map_fn is not None:
            q, k = self.feature_map_fn(q), self.feature_map_fn(k)
        state = last_state["recurrent_state"] if last_state is not None else None
        if mode == "fused_recurrent":
            o, state = fused_recurrent_gla(q, k, v, gk=gk, initial_state=state, output_final_state=use_cache,
                                           cu_seqlens=cu_seqlens)
        elif mode == "fused_chunk":
            o, state = fused_chunk_gla(q, k, v, gk, initial_state=state, output_final_state=use_cache,
                                       cu_seqlens=cu_seqlens, chunk_size=16)
        else:
            o, state = chunk_gla(q, k, v, gk, initial_state=state, output_final_state=use_cache, cu_seqlens=cu_seqlens,
                                 chunk_size=16)
        if past_key_values is not None:
            past_key_values.update(recurrent_state=state, conv_state=conv_states, layer_idx=self.layer_idx, offset=q_len)
        if self.use_output_gate:
            g = self.g_proj(hidden_states)
            if self.fuse_norm_and_gate:
                g = g.reshape(*g.shape[:-1], -1, self.head_v_dim)
                o = self.g_norm_swish_gate(o.contiguous(), g.contiguous()).flatten(-2)
            else:
                o = self.g_norm(o).flatten(-2) * self.gate_fn_act(g)
        else:
            o = self.g_norm(o).flatten(-2)
        return self.o_proj(o), None, past_key_values
