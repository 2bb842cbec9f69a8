"""The `GatedLinearAttention` layer's arithmetic on the CPU, from the layer's own torch submodules
(linears, convolutions) and the oracle's gate, attention and norm: what the layer tests compare with."""
from oracle import aux as OA
from oracle import gla as OG


def layer_on_cpu(layer, x, mode):
    """The layer's arithmetic on the CPU: torch linears / convolutions + oracle gate, attention and norm."""
    q, k, v = layer.q_proj(x), layer.k_proj(x), layer.v_proj(x)
    if layer.use_short_conv:
        q, k, v = layer.q_conv1d(q)[0], layer.k_conv1d(k)[0], layer.v_conv1d(v)[0]
    gk = layer.gk_proj(x)
    q = layer._heads(q, layer.head_k_dim, 1)
    k = layer._heads(k, layer.head_k_dim, layer.num_kv_groups)
    gk = layer._heads(gk, layer.head_k_dim, layer.num_kv_groups)
    v = layer._heads(v, layer.head_v_dim, layer.num_kv_groups)
    gk = OA.gla_gate(gk, layer.gate_logit_normalizer, layer.clamp_min)
    if layer.feature_map_fn is not None:
        q, k = layer.feature_map_fn(q), layer.feature_map_fn(k)
    if mode == "fused_recurrent":
        o, _ = OG.fused_recurrent_gla(q, k, v, gk=gk)
    else:
        o, _ = OG.chunk_gla(q, k, v, gk, chunk_size=16)
    if layer.use_output_gate:
        g = layer.g_proj(x)
        if layer.fuse_norm_and_gate:
            g = g.reshape(*g.shape[:-1], -1, layer.head_v_dim)
            w = layer.g_norm_swish_gate.weight
            o = OA.rmsnorm_gated(o, g, w, layer.g_norm_swish_gate.eps).flatten(-2)
        else:
            o = layer.g_norm(o).flatten(-2) * layer.gate_fn_act(g)
    else:
        o = layer.g_norm(o).flatten(-2)
    return layer.o_proj(o)
