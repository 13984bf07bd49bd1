"""Mufotar, stated plainly: one slow function per mechanism, whole sequences, no cache, no batching.

Nothing here is shared with the package: the functions take the raw ``config.json`` dictionary and a dictionary of
checkpoint tensors by name, and work on one sequence ``[T, width]`` at a time in the dtype they are given (float64 for
an oracle that rounding does not touch). The recurrent mixers are loops over the tokens, the attention builds its mask
as a matrix, the experts are visited token by token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------------------ small pieces
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b, the variance being the mean squared deviation."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([u.new_zeros(taps - 1, C), u])
    y = u.new_zeros(T, C)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return y


# ------------------------------------------------------------------------------------------------------------ attention
def rotate_half(x, positions, dims, base):
    """x [T, heads, dim]: entry i < dims / 2 of a head pairs with entry i + dims / 2; the rest passes."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attention(h, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float):
    """Causal softmax attention over grouped heads, queries and keys normed per head and partly turned."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[f"{p}.q"].T).view(T, H, D)
    k = (h @ t[f"{p}.k"].T).view(T, G, D)
    v = (h @ t[f"{p}.v"].T).view(T, G, DV)
    q = rms_unit(q, eps) * t[f"{p}.q.norm"]
    k = rms_unit(k, eps) * t[f"{p}.k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, int(rot["dims"]), float(rot["base"]))
        k = rotate_half(k, pos, int(rot["dims"]), float(rot["base"]))
    per = H // G
    out = h.new_zeros(T, H, DV)
    visible = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // per
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * DV) @ t[f"{p}.o"].T


# ------------------------------------------------------------------------------------------------------------ selective scan
def selective_scan(h, m: dict, t: Dict[str, torch.Tensor], p: str):
    """A state per channel and state index: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c."""
    T = h.shape[0]
    inner, NS, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ t[f"{p}.in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, t[f"{p}.conv"], t[f"{p}.conv.b"]))
    dbc = x @ t[f"{p}.x"].T
    dt = softplus(dbc[:, :R] @ t[f"{p}.dt"].T + t[f"{p}.dt.b"])
    B, C = dbc[:, R:R + NS], dbc[:, R + NS:R + 2 * NS]
    A = -torch.exp(t[f"{p}.A_log"])
    S = h.new_zeros(inner, NS)
    y = h.new_zeros(T, inner)
    for i in range(T):
        S = torch.exp(dt[i][:, None] * A) * S + (dt[i] * x[i])[:, None] * B[i][None, :]
        y[i] = S @ C[i] + t[f"{p}.D"] * x[i]
    return (y * silu(z)) @ t[f"{p}.o"].T


def parallel_mixer(h, m: dict, t, p: str, eps: float):
    return m["left_scale"] * attention(h, m["left"], t, f"{p}.left", eps) + m["right_scale"] * selective_scan(h, m["right"], t, f"{p}.right")


# ------------------------------------------------------------------------------------------------------------ delta rule
def delta_mixer(h, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float):
    """The gated delta rule with one decay per head."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ t[f"{p}.q"].T, t[f"{p}.q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ t[f"{p}.k"].T, t[f"{p}.k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ t[f"{p}.v"].T, t[f"{p}.v.conv"])).view(T, H, DV)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ t[f"{p}.b"].T)
    g = torch.exp(-torch.exp(t[f"{p}.A_log"]) * softplus(h @ t[f"{p}.a"].T + t[f"{p}.dt_bias"]))
    per = H // G
    o = h.new_zeros(T, H, DV)
    for head in range(H):
        S = h.new_zeros(D, DV)
        kk, qq = k[:, head // per], q[:, head // per]
        for i in range(T):
            S = g[i, head] * S
            u = beta[i, head] * (v[i, head] - S.T @ kk[i])
            S = S + torch.outer(kk[i], u)
            o[i, head] = S.T @ qq[i]
    o = rms_unit(o, eps) * t[f"{p}.norm"]
    o = o.reshape(T, H * DV) * silu(h @ t[f"{p}.g"].T)
    return o @ t[f"{p}.o"].T


# ------------------------------------------------------------------------------------------------------------ feed-forward
def gated_unit(h, t, p: str, act):
    return (act(h @ t[f"{p}.gate"].T) * (h @ t[f"{p}.up"].T)) @ t[f"{p}.down"].T


def route(h, mlp: dict, t, p: str, close_out: Optional[list] = None):
    """(chosen experts [T, top], their weights [T, top]); experts from ``experts`` on are identity experts. ``close_out`` collects,
    per token, whether the last score taken and the first one left out are nearly equal (within a few percent of what a
    rounding of the input to 8 bits moves them by: a score s moves by about s * |dz|)."""
    r = mlp["router"]
    z = h @ t[f"{p}.router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + t[f"{p}.correction"] if f"{p}.correction" in t else s
    top = int(r["top"])
    idx = torch.topk(choice, top, dim=-1).indices
    if close_out is not None:
        if top < choice.shape[-1]:
            order = torch.sort(choice, dim=-1, descending=True)
            gap = order.values[:, top - 1] - order.values[:, top]
            s_edge = torch.gather(s, 1, order.indices[:, top - 1:top + 1]).max(-1).values
            close_out.append(gap < 0.03 * z.abs().max(-1).values.clamp(min=1.0) * s_edge)
        else:
            close_out.append(torch.zeros(h.shape[0], dtype=torch.bool))
    w = torch.gather(s, 1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20)


def experts(h, mlp: dict, t, p: str, close_out: Optional[list] = None):
    E = int(mlp["router"]["experts"])
    idx, w = route(h, mlp, t, p, close_out)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, we in zip(idx[i].tolist(), w[i]):
            y = gated_unit(h[i:i + 1], t, f"{p}.e{e}", silu)[0] if e < E else h[i]
            out[i] = out[i] + we * y
    if mlp.get("shared"):
        out = out + gated_unit(h, t, f"{p}.shared", silu)
    return out


def feed_forward(h, mlp: Optional[dict], t, p: str, close_out: Optional[list] = None):
    if mlp is None:
        return torch.zeros_like(h)
    if mlp.get("kind", "dense") == "dense":
        return gated_unit(h, t, p, gelu_tanh)
    return experts(h, mlp, t, p, close_out)


# ------------------------------------------------------------------------------------------------------------ the model
def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None,
            close_out: Optional[list] = None):
    """Logits ``[T, vocab]`` of one sequence. ``layers_out`` collects the residual stream after every layer, ``close_out`` every
    router's close calls (see ``route``)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        j = layer.get("weights_of")
        p = f"l{i if j is None else j}"
        h = layer_norm(x, t[f"{p}.norm1"], t[f"{p}.norm1.b"], eps)
        if layer["type"] == "delta":
            mix = delta_mixer(h, layer["mixer"], t, f"{p}.mix", eps)
        elif layer["type"] == "parallel":
            mix = parallel_mixer(h, layer["mixer"], t, f"{p}.mix", eps)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        x = x + (mix + feed_forward(h, layer.get("mlp"), t, f"{p}.mlp", close_out))
        if layers_out is not None:
            layers_out.append(x.clone())
    h = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    logits = h @ t["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def bf16_store(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The tensors as a bfloat16 checkpoint would hold them (rounded once), back in float32."""
    return {k: (v.to(torch.bfloat16).float() if v.is_floating_point() else v) for k, v in tensors.items()}
