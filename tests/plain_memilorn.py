"""Memilorn, stated plainly: one slow function per mechanism, whole sequences, no cache, no batching.

Nothing here is shared with the package: the functions take the raw ``config.json`` dictionary and a dictionary of checkpoint
tensors by name, and work on one sequence ``[T, width]`` at a time in the dtype they are given (float64 for an oracle that
rounding does not touch). The matrix memory is a loop over the tokens, the attentions build their masks as matrices, the experts
are visited token by token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------------------ small pieces
def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w, the variance being the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def log_sigmoid(x):
    return torch.minimum(x, torch.zeros_like(x)) - torch.log1p(torch.exp(-x.abs()))


def bounded(x, cap):
    return x if not cap else cap * torch.tanh(x / cap)


# ------------------------------------------------------------------------------------------------------------ matrix memory
def matrix_memory_cell(q, k, v, i_log, f_log):
    """One head. q, k [T, D] (q already scaled), v [T, DV], i_log, f_log [T]: the log gates. Returns o [T, DV].

        m_t = max(f_t + m_(t-1), i_t);  S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T;  n_t likewise with k_t
        o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6),   S_0 = 0, n_0 = 0, m_0 = 0
    """
    T, D = q.shape
    S = q.new_zeros(D, v.shape[1])
    n = q.new_zeros(D)
    m = q.new_zeros(())
    out = []
    for t in range(T):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        keep, take = torch.exp(f_log[t] + m - m_new), torch.exp(i_log[t] - m_new)
        S = keep * S + take * torch.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_new
        out.append((S.T @ q[t]) / (torch.maximum((n @ q[t]).abs(), torch.exp(-m)) + 1e-6))
    return torch.stack(out)


def matrix_memory(h, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float):
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    DV = int(m.get("vdim", D))
    cap = m.get("gate_cap")
    q = (h @ t[f"{p}.q"].T).view(T, H, D) * D ** -0.5
    k = (h @ t[f"{p}.k"].T).view(T, H, D)
    v = (h @ t[f"{p}.v"].T).view(T, H, DV)
    i_log = bounded(h @ t[f"{p}.i"].T + t[f"{p}.i.b"], cap)
    f_log = log_sigmoid(bounded(h @ t[f"{p}.f"].T + t[f"{p}.f.b"], cap))
    o = torch.stack([matrix_memory_cell(q[:, j], k[:, j], v[:, j], i_log[:, j], f_log[:, j]) for j in range(H)], dim=1)   # [T, H, DV]
    o = rms_unit(o, eps).reshape(T, H * DV) * t[f"{p}.norm"] * torch.sigmoid(h @ t[f"{p}.g"].T)
    return o @ t[f"{p}.o"].T


# ------------------------------------------------------------------------------------------------------------ attentions
def causal_mask(T: int):
    return torch.tril(torch.ones(T, T, dtype=torch.bool))


def latent_attention(h, m: dict, t, p: str, eps: float):
    """Queries from the input; keys and values of every head rebuilt from one normed latent per token; no positions."""
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    DV = int(m.get("vdim", D))
    q = (h @ t[f"{p}.q"].T).view(T, H, D)
    c = rms_unit(h @ t[f"{p}.dkv"].T, eps) * t[f"{p}.dkv.norm"]
    k = (c @ t[f"{p}.uk"].T).view(T, H, D)
    v = (c @ t[f"{p}.uv"].T).view(T, H, DV)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    s = s.masked_fill(~causal_mask(T), -math.inf)
    o = torch.einsum("hij,jhv->ihv", torch.softmax(s, dim=-1), v)
    gate = torch.sigmoid(h @ t[f"{p}.g"].T)                      # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * DV) @ t[f"{p}.o"].T


def rotate_neighbours(x, positions, dims: int, base: float):
    """x [T, heads, dim]: entries (2i, 2i + 1) for i < dims / 2 turn by the angle position * base^(-2i / dims); the rest passes."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_softmax(s, sink):
    """Softmax over the last axis of s [H, T, T] whose denominator also holds exp(sink_h); masked entries are -inf."""
    top = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - top))


def talking_attention(h, m: dict, t, p: str):
    """Grouped heads; scores scaled, bounded, then mixed between the heads; causal mask; a sink in the denominator; a gate per head."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    DV = int(m.get("vdim", D))
    pos = torch.arange(T)
    q = (h @ t[f"{p}.q"].T).view(T, H, D)
    k = (h @ t[f"{p}.k"].T).view(T, G, D)
    v = (h @ t[f"{p}.v"].T).view(T, G, DV)
    if m.get("rot"):
        q = rotate_neighbours(q, pos, int(m["rot"]["dims"]), float(m["rot"]["base"]))
        k = rotate_neighbours(k, pos, int(m["rot"]["dims"]), float(m["rot"]["base"]))
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)     # query head h reads key/value head h // (H / G)
    s = bounded(torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"]), m.get("softcap"))
    s = torch.einsum("hg,gij->hij", t[f"{p}.talk"], s)
    s = s.masked_fill(~causal_mask(T), -math.inf)
    o = torch.einsum("hij,jhv->ihv", sink_softmax(s, t[f"{p}.sink"]), v)
    gate = torch.sigmoid(h @ t[f"{p}.g"].T)
    return (o * gate[:, :, None]).reshape(T, H * DV) @ t[f"{p}.o"].T


# ------------------------------------------------------------------------------------------------------------ feed-forward
def clamped_unit(x, t, p: str, limit: float):
    g = torch.clamp(x @ t[f"{p}.gate"].T, max=limit)
    u = torch.clamp(x @ t[f"{p}.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[f"{p}.down"].T


def route(h, mlp: dict, t, p: str, close_out: Optional[list] = None):
    """(chosen experts [T, top], their sigmoid scores [T, top]). ``close_out`` collects, per token, whether the last score taken
    and the first one left out are nearly equal (within a few percent of what a rounding of the input to 8 bits moves them by)."""
    z = h @ t[f"{p}.router"].T
    s = torch.sigmoid(z)
    top = int(mlp["router"]["top"])
    idx = torch.topk(s, top, dim=-1).indices
    if close_out is not None:
        if top < s.shape[-1]:
            order = torch.sort(z, dim=-1, descending=True).values
            close_out.append(order[:, top - 1] - order[:, top] < 0.03 * z.abs().max(-1).values.clamp(min=1.0))
        else:
            close_out.append(torch.zeros(h.shape[0], dtype=torch.bool))
    return idx, torch.gather(s, 1, idx)


def experts(h, mlp: dict, t, p: str, close_out: Optional[list] = None, forced=None, regret_out: Optional[list] = None):
    """sum over the chosen experts of expert(score * h) (the score is on the INPUT, not renormalised), plus the shared unit.
    ``forced [T, top]``: these experts are taken instead of the router's own choice (their weights are still the router's scores of
    them); ``regret_out`` then collects, per token, how far the worst forced expert's router output lies below the worst of the
    router's own choice, in units of the largest output (0 where the choices agree as sets)."""
    idx, w = route(h, mlp, t, p, close_out)
    if forced is not None:
        z = h @ t[f"{p}.router"].T
        forced = torch.as_tensor(forced, dtype=torch.long)
        if regret_out is not None:
            own, theirs = torch.gather(z, 1, idx).min(-1).values, torch.gather(z, 1, forced).min(-1).values
            regret_out.append((own - theirs).clamp(min=0) / z.abs().max(-1).values.clamp(min=1.0))
        idx, w = forced, torch.gather(torch.sigmoid(z), 1, forced)
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, we in zip(idx[i].tolist(), w[i]):
            out[i] = out[i] + clamped_unit((we * h[i])[None], t, f"{p}.e{e}", limit)[0]
    if mlp.get("shared"):
        out = out + clamped_unit(h, t, f"{p}.shared", float(mlp["shared"]["limit"]))
    return out


# ------------------------------------------------------------------------------------------------------------ the model
def running_order(cfg: dict) -> List[tuple]:
    """(layer, opens a further pass) in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for rep in range(times):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def mixer(kind: str, h, m: dict, t, p: str, eps: float):
    if kind == "mlstm":
        return matrix_memory(h, m, t, p, eps)
    if kind == "latent_attention":
        return latent_attention(h, m, t, p, eps)
    if kind == "attention":
        return talking_attention(h, m, t, p)
    raise ValueError(kind)


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, close_out: Optional[list] = None,
            layers_out: Optional[list] = None, forced: Optional[list] = None, regret_out: Optional[list] = None):
    """Logits ``[T, vocab]``. ``forced``: for every run of a feed-forward, in running order, the experts ``[T, top]`` to take instead of
    the router's own choice (what another implementation chose, so that the two can be compared where a choice hung on rounding)."""
    t = {k: v.to(dtype) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    run = 0
    for i, again in running_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}"
        if again:
            x = x + x0
        x = x + t[f"{p}.ls1"] * mixer(layer["type"], layer_norm(x, t[f"{p}.norm1"], eps), layer["mixer"], t, f"{p}.mix", eps)
        if layer.get("mlp"):
            x = x + t[f"{p}.ls2"] * experts(layer_norm(x, t[f"{p}.norm2"], eps), layer["mlp"], t, f"{p}.mlp", close_out,
                                            None if forced is None else forced[run], regret_out)
            run += 1
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, t["final.norm"], eps) @ t["embed"].T
