"""Plain torch statements of what each kernel of the package computes, with the kernels' own signatures.

Two uses. (1) Each function is the reference that the GPU test of the kernel of the same name is
compared with, at sizes other than the engine's. (2) As a stand-in for the kernel library they
let the host side of the engine (step building, block tables, scheduler, replay) run on the CPU in
the tests; the package itself has no such path and refuses to run without its CUDA library.

Everything is computed in float32 whatever the storage dtype, rounding only where the kernels store.
"""
from __future__ import annotations

import math

import torch


class TorchKernels:
    name = "torch-reference"

    def __init__(self):
        self.launches = 0

    def embed(self, token_ids, table, scale=1.0):
        return table[token_ids.long()].float() * scale

    def embed_add(self, token_ids, table, residual, scale=1.0):
        residual += table[token_ids.long()].float() * scale

    def feed_tokens(self, token_ids, source_rows, previous_tokens):
        take = source_rows >= 0
        token_ids[take] = previous_tokens[source_rows[take].long()]

    def zero_fresh_states(self, states, seq_slots, seq_starts, positions):
        for state in states:
            self.zero_fresh_state(state, seq_slots, seq_starts, positions)

    def zero_fresh_state(self, state, seq_slots, seq_starts, positions):
        fresh = positions[seq_starts[: seq_slots.shape[0]].long()] == 0
        state[seq_slots[fresh].long()] = 0

    def rope_tables(self, positions, inv_freq, mult=1.0):
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        return ang.cos() * mult, ang.sin() * mult

    def add_rmsnorm(self, residual, delta, weight, eps, out_dtype):
        if delta is not None:
            residual += delta.float()
        h = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps)
        return (weight.float() * h.to(out_dtype).float()).to(out_dtype)

    def rmsnorm_rows(self, residual, delta, weight, eps, rows, out_dtype):
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
        h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return (weight.float() * h.to(out_dtype).float()).to(out_dtype)

    def linear(self, x, w, out_dtype=None, add_to=None, transient=False):
        y = x.float() @ w.float().T
        if add_to is not None:
            add_to += y
            return None
        return y.to(out_dtype or x.dtype)

    def qkv_rope(self, x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                 write_kv=True, out_dtype=None):
        qkv = self.linear(x, w, out_dtype=out_dtype)
        return self.rope_kv_write(qkv, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size,
                                  write_kv, out_dtype)

    def qkv_attention(self, x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, block_table, token_seq, positions, num_heads,
                      num_kv_heads, head_dim, page_size, scale, window, max_context, batch=None, write_kv=True, out_dtype=None):
        qkv = self.qkv_rope(x, w, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim, page_size, write_kv,
                            out_dtype)
        return self.paged_attention(qkv, k_pool, v_pool, block_table, token_seq, positions, num_heads, num_kv_heads, head_dim, page_size,
                                    scale, window, max_context, batch=batch)

    def rope_kv_write(self, qkv, bias, cos, sin, slot_mapping, k_pool, v_pool, num_heads, num_kv_heads, head_dim,
                      page_size, write_kv=True, out_dtype=None):
        N = qkv.shape[0]
        d, half = head_dim, head_dim // 2
        x = qkv.float()
        if bias is not None:
            x = x + bias.float()
        x = x.view(N, num_heads + 2 * num_kv_heads, d)
        rot = x[:, :num_heads + num_kv_heads]
        x1, x2 = rot[..., :half], rot[..., half:]
        c, s = cos[:, None, :], sin[:, None, :]
        rotated = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
        out = torch.cat((rotated, x[:, num_heads + num_kv_heads:]), dim=1)
        qkv.copy_(out.reshape(N, -1).to(qkv.dtype))
        if write_kv:
            page = (slot_mapping // page_size).long()
            off = (slot_mapping % page_size).long()
            k = qkv.view(N, -1, d)[:, num_heads:num_heads + num_kv_heads]
            v = qkv.view(N, -1, d)[:, num_heads + num_kv_heads:]
            k_pool[page, :, off] = k
            v_pool[page, :, off] = v
        return qkv

    def paged_attention(self, qkv, k_pool, v_pool, block_table, token_seq, positions, num_heads, num_kv_heads, head_dim,
                        page_size, scale, window, max_context, batch=None, num_splits=None):
        N = qkv.shape[0]
        d = head_dim
        rep = num_heads // num_kv_heads
        q = qkv.view(N, -1, d)[:, :num_heads].float()
        out = torch.zeros(N, num_heads, d)
        for t in range(N):
            p = int(positions[t])
            lo = 0 if not window else max(0, p - window + 1)
            keys = torch.arange(lo, p + 1)
            pages = block_table[int(token_seq[t])][(keys // page_size)].long()
            offs = (keys % page_size).long()
            k = k_pool[pages, :, offs].float()  # [S, kvh, d]
            v = v_pool[pages, :, offs].float()
            for h in range(num_heads):
                s = (k[:, h // rep] @ q[t, h]) * scale
                pr = torch.softmax(s, dim=0)
                out[t, h] = pr @ v[:, h // rep]
        return out.reshape(N, num_heads * d).to(qkv.dtype)

    def gate_up_act(self, x, w_gate_up, out_dtype=None, glu=None, activation="silu"):
        if activation == "gelu_tanh":
            gu = self.linear(x, w_gate_up, out_dtype=torch.float32)
            i = gu.shape[1] // 2
            g, u = gu[:, :i], gu[:, i:]
            return (0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3))) * u).to(out_dtype or x.dtype)
        if glu is not None:
            return self.glu_clamped(self.linear(x, w_gate_up, out_dtype=torch.float32), *glu, out_dtype or x.dtype)
        return self.silu_mul(self.linear(x, w_gate_up, out_dtype=torch.float32)).to(out_dtype or x.dtype)

    def silu_mul(self, gu, out_dtype=None):
        i = gu.shape[1] // 2
        g, u = gu[:, :i].float(), gu[:, i:].float()
        return (g * torch.sigmoid(g) * u).to(gu.dtype)

    # ------------------------------------------------------------------ several residual streams
    def zeros_like_rows(self, streams, index=0):
        return torch.zeros(streams.shape[0], streams.shape[-1], dtype=torch.float32)

    def take_result(self, y):
        return y

    def streams_expand(self, x, streams):
        return x[:, None, :].repeat(1, streams, 1).contiguous()

    def streams_update(self, streams, y, mix, coef_out):
        new = torch.einsum("st,nsh->nth", mix.float(), streams) + coef_out.float()[None, :, None] * y.float()[:, None, :]
        streams.copy_(new)

    def streams_norm(self, streams, coef_in, weight, eps, out_dtype, rows=None):
        x = streams if rows is None else streams[rows.long()]
        u = torch.einsum("s,nsh->nh", coef_in.float(), x)
        return (u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(out_dtype)

    def flush(self):
        pass

    # ------------------------------------------------------------------ feed-forward with one product going in
    def linear_act(self, x, w, activation, out_dtype=None):
        z = x.float() @ w.float().T
        if activation != "gelu_tanh":
            raise ValueError(activation)
        y = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
        return y.to(out_dtype or x.dtype)

    # ------------------------------------------------------------------ attention with extras
    def kv_store(self, z, k_col, v_col, slot_mapping, k_pool, v_pool, num_kv_heads, head_dim, v_head_dim, page_size):
        N = z.shape[0]
        page, off = (slot_mapping // page_size).long(), (slot_mapping % page_size).long()
        k_pool[page, :, off] = z[:, k_col:k_col + num_kv_heads * head_dim].reshape(N, num_kv_heads, head_dim).to(k_pool.dtype)
        v_pool[page, :, off] = z[:, v_col:v_col + num_kv_heads * v_head_dim].reshape(N, num_kv_heads, v_head_dim).to(v_pool.dtype)

    def attention_ext(self, q, q_col, num_heads, num_kv_heads, head_dim, v_head_dim, k_pool, v_pool, block_table, token_seq, positions,
                      page_size, scale, window, max_context, temp=(0.0, 0), rel=None, rel_rows=None, sink=None, gate=None, gate_col=0,
                      gate_per_head=False, batch=None, num_splits=None, keep_first=0, chunk=0, softcap=0.0, talk=None):
        N = q.shape[0]
        rep = num_heads // num_kv_heads
        qs = q[:, q_col:q_col + num_heads * head_dim].float().view(N, num_heads, head_dim)
        out = torch.zeros(N, num_heads, v_head_dim)
        for t in range(N):
            p = int(positions[t])
            lo = 0 if not window else max(0, p - window + 1)
            if chunk:
                lo = max(lo, p // chunk * chunk)
            keys = torch.cat([torch.arange(0, min(keep_first, lo)), torch.arange(lo, p + 1)])
            pages = block_table[int(token_seq[t])][(keys // page_size)].long()
            offs = (keys % page_size).long()
            k = k_pool[pages, :, offs].float()                                   # [S, kv heads, head_dim]
            v = v_pool[pages, :, offs].float() if v_pool is not None else k[..., :v_head_dim]
            factor = scale
            if temp[1]:
                factor = scale * (1.0 + temp[0] * math.log((p + 1) // temp[1] + 1))
            mixed = None
            if talk is not None:   # every head's capped scores first, then their mix
                plain = torch.stack([(k[:, g // rep] @ qs[t, g]) * factor for g in range(num_heads)])
                if softcap:
                    plain = softcap * torch.tanh(plain / softcap)
                mixed = talk.float() @ plain
            for h in range(num_heads):
                s = (k[:, h // rep] @ qs[t, h]) * factor
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if mixed is not None:
                    s = mixed[h]
                if rel is not None:
                    dist = p - keys
                    row = torch.where(dist < rel_rows.shape[0], rel_rows.long()[dist.clamp(max=rel_rows.shape[0] - 1)], rel.shape[0] - 1)
                    s = s + rel[row, h].float()
                if sink is not None:
                    top = max(float(s.max()), float(sink[h]))
                    e = torch.exp(s - top)
                    pr = e / (e.sum() + math.exp(float(sink[h]) - top))
                else:
                    pr = torch.softmax(s, dim=0)
                out[t, h] = pr @ v[:, h // rep]
        if gate is not None:
            if gate_per_head:
                out = out * torch.sigmoid(gate[:, gate_col:gate_col + num_heads].float())[:, :, None]
            else:
                out = out * torch.sigmoid(gate[:, gate_col:gate_col + num_heads * v_head_dim].float()).view(N, num_heads, v_head_dim)
        return out.reshape(N, num_heads * v_head_dim).to(q.dtype)

    # ------------------------------------------------------------------ layer norm before and after a sublayer
    @staticmethod
    def _ln(x, w, eps):
        mu = x.mean(-1, keepdim=True)
        d = x - mu
        return d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * w.float()

    def layernorm(self, residual, weight, eps, out_dtype, rows=None, bias=None):
        x = residual if rows is None else residual[rows.long()]
        y = self._ln(x, weight, eps)
        return (y if bias is None else y + bias.float()).to(out_dtype)

    def post_norm_add(self, residual, y, weight, eps):
        residual += self._ln(y.float(), weight, eps)

    def scaled_add(self, residual, y, weight):
        residual += y.float() * weight.float()

    def group_rmsnorm_gate(self, x, gate, gate_col, weight, group_size, eps, gate_first, out_dtype, gate_act="sigmoid"):
        N, C = x.shape
        z = gate[:, gate_col:gate_col + C].float()
        v = x * (z * torch.sigmoid(z)) if gate_first else x
        v = v.view(N, C // group_size, group_size)
        v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).reshape(N, C)
        v = v * (weight.float() if weight.shape[0] == C else weight.float().repeat(C // group_size))
        if not gate_first:
            v = v * (z * torch.sigmoid(z) if gate_act == "silu" else torch.sigmoid(z))
        return v.to(out_dtype)

    def weighted_pair(self, a, b, coef_a, coef_b, add_to):
        add_to += coef_a * a.float() + coef_b * b.float()

    def softcap(self, x, cap):
        return cap * torch.tanh(x / cap)

    def dual_rmsnorm_mix(self, a, b, weight_a, weight_b, eps, coef, add_to):
        a, b = a.float(), b.float()
        add_to += coef * (a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps) * weight_a.float()
                          + b * torch.rsqrt(b.pow(2).mean(-1, keepdim=True) + eps) * weight_b.float())

    def glu_clamped(self, gu, limit, alpha, shift, out_dtype=None):
        i = gu.shape[1] // 2
        g, u = gu[:, :i].float().clamp(max=limit), gu[:, i:].float().clamp(-limit, limit)
        return (g * torch.sigmoid(alpha * g) * (u + shift)).to(out_dtype or gu.dtype)

    def qk_norm_rope_store(self, z, num_heads, num_kv_heads, head_dim, v_head_dim, q_weight, k_weight, eps, cos, sin, rot_dims, interleaved,
                           slot_mapping, k_pool, v_pool, page_size, write_kv=True):
        N = z.shape[0]
        nq, nk = num_heads * head_dim, num_kv_heads * head_dim
        zf = z.float()
        q, k = zf[:, :nq].reshape(N, num_heads, head_dim), zf[:, nq:nq + nk].reshape(N, num_kv_heads, head_dim)
        v = zf[:, nq + nk:nq + nk + num_kv_heads * v_head_dim].reshape(N, num_kv_heads, v_head_dim)
        if q_weight is not None:
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight.float()
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight.float()

        def turn(x):
            if not rot_dims:
                return x
            c, s = cos[:, None, :], sin[:, None, :]
            out = x.clone()
            if interleaved:
                a, b = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
                out[..., 0:rot_dims:2], out[..., 1:rot_dims:2] = a * c - b * s, b * c + a * s
            else:
                h = rot_dims // 2
                a, b = x[..., :h], x[..., h:rot_dims]
                out[..., :h], out[..., h:rot_dims] = a * c - b * s, b * c + a * s
            return out

        q, k = turn(q), turn(k)
        if write_kv:
            page, off = (slot_mapping // page_size).long(), (slot_mapping % page_size).long()
            k_pool[page, :, off] = k.to(k_pool.dtype)
            v_pool[page, :, off] = v.to(v_pool.dtype)
        return q.reshape(N, nq).to(z.dtype)

    # ------------------------------------------------------------------ mixers with a state of fixed size
    @staticmethod
    def _requests(batch):
        starts = [int(x) for x in batch.seq_starts_dev[: batch.num_seqs + 1]]
        slots = [int(x) for x in batch.seq_slots[: batch.num_seqs]]
        return [(slots[r], starts[r], starts[r + 1]) for r in range(batch.num_seqs)]

    def causal_conv(self, z, col, channels, weight, bias, state, batch, activation=None):
        taps = weight.shape[1]
        out = torch.zeros(z.shape[0], channels)
        for slot, s0, s1 in self._requests(batch):
            u = torch.cat([state[slot], z[s0:s1, col:col + channels].float()])       # the last taps - 1 inputs, then the step's rows
            y = torch.zeros(s1 - s0, channels)
            for j in range(taps):
                y = y + u[j:j + s1 - s0] * weight[:, j].float()
            if bias is not None:
                y = y + bias.float()
            out[s0:s1] = y * torch.sigmoid(y) if activation == "silu" else y
            state[slot] = u[u.shape[0] - (taps - 1):]
        return out.to(z.dtype)

    def delta_rule(self, qkv, num_heads, num_kv_heads, head_dim, v_head_dim, a, b, b_col, A_log, dt_bias, state, batch, unit_eps=1e-6,
                   decay_per_head=False):
        N = qkv.shape[0]
        H, G, D, DV = num_heads, num_kv_heads, head_dim, v_head_dim
        x = qkv.float()
        q, k, v = x[:, :G * D].view(N, G, D), x[:, G * D:2 * G * D].view(N, G, D), x[:, 2 * G * D:2 * G * D + H * DV].view(N, H, DV)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * D ** -0.5
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
        beta = torch.sigmoid(b[:, b_col:b_col + H].float())
        if decay_per_head:
            decay = torch.exp(-torch.exp(A_log.float())[None, :] * torch.nn.functional.softplus(a.float() + dt_bias.float()))[:, :, None].expand(N, H, D)
        else:
            decay = torch.exp(-torch.exp(A_log.float())[None, :, None] * torch.nn.functional.softplus(a.float() + dt_bias.float()).view(N, H, D))
        out = torch.zeros(N, H, DV)
        for slot, s0, s1 in self._requests(batch):
            for h in range(H):
                g = h // (H // G)
                S = state[slot, h].T.clone()          # the state is kept column by column: [v_head_dim, head_dim]
                for n in range(s0, s1):
                    S = decay[n, h][:, None] * S
                    u = beta[n, h] * (v[n, h] - S.T @ k[n, g])
                    S = S + torch.outer(k[n, g], u)
                    out[n, h] = S.T @ q[n, g]
                state[slot, h] = S.T
        return out.reshape(N, H * DV)

    def ssm_scan(self, xbc, num_heads, groups, state_size, v_head_dim, dt, dt_col, A_log, dt_bias, skip, state, batch):
        N = xbc.shape[0]
        H, G, NS, DV = num_heads, groups, state_size, v_head_dim
        z = xbc.float()
        x, B, C = z[:, :H * DV].view(N, H, DV), z[:, H * DV:H * DV + G * NS].view(N, G, NS), z[:, H * DV + G * NS:].view(N, G, NS)
        step = torch.nn.functional.softplus(dt[:, dt_col:dt_col + H].float() + dt_bias.float())
        decay = torch.exp(-torch.exp(A_log.float())[None, :] * step)
        out = torch.zeros(N, H, DV)
        for slot, s0, s1 in self._requests(batch):
            for h in range(H):
                g = h // (H // G)
                S = state[slot, h].T.clone()          # kept column by column: [v_head_dim, state_size]
                for n in range(s0, s1):
                    S = decay[n, h] * S + step[n, h] * torch.outer(B[n, g], x[n, h])
                    out[n, h] = S.T @ C[n, g] + skip[h] * x[n, h]
                state[slot, h] = S.T
        return out.reshape(N, H * DV)

    def selective_scan(self, x, dt, bc, b_col, c_col, z, z_col, A_log, dt_bias, skip, state, batch):
        N, C = x.shape
        NS = A_log.shape[1]
        xf = x.float()
        step = torch.nn.functional.softplus(dt.float() + dt_bias.float())
        B, Cc = bc[:, b_col:b_col + NS].float(), bc[:, c_col:c_col + NS].float()
        A = -torch.exp(A_log.float())
        gate = z[:, z_col:z_col + C].float()
        out = torch.zeros(N, C)
        for slot, s0, s1 in self._requests(batch):
            S = state[slot].clone()                  # [channels, state_size]
            for n in range(s0, s1):
                S = torch.exp(step[n][:, None] * A) * S + (step[n] * xf[n])[:, None] * B[n][None, :]
                out[n] = (S @ Cc[n] + skip.float() * xf[n]) * (gate[n] * torch.sigmoid(gate[n]))
            state[slot] = S
        return out.to(x.dtype)

    # ------------------------------------------------------------------ routed experts
    def moe_route(self, logits, correction, top, scoring="softmax"):
        if scoring == "sigmoid":
            s = torch.sigmoid(logits.float())
        else:
            s = torch.softmax(logits.float(), dim=-1)
        choice = s if correction is None else s + correction.float()
        ids = torch.topk(choice, top, dim=-1).indices
        w = torch.gather(s, 1, ids)
        return ids.to(torch.int32), w if scoring == "sigmoid" else w / (w.sum(-1, keepdim=True) + 1e-20)

    def moe_router(self, h, w_router, correction, top, scoring="softmax"):
        return self.moe_route(h.float() @ w_router.float().T, correction, top, scoring)

    def moe_experts(self, h, ids, weights, w_gate_up, w_down, add_to, glu=None, weight_inputs=False):
        E, F = w_gate_up.shape[0], w_gate_up.shape[1] // 2
        x = h.float()
        for t in range(h.shape[0]):
            for k in range(ids.shape[1]):
                e = int(ids[t, k])
                xin = (x[t] * weights[t, k]).to(h.dtype).float() if weight_inputs else x[t]
                if e < E:
                    gu = w_gate_up[e].float() @ xin
                    if glu is None:
                        act = gu[:F] * torch.sigmoid(gu[:F]) * gu[F:]
                    else:
                        limit, alpha, shift = glu
                        g, u = gu[:F].clamp(max=limit), gu[F:].clamp(-limit, limit)
                        act = g * torch.sigmoid(alpha * g) * (u + shift)
                    y = w_down[e].float() @ act.to(h.dtype).float()
                else:
                    y = xin
                add_to[t] += y if weight_inputs else weights[t, k] * y

    # ------------------------------------------------------------------ latent attention
    @staticmethod
    def _turn_pairs(x, cos, sin, dims):
        """Neighbouring pairs (2i, 2i+1) of the first ``dims`` entries of the last axis; cos/sin [N, dims/2] broadcast over the middle axes."""
        if not dims:
            return x
        shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
        c, s = cos.view(shape), sin.view(shape)
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out = x.clone()
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
        return out

    def latent_prepare(self, z, q_rank, kv_rank, rot_dim, rot_dims, q_norm, kv_norm, eps, cos, sin, slot_mapping, kc_pool, page_size, write=True):
        zf = z.float()
        dq, c, r = zf[:, :q_rank], zf[:, q_rank:q_rank + kv_rank], zf[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim]
        cq = dq * torch.rsqrt(dq.pow(2).mean(-1, keepdim=True) + eps) * q_norm.float() if q_rank else None
        if write:
            c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * kv_norm.float()
            r = self._turn_pairs(r, cos, sin, rot_dims)
            page, off = (slot_mapping // page_size).long(), (slot_mapping % page_size).long()
            kc_pool[page, 0, off] = torch.cat([c, r], dim=-1).to(kc_pool.dtype)
        return cq.to(z.dtype) if q_rank else None

    def latent_absorb(self, q, w_uk, cos, sin, num_heads, head_dim, rot_dim, rot_dims, kv_rank):
        N = q.shape[0]
        qf = q.float().view(N, num_heads, head_dim + rot_dim)
        flat = torch.einsum("nhd,hdr->nhr", qf[..., :head_dim], w_uk.float().view(num_heads, head_dim, kv_rank))
        turned = self._turn_pairs(qf[..., head_dim:], cos, sin, rot_dims)
        return torch.cat([flat, turned], dim=-1).reshape(N, -1).to(q.dtype)

    def latent_expand(self, o_lat, w_uv, gate, gate_col, num_heads, kv_rank, v_head_dim):
        N = o_lat.shape[0]
        o = torch.einsum("nhr,hrv->nhv", o_lat.float().view(N, num_heads, kv_rank), w_uv.float().view(num_heads, kv_rank, v_head_dim))
        o = o.reshape(N, -1)
        if gate is not None:
            o = o * torch.sigmoid(gate[:, gate_col:gate_col + num_heads * v_head_dim].float())
        return o.to(o_lat.dtype)

    # ------------------------------------------------------------------ the matrix memory with exponential gates
    def mlstm(self, z, q_col, k_col, v_col, gates, bias_i, bias_f, cap, num_heads, head_dim, v_head_dim, state, mstate, batch):
        H, D, DV = num_heads, head_dim, v_head_dim
        N = z.shape[0]
        zf = z.float()
        q = zf[:, q_col:q_col + H * D].view(N, H, D) * D ** -0.5
        k = zf[:, k_col:k_col + H * D].view(N, H, D)
        v = torch.cat([zf[:, v_col:v_col + H * DV].view(N, H, DV), torch.ones(N, H, 1)], dim=-1)   # the normaliser's column sees v = 1
        xi, xf = gates[:, :H].float() + bias_i.float(), gates[:, H:2 * H].float() + bias_f.float()
        if cap:
            xi, xf = cap * torch.tanh(xi / cap), cap * torch.tanh(xf / cap)
        lf = torch.nn.functional.logsigmoid(xf)
        num, m_out = torch.zeros(N, H, DV + 1), torch.zeros(N, H)
        for slot, s0, s1 in self._requests(batch):
            S, m = state[slot].clone(), mstate[slot].clone()    # S [H, DV + 1, D]
            for t in range(s0, s1):
                m_new = torch.maximum(lf[t] + m, xi[t])
                a, b = torch.exp(lf[t] + m - m_new), torch.exp(xi[t] - m_new)
                S = a[:, None, None] * S + b[:, None, None] * v[t][:, :, None] * k[t][:, None, :]
                m = m_new
                num[t] = torch.einsum("hcd,hd->hc", S, q[t])
                m_out[t] = m
            state[slot], mstate[slot] = S, m
        return num, m_out

    def mlstm_finish(self, num, m, gate, gate_col, weight, eps, out_dtype):
        N, H, DV = num.shape[0], num.shape[1], num.shape[2] - 1
        den = torch.maximum(num[..., DV].abs(), torch.exp(-m)) + 1e-6
        o = num[..., :DV] / den[..., None]
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
        o = o.reshape(N, H * DV) * weight.float() * torch.sigmoid(gate[:, gate_col:gate_col + H * DV].float())
        return o.to(out_dtype)

    def argmax(self, logits):
        return logits.argmax(-1).to(torch.int32)

    def sample(self, logits, temperature, top_k, top_p, uniform):
        from plain_qwen2 import plain_draw

        out = [plain_draw(logits[i].float(), float(temperature[i]), int(top_k[i]), float(top_p[i]), float(uniform[i]))
               for i in range(logits.shape[0])]
        return torch.tensor(out, dtype=torch.int32)
