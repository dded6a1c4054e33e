"""Plain, slow implementation of the Zolulix decoder, used only as the test oracle.

Whole sequences, no cache, no state carried between calls, one function per mechanism, CPU
torch in float64.  It shares no code with the package under test: it reads config.json as a
dictionary and the tensors through plain_model's own safetensors reader.

Notation.  T tokens, width D.  rms(x) = x / sqrt(mean(x^2) + eps) along the last axis.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose weight g is one number."""
    return rms(x, eps) * g


def rotate_pairs(x, positions, base, n_rot):
    """x [T, ..., n]: neighbours (2i, 2i+1), i < n_rot/2, turn by position * base^(-2i/n_rot);
    the rest of the last axis passes."""
    out = x.clone()
    i = torch.arange(n_rot // 2, dtype=F)
    angle = positions.to(F)[:, None] * base ** (-2.0 * i / n_rot)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n_rot // 2]
    c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    a, b = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    out[..., 0:n_rot:2] = a * c - b * s
    out[..., 1:n_rot:2] = b * c + a * s
    return out


def latent_kv(h, W, p, m, eps):
    """(latent c [T, rank], rotated shared key part [T, rot_dim]) of a layer that owns them."""
    T, r = h.shape[0], m["kv_rank"]
    dkv = h @ W[p + "dkv"].T
    c = rms(dkv[:, :r], eps) * W[p + "dkv.norm"]
    kr = rotate_pairs(dkv[:, r:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, W, p, m, c, kr):
    """Attention of the rows h over the latents c and key parts kr (of this layer or another)."""
    T, H, dim, rd, vd = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, dim + rd)
    q_plain = q[..., :dim]
    q_rot = rotate_pairs(q[..., dim:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ W[p + "uk"].T).view(T, H, dim)
    v = (c @ W[p + "uv"].T).view(T, H, vd)
    out = torch.zeros(T, H, vd, dtype=F)
    for i in range(T):
        lo = max(0, i - m["mask"]["size"] + 1)
        for hh in range(H):
            s = (k_plain[lo:i + 1, hh] @ q_plain[i, hh] + kr[lo:i + 1] @ q_rot[i, hh]) * m["scale"]
            w = torch.softmax(s, 0)
            out[i, hh] = w @ v[lo:i + 1, hh]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def mlstm(h, W, p, m, eps):
    """The matrix-memory recurrence, token by token, from a zero state."""
    T, H, dim, vd, cap = h.shape[0], m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ W[p + "q"].T).view(T, H, dim) / math.sqrt(dim)
    k = (h @ W[p + "k"].T).view(T, H, dim)
    v = (h @ W[p + "v"].T).view(T, H, vd)
    gi = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    out = torch.zeros(T, H, vd, dtype=F)
    for hh in range(H):
        S, n, mx = torch.zeros(dim, vd, dtype=F), torch.zeros(dim, dtype=F), torch.zeros((), dtype=F)
        for t in range(T):
            m_new = torch.maximum(gf[t, hh] + mx, gi[t, hh])
            keep, take = torch.exp(gf[t, hh] + mx - m_new), torch.exp(gi[t, hh] - m_new)
            S = keep * S + take * torch.outer(k[t, hh], v[t, hh])
            n = keep * n + take * k[t, hh]
            mx = m_new
            den = torch.maximum((n @ q[t, hh]).abs(), torch.exp(-mx)) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    out = rms(out, eps).reshape(T, H * vd) * W[p + "norm"]
    return (out * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def clamped_glu(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def depth_sum(streams, w):
    return sum(w[j] * x for j, x in enumerate(streams))


def forward(cfg, tensors, tokens, streams_out=None):
    """Logits [T, vocab] (float64) of one whole sequence; `streams_out`, a list, receives what
    each layer hands on."""
    W = {k: v.to(F) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    streams, kept = [x], {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = scalar_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            if "kv_from" in m and m["kv_from"] is not None:
                c, kr = kept[m["kv_from"]]
            else:
                c, kr = kept[i] = latent_kv(h, W, p + "mix.", m, eps)
            y = latent_attention(h, W, p + "mix.", m, c, kr)
        else:
            y = mlstm(h, W, p + "mix.", m, eps)
        x = x + scalar_norm(y, W[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            y = clamped_glu(scalar_norm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"]["limit"])
            x = x + scalar_norm(y, W[p + "norm2b"], eps)
        streams.append(x)
        x = depth_sum(streams, W[p + "dwa"])
        if streams_out is not None:
            streams_out.append(x)
    return scalar_norm(x, W["final.norm"], eps) @ W["head"].T


def greedy_generate(cfg, tensors, prompt, n):
    out, seq = [], list(prompt)
    for _ in range(n):
        t = int(torch.argmax(forward(cfg, tensors, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out
