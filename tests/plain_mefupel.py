"""Plain, slow implementation of the Mefupel decoder, used only as the test oracle.

Whole sequences, no cache, no state carried between calls, one function per mechanism, CPU
torch in float64.  It shares no code with the package under test: it reads config.json as a
dictionary and takes the tensors as a dictionary of torch tensors by name.

Notation.  T tokens, width D, positions 0 .. T-1.  rms(x) = x / sqrt(mean(x^2) + eps) along the
last axis.  A linear weight W is [out, in] and acts as h @ W.T.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms(x, eps) * (1.0 + w)


def _angles(positions, base, n):
    i = torch.arange(n // 2, dtype=F)
    a = positions.to(F)[:, None] * base ** (-2.0 * i / n)
    return torch.cos(a), torch.sin(a)


def rotate(x, positions, base, n_rot, layout, sign=1.0):
    """x [T, heads, n]: the first n_rot coordinates of every head turn, pair i by
    sign * position * base^(-2i/n_rot); pairs are (2i, 2i+1) for layout "interleaved" and
    (i, i + n_rot/2) for "halves".  The rest of a head passes."""
    if n_rot == 0:
        return x.clone()
    c, s = _angles(positions, base, n_rot)
    c, s = c[:, None, :], sign * s[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        a, b = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
        out[..., 0:n_rot:2] = a * c - b * s
        out[..., 1:n_rot:2] = b * c + a * s
    else:
        half = n_rot // 2
        a, b = x[..., :half], x[..., half:n_rot]
        out[..., :half] = a * c - b * s
        out[..., half:n_rot] = b * c + a * s
    return out


def windowed_softmax_attention(q, k, v, scale, window, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Row i attends to j with
    0 <= i - j < window; query head h reads key/value head h // (H/G); `sink` [H] adds exp(sink_h)
    to the softmax's denominator and nothing to its numerator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - m)
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def attention_rotated_values(h, W, p, m):
    """Softmax attention whose values are rotated by their own position before they are summed,
    the sum being turned back by the query's position."""
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    base, n_rot = m["rot"]["base"], m["rot"]["dims"]
    q = rotate((h @ W[p + "q"].T).view(T, H, d), pos, base, n_rot, "interleaved")
    k = rotate((h @ W[p + "k"].T).view(T, G, d), pos, base, n_rot, "interleaved")
    v = rotate((h @ W[p + "v"].T).view(T, G, dv), pos, base, dv, "interleaved")
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"])
    o = rotate(o, pos, base, dv, "interleaved", sign=-1.0)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def sink_attention_keys_as_values(h, W, p, m, eps):
    """Softmax attention with a sink; the values are the key projection as it leaves the matrix,
    queries and keys are normed over the whole projection and then rotated in halves."""
    T, H, G, d = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    base, n_rot = m["rot"]["base"], m["rot"]["dims"]
    q_raw, k_raw = h @ W[p + "q"].T, h @ W[p + "k"].T
    q = rotate((rms(q_raw, eps) * W[p + "q.norm"]).view(T, H, d), pos, base, n_rot, "halves")
    k = rotate((rms(k_raw, eps) * W[p + "k.norm"]).view(T, G, d), pos, base, n_rot, "halves")
    v = k_raw.view(T, G, d)
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], sink=W[p + "sink"])
    return o.reshape(T, H * d) @ W[p + "o"].T


def linear_recurrence(q, k, v, decay):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head from S = 0.
    q, k [T, H, d], v [T, H, dv], decay [T, H, d] (one factor per key channel)."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for hh in range(H):
        S = torch.zeros(d, v.shape[-1], dtype=F)
        for t in range(T):
            S = decay[t, hh][:, None] * S + torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    return out


def gla(h, W, p, m, eps):
    """Gated linear attention: a data-dependent decay per key channel through a low-rank map."""
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, d) / math.sqrt(d)
    k = (h @ W[p + "k"].T).view(T, H, d)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, d)
    o = rms(linear_recurrence(q, k, v, decay), eps) * W[p + "norm"]
    g = h @ W[p + "g"].T
    return (o.reshape(T, H * dv) * g * torch.sigmoid(g)) @ W[p + "o"].T


def retention(h, W, p, m, eps):
    """Linear attention with one fixed decay per head, rotated queries and keys, no denominator."""
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    base, n_rot = m["rot"]["base"], m["rot"]["dims"]
    q = rotate((h @ W[p + "q"].T).view(T, H, d), pos, base, n_rot, "halves")
    k = rotate((h @ W[p + "k"].T).view(T, H, d), pos, base, n_rot, "halves") / math.sqrt(d)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F)[None, :, None].expand(T, H, d)
    o = rms(linear_recurrence(q, k, v, decay), eps)
    g = h @ W[p + "g"].T
    return (o.reshape(T, H * dv) * g * torch.sigmoid(g)) @ W[p + "o"].T


def side_by_side(h, W, p, m, eps):
    """Two mixers on the same input; each result is RMS-normed over the width with its own
    weight, and the mean of the two is the mixer's result."""
    left = sink_attention_keys_as_values(h, W, p + "left.", m["left"], eps)
    right = retention(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * W[p + "left.out"] + rms(right, eps) * W[p + "right.out"])


def polynorm_ff(h, W, p, eps):
    """down(a N(z) + b N(z^2) + c N(z^3) + e), z = up(h), N = division by the row's RMS."""
    z = h @ W[p + "up"].T
    a, b, c, e = W[p + "act"]
    return (a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e) @ W[p + "down"].T


def layer_order(cfg):
    """(layer, pass number or None) in run order; a pass number marks a pass's first layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg, tensors, tokens, streams_out=None):
    """Logits [T, vocab] (float64) of one whole sequence; `streams_out`, a list, receives the
    stream after every layer run."""
    W = {k: v.to(F) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, t in layer_order(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        h = norm_one_plus(x, W[p + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = attention_rotated_values(h, W, p + "mix.", m)
        elif kind == "gla":
            y = gla(h, W, p + "mix.", m, eps)
        elif kind == "parallel":
            y = side_by_side(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            y = y + polynorm_ff(h, W, p + "mlp.", eps)
        x = x + y
        if streams_out is not None:
            streams_out.append(x)
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T


def greedy_generate(cfg, tensors, prompt, n):
    out, seq = [], list(prompt)
    for _ in range(n):
        t = int(torch.argmax(forward(cfg, tensors, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out
