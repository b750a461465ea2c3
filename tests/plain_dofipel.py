"""A plain, slow restatement of the Dofipel design: whole sequences, no cache, no kernels, one function per
mechanism, in the precision of the tensors it is given (the tests use float64). It shares no code with the
library; the tests compare the library with it.

Notation: x [n, d] is the residual stream of one sequence of n tokens at positions 0..n-1; `w` maps checkpoint
names to tensors; `m` is a layer's `mixer` object of config.json and `f` its `mlp` object.

    layer:    u = dyt(x);  x <- x + (mixer(u) + ff(u))           one norm, both branches read it
    output:   logits = E dyt(x) * logit_scale                    E the embedding table
"""
import math

import torch


def dyt(x, alpha, weight, bias):
    """Dynamic tanh: tanh(alpha x) * weight + bias, element by element (no mean, no variance)."""
    return torch.tanh(alpha * x) * weight + bias


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def distance_bucket(n, rows, far):
    """Row of the distance-bias table for distance n >= 0: the first half of the rows one distance each, the
    second half spaced evenly in log(distance) up to `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def window_visible(n, size):
    """[n, n] booleans: query i sees key j when 0 <= i - j < size (size 0: every j <= i)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i - j < size)
    return ok


def softmax_with_sink(scores, ok, sink):
    """p_j = exp(s_j) / (exp(sink) + sum over visible j' of exp(s_j')); sink None = the ordinary softmax."""
    s = scores.masked_fill(~ok, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.expand_as(m))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - m)
    return e / den


def window_attention(u, w, p, m):
    """Grouped-query attention without rotation: capped scores, a learned bias by distance, a sliding window, a
    learned sink per head."""
    n = u.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (u @ w[p + "q"].T).view(n, H, D)
    k = (u @ w[p + "k"].T).view(n, G, D)
    v = (u @ w[p + "v"].T).view(n, G, Dv)
    rel = w[p + "rel"]                                     # [rows, H]
    rows = rel.shape[0]
    ok = window_visible(n, m["mask"]["size"] if m.get("mask") else 0)
    bucket = torch.tensor([[distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(n)]
                           for i in range(n)], dtype=torch.long)
    cap = m["softcap"]
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = cap * torch.tanh(s / cap)
        s = s + rel[:, h][bucket]
        heads.append(softmax_with_sink(s, ok, w[p + "sink"][h]) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def rotate_pairs(x, positions, base, dims):
    """Rotary positions on the first `dims` entries of the last axis of x [n, ..., size]: entries 2i and 2i+1 form
    a pair turned by the angle position * base^(-2i/dims); the rest passes unchanged."""
    n = x.shape[0]
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * freq[None, :]     # [n, dims/2]
    shape = [n] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(a).view(shape), torch.sin(a).view(shape)
    out = x.clone()
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def latent_keys(u, w, p, m, eps):
    """What a latent-attention layer keeps per token: the normed latent c [n, kv_rank] and the rotated key part
    [n, rot_dim] that all heads share."""
    n = u.shape[0]
    r = m["kv_rank"]
    d = u @ w[p + "dkv"].T
    c = rms_norm(d[:, :r], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(d[:, r:], torch.arange(n), m["rot"]["base"], m["rot"]["dims"])
    return c, k_rot


def latent_attention(u, w, p, m, c, k_rot):
    """Causal attention whose keys and values are made from the latent (c, k_rot), with an output gate."""
    n = u.shape[0]
    H, D, R, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (u @ w[p + "q"].T).view(n, H, D + R)
    q_plain = q[..., :D]
    q_rot = rotate_pairs(q[..., D:], torch.arange(n), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).view(n, H, D)
    v = (c @ w[p + "uv"].T).view(n, H, Dv)
    ok = window_visible(n, 0)
    heads = []
    for h in range(H):
        s = (q_plain[:, h] @ k_plain[:, h].T + q_rot[:, h] @ k_rot.T) * m["scale"]
        heads.append(softmax_with_sink(s, ok, None) @ v[:, h])
    o = torch.cat(heads, dim=-1) * torch.sigmoid(u @ w[p + "g"].T)
    return o @ w[p + "o"].T


def gated_ff(u, w, p, act):
    """down(act(gate u) * (up u))."""
    return (act(u @ w[p + "gate"].T) * (u @ w[p + "up"].T)) @ w[p + "down"].T


def route(u, w, p, top):
    """Router: logits = W u + b; the `top` largest are chosen, weighted by the softmax over the chosen logits
    alone. Returns (ids [n, top], weights [n, top])."""
    z = u @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe(u, w, p, f):
    """Weighted sum of each token's chosen experts plus the shared expert that every token uses."""
    idx, wt = route(u, w, p, f["router"]["top"])
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            out[t] += a * gated_ff(u[t:t + 1], w, f"{p}e{e}.", silu)[0]
    if f.get("shared") is not None:
        out = out + gated_ff(u, w, p + "shared.", silu)
    return out


def feed_forward(u, w, p, f):
    if f is None:
        return torch.zeros_like(u)
    if f["kind"] == "dense":
        return gated_ff(u, w, p, gelu_tanh)
    return moe(u, w, p, f)


def forward(w, cfg, tokens, layers_out=None):
    """Logits [n, vocab] of one sequence. `w`: name -> tensor (all of one floating type, tables of integers
    aside). `layers_out`, a list, receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        u = dyt(x, w[p + "norm1.alpha"], w[p + "norm1"], w[p + "norm1.b"])
        if layer["type"] == "attention":
            y = window_attention(u, w, p + "mix.", m)
        else:
            if m.get("kv_from") is None:
                latents[i] = latent_keys(u, w, p + "mix.", m, eps)
            c, k_rot = latents[i if m.get("kv_from") is None else m["kv_from"]]
            y = latent_attention(u, w, p + "mix.", m, c, k_rot)
        x = x + (y + feed_forward(u, w, p + "mlp.", layer.get("mlp")))
        if layers_out is not None:
            layers_out.append(x.clone())
    u = dyt(x, w["final.norm.alpha"], w["final.norm"], w["final.norm.b"])
    return (u @ w["embed"].T) * cfg["logit_scale"]
