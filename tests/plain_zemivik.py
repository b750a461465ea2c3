"""A plain, slow restatement of the Zemivik design: whole sequences, no cache, no kernels, one function per
mechanism, in the precision of the tensors it is given (the tests use float64 or float32). It shares no code
with the library; the tests compare the library with it.

Notation: x [n, d] is the residual stream of one sequence of n tokens at positions 0..n-1.
"""
import math

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis; eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def embed(tokens, table, positions, norm_weight, scale, eps):
    """Token embedding times a constant, plus the learned vector of each position, then the norm."""
    n = len(tokens)
    x = table[torch.as_tensor(tokens, dtype=torch.long)] * scale + positions[:n]
    return rms_norm(x, norm_weight, eps)


def visible(n, window, keep_first):
    """[n, n] booleans: query i sees key j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if window:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_with_sink(scores, ok):
    """p_j = exp(s_j) / (1 + sum over visible j' of exp(s_j')): a sink of score 0 that has no value."""
    s = scores.masked_fill(~ok, -math.inf)
    m = s.max(-1, keepdim=True).values.clamp(min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def blend_values(v, v_first, lam):
    """(1 - lam) v + lam v_first."""
    return (1 - lam) * v + lam * v_first


def attention(x, w, prefix, mixer, eps, v_first):
    """One attention mixer on x. Returns (branch output [n, d], the values it projected before blending)."""
    n = x.shape[0]
    H, G, D, Dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = rms_norm(x @ w[prefix + "q"].T, w[prefix + "q.norm"], eps)        # over all H*D elements at once
    k = rms_norm(x @ w[prefix + "k"].T, w[prefix + "k.norm"], eps)
    v = x @ w[prefix + "v"].T
    projected = v
    if v_first is not None:
        v = blend_values(v, v_first, w[prefix + "vmix"])
    q, k, v = q.view(n, H, D), k.view(n, G, D), v.view(n, G, Dv)
    mask = mixer.get("mask")
    ok = visible(n, mask["size"] if mask else 0, mask["keep_first"] if mask else 0)
    heads = []
    for h in range(H):
        g = h // (H // G)
        p = softmax_with_sink((q[:, h] @ k[:, g].T) * mixer["scale"], ok)
        heads.append(p @ v[:, g])
    o = torch.cat(heads, dim=-1) * torch.sigmoid(x @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T, projected


def dense_mlp(x, w, prefix):
    """down(relu(up x + b)^2) + b."""
    a = torch.relu(x @ w[prefix + "up"].T + w[prefix + "up.b"]) ** 2
    return a @ w[prefix + "down"].T + w[prefix + "down.b"]


def forward(w, cfg, tokens, layers_out=None):
    """Logits [n, vocab] of one sequence. `w`: name -> tensor (all of one floating type)."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w["embed"], w["pos"], w["embed.norm"], cfg["embedding"]["scale"], eps)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        y, projected = attention(x, w, f"l{i}.mix.", m, eps, v_first if m.get("v_mix") else None)
        if m.get("v_mix") and v_first is None:
            v_first = projected
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            x = x + rms_norm(dense_mlp(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x)
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def logits(w, cfg, tokens, dtype=torch.float64):
    return forward({k: v.to(dtype) for k, v in w.items()}, cfg, tokens).float()


def greedy(row):
    return int(row.argmax())


# ------------------------------------------------------------------------------------------ small configurations
def attention_cfg(heads, kv_heads, dim, vdim, scale, v_mix, window=None, keep_first=0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix,
            "mask": None if window is None else {"size": window, "keep_first": keep_first}}


def layer_cfg(mixer, ff):
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model_cfg(vocab, width, max_positions, scale, eps, layers):
    return {"architecture": "Zemivik", "vocab": vocab, "width": width, "max_positions": max_positions,
            "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}


# A: every layer alike; value heads wider than key heads; a short window with three kept tokens; sharp scores.
TINY_A = model_cfg(211, 96, 320, 2.0, 1e-5, [
    layer_cfg(attention_cfg(4, 2, 16, 32, 1.1, True, 40, 3), 160) for _ in range(3)])
# B: every layer different: no mask and no blending; the first blending layer without a feed-forward; a blending
# layer whose window keeps nothing; as many key heads as query heads with head sizes that are no multiples of 8;
# one head; a window of one page exactly.
TINY_B = model_cfg(157, 72, 400, 0.7, 3e-6, [
    layer_cfg(attention_cfg(3, 1, 24, 24, 0.9, False), 100),
    layer_cfg(attention_cfg(2, 2, 20, 12, 1.3, True, 33, 1), None),
    layer_cfg(attention_cfg(4, 2, 8, 12, 1.6, True, 64, 0), 36),
    layer_cfg(attention_cfg(1, 1, 40, 24, 0.8, False, 7, 9), 52),
    layer_cfg(attention_cfg(6, 2, 16, 12, 1.0, True, 100, 64), None)])
# C: the head sizes the tensor-core kernels take (64), six query heads on one key head, a window longer than two
# pages that keeps more than a page, longer sequences.
TINY_C = model_cfg(300, 128, 900, 1.0, 1e-5, [
    layer_cfg(attention_cfg(6, 1, 64, 64, 0.35, True, 150, 70), 256),
    layer_cfg(attention_cfg(2, 1, 64, 64, 0.4, True, 64, 64), 128),
    layer_cfg(attention_cfg(4, 2, 128, 128, 0.2, False, 200, 5), None)])
