"""A plain, slow statement of the Bisodra design, one function per mechanism, in whatever float type it is given.

It shares nothing with the library: tensors come in a dict by checkpoint name, the configuration as the dict that
config.json holds.  Everything runs on one whole sequence at a time, every key of every query spelled out; there is no
cache.

Notation: x [T, W] residual stream of one sequence; W_* weights [out, in]; p positions 0..T-1; i a query's position,
j a key's.
"""
from __future__ import annotations

import math

import torch


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * w with the variance as the mean squared deviation; no bias."""
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(dim=-1, keepdim=True) + eps) * weight


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(h, w_up, w_down):
    """Two matrices with the exact GELU between them; no gate."""
    return gelu_erf(h @ w_up.T) @ w_down.T


def short_conv(u, taps):
    """Causal convolution over time on each channel: y_t = sum_j taps[:, j] u_(t - n + 1 + j), zeros before the start.
    u [T, C], taps [C, n]."""
    n = taps.shape[1]
    padded = torch.cat([u.new_zeros(n - 1, u.shape[1]), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(n):
        out = out + padded[j:j + u.shape[0]] * taps[:, j]
    return out


def slopes(heads: int, dtype):
    """One slope per head for the linear distance bias: 2^(-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def visible_window(T: int, size: int, keep_first: int, rows=None):
    """[rows, T] bool: the query at position i (``rows``; every position 0..T-1 by default) sees key j <= i if it is
    within ``size`` positions or among the first ``keep_first``."""
    i = (torch.arange(T) if rows is None else torch.as_tensor(rows))[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def softmax_with_sink(scores, visible):
    """p_j = exp(s_j) / (1 + sum_visible exp(s_j)): one more term of score 0 that carries no value."""
    masked = scores.masked_fill(~visible, float("-inf"))
    top = torch.clamp(masked.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(masked - top)
    return e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))


def biased_heads(q, k, rows, scale, size, keep_first):
    """Queries q [n, H, d] at positions ``rows`` over the keys k [T, G, d] of their sequence, which are the values too:
    score = q . k * scale - slope_h (i - j), a window that keeps the first keys, softmax with a sink.  [n, H, d]."""
    heads, groups = q.shape[1], k.shape[1]
    rows = torch.as_tensor(rows)
    visible = visible_window(k.shape[0], size if size is not None else k.shape[0], keep_first, rows)
    distance = (rows[:, None] - torch.arange(k.shape[0])[None, :]).to(q.dtype)
    slope = slopes(heads, q.dtype)
    out = torch.zeros_like(q)
    for head in range(heads):
        kv = k[:, head // (heads // groups)]
        scores = (q[:, head] @ kv.T) * scale - slope[head] * distance
        out[:, head] = softmax_with_sink(scores, visible) @ kv
    return out


def window_attention(h, tensors, prefix, mixer):
    """Grouped heads; biased q, k and o; a short convolution on q and k; values are the keys; a linear distance bias;
    a window that keeps the first tokens; softmax with a sink; a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    dt = h.dtype
    heads, groups, dim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"])
    t = lambda name: tensors[f"{prefix}.{name}"].to(dt)
    q = short_conv(h @ t("q").T + t("q.b"), t("q.conv")).view(T, heads, dim)
    k = short_conv(h @ t("k").T + t("k.b"), t("k.conv")).view(T, groups, dim)
    mask = mixer.get("mask") or {}
    out = biased_heads(q, k, torch.arange(T), float(mixer["scale"]), mask.get("size"), int(mask.get("keep_first", 0)))
    gated = out.reshape(T, heads * dim) * torch.sigmoid(h @ t("g").T)
    return gated @ t("o").T + t("o.b")


def yarn_frequencies(rot, dtype=torch.float64):
    """Frequencies of the rotation pairs and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    scaling = rot.get("scaling")
    if not scaling:
        return f.to(dtype), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(dtype), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, rot):
    """x [T, ..., n >= dims]: of the first ``dims`` elements, element i turns with element i + dims / 2 by the angle p f_i."""
    f, magnitude = yarn_frequencies(rot)
    angles = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (angles.cos() * magnitude).to(x.dtype), (angles.sin() * magnitude).to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    dims = int(rot["dims"])
    half = dims // 2
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]          # elements beyond the first ``dims`` pass unchanged
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


def latent_of(h, tensors, prefix, mixer, eps):
    """What a latent-attention layer keeps per token: the normed latent c [T, kv_rank] and the rotated key part
    [T, rot_dim] that all heads share."""
    dt = h.dtype
    rank = int(mixer["kv_rank"])
    down = h @ tensors[f"{prefix}.dkv"].to(dt).T
    c = rms_norm(down[:, :rank], tensors[f"{prefix}.dkv.norm"].to(dt), eps)
    shared = rotate_half(down[:, rank:], torch.arange(h.shape[0]), mixer["rot"])
    return c, shared


def latent_heads(q_plain, q_turned, c, shared, w_uk, w_uv, rows, scale):
    """Queries at positions ``rows`` (q_plain [n, H, d], q_turned [n, H, r] already rotated) over the kept rows of their
    sequence (c [T, rank], shared [T, r]): head h has the keys W_uk_h c | shared and the values W_uv_h c; causal, plain
    softmax.  w_uk [H d, rank], w_uv [H dv, rank].  [n, H, dv]."""
    heads, dim = q_plain.shape[1], q_plain.shape[2]
    T = c.shape[0]
    k_plain = (c @ w_uk.T).view(T, heads, dim)
    values = (c @ w_uv.T).view(T, heads, -1)
    causal = torch.arange(T)[None, :] <= torch.as_tensor(rows)[:, None]
    out = q_plain.new_zeros(q_plain.shape[0], heads, values.shape[-1])
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_turned[:, head] @ shared.T) * scale
        out[:, head] = torch.softmax(scores.masked_fill(~causal, float("-inf")), dim=-1) @ values[:, head]
    return out


def latent_attention(h, tensors, prefix, mixer, eps, kept):
    """Queries through a latent of their own; keys and values expanded per head from ``kept`` = (c, shared rotated
    key part); causal softmax; a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    dt = h.dtype
    heads, dim, rot_dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["rot_dim"]), int(mixer["vdim"])
    t = lambda name: tensors[f"{prefix}.{name}"].to(dt)
    c, shared = kept
    cq = rms_norm(h @ t("dq").T, t("dq.norm"), eps)
    q = (cq @ t("uq").T).view(T, heads, dim + rot_dim)
    q_plain, q_turned = q[..., :dim], rotate_half(q[..., dim:], torch.arange(T), mixer["rot"])
    out = latent_heads(q_plain, q_turned, c, shared, t("uk"), t("uv"), torch.arange(T), float(mixer["scale"]))
    gated = out.reshape(T, heads * vdim) * torch.sigmoid(h @ t("g").T)
    return gated @ t("o").T


def forward(config: dict, tensors: dict, token_ids, dtype=torch.float64, keep_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the stream after every layer)."""
    eps = float(config["norm"]["eps"])
    table = tensors["embed"].to(dtype)
    x = table[torch.as_tensor(token_ids, dtype=torch.long)] * float(config["embedding"]["scale"])
    kept_by_layer: dict[int, tuple] = {}
    streams = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}"
        norm = lambda name: tensors[f"{prefix}.{name}"].to(dtype)
        h = layer_norm(x, norm("norm1"), eps)
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            y = window_attention(h, tensors, f"{prefix}.mix", mixer)
        elif layer["type"] == "latent_attention":
            if mixer.get("kv_from") is None:
                kept_by_layer[index] = latent_of(h, tensors, f"{prefix}.mix", mixer, eps)
                kept = kept_by_layer[index]
            else:
                kept = kept_by_layer[int(mixer["kv_from"])]
            y = latent_attention(h, tensors, f"{prefix}.mix", mixer, eps, kept)
        else:
            raise ValueError(f"no mixer {layer['type']!r}")
        x = x + layer_norm(y, norm("norm1b"), eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, norm("norm2"), eps)
            y = dense_ff(h, tensors[f"{prefix}.mlp.up"].to(dtype), tensors[f"{prefix}.mlp.down"].to(dtype))
            x = x + layer_norm(y, norm("norm2b"), eps)
        streams.append(x)
    logits = layer_norm(x, tensors["final.norm"].to(dtype), eps) @ table.T * float(config["logit_scale"])
    return (logits, torch.stack(streams)) if keep_layers else logits
