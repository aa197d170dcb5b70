"""A plain, slow statement of the Regupel design, one function per mechanism, in float64 on the CPU.

It shares no code with the package: tensors come in as a dict name -> tensor, the configuration as the dict that
config.json holds.  Every sequence is run by itself, token after token where a mechanism is recurrent.

The design: x = embed[token] * embedding.scale; every layer adds m * LN1(mixer(x)) and then m * LN2(ff(x)) (the
sublayers read the stream itself; the layer norms have a weight and a bias; m = residual_mult); the logits are
embed LN_final(x) * logit_scale.  Mixer ``attention``: grouped heads, rotate-half rotation of the first rot.dims
elements with frequencies stretched by wavelength, q and k divided by their root mean square per head after the
rotation, a sliding window, a softmax whose denominator also holds exp(sink_h), heads times sigmoid(W_g h)_h.
Mixer ``parallel``: left, an attention whose q and k are RMS-normed over the whole projection with a weight, no
rotation, a window that also keeps the first tokens; right, a linear attention with a constant decay per head,
S <- decay S + k v^T, o = S^T q on SiLU'd projections, RMS-normed over all heads with a weight, times sigmoid(W_g h);
the two are mixed with two constants.  Feed-forward: experts chosen by a sigmoid router, the score multiplying the
expert's input, plus a shared expert.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def stretched_frequencies(dims: int, base: float, scaling) -> torch.Tensor:
    """f_i = base^(-2i/dims); a pair whose wavelength 2 pi / f is below original/high keeps f, above original/low turns
    at f / factor, and between the two blends them linearly in original / wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate(x, positions, freqs, dims):
    """x [T, heads, dim]: element i < dims/2 turns together with element i + dims/2 by the angle position * f_i."""
    if dims == 0:
        return x
    half = dims // 2
    angle = positions.to(F)[:, None] * freqs[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, x[..., dims:]), dim=-1)


def masked_softmax_attention(q, k, v, scale, window, keep_first, sinks):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one sequence from its start.  Query i sees key j <= i with
    i - j < window (None: all) or j < keep_first.  sinks [H] or None: exp(sink) joins the denominator."""
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F)
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    for h in range(heads):
        g = h // group
        score = (q[:, h] @ k[:, g].T) * scale
        score = score.masked_fill(~seen, -math.inf)
        top = score.max(-1, keepdim=True).values
        if sinks is not None:
            top = torch.maximum(top, sinks[h].expand_as(top))
        weight = torch.exp(score - top)
        denominator = weight.sum(-1, keepdim=True)
        if sinks is not None:
            denominator = denominator + torch.exp(sinks[h] - top)
        out[:, h] = (weight / denominator) @ v[:, g]
    return out


def attention_mixer(h, t, prefix, m, eps):
    tokens = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[prefix + ".q"].T).view(tokens, heads, dim)
    k = (h @ t[prefix + ".k"].T).view(tokens, kv, dim)
    v = (h @ t[prefix + ".v"].T).view(tokens, kv, vdim)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        freqs = stretched_frequencies(dims, float(rot["base"]), rot.get("scaling"))
        positions = torch.arange(tokens)
        q, k = rotate(q, positions, freqs, dims), rotate(k, positions, freqs, dims)
    q, k = rms_divide(q, eps), rms_divide(k, eps)
    mask = m.get("mask") or {}
    out = masked_softmax_attention(q, k, v, float(m["scale"]), mask.get("size"), int(mask.get("keep_first", 0)), t[prefix + ".sink"])
    gate = torch.sigmoid(h @ t[prefix + ".g"].T)                 # [T, heads]
    out = out * gate[:, :, None]
    return out.reshape(tokens, heads * vdim) @ t[prefix + ".o"].T


def left_mixer(h, t, prefix, m, eps):
    tokens = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_divide(h @ t[prefix + ".q"].T, eps) * t[prefix + ".q.norm"]
    k = rms_divide(h @ t[prefix + ".k"].T, eps) * t[prefix + ".k.norm"]
    v = (h @ t[prefix + ".v"].T).view(tokens, kv, vdim)
    mask = m.get("mask") or {}
    out = masked_softmax_attention(q.view(tokens, heads, dim), k.view(tokens, kv, dim), v, float(m["scale"]), mask.get("size"),
                                   int(mask.get("keep_first", 0)), None)
    return out.reshape(tokens, heads * vdim) @ t[prefix + ".o"].T


def decayed_linear_attention(q, k, v, decay):
    """q, k [T, H, d], v [T, H, dv], decay [H]: S_t = decay S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t."""
    tokens, heads, dim = q.shape
    state = torch.zeros(heads, dim, v.shape[-1], dtype=F)
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F)
    for step in range(tokens):
        state = decay[:, None, None] * state + k[step][:, :, None] * v[step][:, None, :]
        out[step] = torch.einsum("hdv,hd->hv", state, q[step])
    return out


def right_mixer(h, t, prefix, m, eps):
    tokens = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ t[prefix + ".q"].T).view(tokens, heads, dim)
    k = silu(h @ t[prefix + ".k"].T).view(tokens, heads, dim)
    v = silu(h @ t[prefix + ".v"].T).view(tokens, heads, vdim)
    out = decayed_linear_attention(q, k, v, torch.tensor([float(d) for d in m["decay"]], dtype=F)).reshape(tokens, heads * vdim)
    out = rms_divide(out, eps) * t[prefix + ".norm"] * torch.sigmoid(h @ t[prefix + ".g"].T)
    return out @ t[prefix + ".o"].T


def parallel_mixer(h, t, prefix, m, eps):
    return float(m["left_scale"]) * left_mixer(h, t, prefix + ".left", m["left"], eps) + \
        float(m["right_scale"]) * right_mixer(h, t, prefix + ".right", m["right"], eps)


def expert(h, t, prefix):
    return (silu(h @ t[prefix + ".gate"].T) * (h @ t[prefix + ".up"].T)) @ t[prefix + ".down"].T


def routed_feed_forward(h, t, prefix, mlp, margins: list | None = None):
    """``margins`` collects, per position, how clear the router's choice is: the gap between the last chosen logit and the
    first one left out, over the root mean square of the position's logits (infinite where every expert is chosen)."""
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ t[prefix + ".router"].T
    scores = torch.sigmoid(logits)
    if margins is not None:
        ordered = logits.sort(dim=-1, descending=True).values
        gap = ordered[:, top - 1] - ordered[:, top] if top < experts else torch.full((h.shape[0],), math.inf, dtype=F)
        margins.append(gap / (logits.pow(2).mean(-1).sqrt() + 1e-30))
    out = torch.zeros_like(h)
    for row in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(logits[row, e]), e))[:top]      # the scores' order is the logits' order
        for e in order:
            out[row] += expert(scores[row, e] * h[row], t, f"{prefix}.e{e}")
    if mlp.get("shared") is not None:
        out = out + expert(h, t, prefix + ".shared")
    return out


def forward(config, tensors, tokens, layers_out: list | None = None, margins: list | None = None):
    """Logits [T, vocab] of one sequence from its start; ``layers_out`` collects the stream after every layer run,
    ``margins`` the clearness of every router's choice per position (see ``routed_feed_forward``)."""
    t = {name: value.to(F) for name, value in tensors.items()}
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float((config.get("embedding") or {}).get("scale", 1.0))
    for index, entry in enumerate(config["layers"]):
        owner = entry.get("weights_of", index)
        p = f"l{owner}"
        mixer = attention_mixer if entry["type"] == "attention" else parallel_mixer
        x = x + mult * layer_norm(mixer(x, t, p + ".mix", entry["mixer"], eps), t[p + ".norm1"], t[p + ".norm1.b"], eps)
        if entry.get("mlp") is not None:
            x = x + mult * layer_norm(routed_feed_forward(x, t, p + ".mlp", entry["mlp"], margins), t[p + ".norm2"], t[p + ".norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    return (x @ t["embed"].T) * float(config.get("logit_scale", 1.0))
