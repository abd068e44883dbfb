"""The Zozezen decoder written out plainly: one function per mechanism, whole sequences, float64.

The oracle of the Zozezen tests.  It shares no code with the package: it reads ``config.json`` as a nested
mapping, takes tensors by their checkpoint names, computes a whole sequence at once (no cache, no state carried
between calls, no batching), walks the recurrence token by token and the experts token by token.

Notation: ``x`` is the residual stream ``[n, width]``, ``h`` a sublayer's normed input.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F64 = torch.float64


def load_folder(folder, dtype=F64):
    from safetensors.torch import load_file

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    tensors = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in
               load_file(str(folder / "model.safetensors")).items()}
    return config, tensors


# --------------------------------------------------------------------------- small pieces


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    """The model's norm: the stored weight lies around zero and stands for 1 + weight."""
    return unit_rms(x, eps) * (1.0 + weight)


def norm_plain(x, weight, eps):
    return unit_rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_half_split(x, positions, dims, base):
    """Rotates the first ``dims`` entries of the last dimension of ``x [n, heads, d]``; entry i pairs with entry
    i + dims/2 and turns by the angle ``position * base^(-2i/dims)``."""
    half = dims // 2
    freqs = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angles = positions.to(F64)[:, None] * freqs[None, :]
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------- attention


def attention_keys_values(h, w, prefix, mixer, eps, positions):
    """The keys (normed, rotated) ``[n, G, dim]`` and values ``[n, G, vdim]`` that a layer with projections of its
    own makes from its input."""
    n = h.shape[0]
    G, dim, vdim = int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    k = (h @ w[prefix + "mix.k"].T).view(n, G, dim)
    v = (h @ w[prefix + "mix.v"].T).view(n, G, vdim)
    k = norm_plain(k, w[prefix + "mix.k.norm"], eps)
    k = rotate_half_split(k, positions, int(mixer["rot"]["dims"]), float(mixer["rot"]["base"]))
    return k, v


def attention(h, w, prefix, mixer, eps, positions, keys, values, window=None):
    """Causal attention of every row of ``h`` over ``keys``/``values`` of the same rows, with a sink in the softmax's
    denominator and a gate per head.  Returns ``[n, width]``."""
    n = h.shape[0]
    H, G, dim, vdim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    q = (h @ w[prefix + "mix.q"].T).view(n, H, dim)
    q = norm_plain(q, w[prefix + "mix.q.norm"], eps)
    q = rotate_half_split(q, positions, int(mixer["rot"]["dims"]), float(mixer["rot"]["base"]))
    gate = torch.sigmoid(h @ w[prefix + "mix.g"].T)                     # [n, H]
    out = torch.zeros(n, H, vdim, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ keys[:, g].T) * float(mixer["scale"])      # [n, n]
        i = positions[:, None]
        j = positions[None, :]
        visible = j <= i
        if window:
            visible = visible & (j > i - window)
        scores = scores.masked_fill(~visible, -math.inf)
        # softmax with a sink of score 0 that carries no value: 1 is added to the denominator
        top = torch.clamp(scores.max(dim=-1, keepdim=True).values, min=0.0)
        e = torch.exp(scores - top)
        p = e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))
        out[:, head] = (p @ values[:, g]) * gate[:, head:head + 1]
    return out.reshape(n, H * vdim) @ w[prefix + "mix.o"].T


# --------------------------------------------------------------------------- the state-space mixer


def causal_convolution(u, weight, bias):
    """Per channel: out[t] = bias + sum_k weight[:, k] * u[t - (taps - 1 - k)], zeros before the start."""
    n, taps = u.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    out = bias.expand(n, -1).clone()
    for k in range(taps):
        out = out + padded[k:k + n] * weight[:, k]
    return out


def state_space(h, w, prefix, mixer, eps):
    """The selective state-space mixer, walked token by token.  Returns ``[n, width]``."""
    n = h.shape[0]
    H, P, N, G = int(mixer["heads"]), int(mixer["vdim"]), int(mixer["state"]), int(mixer["groups"])
    inner = H * P
    proj = h @ w[prefix + "mix.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_convolution(xbc, w[prefix + "mix.conv"], w[prefix + "mix.conv.b"]))
    xs = xbc[:, :inner].view(n, H, P)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = softplus(dt + w[prefix + "mix.dt_bias"])                       # [n, H]
    decay = torch.exp(-torch.exp(w[prefix + "mix.A_log"]) * dt)         # [n, H]
    y = torch.zeros(n, H, P, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(n):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], xs[t, head])
            y[t, head] = S.T @ C[t, g] + w[prefix + "mix.D"][head] * xs[t, head]
    y = y.reshape(n, inner) * silu(z)
    parts = int(mixer["norm_groups"])
    y = unit_rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[prefix + "mix.norm"]
    return y @ w[prefix + "mix.o"].T


# --------------------------------------------------------------------------- feed-forward


def clamped_expert(h, gate_w, up_w, down_w, limit):
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down_w.T


def route(h, w, prefix, mlp):
    """Per token the chosen router outputs and their weights: ``(ids [n, top], weights [n, top], smallest gap)``.
    The gap is the distance between the weakest chosen and the strongest unchosen choice score (after the group
    limit), for tests that must not rest on a close call."""
    router = mlp["router"]
    top = int(router["top"])
    total = int(router["experts"]) + int(router.get("identity", 0) or 0)
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    scores = torch.softmax(h @ w[prefix + "mlp.router"].T, dim=-1)      # [n, total]
    choice = scores + w[prefix + "mlp.correction"]
    n = h.shape[0]
    group_best = choice.view(n, count, total // count).max(dim=-1).values
    kept = torch.zeros(n, count, dtype=torch.bool)
    kept.scatter_(1, torch.topk(group_best, keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(n, count, total // count).reshape(n, total)
    limited = choice.masked_fill(~allowed, -math.inf)
    ranked = torch.sort(limited, dim=-1, descending=True)
    ids = ranked.indices[:, :top]
    gap = math.inf
    if top < total:
        gap = float((ranked.values[:, top - 1] - ranked.values[:, top]).min())
    if keep < count:
        best = torch.sort(group_best, dim=-1, descending=True).values
        gap = min(gap, float((best[:, keep - 1] - best[:, keep]).min()))
    return ids, torch.gather(scores, 1, ids), gap


def mixture(h, w, prefix, mlp):
    """Routed experts (some of them identities), unrenormalised weights, plus a gated shared expert."""
    router = mlp["router"]
    real = int(router["experts"])
    limit = float(mlp["expert"]["limit"])
    ids, weights, _gap = route(h, w, prefix, mlp)
    out = torch.zeros(h.shape[0], h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t].tolist(), weights[t].tolist()):
            if e >= real:
                out[t] += weight * h[t]
            else:
                p = f"{prefix}mlp.e{e}."
                out[t] += weight * clamped_expert(h[t:t + 1], w[p + "gate"], w[p + "up"], w[p + "down"], limit)[0]
    shared = mlp.get("shared")
    if shared:
        p = prefix + "mlp.shared."
        y = clamped_expert(h, w[p + "gate"], w[p + "up"], w[p + "down"], float(shared["limit"]))
        out = out + y * torch.sigmoid(h @ w[p + "sg"].T)
    return out


# --------------------------------------------------------------------------- the model


def forward(tokens, w, config, return_layers=False):
    """float64 logits ``[n, vocab]`` of a whole sequence (and the stream after every layer)."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = w["embed"][tokens]
    kept = {}                     # layer index -> (keys, values) for layers that lend theirs
    stream = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        mixer = layer["mixer"]
        h = norm_one_plus(x, w[prefix + "norm1"], eps)
        if layer["type"] == "attention":
            source = mixer.get("kv_from")
            if source is None:
                kept[index] = attention_keys_values(h, w, prefix, mixer, eps, positions)
                source = index
            keys, values = kept[source]
            mixed = attention(h, w, prefix, mixer, eps, positions, keys, values)
        elif layer["type"] == "mamba2":
            mixed = state_space(h, w, prefix, mixer, eps)
        else:
            raise ValueError(f"unknown mixer {layer['type']!r}")
        x = x + norm_one_plus(mixed, w[prefix + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = norm_one_plus(x, w[prefix + "norm2"], eps)
            x = x + norm_one_plus(mixture(h, w, prefix, layer["mlp"]), w[prefix + "norm2b"], eps)
        stream.append(x)
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
    return (logits, stream) if return_layers else logits
