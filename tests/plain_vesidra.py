"""The Vesidra decoder written out plainly: one function per mechanism, whole sequences, float64.

The oracle of the Vesidra tests.  It shares no code with the package: it reads ``config.json`` as a
nested mapping, takes tensors by their checkpoint names and computes every key and value of a
sequence in full (no cache, no absorbed projections, no batching).

Notation: ``h`` is a layer's normed input ``[n, width]``; ``H`` heads; per head ``dim`` unrotated and
``rot_dim`` rotated query/key dimensions, ``vdim`` value dimensions; ``kv_rank`` the latent size.
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


# --------------------------------------------------------------------------- mechanisms


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def rotary_frequencies(rot):
    """(frequencies [dims/2], magnitude) of a rotation ``rot = {base, dims, scaling}``.

    Unscaled: f_i = base^(-2i/dims).  With ``scaling = {factor, original, fast, slow}`` the frequency of pair i
    becomes f_i / factor * ramp_i + f_i * (1 - ramp_i), where ramp runs from 0 at pair ``lo`` to 1 at pair ``hi``
    and lo, hi are the pairs that turn ``fast`` and ``slow`` times within ``original`` positions; cosines and
    sines are multiplied by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return torch.tensor(freqs, dtype=F64), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    scaled = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        scaled.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(scaled, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """Rotates the first ``rot['dims']`` entries of the last dimension of ``x [n, ..., d]``: entry i is paired
    with entry i + dims/2; the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a)."""
    dims = int(rot["dims"])
    half = dims // 2
    freqs, magnitude = rotary_frequencies(rot)
    angles = positions.to(F64)[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = (angles.cos() * magnitude).view(shape), (angles.sin() * magnitude).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def latent_attention(h, w, prefix, mixer, eps, positions, window=None):
    """The mixer on a whole sequence; every token's key and value are recomputed from its latent.  (``window``: a query
    sees only the last ``window`` keys; the design itself has none, the engine's part takes one as an option.)"""
    n = h.shape[0]
    heads, dim, rot_dim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["rot_dim"])
    vdim, rank = int(mixer["vdim"]), int(mixer["kv_rank"])
    q = (h @ w[prefix + "q"].T).view(n, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, mixer["rot"])
    down = h @ w[prefix + "dkv"].T
    latent = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    k_rot = rotate(down[:, rank:], positions, mixer["rot"])                   # one rotated key part for all heads
    k_plain = (latent @ w[prefix + "uk"].T).view(n, heads, dim)
    values = (latent @ w[prefix + "uv"].T).view(n, heads, vdim)
    gate = torch.sigmoid(h @ w[prefix + "g"].T) if prefix + "g" in w else torch.ones(n, heads, dtype=h.dtype)
    visible = positions[None, :] <= positions[:, None]
    if window:
        visible = visible & (positions[None, :] > positions[:, None] - window)
    out = torch.zeros(n, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * float(mixer["scale"])
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, head] = (torch.softmax(scores, dim=-1) @ values[:, head]) * gate[:, head:head + 1]
    return out.reshape(n, heads * vdim) @ w[prefix + "o"].T


def dense_feed_forward(h, w, prefix):
    gate = h @ w[prefix + "gate"].T
    return (gate * torch.sigmoid(gate) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def squared_relu_expert(h, up, down):
    return torch.relu(h @ up.T).pow(2) @ down.T


def routed_feed_forward(h, w, prefix, mlp):
    """Every token goes to the ``top`` experts with the largest router logits, weighted by the softmax over those
    logits alone; a shared expert, if any, is added for every token.  Also returns the smallest gap between the
    last chosen and the first unchosen logit (how far the routing is from a tie)."""
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ w[prefix + "router"].T + w[prefix + "router.b"]
    ranked = logits.sort(dim=-1, descending=True)
    gap = float((ranked.values[:, top - 1] - ranked.values[:, top]).min()) if top < experts else math.inf
    weights = torch.softmax(ranked.values[:, :top], dim=-1)
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(ranked.indices[t, j])
            out[t] += weights[t, j] * squared_relu_expert(h[t:t + 1], w[f"{prefix}e{e}.up"], w[f"{prefix}e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + squared_relu_expert(h, w[prefix + "shared.up"], w[prefix + "shared.down"])
    return out, gap


# --------------------------------------------------------------------------- the model


def forward(tokens, w, config, return_layers=False):
    """float64 logits ``[n, vocab]`` of one whole sequence (and, on request, the residual stream after every layer
    and the smallest routing gap met)."""
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(tokens)] * float(config["embedding"]["scale"])
    eps = float(config["norm"]["eps"])
    streams, gap = [], math.inf
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        h = rms_norm(x, w[prefix + "norm1"], eps)
        if layer["type"] != "latent_attention":
            raise ValueError(f"unknown mixer {layer['type']!r}")
        update = latent_attention(h, w, prefix + "mix.", layer["mixer"], eps, positions)
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] == "dense":
                update = update + dense_feed_forward(h, w, prefix + "mlp.")
            elif mlp["kind"] == "moe":
                routed, layer_gap = routed_feed_forward(h, w, prefix + "mlp.", mlp)
                update, gap = update + routed, min(gap, layer_gap)
            else:
                raise ValueError(f"unknown feed-forward {mlp['kind']!r}")
        x = x + update
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    if return_layers:
        return logits, torch.stack(streams), gap
    return logits
