"""Plain, slow forward pass of the Pemezen design: whole sequences, no cache, CPU only.

One function per mechanism, written from the design's equations, computing with torch
on the CPU in float64 (or float32).  It shares no code with the product package: it reads
config.json with json and the weights with the `safetensors` library.

Notation: h is what a sublayer reads, x the residual stream, t a token's index in its
sequence (its position, from 0), W a weight stored [out, in] and applied as W h.
"""
from __future__ import annotations

import json
import math
import os

import torch


def read_model(folder: str, dtype=torch.float64):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return config, weights


# -- norms ----------------------------------------------------------------------------------
def grouped_rms_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis is cut into `groups` equal consecutive parts; each part is divided by its own
    sqrt(mean(part^2) + eps); the whole is multiplied by w."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(shape) * w


# -- short causal convolution over time ---------------------------------------------------------
def causal_conv(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start; the last
    column of w multiplies the current token."""
    T, C = h.shape
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    if bias is not None:
        out = out + bias
    return out


# -- rotary positions with YaRN scaling -----------------------------------------------------------
def yarn_frequencies(dims: int, base: float, scaling: dict | None):
    """(f [dims/2], m): the angle of pair i at position p is p * f[i]; cos and sin are multiplied by m."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    fast, slow = float(scaling["fast"]), float(scaling["slow"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=torch.float64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, f: torch.Tensor, m: float, dims: int) -> torch.Tensor:
    """v [T, ..., n]: of the last axis, the first `dims` entries are rotated, (2i, 2i+1) a pair; the rest stay."""
    out = v.clone()
    ang = positions.to(torch.float64)[:, None] * f[None, :]              # [T, dims/2]
    cos, sin = (torch.cos(ang) * m).to(v.dtype), (torch.sin(ang) * m).to(v.dtype)
    while cos.dim() < v.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


# -- latent attention ---------------------------------------------------------------------------------
def latent_attention(h: torch.Tensor, W: dict, mixer: dict, gate: str | None, eps: float, window: int = 0,
                     return_weights: bool = False) -> torch.Tensor:
    """h [T, width] of ONE sequence from position 0.  W: this mixer's tensors by their short names.
    gate: "element" (sigmoid(W_g h) has one entry per output channel), "head" (one per head) or None.
    window > 0: position t sees only the keys s with t - window < s <= t (the design itself has none)."""
    T = h.shape[0]
    H, dim, rot, vdim, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    pos = torch.arange(T)
    q = (h @ W["q"].T).reshape(T, H, dim + rot)
    down = h @ W["dkv"].T
    c = down[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * W["dkv.norm"]
    k_rot = down[:, rank:]
    f, m = yarn_frequencies(mixer["rot"]["dims"], mixer["rot"]["base"], mixer["rot"].get("scaling"))
    q_rot = rotate_pairs(q[..., dim:], pos, f, m, mixer["rot"]["dims"])
    k_rot = rotate_pairs(k_rot, pos, f, m, mixer["rot"]["dims"])
    k = (c @ W["uk"].T).reshape(T, H, dim)
    v = (c @ W["uv"].T).reshape(T, H, vdim)
    scores = (torch.einsum("thd,shd->hts", q[..., :dim], k) + torch.einsum("thd,sd->hts", q_rot, k_rot)) * mixer["scale"]
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible = visible & (pos[None, :] > pos[:, None] - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    if return_weights:
        return p
    out = torch.einsum("hts,shd->thd", p, v)
    if gate is not None:
        g = torch.sigmoid(h @ W["g"].T)
        out = out * (g.reshape(T, H, vdim) if gate == "element" else g.reshape(T, H, 1))
    return out.reshape(T, H * vdim) @ W["o"].T


# -- the recurrent block with a real-gated linear recurrent unit ------------------------------------------
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rglru(h: torch.Tensor, W: dict, mixer: dict) -> torch.Tensor:
    T = h.shape[0]
    width, blocks = mixer["width"], mixer["blocks"]
    bw = width // blocks
    y = gelu_tanh(h @ W["y"].T + W["y.b"])
    u = causal_conv(h @ W["x"].T + W["x.b"], W["conv"], W["conv.b"])
    ub = u.reshape(T, blocks, bw)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W["ra"], ub) + W["ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W["ri"], ub) + W["ri.b"]).reshape(T, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(W["lam"])
    a = torch.exp(log_a)
    S = torch.zeros(width, dtype=h.dtype)
    out = torch.zeros(T, width, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W["o"].T


# -- feed-forward ----------------------------------------------------------------------------------------
def xielu(z: torch.Tensor, p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    sp = torch.nn.functional.softplus
    pos = sp(p) * z * z + z / 2
    neg = (0.5 + sp(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(h: torch.Tensor, W: dict) -> torch.Tensor:
    return xielu(h @ W["up"].T, W["act"][0], W["act"][1]) @ W["down"].T


# -- the model -----------------------------------------------------------------------------------------------
def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer)."""
    dtype = weights["embed"].dtype
    groups, eps = config["norm"]["groups"], config["norm"]["eps"]
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    norm = lambda v, name: grouped_rms_norm(v, weights[name], groups, eps)
    after = []
    for l, layer in enumerate(config["layers"]):
        p = f"l{l}."
        h = norm(x, p + "norm1")
        h = h + causal_conv(h, weights[p + "canon1"])
        kind = layer["type"]
        if kind == "latent_attention":
            m = latent_attention(h, sub(weights, p + "mix."), layer["mixer"], "element", eps)
        elif kind == "latent_attention_2":
            m = latent_attention(h, sub(weights, p + "mix."), layer["mixer"], "head", eps)
        elif kind == "rglru":
            m = rglru(h, sub(weights, p + "mix."), layer["mixer"])
        else:
            raise ValueError(kind)
        x = x + norm(m, p + "norm1b")
        if layer.get("mlp") is not None:
            h = norm(x, p + "norm2")
            h = h + causal_conv(h, weights[p + "canon2"])
            x = x + norm(dense_ff(h, sub(weights, p + "mlp.")), p + "norm2b")
        after.append(x.clone())
    logits = norm(x, "final.norm") @ weights["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(config: dict, weights: dict, prompt, new_tokens: int) -> list:
    toks, out = list(prompt), []
    for _ in range(new_tokens):
        nxt = int(forward(config, weights, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
