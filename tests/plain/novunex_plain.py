"""Plain, slow forward pass of the Novunex design: whole sequences, no cache, CPU only.

One function per mechanism, written from the design's equations, computing with torch on
the CPU in float64 (or float32).  It shares no code with the product package: it reads
config.json with json and the weights with the `safetensors` library.

Notation: x is the residual stream [T, width] and also what every sublayer reads (this design
has no norm in front of a sublayer, only one behind it); t is a token's index in its sequence
(its position, from 0); W is a weight stored [out, in] and applied as W h.
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


# -- norm -----------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Over the last axis: x / sqrt(mean(x^2) + eps) * w."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


# -- rotary positions --------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> torch.Tensor:
    """f [dims/2] with f_i = base^(-2i/dims).  With `scaling` = (factor, low, high, original) a frequency is judged by its
    wavelength l = 2 pi / f: short ones (l < original/high) stay, long ones (l > original/low) are divided by factor, and
    between the two the frequency slides from one to the other with s = (original/l - low) / (high - low)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f:
            l = 2.0 * math.pi / fi
            if l < original / high:
                out.append(fi)
            elif l > original / low:
                out.append(fi / factor)
            else:
                s = (original / l - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=torch.float64)


def rotate(v: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """v [T, heads, d]: of each head's first 2*len(freqs) entries, entry i and entry i + len(freqs) are a pair (a, b)
    that becomes (a cos - b sin, b cos + a sin) with the angle position * f_i; the other entries stay."""
    half = freqs.shape[0]
    if half == 0:
        return v
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    c, s = torch.cos(ang).to(v.dtype)[:, None, :], torch.sin(ang).to(v.dtype)[:, None, :]
    a, b = v[..., :half], v[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., 2 * half:]], dim=-1)


# -- attention ---------------------------------------------------------------------------------
def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: bool) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query head h reads key/value head h // (H/G); token t
    sees tokens 0..t.  With `sink` the softmax has one more term in its denominator, of score 0 and without a value:
    p_j = exp(s_j) / (1 + sum_j exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, h]) * scale
            m = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - m)
            denom = e.sum() + (math.exp(-m) if sink else 0.0)
            out[t, h] = (e / denom) @ v[:t + 1, g]
    return out


def keys_and_values(x: torch.Tensor, w: dict, p: str, m: dict, kind: str, eps: float, positions: torch.Tensor):
    """What a layer with projections of its own leaves for itself (and for a layer that names it in `kv_from`):
    keys after their norm and rotation, and values."""
    T, G, d, dv = x.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = x @ w[p + "k"].T
    v = (x @ w[p + "v"].T).reshape(T, G, dv)
    if kind == "attention":
        k = rms_norm(k.reshape(T, G, d), w[p + "k.norm"], eps)          # per head, one gain of d entries for all heads
    else:
        k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, d)          # over the whole projection, a gain as wide as it
    rot = m["rot"]
    k = rotate(k, positions, rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling") if kind == "attention_2" else None))
    return k, v


def attention_mixer(x: torch.Tensor, w: dict, p: str, m: dict, kind: str, eps: float, positions: torch.Tensor, kv) -> torch.Tensor:
    """The mixer of one layer; `kv` = (keys, values) as keys_and_values() made them, this layer's or another's."""
    T, H, d = x.shape[0], m["heads"], m["dim"]
    q = x @ w[p + "q"].T
    if kind == "attention":
        q = rms_norm(q.reshape(T, H, d), w[p + "q.norm"], eps)
    else:
        q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)
    rot = m["rot"]
    q = rotate(q, positions, rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling") if kind == "attention_2" else None))
    o = causal_attention(q, kv[0], kv[1], float(m["scale"]), sink=(kind == "attention"))
    return o.reshape(T, -1) @ w[p + "o"].T


# -- feed-forward ---------------------------------------------------------------------------------
def relu_squared_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
    """(chosen [T, top], weights [T, top]): scores are the softmax of the router's outputs over ALL of them; the `top`
    largest of score + correction are chosen; a chosen output's weight is its score, without the correction and without
    renormalising."""
    s = torch.softmax(h @ router.T, dim=-1)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    return chosen, torch.gather(s, -1, chosen)


def mixture(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    """Of the router's outputs the first `experts` name experts with tensors, the last `identity` name experts whose
    output is their input.  A shared expert, if the layer has one, runs for every token with weight 1."""
    r = mlp["router"]
    E = r["experts"]
    chosen, weights = route(h, w[p + "router"], w[p + "correction"], r["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            if e < E:
                out[t] += g * relu_squared_expert(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
            else:
                out[t] += g * h[t]
    if mlp.get("shared"):
        out = out + relu_squared_expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# -- the model ------------------------------------------------------------------------------------
def forward(config: dict, w: dict, tokens: list[int], layers_out: bool = False):
    """Logits [T, vocab] of one sequence; with `layers_out` also the residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    positions = torch.arange(len(tokens))
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        if m.get("kv_from") is None:
            kept[i] = keys_and_values(x, w, p + "mix.", m, kind, eps, positions)
            kv = kept[i]
        else:
            kv = kept[m["kv_from"]]
        x = x + rms_norm(attention_mixer(x, w, p + "mix.", m, kind, eps, positions, kv), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(mixture(x, w, p + "mlp.", layer["mlp"]), w[p + "norm2"], eps)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if layers_out else logits


def greedy(config: dict, weights: dict, prompt, new_tokens: int) -> list:
    toks, out = list(prompt), []
    for _ in range(new_tokens):
        nxt = int(forward(config, weights, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
