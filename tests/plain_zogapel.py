"""A plain, slow statement of the Zogapel decoder: one function per mechanism, 64-bit arithmetic,
token by token and key by key, its own safetensors reader. It shares no code with the package.

A layer is  x <- x + post1(mixer(pre1(x)));  x <- x + post2(ff(pre2(x)))  with RMS norms whose
weights are stored around zero. The mixer is a gated delta rule behind short convolutions, or a
windowed softmax attention whose values are its unrotated keys, with partly rotated heads, scaled
frequencies and an output gate. The feed-forward is a two-matrix layer with the tanh form of gelu,
or a routed mixture of gated experts.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F = torch.float64


# ----------------------------------------------------------------------------- reading a folder

def read_safetensors(path) -> dict:
    data = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + n])
    out = {}
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[8 + n + a:8 + n + b]), dtype=kinds[info["dtype"]])
        out[name] = t.reshape(info["shape"]).to(F)
    return out


def read_model(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ----------------------------------------------------------------------------- small pieces

def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + weight), over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + weight)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, taps):
    """u [T, C], taps [C, K] with the last column at the current token; zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(K):
            s = t - (K - 1 - j)
            if s >= 0:
                out[t] += taps[:, j] * u[s]
    return out


# ----------------------------------------------------------------------------- rotation

def rotary_frequencies(rot):
    """One frequency per pair and the factor of cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    scaling = rot.get("scaling")
    if not scaling:
        return torch.tensor(freq, dtype=F), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    fast, slow = float(scaling["fast"]), float(scaling["slow"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(fast)), 0)
    hi = min(math.ceil(dim_of(slow)), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(freq[i] / factor * ramp + freq[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate(x, position, freq, magnitude):
    """x [..., dim]: the first 2 * len(freq) elements rotate, element i with element i + half."""
    half = freq.numel()
    angle = position * freq
    c, s = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    out = x.clone()
    a, b = x[..., :half], x[..., half:2 * half]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- mixers

def attention_mixer(h, m, w, p):
    """h [T, width] of one sequence from position 0. m: the mixer's sizes; w: tensors; p: name prefix."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = k.clone()                                   # the values are the keys as projected
    rot = m.get("rot")
    if rot:
        freq, magnitude = rotary_frequencies(rot)
        for t in range(T):
            q[t] = rotate(q[t], float(t), freq, magnitude)
            k[t] = rotate(k[t], float(t), freq, magnitude)
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    scale = float(m["scale"])
    out = torch.zeros(T, H, D, dtype=F)
    for t in range(T):
        first = max(0, t - window + 1) if window else 0
        for a in range(H):
            g = a // (H // G)
            scores = (k[first:t + 1, g] @ q[t, a]) * scale
            weights = torch.softmax(scores, 0)
            out[t, a] = weights @ v[first:t + 1, g]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * D) * gate) @ w[p + "o"].T


def delta_mixer(h, m, w, p, eps):
    """The gated delta rule over one sequence from its start (state zero)."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                        # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=F)
    S = torch.zeros(H, D, V, dtype=F)
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = decay[t, a] * S[a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, g])
            S[a] = S[a] + torch.outer(k[t, g], u)
            out[t, a] = S[a].T @ q[t, g]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w[p + "norm"]
    return (out * gate).reshape(T, H * V) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forwards

def dense_ff(h, w, p):
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def routed_ff(h, f, w, p, margins=None):
    """`margins` (a list) receives, per token, how far the last chosen logit lies above the first one
    that is not chosen (infinite where every expert is chosen)."""
    experts, top = int(f["router"]["experts"]), int(f["router"]["top"])
    logits = h @ w[p + "router"].T + w[p + "router.b"]
    if margins is not None:
        ranked = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < experts else torch.full((h.shape[0],), math.inf, dtype=F))
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        share = torch.softmax(logits[t, chosen], 0)
        for e, s in zip(chosen.tolist(), share):
            q = p + f"e{e}."
            out[t] += s * ((silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    return out


# ----------------------------------------------------------------------------- the model

def forward(config, w, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence from its first token; `layers_out` (a list) receives the
    stream after every layer, `margins` (a list) every routed layer's margins of choice."""
    eps = float(config["norm"]["eps"])
    scale = float(config.get("embedding", {}).get("scale", 1.0)) if config.get("embedding") else 1.0
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * scale
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(h, layer["mixer"], w, p + "mix.")
        elif layer["type"] == "delta":
            y = delta_mixer(h, layer["mixer"], w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        f = layer.get("mlp")
        if f is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            y = dense_ff(h, w, p + "mlp.") if f.get("kind", "dense") == "dense" else routed_ff(h, f, w, p + "mlp.", margins)
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T


def greedy(config, w, prompt, n_new):
    """The n_new tokens that follow the prompt when the largest logit is taken every time."""
    tokens, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(torch.argmax(forward(config, w, tokens)[-1])))
        tokens.append(out[-1])
    return out


def closest_call(config, w, tokens):
    """Per token, the smallest margin by which any routed layer chose its experts."""
    margins = []
    forward(config, w, tokens, margins=margins)
    if not margins:
        return torch.full((len(tokens),), math.inf, dtype=F)
    return torch.stack(margins).min(dim=0).values
