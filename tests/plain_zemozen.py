"""A plain, slow statement of the Zemozen decoder: one function per mechanism, 64-bit arithmetic,
token by token and key by key, its own safetensors reader. It shares no code with the package.

A layer is  x <- x + m * mixer(norm1(x));  x <- x + m * ff(norm2(x))  with RMS norms and one constant m.
The mixer is a windowed softmax attention (heads normed one by one before a half-split rotation with
stretched positions, values blended with those of the first such layer, a sigmoid gate per head), or
two mixers side by side: a windowed attention with interleaved rotation, soft-capped scores and a
softmax whose denominator holds a one, beside a state-space recurrence with a scalar decay per head
(convolution, silu, softplus step, gate, grouped norm). The feed-forward is a routed mixture of gated
experts chosen by softmax scores plus a correction, some of which hand their input through.
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
    """x / sqrt(mean(x^2) + eps) * weight, over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, taps, bias):
    """u [T, C], taps [C, K] with the last column at the current token; zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    out = bias.expand(T, C).clone()
    for t in range(T):
        for j in range(K):
            s = t - (K - 1 - j)
            if s >= 0:
                out[t] += taps[:, j] * u[s]
    return out


# ----------------------------------------------------------------------------- rotation

def rotary_frequencies(rot):
    """One frequency per pair: base^(-2i/dims), all divided by the scaling factor if there is one."""
    dims, base = int(rot["dims"]), float(rot["base"])
    factor = float(rot["scaling"]["factor"]) if rot.get("scaling") else 1.0
    return torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(dims // 2)], dtype=F)


def rotate(x, position, freq, interleaved):
    """x [..., dim]: the first 2 * len(freq) elements rotate; pairs (i, i + half) or (2i, 2i + 1)."""
    half = freq.numel()
    angle = position * freq
    c, s = torch.cos(angle), torch.sin(angle)
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = a * c - b * s
        out[..., 1:2 * half:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:2 * half]
        out[..., :half] = a * c - b * s
        out[..., half:2 * half] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- mixers

def attention_mixer(h, m, w, p, eps, interleaved, v_first=None, values_out=None, one_more=False):
    """h [T, width] of one sequence from position 0. m: the mixer's sizes; w: tensors; p: name prefix.
    `v_first` [T, G, V]: the values to blend in (None: none). `values_out` (a list) receives this layer's
    values as projected. `one_more`: the softmax's denominator holds a one besides the keys' terms. From m: a
    soft cap on the scores where it names one; a gate per head where the tensor exists."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    if values_out is not None:
        values_out.append(v.clone())
    if v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        freq = rotary_frequencies(rot)
        for t in range(T):
            q[t] = rotate(q[t], float(t), freq, interleaved)
            k[t] = rotate(k[t], float(t), freq, interleaved)
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    scale = float(m["scale"])
    cap = float(m["softcap"]) if m.get("softcap") else 0.0
    out = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        first = max(0, t - window + 1) if window else 0
        for a in range(H):
            g = a // (H // G)
            scores = (k[first:t + 1, g] @ q[t, a]) * scale
            if cap:
                scores = cap * torch.tanh(scores / cap)
            if one_more:
                e = torch.exp(scores)
                weights = e / (1.0 + e.sum())
            else:
                weights = torch.softmax(scores, 0)
            out[t, a] = weights @ v[first:t + 1, g]
    if p + "g" in w:
        out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].T


def state_space_mixer(h, m, w, p, eps, state_out=None):
    """The scalar-decay state-space recurrence over one sequence from its start (state zero)."""
    T = h.shape[0]
    H, V, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner, parts = H * V, int(m["norm_groups"])
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                                  # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, V, dtype=F)
    S = torch.zeros(H, N, V, dtype=F)
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = decay[t, a] * S[a] + dt[t, a] * torch.outer(B[t, g], x[t, a])
            y[t, a] = S[a].T @ C[t, g] + w[p + "D"][a] * x[t, a]
    if state_out is not None:
        state_out.append(S.clone())
    y = y.reshape(T, inner) * silu(z)
    y = y.view(T, parts, inner // parts)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return (y.reshape(T, inner) * w[p + "norm"]) @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward

def router(h, f, w, p):
    """Per token: the chosen experts in order of choice, their weights, and the margin of the choice."""
    top, hand_through = int(f["router"]["top"]), int(f["router"].get("identity", 0))
    scores = torch.softmax(h @ w[p + "router"].T, -1)
    choice = scores + w[p + "correction"]
    ranked = torch.sort(choice, dim=-1, descending=True)
    chosen = ranked.indices[:, :top]
    share = torch.gather(scores, 1, chosen)
    share = share / (share.sum(-1, keepdim=True) + 1e-20)
    n = scores.shape[1]
    margin = ranked.values[:, top - 1] - ranked.values[:, top] if top < n else torch.full((h.shape[0],), math.inf, dtype=F)
    return chosen, share, margin, n - hand_through


def routed_ff(h, f, w, p, margins=None):
    chosen, share, margin, real = router(h, f, w, p)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), share[t]):
            if e >= real:
                out[t] += s * h[t]
                continue
            q = p + f"e{e}."
            out[t] += s * ((silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    return out


# ----------------------------------------------------------------------------- the model

def forward(config, w, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence from its first token; `layers_out` (a list) receives the
    stream after every layer, `margins` (a list) every routed layer's margins of choice."""
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    scale = float(config["embedding"]["scale"]) if config.get("embedding") else 1.0
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * scale
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            if m.get("v_mix"):
                got = []
                y = attention_mixer(h, m, w, p + "mix.", eps, False, v_first, got)
                if v_first is None:
                    v_first = got[0]
            else:
                y = attention_mixer(h, m, w, p + "mix.", eps, False)
        elif layer["type"] == "parallel":
            y = float(m["left_scale"]) * attention_mixer(h, m["left"], w, p + "mix.left.", eps, True, one_more=True) + \
                float(m["right_scale"]) * state_space_mixer(h, m["right"], w, p + "mix.right.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * y
        f = layer.get("mlp")
        if f is not None:
            x = x + mult * routed_ff(rms_norm(x, w[p + "norm2"], eps), f, w, p + "mlp.", margins)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


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
