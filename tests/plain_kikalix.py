"""A plain, slow float64 implementation of the Kikalix decoder, written from its equations.

One function per mechanism, token by token where the design is recurrent, no cache and no
batching: the whole sequence is recomputed from its first token. It shares no code with the
library; the tests compare the library's logits and intermediate tensors with it.

Notation: h is a mixer's or feed-forward's input [T, width]; W x means x @ W.T for a matrix
stored [out, in]; positions count from 0.
"""
import json
import os
import struct

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- reading a folder
def read_model(folder):
    """(config dict, name -> float64 tensor) of a model folder with one model.safetensors."""
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        (size,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(size))
        data = handle.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        raw = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[entry["dtype"]])
        tensors[name] = raw.reshape(entry["shape"]).to(F64)
    return config, tensors


# --------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm that multiplies by 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


# --------------------------------------------------------------------------- windowed attention with a distance penalty
def distance_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def biased_window_attention(h, w, p, m):
    """Grouped-query softmax attention, no rotation; score_ij = q_i.k_j * scale - slope_h (i - j),
    query i sees keys j with 0 <= i - j < window."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window = m["mask"]["size"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    slopes = distance_slopes(H)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            scores = (k[lo:i + 1, g] @ q[i, head]) * m["scale"]
            scores = scores - slopes[head] * (i - torch.arange(lo, i + 1, dtype=F64))
            weights = torch.softmax(scores, dim=0)
            out[i, head] = weights @ v[lo:i + 1, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# --------------------------------------------------------------------------- gated delta rule
def causal_conv_silu(x, taps):
    """x [T, C], taps [C, n]: y_t = silu(sum_j taps[:, n-1-j] x_(t-j)), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(n):
            if t - j >= 0:
                y[t] += taps[:, n - 1 - j] * x[t - j]
    return silu(y)


def gated_delta_rule(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).reshape(T, G, d)
    k = causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).reshape(T, G, d)
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                     # [T, H]
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, d)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * step)        # [T, H, d]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = unit_rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * dv) @ w[p + "o"].T


# --------------------------------------------------------------------------- retention
def rotate_half(x, positions, dims, base):
    """x [T, heads, d]: the first `dims` dimensions of each head turn, i paired with i + dims/2."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def retention(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = rotate_half((h @ w[p + "q"].T).reshape(T, H, d), positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((h @ w[p + "k"].T).reshape(T, H, d), positions, m["rot"]["dims"], m["rot"]["base"]) * d ** -0.5
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = unit_rms(out, eps).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# --------------------------------------------------------------------------- mixture of experts
def clamped_expert(x, w, p, limit):
    g = torch.clamp(x @ w[p + "gate"].T, max=limit)
    u = torch.clamp(x @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def mixture_of_experts(h, w, p, f):
    experts, top, limit = f["router"]["experts"], f["router"]["top"], f["expert"]["limit"]
    logits = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(logits[t], top).indices
        weights = torch.softmax(logits[t][chosen], dim=0)
        for e, a in zip(chosen.tolist(), weights):
            out[t] += a * clamped_expert(h[t], w, f"{p}e{e}.", limit)
    return out


# --------------------------------------------------------------------------- the decoder
def mixer(kind, h, w, p, m, eps):
    if kind == "retention":
        return retention(h, w, p, m, eps)
    if kind == "parallel":
        left = biased_window_attention(h, w, p + "left.", m["left"])
        right = gated_delta_rule(h, w, p + "right.", m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    raise ValueError(kind)


def layer(x, w, index, spec, eps):
    p = f"l{index}."
    x = x + mixer(spec["type"], offset_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    if spec.get("mlp") is not None:
        x = x + mixture_of_experts(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.", spec["mlp"])
    return x


def layer_runs(config):
    """(layer index, pass number or None) in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(config, w, tokens, streams=None):
    """float64 logits [T, vocab] of one sequence; `streams` (a list) receives the residual stream
    after every layer run."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for index, loop_pass in layer_runs(config):
        if loop_pass is not None:
            x = x + w["loop.step"][loop_pass]
        x = layer(x, w, index, config["layers"][index], eps)
        if streams is not None:
            streams.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T
