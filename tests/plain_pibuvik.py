"""A plain, slow float64 implementation of the Pibuvik decoder, written from its equations.

One function per mechanism, no cache and no batching: the whole sequence is recomputed from
its first token, the recurrent layer token by token. It shares no code with the library; the
tests compare the library's logits and intermediate tensors with it.

Notation: h is a mixer's or feed-forward's input [T, width]; W x means x @ W.T for a matrix
stored [out, in]; positions count from 0.
"""
import json
import math
import os
import struct

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


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def rotate_half(x, positions, dims, base):
    """Rotate the first `dims` dimensions of x [T, ..., n]: dimension i pairs with i + dims/2,
    angle = position * base^(-2i/dims)."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    angle = positions.to(F64)[:, None] * freq[None, :]
    while angle.dim() < x.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- the recurrent mixer
def causal_conv(x, taps, bias):
    """y_t[c] = bias[c] + sum_j taps[c, j] x_(t - (n-1) + j)[c], zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=F64), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(n):
        out = out + padded[j:j + T] * taps[:, j]
    return out + bias


def gated_linear_recurrence(h, w, p, m, decay_factor=8.0):
    """Two branches of `width` channels: y = gelu_tanh(W_y h + b_y), u = conv(W_x h + b_x). Per
    block of channels, gates r = sigmoid(A_b u_b + a_b), i = sigmoid(B_b u_b + b_b);
    a = exp(-decay_factor r softplus(lam)); S_t = a S_(t-1) + sqrt(1 - a^2) i u; out = W_o (S y)."""
    T, width, blocks = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    size = width // blocks
    ub = u.reshape(T, blocks, size)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, width)
    log_a = -decay_factor * r * softplus(w[p + "lam"])
    a = torch.exp(log_a)
    state = torch.zeros(width, dtype=F64)
    out = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        state = a[t] * state + torch.sqrt(1.0 - a[t] ** 2) * (i[t] * u[t])
        out[t] = state
    return (out * y) @ w[p + "o"].T


# --------------------------------------------------------------------------- attention with a sink
def sink_attention(h, w, p, m):
    """Grouped-query causal attention whose values are its keys; no rotation; the query at
    position t is multiplied by 1 + coef ln(floor((t + 1) / every) + 1); the softmax's
    denominator also holds exp(sink_head)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d)
    k = (h @ w[p + "k"].T).reshape(T, G, d)
    temp = m.get("q_temp")
    if temp:
        factor = torch.tensor([1.0 + temp["coef"] * math.log((t + 1) // temp["every"] + 1) for t in range(T)],
                              dtype=F64)
        q = q * factor[:, None, None]
    out = torch.zeros(T, H, d, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        sink = w[p + "sink"][head]
        for t in range(T):
            scores = (k[:t + 1, g] @ q[t, head]) * m["scale"]
            top = torch.maximum(scores.max(), sink)
            e = torch.exp(scores - top)
            out[t, head] = (e[:, None] * k[:t + 1, g]).sum(0) / (e.sum() + torch.exp(sink - top))
    return out.reshape(T, H * d) @ w[p + "o"].T


# --------------------------------------------------------------------------- latent attention
def latent_keys(h, w, p, m, eps):
    """(c [T, kv_rank], rotated shared key part [T, rot_dim]) of a layer with a W_dkv."""
    T = h.shape[0]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :m["kv_rank"]], w[p + "dkv.norm"], eps)
    shared = rotate_half(down[:, m["kv_rank"]:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    return c, shared


def latent_attention(h, w, p, m, eps, kept):
    """Queries through a normed latent; keys and values from the latent c (`kept` = (c, rotated
    key part), this layer's or the layer's it reads from); sliding window; sigmoid gate per head."""
    T = h.shape[0]
    H, d, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, shared = kept
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + r)
    q_plain = q[..., :d]
    q_rot = rotate_half(q[..., d:], torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)
    window = m["mask"]["size"] if "mask" in m else T   # without a mask every earlier position is seen
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        for t in range(T):
            lo = max(0, t - window + 1)
            scores = (k_plain[lo:t + 1, head] @ q_plain[t, head] + shared[lo:t + 1] @ q_rot[t, head]) * m["scale"]
            out[t, head] = torch.softmax(scores, dim=0) @ v[lo:t + 1, head]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forward
def clamped_gate_mlp(h, w, p, f, alpha=1.702):
    g = torch.clamp(h @ w[p + "gate"].T, max=f["limit"])
    u = torch.clamp(h @ w[p + "up"].T, min=-f["limit"], max=f["limit"])
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)) @ w[p + "down"].T


# --------------------------------------------------------------------------- the model
def forward(config, w, tokens, streams=None, float_dtype=F64):
    """Logits [T, vocab] of one sequence; `streams` (a list) receives the residual stream after
    every layer."""
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    kept = {}
    for index, spec in enumerate(config["layers"]):
        p = f"l{index}."
        m = spec["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if spec["type"] == "rglru":
            mixed = gated_linear_recurrence(h, w, p + "mix.", m)
        elif spec["type"] == "attention":
            mixed = sink_attention(h, w, p + "mix.", m)
        elif spec["type"] == "latent_attention":
            if "kv_from" in m:
                source = kept[m["kv_from"]]
            else:
                source = kept[index] = latent_keys(h, w, p + "mix.", m, eps)
            mixed = latent_attention(h, w, p + "mix.", m, eps, source)
        else:
            raise ValueError(spec["type"])
        x = x + mult * rms_norm(mixed, w[p + "norm1b"], eps)
        if spec.get("mlp") is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + mult * rms_norm(clamped_gate_mlp(h, w, p + "mlp.", spec["mlp"]), w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T * config["logit_scale"]
