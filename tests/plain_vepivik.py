"""A plain, slow Vepivik: whole sequences, no cache, explicit loops, one function per mechanism.

The oracle of the Vepivik tests.  It shares no code with the package: it reads a model folder with its own
safetensors reader and computes every position from all tokens before it.  ``dtype`` is the arithmetic
(float64 in most tests).

Notation: T tokens, H query heads, G key/value heads, d key size, e value size, r latent size, p rotated size.
"""

from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


def read_folder(path):
    """(config dictionary, name -> float64 tensor) of a model folder."""
    with open(os.path.join(path, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = blob[8 + n + a:8 + n + b]
        kind = info["dtype"]
        if kind == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32).astype(np.float64)
        elif kind == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {kind}")
        tensors[name] = torch.from_numpy(arr.reshape(info["shape"]).copy())
    return config, tensors


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def softmax_rows(z):
    z = z - z.max(dim=-1, keepdim=True).values
    e = torch.exp(z)
    return e / e.sum(dim=-1, keepdim=True)


def windowed_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, H, d], v [T, H, e] (already one key head per query head); position i sees j with
    0 <= i - j < window.  Returns [T, H, e]."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)
        for h in range(H):
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            w = softmax_rows(s[None])[0]
            out[i, h] = w @ v[lo:i + 1, h]
    return out


def attention_mixer(h, t, prefix, m):
    """Grouped-query attention without positions and with a sliding window."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ t[prefix + "q"].T).reshape(T, H, d)
    k = (h @ t[prefix + "k"].T).reshape(T, G, d)
    v = (h @ t[prefix + "v"].T).reshape(T, G, e)
    group = [hh // (H // G) for hh in range(H)]
    o = windowed_attention(q, k[:, group], v[:, group], m["scale"], m["mask"]["size"])
    return o.reshape(T, H * e) @ t[prefix + "o"].T


def rotary_frequencies(rot):
    """Angles per position of the rot['dims'] / 2 pairs, and the factor on cosine and sine."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0

    def dim_of(turns):
        return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(sc["fast"])), 0)
    hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, ..., n]: the first rot['dims'] of the last axis turn, element 2i with element 2i + 1."""
    f, mag = rotary_frequencies(rot)
    out = x.clone()
    for ti, p in enumerate(positions):
        for i, fi in enumerate(f):
            a = p * fi
            c, s = math.cos(a) * mag, math.sin(a) * mag
            u, v = x[ti, ..., 2 * i].clone(), x[ti, ..., 2 * i + 1].clone()
            out[ti, ..., 2 * i] = u * c - v * s
            out[ti, ..., 2 * i + 1] = v * c + u * s
    return out


def latent_of(h, t, prefix, m, eps):
    """The normed latent c [T, r] and the rotated shared key part [T, p] of the layer that owns them."""
    r = m["kv_rank"]
    z = h @ t[prefix + "dkv"].T
    c = rms_norm(z[:, :r], t[prefix + "dkv.norm"], eps)
    kr = rotate_pairs(z[:, r:], range(h.shape[0]), m["rot"])
    return c, kr


def latent_attention_mixer(h, t, prefix, m, eps, latent):
    """Attention whose keys and values are expanded from a latent per token; ``latent`` = (c, kr)."""
    H, d, p, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    c, kr = latent
    q = (h @ t[prefix + "q"].T).reshape(T, H, d + p)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], range(T), m["rot"])
    k_plain = (c @ t[prefix + "uk"].T).reshape(T, H, d)
    v = (c @ t[prefix + "uv"].T).reshape(T, H, e)
    qq = torch.cat([q_plain, q_rot], dim=-1)
    kk = torch.cat([k_plain, kr[:, None, :].expand(T, H, p)], dim=-1)
    o = windowed_attention(qq, kk, v, m["scale"], m["mask"]["size"]).reshape(T, H * e)
    o = o * torch.sigmoid(h @ t[prefix + "g"].T)
    return o @ t[prefix + "o"].T


def expert(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def routing(h, router, top):
    """Chosen experts [T, top] and their weights: softmax over all, the largest ``top``, divided by their sum."""
    s = softmax_rows(h @ router.T)
    chosen = torch.topk(s, top, dim=-1)
    w = chosen.values / (chosen.values.sum(dim=-1, keepdim=True) + 1e-20)
    return chosen.indices, w


def mixture_of_experts(h, t, prefix, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, w = routing(h, t[prefix + "router"], top)
    out = torch.zeros_like(h)
    for ti in range(h.shape[0]):
        for j in range(top):
            e = int(idx[ti, j])
            out[ti] += w[ti, j] * expert(h[ti:ti + 1], t[f"{prefix}e{e}.up"], t[f"{prefix}e{e}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, t[prefix + "shared.up"], t[prefix + "shared.down"])
    return out


def forward(config, tensors, tokens, dtype=torch.float64):
    """(logits [T, vocab], the stream after every layer [L, T, width])."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][torch.tensor(list(tokens))] * config["embedding"]["scale"]
    latents, taps = {}, []
    for i, layer in enumerate(config["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, t[pre + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(h, t, pre + "mix.", m)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                latents[i] = latent_of(h, t, pre + "mix.", m, eps)
            y = latent_attention_mixer(h, t, pre + "mix.", m, eps, latents[m["kv_from"] if m.get("kv_from") is not None else i])
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + mixture_of_experts(rms_norm(x, t[pre + "norm2"], eps), t, pre + "mlp.", layer["mlp"])
        taps.append(x.clone())
    logits = rms_norm(x, t["final.norm"], eps) @ t["embed"].T
    return logits, torch.stack(taps)


def greedy(config, tensors, prompt, n_new, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(n_new):
        logits, _ = forward(config, tensors, tokens, dtype)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]
