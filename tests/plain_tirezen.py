"""Plain, slow Tirezen decoder: whole sequences, no cache, ordinary torch on the CPU.

The oracle of the Tirezen tests.  It shares no code with the ``yalis_b200``
package: it reads ``config.json`` and ``model.safetensors`` itself and computes
every mechanism token by token with explicit loops, one function per mechanism.
All arithmetic runs in the dtype of the weights handed in (float32 or float64).

The design, in this file's notation (h: a layer's normed input, p: position):

* layer:       h = rms(x) * (1 + w_norm);  x <- x + mixer(h) + mlp(h)
* loop:        layers [start, stop) run ``times`` times with the same weights and
               a state of their own per pass; before pass t: x <- x + e (t > 0,
               e = the embedding rows) and then x <- x + step[t]
* retention:   S_p = d_head * S_(p-1) + k_p v_p^T,  o_p = S_p^T q_p, rotary q and k,
               k / sqrt(dim); o / rms(o) * silu(W_g h); W_o
* delta:       short causal convolution + silu on q, k, v; q, k to unit length;
               S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
* parallel:    left_scale * softmax attention (query/key norm, rotary, soft cap,
               one extra 1 in the denominator) + right_scale * delta rule with a
               decay per key channel and low-rank gates
* mlp:         W_down gelu(W_up h), the erf gelu
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List

import torch

_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F64": torch.float64, "I32": torch.int32,
              "I64": torch.int64, "F16": torch.float16}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Every tensor of model.safetensors by name (own reader: 8 bytes of length, a JSON header, raw data)."""
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return out


# ---- small pieces --------------------------------------------------------------------------

def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim], positions 0..T-1: the first rot['dims'] sizes turn, i paired with i + dims/2."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    T = x.shape[0]
    out = x.clone()
    for p in range(T):
        for i in range(half):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[p, :, i].clone(), x[p, :, i + half].clone()
            out[p, :, i] = u * c - v * s
            out[p, :, i + half] = v * c + u * s
    return out


def short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y_t = sum_j taps[:, K-1-j] x_(t-j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            if t - j >= 0:
                y[t] += taps[:, K - 1 - j] * x[t - j]
    return y


# ---- mixers ----------------------------------------------------------------------------------

def retention(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, D)
    k = (h @ w[pre + "k"].T).reshape(T, H, D)
    v = (h @ w[pre + "v"].T).reshape(T, H, V)
    q, k = rotate(q, m["rot"]), rotate(k, m["rot"]) * D ** -0.5
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][hd]) * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = rms(out, eps).reshape(T, H * V) * silu(h @ w[pre + "g"].T)
    return out @ w[pre + "o"].T


def delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """q, k [T, H, D] (already per value head), v [T, H, V], beta [T, H], g [T, H] or [T, H, D]."""
    T, H, D = q.shape
    V = v.shape[2]
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=q.dtype)
        for t in range(T):
            gt = g[t, hd]
            S = S * (gt[:, None] if gt.dim() == 1 else gt)
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, hd])
            S = S + torch.outer(k[t, hd], u)
            out[t, hd] = S.T @ q[t, hd]
    return out


def _delta_inputs(h, w, pre, m):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    per = H // G
    q = q.repeat_interleave(per, dim=1)
    k = k.repeat_interleave(per, dim=1)
    beta = torch.sigmoid(h @ w[pre + "b"].T)
    return q, k, v, beta


def delta(h, w, pre, m, eps) -> torch.Tensor:
    T = h.shape[0]
    H, V = m["heads"], m["vdim"]
    q, k, v, beta = _delta_inputs(h, w, pre, m)
    g = torch.exp(-torch.exp(w[pre + "A_log"]) * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    o = rms(o, eps) * w[pre + "norm"]
    o = o.reshape(T, H * V) * silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def delta_channelwise(h, w, pre, m, eps) -> torch.Tensor:
    """The delta rule with a decay per head and key channel, and low-rank decay and gate projections."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q, k, v, beta = _delta_inputs(h, w, pre, m)
    a = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]
    g = torch.exp(-torch.exp(w[pre + "A_log"])[None, :, None] * softplus(a).reshape(T, H, D))
    o = delta_rule(q, k, v, beta, g)
    o = rms(o, eps) * w[pre + "norm"]
    o = o.reshape(T, H * V) * torch.sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T)
    return o @ w[pre + "o"].T


def capped_sink_attention(h, w, pre, m, eps) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).reshape(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).reshape(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).reshape(T, G, V)
    q = rotate(rms(q, eps) * w[pre + "q.norm"], m["rot"])
    k = rotate(rms(k, eps) * w[pre + "k.norm"], m["rot"])
    cap, scale = float(m["softcap"]), float(m["scale"])
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        for t in range(T):
            s = (k[: t + 1, kv] @ q[t, hd]) * scale
            s = cap * torch.tanh(s / cap)
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[t, hd] = p @ v[: t + 1, kv]
    return out.reshape(T, H * V) @ w[pre + "o"].T


def mixer(kind: str, h, w, pre, m, eps) -> torch.Tensor:
    if kind == "retention":
        return retention(h, w, pre, m, eps)
    if kind == "delta":
        return delta(h, w, pre, m, eps)
    if kind == "parallel":
        left = capped_sink_attention(h, w, pre + "left.", m["left"], eps)
        right = delta_channelwise(h, w, pre + "right.", m["right"], eps)
        return float(m["left_scale"]) * left + float(m["right_scale"]) * right
    raise ValueError(f"unknown mixer {kind!r}")


def mlp(h, w, pre, spec) -> torch.Tensor:
    if spec is None:
        return torch.zeros_like(h)
    assert spec["kind"] == "dense"
    return gelu_erf(h @ w[pre + "up"].T) @ w[pre + "down"].T


# ---- the model -----------------------------------------------------------------------------------

def layer_order(cfg: dict) -> List[tuple]:
    """(layer index, pass number or None, first of its pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    order += [(i, None, False) for i in range(b, n)]
    return order


def forward(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict, layers_out: list = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  ``layers_out`` collects the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    e = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = e.clone()
    for i, t, first in layer_order(cfg):
        if first:
            if t > 0:
                x = x + e
            x = x + w["loop.step"][t]
        L = cfg["layers"][i]
        pre = f"l{i}."
        h = norm_one_plus(x, w[pre + "norm1"], eps)
        x = x + (mixer(L["type"], h, w, pre + "mix.", L["mixer"], eps) + mlp(h, w, pre + "mlp.", L.get("mlp")))
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, w["final.norm"], eps) @ w["head"].T


def greedy(tokens: List[int], n_new: int, w, cfg) -> List[int]:
    seq = list(tokens)
    for _ in range(n_new):
        seq.append(int(forward(seq, w, cfg)[-1].argmax()))
    return seq[len(tokens):]
