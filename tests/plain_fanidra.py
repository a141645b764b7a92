"""A plain, slow Fanidra: whole sequences, no cache, one function per mechanism.

This file is the tests' oracle for the Fanidra design.  It shares no code with
the package: it reads config.json and the safetensors file itself and computes
with numpy in float64, token by token where that is the clearest way to say
what is meant.  The notation, for a sequence of T tokens at positions 0..T-1:

  layer          x <- x + m * N1(mixer(c(x)));  x <- x + m * N2(ff(x))
  N(y)           g * y / sqrt(mean(y^2) + eps), g one number
  c(h)           h + conv(h): a causal convolution over time per channel
  conv(u)_t      sum_j w[:, j] * u[t - taps + 1 + j], zero before the sequence
  attention      two score maps per head over the same values, each a softmax of
                 cap * tanh(scale * q.k / cap) over the keys of the query's own
                 block of positions (blocks of `mask.size`, counted from 0);
                 out = rms(a1 - lam * a2) * (1 - diff)
  hgrn2          S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,  o_t = S_t^T q_t
  feed-forward   down(gelu_tanh(gate h) * (up h))
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_safetensors(path):
    """name -> float64 (or integer) array."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        b, e = rec["data_offsets"]
        raw = data[b:e]
        if rec["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        elif rec["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype=np.float32).astype(np.float64)
        elif rec["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype=np.int32)
        else:
            raise ValueError(f"unexpected tensor type {rec['dtype']}")
        out[name] = arr.reshape(rec["shape"])
    return out


def load_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------

def rms(y, eps):
    """y / sqrt(mean(y^2) + eps) over the last axis."""
    return y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + eps)


def scalar_norm(y, g, eps):
    return rms(y, eps) * float(g)


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u[t - taps + 1 + j], zeros before t = 0."""
    T, taps = u.shape[0], w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotate_pairs(u, positions, dims, base):
    """u [T, ..., dim]: the first `dims` dimensions turned in pairs (2i, 2i+1) by p * base^(-2i/dims)."""
    out = u.copy()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = np.asarray(positions, dtype=np.float64) * f
        shape = (len(positions),) + (1,) * (u.ndim - 2)
        c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
        x, y = u[..., 2 * i], u[..., 2 * i + 1]
        out[..., 2 * i] = x * c - y * s
        out[..., 2 * i + 1] = y * c + x * s
    return out


def diff_lambda(w, p, diff):
    return (math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"])))
            + diff)


def differential_attention(h, w, p, mx, eps):
    """h [T, width] -> [T, width]; p is the tensor prefix '<layer>.mix.', mx the mixer's sizes and constants."""
    q = causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])
    k = causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])
    v = causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])
    rot = mx.get("rot") or {"dims": 0, "base": 1.0}
    out = attend_two_maps(q, k, v, mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"],
                          w[p + "q.norm"], w[p + "k.norm"], eps, rot["dims"], rot["base"], mx["scale"],
                          mx.get("softcap", 0.0), mx["mask"]["size"] if mx.get("mask") else None,
                          diff_lambda(w, p, mx["diff"]), 1.0 - mx["diff"])
    return out @ w[p + "o"].T


def attend_two_maps(q, k, v, H, G, d, dv, q_norm, k_norm, eps, rot_dims, rot_base, scale, cap, block, lam, out_scale):
    """q [T, H*2*d], k [T, G*2*d], v [T, G*dv] after their convolutions -> [T, H*dv]: norm and rotation of the
    queries and keys, the two capped softmax maps per head over the keys of the query's block, their difference,
    the RMS norm of each head's result."""
    T = q.shape[0]
    q = rms(q.reshape(T, H, 2, d), eps) * q_norm
    k = rms(k.reshape(T, G, 2, d), eps) * k_norm
    v = v.reshape(T, G, dv)
    pos = np.arange(T)
    if rot_dims:
        q = rotate_pairs(q, pos, rot_dims, rot_base)
        k = rotate_pairs(k, pos, rot_dims, rot_base)
    out = np.zeros((T, H, dv))
    for t in range(T):
        lo = (t // block) * block if block else 0
        for hd in range(H):
            g = hd // (H // G)
            maps = []
            for a in range(2):
                s = (k[lo:t + 1, g, a] @ q[t, hd, a]) * scale
                if cap:
                    s = cap * np.tanh(s / cap)
                e = np.exp(s - s.max())
                maps.append((e / e.sum()) @ v[lo:t + 1, g])
            out[t, hd] = rms(maps[0] - lam * maps[1], eps) * out_scale
    return out.reshape(T, H * dv)


def hgrn2(h, w, p, mx, eps):
    """h [T, width] -> [T, width]; the state S [heads, dim, vdim] starts at zero."""
    out = gated_recurrence(h @ w[p + "q"].T, h @ w[p + "f"].T, h @ w[p + "v"].T, w[p + "f.b"], w[p + "lower"],
                           w[p + "norm"], mx["heads"], mx["dim"], mx["vdim"], eps)
    return out @ w[p + "o"].T


def gated_recurrence(zq, zf, v, f_bias, lower, norm_w, H, d, dv, eps):
    """zq, zf [T, H*d], v [T, H*dv] (the three projections) -> [T, H*dv]."""
    T = zq.shape[0]
    q = silu(zq).reshape(T, H, d)
    v = v.reshape(T, H, dv)
    f = (lower + (1.0 - lower) * sigmoid(zf + f_bias)).reshape(T, H, d)
    S = np.zeros((H, d, dv))
    out = np.zeros((T, H, dv))
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return (rms(out, eps) * norm_w).reshape(T, H * dv)


def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] for one whole sequence (and the residual stream after every layer)."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = x + causal_conv(x, w[p + "canon1"]) if cfg.get("canon") else x
        if layer["type"] == "attention":
            y = differential_attention(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "hgrn2":
            y = hgrn2(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + m * scalar_norm(y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']}")
            x = x + m * scalar_norm(feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
        layers.append(x.copy())
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(layers)) if return_layers else logits
