"""A plain, slow Pikadra: whole sequences, no cache, one function per mechanism.

This file is the tests' oracle for the Pikadra design.  It shares no code with
the package: it reads config.json and the safetensors file itself and computes
with numpy in float64.  The notation, for a sequence of T tokens at positions
0..T-1 (x: the residual stream [T, width], x0: the scaled embedding rows):

  order of layers  the layers before `loop.start` once; then `loop.times` passes over
                   layers start..stop-1 with the same weights, each pass opened by
                   x <- W_in [x ; x0] + step[pass]; then the layers from `loop.stop` on
  layer            h = N(x);  x <- x + (mixer(h) + ff(h))         (both read the same h)
  N(y)             y / sqrt(mean(y^2) + eps) * (1 + w)
  latent attention queries through a normed latent, keys and values from one normed latent per
                   token plus one rotated key part shared by the heads; softmax with a per-head
                   sink in the denominator; a sigmoid gate per head on the result
  feed-forward     down(silu(gate h) * (up h)), dense or as a routed mixture plus a gated shared one
  output           N(x) with the final weight, product with the embedding table, scale, tanh cap
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


def offset_norm(y, w, eps):
    """The norm of the layers: the checkpoint keeps the weight minus one."""
    return rms(y, eps) * (1.0 + w)


def weighted_norm(y, w, eps):
    """The latents' norm: the stored weight is used as it is."""
    return rms(y, eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotate_halves(u, positions, dims, base):
    """u [T, ..., n]: of the first `dims` dimensions, i is paired with i + dims/2 and the pair turned by
    p * base^(-2i/dims); the other dimensions pass unchanged."""
    out = u.copy()
    half = dims // 2
    p = np.asarray(positions, dtype=np.float64).reshape((len(positions),) + (1,) * (u.ndim - 2))
    for i in range(half):
        a = p * base ** (-2.0 * i / dims)
        c, s = np.cos(a), np.sin(a)
        lo, hi = u[..., i], u[..., i + half]
        out[..., i] = lo * c - hi * s
        out[..., i + half] = hi * c + lo * s
    return out


def sink_softmax(scores, sink):
    """scores [T, T] already masked with -inf where a key is not seen; the denominator also holds exp(sink)."""
    m = np.maximum(scores.max(axis=-1, keepdims=True), sink)
    e = np.exp(scores - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def latent_attention(h, w, p, mx, eps, positions=None):
    """h [T, width] -> [T, width]; p is the tensor prefix '<layer>.mix.', mx the mixer's sizes and constants."""
    T = h.shape[0]
    H, d, r, vd, kr = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    rot = mx.get("rot") or {"dims": 0, "base": 1.0}          # no rotated part: nothing is turned
    pos = np.arange(T) if positions is None else np.asarray(positions)
    cq = weighted_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_halves(q[..., d:], pos, rot["dims"], rot["base"])
    dkv = h @ w[p + "dkv"].T
    c = weighted_norm(dkv[:, :kr], w[p + "dkv.norm"], eps)
    k_rot = rotate_halves(dkv[:, kr:], pos, rot["dims"], rot["base"])          # one per token, for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, vd)
    gate = sigmoid(h @ w[p + "g"].T)                                          # [T, H]
    seen = pos[None, :] <= pos[:, None]
    out = np.zeros((T, H, vd))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * mx["scale"]
        s = np.where(seen, s, -np.inf)
        out[:, a] = sink_softmax(s, float(w[p + "sink"][a])) @ v[:, a]
        out[:, a] *= gate[:, a:a + 1]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def gated_unit(h, w, p):
    """down(silu(gate h) * (up h)) with the tensors p + 'gate' / 'up' / 'down'."""
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w_router, top):
    """-> (experts [T, top], weights [T, top]): softmax over all experts, the `top` largest, not renormalised.
    Ties go to the lower index."""
    z = h @ w_router.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def mixture(h, w, p, mlp):
    """The routed experts' weighted sum plus the shared expert times its gate."""
    experts, weights = route(h, w[p + "router"], mlp["router"]["top"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, g in zip(experts[t], weights[t]):
            out[t] += g * gated_unit(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out += gated_unit(h, w, p + "shared.") * sigmoid(h @ w[p + "shared.sg"].T)
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return gated_unit(h, w, p)
    return mixture(h, w, p, mlp)


def layer(x, w, i, spec, eps, positions=None):
    h = offset_norm(x, w[f"l{i}.norm1"], eps)
    y = latent_attention(h, w, f"l{i}.mix.", spec["mixer"], eps, positions)
    if spec.get("mlp") is not None:
        y = y + feed_forward(h, w, f"l{i}.mlp.", spec["mlp"])
    return x + y


def layer_runs(cfg):
    """The order in which layers run: (layer index, pass number or None, whether the pass opens here)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0.copy()
    after = []
    for i, t, opens in layer_runs(cfg):
        if opens:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(x, w, i, cfg["layers"][i], eps)
        after.append(x.copy())
    y = offset_norm(x, w["final.norm"], eps)
    logits = y @ w["embed"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(after)) if return_layers else logits


def greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
