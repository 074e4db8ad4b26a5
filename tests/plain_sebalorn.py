"""A plain, slow restatement of the Sebalorn design in PyTorch on the CPU, one function per
mechanism, written from the design's equations and sharing no code with the engine.  Whole
sequences only: no cache and no state handed between calls; every key is recomputed and every
recurrence starts at zero.  `dtype` is the arithmetic type (float64 for an oracle).

Notation: T tokens, W model width, H query heads, G key/value heads; weights are [out, in]
and applied as x @ w.T; positions count from 0.  A layer is x <- x + mixer(n) + ff(n) with
n = unit_rms(x) * (1 + w_norm): one norm feeds both sublayers.  A run of layers may repeat
with the same weights; before each repetition a learned vector is added to x.
"""
from __future__ import annotations

import json
import math
import os

import torch


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x, weight, eps):
    return unit_rms(x, eps) * weight


def norm_around_zero(x, weight, eps):
    return unit_rms(x, eps) * (1.0 + weight)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


# ---- rotations ----------------------------------------------------------------------------

def angles(positions, dims, base, dtype):
    i = torch.arange(dims // 2, dtype=dtype)
    return positions.to(dtype)[:, None] * (base ** (-2.0 * i / dims))[None, :]


def turn_halves(x, positions, dims, base):
    """x [T, heads, n]: of the first `dims` features, feature i pairs with i + dims / 2."""
    if not dims:
        return x
    a = angles(positions, dims, base, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def turn_neighbours(x, positions, dims, base):
    """x [T, heads, n]: of the first `dims` features, feature 2i pairs with 2i + 1."""
    if not dims:
        return x
    a = angles(positions, dims, base, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    return torch.cat([torch.stack([u * c - v * s, v * c + u * s], -1).flatten(-2), x[..., dims:]], -1)


# ---- softmax over the earlier tokens, with or without a term that has no key ----------------

def causal_weights(scores, sink=None):
    """scores [H, T, T] -> weights; row i sees j <= i.  `sink` [H]: exp(sink) joins every row's
    denominator once, unscaled, with no value."""
    t = scores.shape[-1]
    seen = torch.ones(t, t, dtype=torch.bool).tril()
    scores = scores.masked_fill(~seen, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(scores - top)
    total = e.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink[:, None, None] - top)
    return e / total


# ---- mixers ---------------------------------------------------------------------------------

def grouped_attention(h, w, m, eps, prefix):
    """Grouped queries; q and k normed over the WHOLE projection (all heads at once, plain
    weights), then split-half rotation of the first rot.dims features of each head; ordinary
    softmax; every head's result times the sigmoid of one logit."""
    t = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, E = m.get("kv_heads", H), m.get("vdim", D)
    pos = torch.arange(t)
    q = norm_plain(h @ w[prefix + "q"].T, w[prefix + "q.norm"], eps).view(t, H, D)
    k = norm_plain(h @ w[prefix + "k"].T, w[prefix + "k.norm"], eps).view(t, G, D)
    v = (h @ w[prefix + "v"].T).view(t, G, E)
    rot = m.get("rot")
    if rot:
        q = turn_halves(q, pos, rot["dims"], rot["base"])
        k = turn_halves(k, pos, rot["dims"], rot["base"])
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    p = causal_weights(torch.einsum("ihd,jhd->hij", q, k) * m["scale"])
    o = torch.einsum("hij,jhe->ihe", p, v)
    o = o * sigmoid(h @ w[prefix + "g"].T)[:, :, None]
    return o.reshape(t, H * E) @ w[prefix + "o"].T


def latent_attention(h, w, m, eps, prefix):
    """Queries and keys/values through latents; one rotated key part for all heads
    (neighbouring pairs); a sink in the softmax; a gate feature by feature."""
    t = h.shape[0]
    H, D, R, E, C = m["heads"], m["dim"], m["rot_dim"], m.get("vdim", m["dim"]), m["kv_rank"]
    pos = torch.arange(t)
    rot = m.get("rot")
    cq = norm_plain(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
    q = (cq @ w[prefix + "uq"].T).view(t, H, D + R)
    down = h @ w[prefix + "dkv"].T
    c = norm_plain(down[:, :C], w[prefix + "dkv.norm"], eps)
    shared = down[:, C:].view(t, 1, R)
    q_plain, q_rot = q[..., :D], q[..., D:]
    if rot and R:
        q_rot = turn_neighbours(q_rot, pos, rot["dims"], rot["base"])
        shared = turn_neighbours(shared, pos, rot["dims"], rot["base"])
    k_plain = (c @ w[prefix + "uk"].T).view(t, H, D)
    v = (c @ w[prefix + "uv"].T).view(t, H, E)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
              + torch.einsum("ihr,jr->hij", q_rot, shared[:, 0])) * m["scale"]
    p = causal_weights(scores, sink=w[prefix + "sink"])
    o = torch.einsum("hij,jhe->ihe", p, v).reshape(t, H * E)
    o = o * sigmoid(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T


def retention(h, w, m, eps, prefix):
    """Linear attention with a fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T,
    o_t = S_t^T q_t; no softmax, no denominator.  Token by token, the state from zero."""
    t = h.shape[0]
    H, D, E = m["heads"], m["dim"], m.get("vdim", m["dim"])
    pos = torch.arange(t)
    q = (h @ w[prefix + "q"].T).view(t, H, D)
    k = (h @ w[prefix + "k"].T).view(t, H, D)
    v = (h @ w[prefix + "v"].T).view(t, H, E)
    rot = m.get("rot")
    if rot:
        q = turn_halves(q, pos, rot["dims"], rot["base"])
        k = turn_halves(k, pos, rot["dims"], rot["base"])
    k = k * D ** -0.5
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    state = torch.zeros(H, D, E, dtype=h.dtype)
    o = torch.zeros(t, H, E, dtype=h.dtype)
    for i in range(t):
        state = decay[:, None, None] * state + k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hde,hd->he", state, q[i])
    o = unit_rms(o, eps).reshape(t, H * E)
    z = h @ w[prefix + "g"].T
    return (o * (z * sigmoid(z))) @ w[prefix + "o"].T


MIXERS = {"attention": grouped_attention, "latent_attention": latent_attention, "retention": retention}


def dense_feed_forward(h, w, prefix):
    """W_down relu(W_up h)^2."""
    return torch.relu(h @ w[prefix + "up"].T) ** 2 @ w[prefix + "down"].T


# ---- the model ------------------------------------------------------------------------------

def run_list(config):
    """[(layer, number of the pass or None, first of its pass)]: the layers start .. stop - 1
    run `times` times in a row, the rest once."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, None, False) for i in range(start)]
    for t in range(times):
        out += [(i, t, i == start) for i in range(start, stop)]
    return out + [(i, None, False) for i in range(stop, n)]


def forward(config, w, tokens, dtype=torch.float64, residuals=None):
    """Logits [T, vocab] of one whole sequence.  `residuals`: a list that receives x after
    every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    for i, number, first in run_list(config):
        layer = config["layers"][i]
        if first:
            x = x + w["loop.step"][number]
        n = norm_around_zero(x, w[f"l{i}.norm1"], eps)
        y = MIXERS[layer["type"]](n, w, layer["mixer"], eps, f"l{i}.mix.")
        if layer.get("mlp") is not None:
            y = y + dense_feed_forward(n, w, f"l{i}.mlp.")
        x = x + y
        if residuals is not None:
            residuals.append(x.clone())
    z = norm_around_zero(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def load_folder(path):
    """(config, tensors) of a model folder; reads the safetensors container itself."""
    import numpy as np
    with open(os.path.join(path, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype=np.uint8).copy()
        if meta["dtype"] == "BF16":
            t = torch.from_numpy(raw).view(torch.bfloat16)
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(raw).view(torch.float32)
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(raw).view(torch.int32)
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = t.reshape(meta["shape"])
    return config, out


def greedy(config, w, prompt, n, dtype=torch.float64):
    """`n` tokens after `prompt`, each the largest logit (the lowest index on ties); the whole
    sequence is run again for every token."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(torch.argmax(forward(config, w, tokens, dtype)[-1])))
    return tokens[len(prompt):]
