"""A plain, slow restatement of the Nipapel design in PyTorch on the CPU, one function per
mechanism, written from the design's equations and sharing no code with the engine.  Whole
sequences only: no cache, nothing handed between calls; every key is recomputed.  `dtype` is
the arithmetic type (float64 for an oracle).

Notation: T tokens, W model width, H query heads, G key/value heads; weights are [out, in]
and applied as x @ w.T; positions count from 0.  A layer is x <- x + mixer(n) + ff(n) with
n = unit_rms(x) * (1 + w_norm): one norm feeds both sublayers.
"""
from __future__ import annotations

import json
import os

import torch


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x, weight, eps):
    """unit rms times the stored weight."""
    return unit_rms(x, eps) * weight


def norm_around_zero(x, weight, eps):
    """unit rms times (1 + the stored weight): the weight is kept around zero."""
    return unit_rms(x, eps) * (1.0 + weight)


# ---- rotations ----------------------------------------------------------------------------

def frequencies(dims, base, dtype):
    i = torch.arange(dims // 2, dtype=dtype)
    return base ** (-2.0 * i / dims)


def turn_split_halves(x, positions, dims, base):
    """x [T, heads, n]: of the first `dims` features, feature i pairs with i + dims/2."""
    half = dims // 2
    ang = positions.to(x.dtype)[:, None] * frequencies(dims, base, x.dtype)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def turn_neighbours(x, positions, dims, base):
    """x [T, heads, n]: of the first `dims` features, feature 2i pairs with 2i + 1."""
    ang = positions.to(x.dtype)[:, None] * frequencies(dims, base, x.dtype)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], -1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], -1)


# ---- masks ----------------------------------------------------------------------------------

def visible(positions, size, keep_first=0):
    """[T, T] bool: row i sees column j when j <= i and (i - j < size or j < keep_first)."""
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def softmax_over_visible(scores, seen):
    """scores [H, T, T]; ordinary softmax over the visible keys of every row."""
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.softmax(scores, -1)


# ---- mixers ---------------------------------------------------------------------------------

def attention(h, w, cfg, eps, positions):
    """Grouped-query attention: per-head RMS norm of q and k (one weight for all heads, plain),
    then the rotation of split halves, a window that keeps the first tokens, softmax, W_o."""
    T = h.shape[0]
    H, G, D = cfg["heads"], cfg.get("kv_heads", cfg["heads"]), cfg["dim"]
    E = cfg.get("vdim", D)
    q = (h @ w["q"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, G, D)
    v = (h @ w["v"].T).view(T, G, E)
    q = norm_plain(q, w["q.norm"], eps)
    k = norm_plain(k, w["k.norm"], eps)
    rot = cfg.get("rot")
    if rot:
        q = turn_split_halves(q, positions, rot["dims"], rot["base"])
        k = turn_split_halves(k, positions, rot["dims"], rot["base"])
    mask = cfg.get("mask") or {}
    seen = visible(positions, mask.get("size"), mask.get("keep_first", 0))
    rep = H // G
    k = k.repeat_interleave(rep, 1)
    v = v.repeat_interleave(rep, 1)
    p = softmax_over_visible(torch.einsum("thd,shd->hts", q, k) * cfg["scale"], seen)
    o = torch.einsum("hts,she->the", p, v).reshape(T, H * E)
    return o @ w["o"].T


def latent_rows(h, w, cfg, eps, positions):
    """What a latent-attention layer leaves for its own and other layers' keys:
    (normed latent [T, rank], rotated shared key part [T, rot_dim])."""
    C, R = cfg["kv_rank"], cfg["rot_dim"]
    both = h @ w["dkv"].T
    c = norm_plain(both[:, :C], w["dkv.norm"], eps)
    part = turn_neighbours(both[:, None, C:], positions, cfg["rot"]["dims"], cfg["rot"]["base"])[:, 0]
    return c, part


def latent_attention(h, w, cfg, eps, positions, rows):
    """`rows`: the (latent, rotated key part) this layer reads: its own or another layer's."""
    T = h.shape[0]
    H, D, R = cfg["heads"], cfg["dim"], cfg["rot_dim"]
    E = cfg.get("vdim", D)
    c, part = rows
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, D + R)
    q_plain = q[..., :D]
    q_turned = turn_neighbours(q[..., D:], positions, cfg["rot"]["dims"], cfg["rot"]["base"])
    k_plain = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, E)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain)
              + torch.einsum("thr,sr->hts", q_turned, part)) * cfg["scale"]
    seen = visible(positions, (cfg.get("mask") or {}).get("size"))
    p = softmax_over_visible(scores, seen)
    o = torch.einsum("hts,she->the", p, v).reshape(T, H * E)
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ---- feed-forwards ----------------------------------------------------------------------------

def capped_glu(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, bias, top):
    """Chosen experts [T, top] (largest logits first) and the softmax over the chosen logits."""
    z = h @ router.T + bias
    best, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(best, -1)


def experts(h, w, cfg):
    top = cfg["router"]["top"]
    idx, weight = route(h, w["router"], w["router.b"], top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += weight[t, j] * capped_glu(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                                cfg["expert"]["limit"])[0]
    return out


def feed_forward(h, w, cfg):
    if cfg is None:
        return torch.zeros_like(h)
    if cfg["kind"] == "dense":
        return capped_glu(h, w["gate"], w["up"], w["down"], cfg["limit"])
    return experts(h, w, cfg)


# ---- the model ----------------------------------------------------------------------------------

def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] for one sequence.  `layers_out`: a list that receives the residual
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    t = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(t))
    x = norm_around_zero(w["embed"][t], w["embed.norm"], eps)
    left = {}
    for i, layer in enumerate(cfg["layers"]):
        n = norm_around_zero(x, w[f"l{i}.norm1"], eps)
        mw, m = sub(w, f"l{i}.mix."), layer["mixer"]
        if layer["type"] == "attention":
            y = attention(n, mw, m, eps, positions)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is not None:
                rows = left[m["kv_from"]]
            else:
                rows = left[i] = latent_rows(n, mw, m, eps, positions)
            y = latent_attention(n, mw, m, eps, positions, rows)
        else:
            raise ValueError(layer["type"])
        x = x + (y + feed_forward(n, sub(w, f"l{i}.mlp."), layer.get("mlp")))
        if layers_out is not None:
            layers_out.append(x)
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T


def read_folder(model_dir):
    """config.json and the tensors of model.safetensors (own reader of the container)."""
    import numpy as np
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = np.frombuffer(data[a:b], dtype=np.uint8)
        if info["dtype"] == "BF16":
            wide = (raw.view("<u2").astype(np.uint32) << 16).view("<f4")
            out[name] = torch.from_numpy(wide.copy()).view(info["shape"])
        elif info["dtype"] == "F32":
            out[name] = torch.from_numpy(raw.view("<f4").copy()).view(info["shape"])
        elif info["dtype"] == "I32":
            out[name] = torch.from_numpy(raw.view("<i4").copy()).view(info["shape"])
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
    return cfg, out


def greedy(cfg, weights, prompt, n_new, dtype=torch.float64):
    """The prompt's continuation by the largest logit (the lower index on ties), the whole
    sequence run again for every token."""
    tokens, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, weights, tokens, dtype)[-1]))
        out.append(nxt)
        tokens.append(nxt)
    return out
