"""Small Nipapel configurations for the tests.  They differ from one another in every size
and option: layer order, head counts and groups, key, value and rotated sizes, the latents'
ranks, windows and kept first tokens, which layers read another layer's cached rows (with a
window of their own), dense and routed feed-forwards and layers without one, limits, page
sizes."""
from __future__ import annotations

import os

STD = 0.08       # wider than an initialiser's 0.02, so a wrong key, window or gate moves the logits


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base, size, keep_first, mlp):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if kv_heads is not None:
        mixer["kv_heads"] = kv_heads
    if keep_first is not None:
        mixer["mask"]["keep_first"] = keep_first
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot, vdim, rank, q_rank, scale, base, size, mlp, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
             "scale": scale, "rot": {"base": base, "dims": rot}, "mask": {"size": size}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


CASES = {
    # attention first; a reader whose window is wider than its owner's; a layer without a
    # feed-forward; a second owner with rows of another size (pages of its own)
    "ni-a": dict(seed=3, page_tokens=16, config={
        "architecture": "Nipapel", "vocab": 300, "width": 64, "norm": {"eps": 1e-6},
        "layers": [attention(4, 2, 16, 24, 0.3, 8, 10000.0, 20, 3, moe(6, 2, 40, 1.5)),
                   latent(2, 24, 8, 16, 40, 24, 0.2, 5000.0, 33, dense(96, 0.8)),
                   latent(3, 24, 8, 8, 40, 16, 0.25, 5000.0, 50, moe(6, 2, 40, 1.5), kv_from=1),
                   attention(2, None, 32, 32, 0.2, 32, 500.0, 9, None, None),
                   latent(2, 16, 16, 24, 48, 40, 0.25, 300.0, 12, dense(72, 3.0))]}),
    # a latent layer first and its reader right behind it, then a second reader far away with
    # a narrower window; sizes that are no multiples of 8; one head, one expert of one
    "ni-b": dict(seed=4, page_tokens=8, config={
        "architecture": "Nipapel", "vocab": 211, "width": 44, "norm": {"eps": 1e-5},
        "layers": [latent(1, 10, 6, 14, 21, 9, 0.3, 100.0, 40, moe(1, 1, 20, 0.5)),
                   latent(5, 4, 6, 6, 21, 13, 0.5, 100.0, 40, None, kv_from=0),
                   attention(3, 1, 12, 12, 0.35, 4, 3000.0, 17, 17, dense(52, 1.1)),
                   latent(2, 12, 6, 10, 21, 30, 0.3, 100.0, 7, moe(3, 3, 12, 2.0), kv_from=0)]}),
    # sizes that let the bfloat16 products and both attentions run on the tensor cores
    "ni-c": dict(seed=5, page_tokens=16, config={
        "architecture": "Nipapel", "vocab": 400, "width": 128, "norm": {"eps": 1e-5},
        "layers": [latent(4, 32, 32, 32, 96, 64, 0.15, 9000.0, 70, moe(8, 2, 80, 1.7)),
                   attention(4, 2, 64, 64, 0.11, 48, 40000.0, 70, 5, dense(272, 0.9)),
                   latent(4, 32, 32, 32, 96, 64, 0.15, 9000.0, 70, moe(8, 2, 80, 1.7), kv_from=0)]}),
}


def make_folder(tmp_path, name, config=None, seed=None) -> str:
    from crucible_b200.weights import write_random_model
    out = os.path.join(str(tmp_path), name)
    case = CASES.get(name, {})
    write_random_model(config or case["config"], out, case.get("seed", 0) if seed is None else seed, std=STD)
    return out
