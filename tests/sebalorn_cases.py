"""Small Sebalorn configurations for the tests.  They differ from one another in every size
and option: layer order, which layers repeat and how often, head counts and groups, key, value
and rotated sizes, the latents' ranks, decays, the embedding's scale, the logits' cap, layers
without a feed-forward, page sizes."""
from __future__ import annotations

import os

STD = 0.08       # wider than an initialiser's 0.02, so a wrong key, state or gate moves the logits


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base, mlp):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "scale": scale}
    if kv_heads is not None:
        mixer["kv_heads"] = kv_heads
    if rot_dims is not None:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot, vdim, rank, q_rank, scale, base, mlp):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
             "scale": scale}
    if rot:
        mixer["rot"] = {"base": base, "dims": rot}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def retention(heads, dim, vdim, decay, rot_dims, base, mlp):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims is not None:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "retention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(vocab, width, eps, scale, cap, layers, loop):
    out = {"architecture": "Sebalorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": layers}
    if cap is not None:
        out["logit_softcap"] = cap
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CASES = {
    # the repeated run is in the middle and holds all three mixers; a layer without a feed-forward
    "se-a": dict(seed=3, page_tokens=16, config=model(300, 64, 1e-6, 8.0, 20.0, [
        retention(4, 16, 24, [0.9, 0.99, 1.0, 0.5], 8, 10000.0, dense(96)),
        attention(4, 2, 16, 24, 0.5, 8, 10000.0, dense(80)),
        latent(2, 24, 8, 16, 40, 24, 0.3, 5000.0, None),
        retention(2, 24, 8, [0.97, 0.999], 24, 300.0, dense(72)),
        attention(2, None, 32, 32, 0.4, 32, 500.0, dense(40))], (1, 4, 2))),
    # the repeated run starts at the first layer and runs three times; sizes that are no
    # multiples of 8; one head; no rotation on one layer; no cap on the logits
    "se-b": dict(seed=4, page_tokens=8, config=model(211, 44, 1e-5, 3.5, None, [
        latent(1, 10, 6, 14, 21, 9, 0.4, 100.0, dense(52)),
        retention(3, 10, 6, [0.8, 0.95, 0.9], None, 1.0, None),
        attention(3, 1, 12, 20, 0.6, 4, 3000.0, dense(36)),
        latent(5, 4, 2, 6, 13, 30, 0.7, 50.0, dense(20))], (0, 2, 3))),
    # sizes that let the bfloat16 products and attentions run on the tensor cores; the repeated
    # run is the last layer alone
    "se-c": dict(seed=5, page_tokens=16, config=model(400, 128, 1e-5, 11.3, 50.0, [
        latent(4, 32, 32, 32, 96, 64, 0.2, 9000.0, dense(272)),
        attention(4, 2, 64, 64, 0.2, 48, 40000.0, dense(256)),
        retention(4, 32, 64, [0.9, 0.97, 0.99, 0.999], 16, 7000.0, dense(128))], (2, 3, 2))),
    # no repeated run at all, every mixer once
    "se-d": dict(seed=6, page_tokens=32, config=model(150, 48, 1e-6, 1.0, 5.0, [
        attention(6, 3, 8, 8, 0.9, 8, 77.0, None),
        retention(1, 40, 12, [0.93], 20, 77.0, dense(64)),
        latent(3, 8, 0, 8, 16, 8, 0.5, 1.0, dense(64))], None)),
}


def make_folder(tmp_path, name, config=None, seed=None) -> str:
    from crucible_b200.weights import write_random_model
    out = os.path.join(str(tmp_path), name)
    case = CASES.get(name, {})
    write_random_model(config or case["config"], out, case.get("seed", 0) if seed is None else seed, std=STD)
    return out
