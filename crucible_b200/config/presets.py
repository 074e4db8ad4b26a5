"""Named shapes, as config.json dictionaries.

These are data for the benchmark, the command line and the tests, not defaults
of the engine: every one goes through the same `parse_config` as a model
folder's config.json does.  The 120m entry is the reference's `PRESETS["120m"]`
(`model.py:387-391`) with the benchmark's KV-head count, context and epsilon.
"""
from __future__ import annotations


def _crucible(vocab, layers, heads, kv_heads, width, head_dim, inter, ctx, theta, eps, tie):
    label = "mha" if kv_heads == heads else ("mqa" if kv_heads == 1 else "gqa")
    return {
        "architectures": ["CrucibleGPT"], "vocab_size": vocab, "n_layer": layers,
        "n_head": heads, "n_kv_head": kv_heads, "n_embd": width, "head_dim": head_dim,
        "intermediate_size": inter, "block_size": ctx, "dropout": 0.0, "bias": False,
        "attention": label, "pos_encoding": "rope", "activation": "swiglu",
        "norm": "rmsnorm", "norm_placement": "pre", "rope_theta": theta,
        "rms_norm_eps": eps, "tie_word_embeddings": tie,
    }


def _llama(vocab, layers, heads, kv_heads, width, head_dim, inter, ctx, theta, eps, tie):
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": vocab,
        "hidden_size": width, "num_hidden_layers": layers, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter,
        "max_position_embeddings": ctx, "hidden_act": "silu", "rope_theta": theta,
        "rms_norm_eps": eps, "tie_word_embeddings": tie,
    }


SHAPES = {
    "tiny-a": _crucible(256, 2, 4, 2, 64, 16, 176, 128, 10000.0, 1e-5, True),
    "tiny-b": _crucible(509, 3, 3, 1, 96, 32, 320, 192, 500000.0, 1e-6, False),
    "120m": _crucible(50304, 12, 12, 4, 768, 64, 2048, 4096, 10000.0, 1e-5, True),
    "llama-1b": _llama(128256, 16, 32, 8, 2048, 64, 8192, 8192, 500000.0, 1e-5, True),
    "llama-8b": _llama(128256, 32, 32, 8, 4096, 128, 14336, 8192, 500000.0, 1e-5, False),
}


def shape(name: str) -> dict:
    try:
        return dict(SHAPES[name])
    except KeyError:
        raise KeyError(f"unknown shape {name!r}; known: {sorted(SHAPES)}") from None


def vuvosun(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, vocab: int,
            layers: int = 4, window: int = 1024, keep_first: int = 4, streams: int = 4) -> dict:
    """A Vuvosun config.json of a real model's proportions: `layers` layers that alternate
    mLSTM (no feed-forward) and parallel attention + delta rule (dense feed-forward), every
    mixer `heads * head_dim` wide."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
            "scale": head_dim ** -0.5, "rot": {"base": 10000.0, "dims": head_dim // 2},
            "mask": {"size": window, "keep_first": keep_first}}
    right = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "conv": 4}
    parallel = {"type": "parallel", "mlp": {"kind": "dense", "ff": ff},
                "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.7}}
    mlstm = {"type": "mlstm", "mlp": None,
             "mixer": {"heads": heads, "dim": head_dim, "vdim": head_dim, "gate_cap": 15.0}}
    return {"architecture": "Vuvosun", "vocab": vocab, "width": width, "streams": streams,
            "norm": {"eps": 1e-5}, "layers": [mlstm if i % 2 == 0 else parallel for i in range(layers)]}


# sizes at which the two designs are compared: (width, heads, kv heads, head size, ff, vocabulary)
COMPARISON_SIZES = {"w1024": (1024, 8, 2, 128, 2816, 32000), "w2048": (2048, 16, 4, 128, 5632, 32000)}

SHAPES["vuvosun-w1024"] = vuvosun(*COMPARISON_SIZES["w1024"])
SHAPES["vuvosun-w2048"] = vuvosun(*COMPARISON_SIZES["w2048"])


def futepel(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, vocab: int,
            layers: int = 4, experts: int = 8, top: int = 2, max_positions: int = 8192) -> dict:
    """A Futepel config.json of a real model's proportions: `layers` layers that take turns as
    state space + dense feed-forward, wkv + experts, wkv + dense, latent attention + experts;
    every mixer `heads * head_dim` wide (the wkv heads are 64 wide), the latent's cached row
    256 features (192 of latent, 64 rotated), `experts` experts of half the dense width of which
    a token uses `top`, beside a shared one of that width."""
    inner = heads * head_dim
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff // 2},
           "shared": {"ff": ff // 2}}
    mamba = {"type": "mamba2", "mlp": dense,
             "mixer": {"heads": heads, "vdim": head_dim, "state": 128, "groups": max(1, kv_heads // 2),
                       "conv": 4, "norm_groups": 1}}
    wkv = {"type": "wkv", "mixer": {"heads": inner // 64, "dim": 64, "decay_rank": 64}}
    latent = {"type": "latent_attention", "mlp": moe,
              "mixer": {"heads": heads, "dim": head_dim, "rot_dim": 64, "vdim": head_dim, "kv_rank": 192,
                        "scale": (head_dim + 64) ** -0.5,
                        "rot": {"base": 10000.0, "dims": 64,
                                "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}}
    cycle = [mamba, dict(wkv, mlp=moe), dict(wkv, mlp=dense), latent]
    return {"architecture": "Futepel", "vocab": vocab, "width": width, "max_positions": max_positions,
            "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 1000003,
                                                                       "mul_cur": 31}},
            "layers": [cycle[i % 4] for i in range(layers)]}


SHAPES["futepel-w1024"] = futepel(*COMPARISON_SIZES["w1024"])
SHAPES["futepel-w2048"] = futepel(*COMPARISON_SIZES["w2048"])


def nipapel(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, vocab: int,
            layers: int = 4, experts: int = 8, top: int = 2, window: int = 1024, keep_first: int = 8) -> dict:
    """A Nipapel config.json of a real model's proportions: `layers` layers that take turns as
    latent attention + dense feed-forward, attention + experts, latent attention that reads the
    first one's cached rows + experts, attention + dense; every mixer `heads * head_dim` wide,
    the latent's cached row 256 features (192 of latent, 64 rotated), the queries' latent half
    the model's width, `experts` experts of half the dense width of which a token uses `top`."""
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff // 2, "limit": 7.0}}
    latent = {"heads": heads, "dim": head_dim, "rot_dim": 64, "vdim": head_dim, "kv_rank": 192,
              "q_rank": width // 2, "scale": (head_dim + 64) ** -0.5, "rot": {"base": 10000.0, "dims": 64},
              "mask": {"size": window}}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
                 "scale": head_dim ** -0.5, "rot": {"base": 10000.0, "dims": head_dim // 2},
                 "mask": {"size": window, "keep_first": keep_first}}
    out = []
    for i in range(layers):
        if i % 4 == 0:
            out.append({"type": "latent_attention", "mixer": dict(latent), "mlp": dense})
        elif i % 4 == 2:
            out.append({"type": "latent_attention", "mixer": dict(latent, kv_from=i - 2), "mlp": moe})
        else:
            out.append({"type": "attention", "mixer": dict(attention), "mlp": moe if i % 4 == 1 else dense})
    return {"architecture": "Nipapel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": out}


SHAPES["nipapel-w1024"] = nipapel(*COMPARISON_SIZES["w1024"])
SHAPES["nipapel-w2048"] = nipapel(*COMPARISON_SIZES["w2048"])


def sebalorn(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, vocab: int,
             layers: int = 4, passes: int = 1) -> dict:
    """A Sebalorn config.json of a real model's proportions: `layers` layers that take turns as
    attention (q and k normed over the whole projection, a gate per head) + dense feed-forward,
    retention + dense, latent attention with a sink + dense, attention + dense; every mixer
    `heads * head_dim` wide, the latent's cached row 256 features (192 of latent, 64 rotated),
    the queries' latent half the model's width.  Layers 1 and 2 form the repeated run, `passes`
    times (1: every layer runs once, so the model does the work of `layers` layers)."""
    dense = {"kind": "dense", "ff": ff}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim,
                 "scale": head_dim ** -0.5, "rot": {"base": 10000.0, "dims": head_dim // 2}}
    retention = {"heads": heads, "dim": head_dim, "vdim": head_dim,
                 "decay": [1.0 - 2.0 ** (-4 - 0.75 * (i % 8)) for i in range(heads)],
                 "rot": {"base": 10000.0, "dims": head_dim}}
    latent = {"heads": heads, "dim": head_dim, "rot_dim": 64, "vdim": head_dim, "kv_rank": 192,
              "q_rank": width // 2, "scale": (head_dim + 64) ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
    cycle = [("attention", attention), ("retention", retention), ("latent_attention", latent),
             ("attention", attention)]
    out = {"architecture": "Sebalorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
           "embedding": {"scale": float(width) ** 0.5}, "logit_softcap": 50.0,
           "layers": [{"type": cycle[i % 4][0], "mixer": dict(cycle[i % 4][1]), "mlp": dense}
                      for i in range(layers)]}
    if layers >= 3:
        out["loop"] = {"start": 1, "stop": 3, "times": passes}
    return out


SHAPES["sebalorn-w1024"] = sebalorn(*COMPARISON_SIZES["w1024"])
SHAPES["sebalorn-w2048"] = sebalorn(*COMPARISON_SIZES["w2048"])
