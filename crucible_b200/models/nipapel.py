"""Nipapel: a decoder whose layers are listed one by one in config.json; every layer has ONE
norm that both of its sublayers read (x += mixer(n) + ff(n), n = norm(x)), and every norm's
weight is stored around zero (the gain is 1 + weight).

config.json: `vocab`, `width`, `norm.eps` and `layers`, a list of {`type`, `mixer`, `mlp`}.
Layer types:
  `attention`: grouped-query attention (`heads`, `kv_heads`, `dim`, `vdim`, `scale`) with an RMS
      norm of every q and k head (one weight over `dim` for all heads, stored as the gain
      itself), the rotation of split halves on the first `rot.dims` features (`rot.base`), and
      a window `mask.size` that keeps the first `mask.keep_first` tokens visible;
  `latent_attention`: attention over a cached latent (`heads`, `dim`, `rot_dim`, `vdim`,
      `kv_rank`, `scale`, `rot` = {`base`, `dims`}) whose queries go through a latent of their
      own (`q_rank`), with the rotation of neighbouring pairs on the rotated part, a window
      `mask.size`, and a sigmoid gate with a logit for every output feature.  `kv_from`: j
      means the layer has no latent projection of its own and reads the rows layer j cached.
`mlp` is null, {`kind`: "dense", `ff`, `limit`} or {`kind`: "moe", `router`: {`experts`, `top`},
`expert`: {`ff`, `limit`}}: gated feed-forwards with the capped pair g' = min(g, limit),
u' = clamp(u, -limit, limit), y = g' sigmoid(1.702 g') (u' + 1); the router has a bias.
The embedding's rows pass the model's norm; the head is a matrix of its own.
Tensors: `embed`, `embed.norm`, `final.norm`, `head`, and per layer i `l<i>.norm1`,
`l<i>.mix.*`, `l<i>.mlp.*`.  The design names no longest context.
"""
from __future__ import annotations

import copy
from collections.abc import Mapping as _Mapping
from typing import Any, Mapping

from ..config.model_config import (UNBOUNDED_CONTEXT, ConfigError, EndSpec, FeedForwardSpec, KeyReader,
                                   LayerSpec, MixerSpec, ModelConfig, NormSpec, PositionSpec, RunEntry)
from ..config.registry import Architecture, register_architecture

# constants the design fixes: the sigmoid's slope and the offset of the linear half
GLU_ALPHA = 1.702
GLU_OFFSET = 1.0


class _Names(_Mapping):
    """Part-local tensor names to this family's checkpoint names, by rule."""
    _FIXED = {"embedding.table": "embed", "embedding.norm_gain": "embed.norm",
              "final_norm.gain": "final.norm", "head.weight": "head", "layer.norm.gain": "l{layer}.norm1"}
    _PREFIXES = (("layer.mixer.", "l{layer}.mix."), ("layer.feed_forward.", "l{layer}.mlp."))

    def __getitem__(self, key):
        if key in self._FIXED:
            return self._FIXED[key]
        for local, stored in self._PREFIXES:
            if key.startswith(local):
                return stored + key[len(local):]
        raise KeyError(key)

    def __iter__(self):
        return iter(self._FIXED)

    def __len__(self):
        return len(self._FIXED)


def _section(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object")
    return v


def _count(raw: Mapping[str, Any], key: str, where: str, default: int = 0) -> int:
    """An integer that may be zero."""
    v = raw.get(key, default)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"{where}: {key!r} must be a non-negative integer, got {v!r}")
    return v


def _rotation(raw, kind: str, most: int, where: str):
    if raw.get("rot") is None:
        return None
    rot = KeyReader(_section(raw, "rot", where), where + ".rot")
    dims = _count(raw["rot"], "dims", where + ".rot", most)
    if dims % 2 or dims > most:
        raise ConfigError(f"{where}.rot: 'dims' must be even and at most {most}, got {dims}")
    if dims == 0:
        return None
    return PositionSpec(kind=kind, rotary_dim=dims, theta=rot.number("base"), max_positions=0)


def _mask(raw, where: str):
    """(window or None, kept first tokens)."""
    if raw.get("mask") is None:
        return None, 0
    mask = KeyReader(_section(raw, "mask", where), where + ".mask")
    window = mask.integer("size") if mask.has("size") else None
    return window, _count(raw["mask"], "keep_first", where + ".mask")


def _attention(raw, width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    dim, heads = r.integer("dim"), r.integer("heads")
    window, keep_first = _mask(raw, where)
    return MixerSpec(kind="sink_attention", width=width, n_heads=heads, n_kv_heads=r.integer("kv_heads", heads),
                     head_dim=dim, softmax_scale=r.number("scale"), window=window,
                     position=_rotation(raw, "rope_halves", dim, where),
                     extra=(("value_dim", r.integer("vdim", dim)), ("keep_first", keep_first if window else 0),
                            ("sink", False), ("gate", False), ("value_norm_eps", None), ("qk_norm_eps", eps)))


def _latent(raw, width: int, eps: float, where: str, n_before: int):
    """(MixerSpec without its cache window, the layer whose rows it reads or None)."""
    r = KeyReader(raw, where)
    dim, rot_dim = r.integer("dim"), _count(raw, "rot_dim", where)
    window, keep_first = _mask(raw, where)
    if keep_first:
        raise ConfigError(f"{where}.mask: latent attention keeps no first tokens")
    source = raw.get("kv_from")
    if source is not None and (isinstance(source, bool) or not isinstance(source, int)
                               or not 0 <= source < n_before):
        raise ConfigError(f"{where}: 'kv_from' must name an earlier layer, got {source!r}")
    extra = (("rot_dim", rot_dim), ("value_dim", r.integer("vdim", dim)), ("kv_rank", r.integer("kv_rank")),
             ("norm_eps", eps), ("gate", "element"), ("q_rank", r.integer("q_rank")),
             ("reads_other", source is not None))
    spec = MixerSpec(kind="latent_attention", width=width, n_heads=r.integer("heads"), n_kv_heads=1, head_dim=dim,
                     softmax_scale=r.number("scale"), window=window,
                     position=_rotation(raw, "rope_interleaved", rot_dim, where) if rot_dim else None, extra=extra)
    return spec, source


def _feed_forward(mlp, width: int, where: str) -> FeedForwardSpec:
    if mlp is None:
        return FeedForwardSpec(kind="none", width=width, intermediate=0)
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where}: 'mlp' must be an object or null")
    m = KeyReader(mlp, where)
    kind = m.choice("kind", ("dense", "moe"))
    if kind == "dense":
        return FeedForwardSpec(kind="glu_capped", width=width, intermediate=m.integer("ff"),
                               extra=(("limit", m.number("limit")), ("alpha", GLU_ALPHA), ("offset", GLU_OFFSET)))
    router = KeyReader(_section(mlp, "router", where), where + ".router")
    expert = KeyReader(_section(mlp, "expert", where), where + ".expert")
    experts, top = router.integer("experts"), router.integer("top")
    if top > experts:
        raise ConfigError(f"{where}.router: 'top' ({top}) exceeds 'experts' ({experts})")
    return FeedForwardSpec(kind="moe", width=width, intermediate=expert.integer("ff"),
                           extra=(("experts", experts), ("top", top), ("shared_intermediate", None),
                                  ("router_bias", True),
                                  ("pair", (expert.number("limit"), GLU_ALPHA, GLU_OFFSET))))


def _with(spec: MixerSpec, key: str, value) -> MixerSpec:
    from dataclasses import replace
    return replace(spec, extra=tuple((k, v) for k, v in spec.extra if k != key) + ((key, value),))


def _parse(raw: Mapping[str, Any]) -> ModelConfig:
    r = KeyReader(raw)
    width, vocab = r.integer("width"), r.integer("vocab")
    eps = KeyReader(_section(raw, "norm", "config.json"), "config.json norm").number("eps")
    entries = raw.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    norm = NormSpec(kind="rmsnorm_offset", width=width, eps=eps)
    mixers, sources, ffns = [], [], []
    for i, entry in enumerate(entries):
        where = f"config.json layers[{i}]"
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"{where}: a layer is an object with a 'type'")
        kind, mraw = entry["type"], _section(entry, "mixer", where)
        if kind == "attention":
            mixers.append(_attention(mraw, width, eps, where + ".mixer"))
            sources.append(None)
        elif kind == "latent_attention":
            spec, source = _latent(mraw, width, eps, where + ".mixer", i)
            mixers.append(spec)
            sources.append(source)
        else:
            raise ConfigError(f"{where}: unknown layer type {kind!r} (this engine runs 'attention' "
                              f"and 'latent_attention')")
        ffns.append(_feed_forward(entry.get("mlp"), width, where + ".mlp"))
    # a layer that reads another layer's rows: that layer has rows of its own, of the same
    # sizes and rotation; the pages are kept for the widest window among their readers
    keep = {}
    for i, source in enumerate(sources):
        if source is None:
            continue
        where = f"config.json layers[{i}].mixer"
        own, other = mixers[i], mixers[source]
        if other.kind != "latent_attention" or sources[source] is not None:
            raise ConfigError(f"{where}: 'kv_from' must name a latent-attention layer with rows of its own")
        if (own.option("kv_rank"), own.option("rot_dim"), own.position) != \
                (other.option("kv_rank"), other.option("rot_dim"), other.position):
            raise ConfigError(f"{where}: 'kv_rank', 'rot_dim' and 'rot' must equal those of layer {source}")
        keep.setdefault(source, [other.window]).append(own.window)
    for source, windows in keep.items():
        widest = None if any(w is None for w in windows) else max(windows)
        for i in [source] + [j for j, src in enumerate(sources) if src == source]:
            mixers[i] = _with(mixers[i], "cache_window", widest)
    layers = tuple(LayerSpec(arrangement="parallel", mixer=m, feed_forward=f, norms=(("norm", norm),))
                   for m, f in zip(mixers, ffns))
    return ModelConfig(
        architecture="Nipapel", vocab_size=vocab, hidden_size=width, max_context=UNBOUNDED_CONTEXT,
        tie_word_embeddings=False, layers=layers,
        run_order=tuple(RunEntry(layer=i, cache_of=s) for i, s in enumerate(sources)), final_norm=norm,
        embedding=EndSpec("token_normed_streams", (("eps", eps), ("streams", None), ("gain_offset", 1.0))),
        tensor_names=_Names(), raw=copy.deepcopy(dict(raw)))


def _describe(cfg: ModelConfig) -> dict:
    out = copy.deepcopy(dict(cfg.raw))
    out["architecture"] = "Nipapel"
    return out


register_architecture(Architecture("Nipapel", _parse, _describe))
