"""Sebalorn: a decoder whose layers are listed one by one in config.json; every layer has ONE
norm that both of its sublayers read (x += mixer(n) + ff(n), n = norm(x)); every norm's weight
is stored around zero (the gain is 1 + weight); a run of layers may repeat with the same weights.

config.json: `vocab`, `width`, `norm.eps`, `embedding.scale`, `logit_softcap`, `layers` (a list
of {`type`, `mixer`, `mlp`}) and `loop` = {`start`, `stop`, `times`}: the layers start .. stop - 1
run `times` times in a row, each pass with keys and state of its own, and before each pass row t
of the tensor `loop.step` [times, width] is added to the residual.  Layer types:
  `attention`: grouped-query attention (`heads`, `kv_heads`, `dim`, `vdim`, `scale`) whose q and
      k are normed over the whole projection (all heads at once; weights `q.norm`, `k.norm` stored
      as the gains themselves) before the rotation of split halves on the first `rot.dims`
      features of each head (`rot.base`); ordinary softmax over all earlier keys; each head's
      result times the sigmoid of one logit (`g` [heads, width]);
  `latent_attention`: attention over a cached latent (`heads`, `dim`, `rot_dim`, `vdim`,
      `kv_rank`, `scale`, `rot` = {`base`, `dims`}) whose queries go through a latent of their own
      (`q_rank`), with the rotation of neighbouring pairs on the rotated part, a learned sink per
      head in the softmax's denominator, and a sigmoid gate with a logit for every output feature;
  `retention`: linear attention with a fixed decay per head (`heads`, `dim`, `vdim`, `decay`: one
      number a head, `rot`): split-half rotation of q and k, k times dim^-1/2, S <- decay S + k v^T,
      o = S^T q, each head's o divided by its root mean square, times silu(W_g h).
`mlp` is null or {`kind`: "dense", `ff`}: W_down relu(W_up h)^2.  The embedding's rows are
multiplied by `embedding.scale`; the head is a matrix of its own and the logits pass
cap * tanh(logits / cap).  Tensors: `embed`, `loop.step`, `final.norm`, `head`, and per layer i
`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`.  The design names no longest context.
"""
from __future__ import annotations

import copy
from collections.abc import Mapping as _Mapping
from typing import Any, Mapping

from ..config.model_config import (UNBOUNDED_CONTEXT, ConfigError, EndSpec, FeedForwardSpec, KeyReader,
                                   LayerSpec, MixerSpec, ModelConfig, NormSpec, PositionSpec, RunEntry)
from ..config.registry import Architecture, register_architecture

LOOP_VECTORS = "loop_step"      # the model's table of the vectors added before each pass


class _Names(_Mapping):
    """Part-local tensor names to this family's checkpoint names, by rule."""
    _FIXED = {"embedding.table": "embed", "final_norm.gain": "final.norm", "head.weight": "head",
              "layer.norm.gain": "l{layer}.norm1", f"vectors.{LOOP_VECTORS}": "loop.step"}
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


def _count(raw: Mapping[str, Any], key: str, where: str, default=None) -> int:
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


def _attention(raw, width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    dim, heads = r.integer("dim"), r.integer("heads")
    kv_heads = r.integer("kv_heads", heads)
    if heads % kv_heads:
        raise ConfigError(f"{where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    return MixerSpec(kind="sink_attention", width=width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim,
                     softmax_scale=r.number("scale"), window=None,
                     position=_rotation(raw, "rope_halves", dim, where),
                     extra=(("value_dim", r.integer("vdim", dim)), ("keep_first", 0), ("sink", False),
                            ("gate", "head"), ("value_norm_eps", None), ("qk_norm_eps", eps),
                            ("qk_norm_whole", True)))


def _latent(raw, width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    dim, rot_dim = r.integer("dim"), _count(raw, "rot_dim", where)
    if rot_dim % 2:
        raise ConfigError(f"{where}: 'rot_dim' must be even, got {rot_dim}")
    extra = (("rot_dim", rot_dim), ("value_dim", r.integer("vdim", dim)), ("kv_rank", r.integer("kv_rank")),
             ("norm_eps", eps), ("gate", "element"), ("q_rank", r.integer("q_rank")), ("sink", True))
    return MixerSpec(kind="latent_attention", width=width, n_heads=r.integer("heads"), n_kv_heads=1,
                     head_dim=dim, softmax_scale=r.number("scale"), window=None,
                     position=_rotation(raw, "rope_interleaved", rot_dim, where) if rot_dim else None,
                     extra=extra)


def _retention(raw, width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    dim, heads = r.integer("dim"), r.integer("heads")
    decay = raw.get("decay")
    if (not isinstance(decay, list) or len(decay) != heads
            or any(isinstance(x, bool) or not isinstance(x, (int, float)) or not 0.0 <= x <= 1.0 for x in decay)):
        raise ConfigError(f"{where}: 'decay' must list one number in [0, 1] for each of the {heads} heads")
    return MixerSpec(kind="retention", width=width, n_heads=heads, n_kv_heads=heads, head_dim=dim,
                     position=_rotation(raw, "rope_halves", dim, where),
                     extra=(("value_dim", r.integer("vdim", dim)), ("norm_eps", eps),
                            ("decay", tuple(float(x) for x in decay))))


_MIXERS = {"attention": _attention, "latent_attention": _latent, "retention": _retention}


def _feed_forward(mlp, width: int, where: str) -> FeedForwardSpec:
    if mlp is None:
        return FeedForwardSpec(kind="none", width=width, intermediate=0)
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where}: 'mlp' must be an object or null")
    m = KeyReader(mlp, where)
    m.choice("kind", ("dense",))
    return FeedForwardSpec(kind="dense_act", width=width, intermediate=m.integer("ff"),
                           extra=(("activation", "relu2"),))


def _run_order(raw, n_layers: int):
    """(run order, rows of the passes' vectors): the looped layers once per pass, each pass a
    copy with keys and state of its own; the pass's vector is added before its first layer."""
    loop = raw.get("loop")
    if loop is None:
        return tuple(RunEntry(layer=i) for i in range(n_layers)), 0
    where = "config.json loop"
    if not isinstance(loop, dict):
        raise ConfigError(f"{where}: must be an object")
    start, stop = _count(loop, "start", where), _count(loop, "stop", where)
    times = KeyReader(loop, where).integer("times")
    if not start <= stop <= n_layers:
        raise ConfigError(f"{where}: 'start' <= 'stop' <= the number of layers, got {start} and {stop}")
    if start == stop:
        # an empty run: nothing repeats and no vector is ever added (the table is still the model's)
        return tuple(RunEntry(layer=i) for i in range(n_layers)), times
    order = [RunEntry(layer=i) for i in range(start)]
    for t in range(times):
        order += [RunEntry(layer=i, copy=t, add=(LOOP_VECTORS, t) if i == start else None)
                  for i in range(start, stop)]
    order += [RunEntry(layer=i) for i in range(stop, n_layers)]
    return tuple(order), times


def _parse(raw: Mapping[str, Any]) -> ModelConfig:
    r = KeyReader(raw)
    width, vocab = r.integer("width"), r.integer("vocab")
    eps = KeyReader(_section(raw, "norm", "config.json"), "config.json norm").number("eps")
    scale = 1.0
    if raw.get("embedding") is not None:
        scale = KeyReader(_section(raw, "embedding", "config.json"), "config.json embedding").number("scale", 1.0)
    cap = r.number("logit_softcap") if r.has("logit_softcap") else None
    entries = raw.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    norm = NormSpec(kind="rmsnorm_offset", width=width, eps=eps)
    layers = []
    for i, entry in enumerate(entries):
        where = f"config.json layers[{i}]"
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"{where}: a layer is an object with a 'type'")
        kind = entry["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"{where}: unknown layer type {kind!r} (this engine runs {sorted(_MIXERS)})")
        mixer = _MIXERS[kind](_section(entry, "mixer", where), width, eps, where + ".mixer")
        layers.append(LayerSpec(arrangement="parallel", mixer=mixer,
                                feed_forward=_feed_forward(entry.get("mlp"), width, where + ".mlp"),
                                norms=(("norm", norm),)))
    order, times = _run_order(raw, len(layers))
    return ModelConfig(
        architecture="Sebalorn", vocab_size=vocab, hidden_size=width, max_context=UNBOUNDED_CONTEXT,
        tie_word_embeddings=False, layers=tuple(layers), run_order=order, final_norm=norm,
        embedding=EndSpec("token_hashed_positions", (("scale", scale), ("bigram", None), ("max_positions", None))),
        head=EndSpec("linear", (("softcap", cap),)),
        vectors=((LOOP_VECTORS, times),) if times else (),
        tensor_names=_Names(), raw=copy.deepcopy(dict(raw)))


def _describe(cfg: ModelConfig) -> dict:
    out = copy.deepcopy(dict(cfg.raw))
    out["architecture"] = "Sebalorn"
    return out


register_architecture(Architecture("Sebalorn", _parse, _describe))
