"""Futepel: a decoder whose layers are listed one by one in config.json, each a pre-norm
layer with one of three mixers and a dense or routed feed-forward (or none).

config.json: `vocab`, `width`, `norm.eps`, `max_positions` (rows of the learned position
table), `embedding` = {`scale`, `bigram`: {`buckets`, `mul_prev`, `mul_cur`}} and `layers`, a
list of {`type`, `mixer`, `mlp`}.  Layer types:
  `wkv`: time mixing with a decay per key channel (`heads`, `dim`);
  `latent_attention`: attention over a cached latent (`heads`, `dim`, `rot_dim`, `vdim`,
      `kv_rank`, `scale`, `rot` = {`base`, `dims`, `scaling`: {`factor`, `original`, `fast`,
      `slow`} or absent}), causal over all earlier tokens, with a sigmoid gate per head;
  `mamba2`: the state-space mixer (`heads`, `vdim`, `state`, `groups`, `conv`, `norm_groups`).
`mlp` is null, {`kind`: "dense", `ff`} (activation: squared ReLU) or {`kind`: "moe",
`router`: {`experts`, `top`}, `expert`: {`ff`}, `shared`: {`ff`} or absent}.
Tensors: `embed`, `bigram`, `pos`, `final.norm`, `head`, and per layer i `l<i>.norm1|norm2`,
`l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

import copy
from collections.abc import Mapping as _Mapping
from typing import Any, Mapping

from ..config.model_config import (UNBOUNDED_CONTEXT, ConfigError, EndSpec, FeedForwardSpec, KeyReader,
                                   LayerSpec, MixerSpec, ModelConfig, NormSpec, PositionSpec, RunEntry)
from ..config.registry import Architecture, register_architecture


class _Names(_Mapping):
    """Part-local tensor names to this family's checkpoint names, by rule."""
    _FIXED = {"embedding.table": "embed", "embedding.bigram": "bigram", "embedding.positions": "pos",
              "final_norm.gain": "final.norm", "head.weight": "head"}
    _PREFIXES = (("layer.mixer.", "l{layer}.mix."), ("layer.feed_forward.", "l{layer}.mlp."))
    _NORMS = {"layer.mixer_norm.gain": "l{layer}.norm1", "layer.feed_forward_norm.gain": "l{layer}.norm2"}

    def __getitem__(self, key):
        if key in self._FIXED:
            return self._FIXED[key]
        if key in self._NORMS:
            return self._NORMS[key]
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


def _whole(raw: Mapping[str, Any], key: str, where: str) -> int:
    """An integer that may be zero or negative (a multiplier of a hash)."""
    v = raw.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"{where}: {key!r} must be an integer, got {v!r}")
    return v


def _mixer(kind: str, raw: Mapping[str, Any], width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    if kind == "wkv":
        extra = (("norm_eps", eps),) + ((("decay_rank", r.integer("decay_rank")),) if r.has("decay_rank") else ())
        return MixerSpec(kind="wkv", width=width, n_heads=r.integer("heads"), n_kv_heads=r.integer("heads"),
                         head_dim=r.integer("dim"), extra=extra)
    if kind == "mamba2":
        heads = r.integer("heads")
        return MixerSpec(kind="mamba2", width=width, n_heads=heads, n_kv_heads=r.integer("groups", 1),
                         head_dim=r.integer("state"),
                         extra=(("value_dim", r.integer("vdim")), ("conv_taps", r.integer("conv")),
                                ("norm_groups", r.integer("norm_groups", 1)), ("norm_eps", eps)))
    if kind == "latent_attention":
        rot_dim = r.integer("rot_dim") if r.has("rot_dim") else 0
        position = None
        if rot_dim:
            rot = KeyReader(_section(raw, "rot", where), where + ".rot")
            dims = rot.integer("dims", rot_dim)
            if dims > rot_dim or dims % 2:
                raise ConfigError(f"{where}.rot: 'dims' must be even and at most 'rot_dim' ({rot_dim}), got {dims}")
            scaling = None
            if raw["rot"].get("scaling") is not None:
                sc = KeyReader(_section(raw["rot"], "scaling", where + ".rot"), where + ".rot.scaling")
                scaling = tuple((k, sc.number(k)) for k in ("factor", "original", "fast", "slow"))
            position = PositionSpec(kind="rope_yarn", rotary_dim=dims, theta=rot.number("base"),
                                    max_positions=0, scaling=scaling)
        dim = r.integer("dim")
        return MixerSpec(kind="latent_attention", width=width, n_heads=r.integer("heads"), n_kv_heads=1,
                         head_dim=dim, softmax_scale=r.number("scale"), position=position,
                         extra=(("rot_dim", rot_dim), ("value_dim", r.integer("vdim", dim)),
                                ("kv_rank", r.integer("kv_rank")), ("norm_eps", eps), ("gate", True)))
    raise ConfigError(f"{where}: unknown layer type {kind!r} (this engine runs 'wkv', "
                      f"'latent_attention' and 'mamba2')")


def _feed_forward(mlp, width: int, where: str) -> FeedForwardSpec:
    if mlp is None:
        return FeedForwardSpec(kind="none", width=width, intermediate=0)
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where}: 'mlp' must be an object or null")
    m = KeyReader(mlp, where)
    kind = m.choice("kind", ("dense", "moe"))
    if kind == "dense":
        return FeedForwardSpec(kind="dense_act", width=width, intermediate=m.integer("ff"),
                               extra=(("activation", "relu2"),))
    router = KeyReader(_section(mlp, "router", where), where + ".router")
    expert = KeyReader(_section(mlp, "expert", where), where + ".expert")
    experts, top = router.integer("experts"), router.integer("top")
    if top > experts:
        raise ConfigError(f"{where}.router: 'top' ({top}) exceeds 'experts' ({experts})")
    shared = None
    if mlp.get("shared") is not None:
        shared = KeyReader(_section(mlp, "shared", where), where + ".shared").integer("ff")
    return FeedForwardSpec(kind="moe", width=width, intermediate=expert.integer("ff"),
                           extra=(("experts", experts), ("top", top), ("shared_intermediate", shared)))


def _parse(raw: Mapping[str, Any]) -> ModelConfig:
    r = KeyReader(raw)
    width, vocab = r.integer("width"), r.integer("vocab")
    eps = KeyReader(_section(raw, "norm", "config.json"), "config.json norm").number("eps")
    max_positions = r.integer("max_positions") if r.has("max_positions") else None
    emb = raw.get("embedding") or {}
    if not isinstance(emb, dict):
        raise ConfigError("config.json: 'embedding' must be an object")
    bigram = None
    if emb.get("bigram") is not None:
        b = _section(emb, "bigram", "config.json embedding")
        where = "config.json embedding.bigram"
        bigram = (KeyReader(b, where).integer("buckets"), _whole(b, "mul_prev", where), _whole(b, "mul_cur", where))
    scale = KeyReader(emb, "config.json embedding").number("scale", 1.0)
    entries = raw.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    norm = NormSpec(kind="rmsnorm", width=width, eps=eps)
    layers = []
    for i, entry in enumerate(entries):
        where = f"config.json layers[{i}]"
        if not isinstance(entry, dict) or not isinstance(entry.get("type"), str):
            raise ConfigError(f"{where}: a layer is an object with a 'type'")
        mixer = _mixer(entry["type"], _section(entry, "mixer", where), width, eps, where + ".mixer")
        ffn = _feed_forward(entry.get("mlp"), width, where + ".mlp")
        norms = (("mixer_norm", norm),) + ((("feed_forward_norm", norm),) if ffn.kind != "none" else ())
        layers.append(LayerSpec(arrangement="pre_norm", mixer=mixer, feed_forward=ffn, norms=norms))
    return ModelConfig(
        architecture="Futepel", vocab_size=vocab, hidden_size=width,
        max_context=max_positions if max_positions is not None else UNBOUNDED_CONTEXT,
        tie_word_embeddings=False, layers=tuple(layers),
        run_order=tuple(RunEntry(layer=i) for i in range(len(layers))), final_norm=norm,
        embedding=EndSpec("token_hashed_positions", (("scale", scale), ("bigram", bigram),
                                                     ("max_positions", max_positions))),
        tensor_names=_Names(), raw=copy.deepcopy(dict(raw)))


def _describe(cfg: ModelConfig) -> dict:
    out = copy.deepcopy(dict(cfg.raw))
    out["architecture"] = "Futepel"
    return out


register_architecture(Architecture("Futepel", _parse, _describe))
