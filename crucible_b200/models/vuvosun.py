"""Vuvosun: a decoder whose layers are listed one by one in config.json, each with a
mixer of its own kind, over a residual of several streams (hyper-connections).

config.json: `vocab`, `width`, `norm.eps`, `streams` and `layers`, a list of
{`type`, `mixer`, `mlp`}.  Layer types:
  `parallel`: two mixers side by side on the same input, `mixer.left` (attention with
      a window that keeps the first tokens, a sink, unit-rms values, interleaved rotary
      pairs on the first `rot.dims` features, a sigmoid output gate) and `mixer.right`
      (the gated delta rule with short convolutions), summed with `left_scale` and
      `right_scale`;
  `mlstm`: the matrix memory of the xLSTM with capped exponential gates.
`mlp` is null (the layer has no feed-forward sublayer) or {`kind`: "dense", `ff`}: a
dense feed-forward with the PolyNorm activation.  The embedding's rows pass an RMS
norm; the head is the embedding table.  Tensors: `embed`, `embed.norm`, `final.norm`,
and per layer i `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.hc1|hc2.in|out|mix`.
The design names no longest context.
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
    _FIXED = {"embedding.table": "embed", "embedding.norm_gain": "embed.norm",
              "final_norm.gain": "final.norm"}
    _PREFIXES = (("layer.mixer.", "l{layer}.mix."), ("layer.feed_forward.", "l{layer}.mlp."),
                 ("layer.arrangement.", "l{layer}."))

    def __getitem__(self, key):
        if key in self._FIXED:
            return self._FIXED[key]
        for local, stored in self._PREFIXES:
            if key.startswith(local):
                return stored + key[len(local):]
        if key.startswith("layer.") and key.endswith(".gain"):
            return "l{layer}." + key[len("layer."):-len(".gain")]
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


def _attention(raw: Mapping[str, Any], width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    dim = r.integer("dim")
    position = None
    if raw.get("rot") is not None:
        rot = KeyReader(_section(raw, "rot", where), where + ".rot")
        dims = rot.integer("dims")
        if dims % 2 or dims > dim:
            raise ConfigError(f"{where}.rot: 'dims' must be even and at most 'dim', got {dims}")
        position = PositionSpec(kind="rope_interleaved", rotary_dim=dims, theta=rot.number("base"),
                                max_positions=0)
    window, keep_first = None, 0
    if raw.get("mask") is not None:
        mask = KeyReader(_section(raw, "mask", where), where + ".mask")
        window = mask.integer("size")
        kf = raw["mask"].get("keep_first", 0)
        if isinstance(kf, bool) or not isinstance(kf, int) or kf < 0:
            raise ConfigError(f"{where}.mask: 'keep_first' must be a non-negative integer, got {kf!r}")
        keep_first = kf
    heads = r.integer("heads")
    return MixerSpec(kind="sink_attention", width=width, n_heads=heads,
                     n_kv_heads=r.integer("kv_heads", heads), head_dim=dim,
                     softmax_scale=r.number("scale"), window=window, position=position,
                     extra=(("value_dim", r.integer("vdim", dim)), ("keep_first", keep_first),
                            ("sink", True), ("gate", True), ("value_norm_eps", eps)))


def _delta(raw: Mapping[str, Any], width: int, eps: float, where: str) -> MixerSpec:
    r = KeyReader(raw, where)
    dim, heads = r.integer("dim"), r.integer("heads")
    return MixerSpec(kind="gated_delta", width=width, n_heads=heads,
                     n_kv_heads=r.integer("kv_heads", heads), head_dim=dim,
                     extra=(("value_dim", r.integer("vdim", dim)), ("conv_taps", r.integer("conv")),
                            ("norm_eps", eps)))


def _mixer(kind: str, raw: Mapping[str, Any], width: int, eps: float, where: str) -> MixerSpec:
    if kind == "parallel":
        r = KeyReader(raw, where)
        left = _attention(_section(raw, "left", where), width, eps, where + ".left")
        right = _delta(_section(raw, "right", where), width, eps, where + ".right")
        return MixerSpec(kind="parallel", width=width,
                         extra=(("branches", (("left", left, _plain_number(raw, "left_scale", where)),
                                              ("right", right, _plain_number(raw, "right_scale", where)))),))
    if kind == "mlstm":
        r = KeyReader(raw, where)
        dim, heads = r.integer("dim"), r.integer("heads")
        return MixerSpec(kind="mlstm", width=width, n_heads=heads, n_kv_heads=heads, head_dim=dim,
                         extra=(("value_dim", r.integer("vdim", dim)), ("gate_cap", r.number("gate_cap")),
                                ("norm_eps", eps)))
    raise ConfigError(f"{where}: unknown layer type {kind!r} (this engine runs 'parallel' and 'mlstm')")


def _plain_number(raw, key, where) -> float:
    v = raw.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: {key!r} must be a number, got {v!r}")
    return float(v)


def _parse(raw: Mapping[str, Any]) -> ModelConfig:
    r = KeyReader(raw)
    width, vocab = r.integer("width"), r.integer("vocab")
    eps = KeyReader(_section(raw, "norm", "config.json"), "config.json norm").number("eps")
    streams = r.integer("streams") if r.has("streams") else None
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
        mlp = entry.get("mlp")
        if mlp is None:
            ffn = FeedForwardSpec(kind="none", width=width, intermediate=0)
            norms = (("norm1", norm),)
        else:
            m = KeyReader(mlp, where + ".mlp")
            m.choice("kind", ("dense",))
            ffn = FeedForwardSpec(kind="polynorm", width=width, intermediate=m.integer("ff"),
                                  extra=(("norm_eps", eps),))
            norms = (("norm1", norm), ("norm2", norm))
        layers.append(LayerSpec(arrangement="hyper_connections", mixer=mixer, feed_forward=ffn,
                                norms=norms, extra=(("streams", streams or 1),
                                                    ("learned", streams is not None))))
    return ModelConfig(
        architecture="Vuvosun", vocab_size=vocab, hidden_size=width, max_context=UNBOUNDED_CONTEXT,
        tie_word_embeddings=True, layers=tuple(layers),
        run_order=tuple(RunEntry(layer=i) for i in range(len(layers))), final_norm=norm,
        embedding=EndSpec("token_normed_streams", (("eps", eps), ("streams", streams or 1))),
        tensor_names=_Names(), raw=copy.deepcopy(dict(raw)))


def _describe(cfg: ModelConfig) -> dict:
    out = copy.deepcopy(dict(cfg.raw))
    out["architecture"] = "Vuvosun"
    return out


register_architecture(Architecture("Vuvosun", _parse, _describe))
