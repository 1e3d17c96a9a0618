"""Dokodra: a decoder whose layers are listed one by one in config.json, each a pre-norm block around one
of three mixers and, optionally, a bounded gated feed-forward.

config.json keys read: ``architecture``, ``width``, ``vocab``, ``embedding.scale``, ``norm.eps``,
``logit_softcap`` and ``layers``: per layer ``type`` (``latent_attention`` | ``latent_attention_2`` |
``mamba2``), ``mixer`` (the mixer's sizes) and ``mlp`` (``{kind: dense, ff, limit}`` or null).

* ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale, rot.{base, dims}``, optional
  ``kv_from: j`` (no down-projection of its own: it reads the cache rows of layer ``j``).
* ``latent_attention_2``: the same with ``q_rank`` (queries through a normed latent) and a sink logit per
  head in the softmax's denominator.
* ``mamba2``: ``heads, vdim, state, groups, conv, norm_groups``.

Every layer norm and the final norm multiply by ``1 + w`` (weights stored around zero) in float32; the
embedding is scaled by a constant; the logits pass ``c * tanh(x / c)``.  Tensor names: ``embed``,
``head``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate, up, down}``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..config.model_config import ConfigError
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

#: constants the design fixes for its dense feed-forward: g * sigmoid(1.702 g) * (u + 1)
FFN_ALPHA = 1.702
FFN_SHIFT = 1.0

ATTENTION_TYPES = ("latent_attention", "latent_attention_2")
LAYER_TYPES = ATTENTION_TYPES + ("mamba2",)


def _need(d: dict[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"{where}: no '{key}'")
    return d[key]


@dataclass
class DokodraConfig:
    hidden_size: int
    vocab_size: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: float
    layers: list[dict[str, Any]] = field(default_factory=list)
    architectures: list[str] = field(default_factory=lambda: ["Dokodra"])

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config") -> "DokodraConfig":
        layers = _need(raw, "layers", where)
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            at = f"{where}: layers[{i}]"
            kind = _need(layer, "type", at)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: {LAYER_TYPES}")
            m = _need(layer, "mixer", at)
            if kind == "mamba2":
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    _need(m, key, at + ".mixer")
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"{at}: groups must divide heads, norm_groups the inner width")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"):
                    _need(m, key, at + ".mixer")
                _need(m["rot"], "base", at + ".mixer.rot")
                _need(m["rot"], "dims", at + ".mixer.rot")
                if kind == "latent_attention_2":
                    _need(m, "q_rank", at + ".mixer")
                src = m.get("kv_from")
                if src is not None:
                    if not (isinstance(src, int) and 0 <= src < i) or layers[src].get("type") not in ATTENTION_TYPES \
                            or layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{at}: kv_from must name an earlier attention layer with a down-projection of its own")
                    theirs = layers[src]["mixer"]
                    if (theirs["kv_rank"], theirs["rot_dim"], theirs["rot"]) != (m["kv_rank"], m["rot_dim"], m["rot"]):
                        raise ConfigError(f"{at}: kv_from layer {src} has another latent size or rotation")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{at}: mlp.kind {mlp.get('kind')!r} is not supported (dense only)")
                _need(mlp, "ff", at + ".mlp")
                _need(mlp, "limit", at + ".mlp")
            out.append({"type": kind, "mixer": dict(m), "mlp": dict(mlp) if mlp is not None else None})
        return cls(hidden_size=int(_need(raw, "width", where)), vocab_size=int(_need(raw, "vocab", where)),
                   embedding_scale=float(_need(_need(raw, "embedding", where), "scale", where + ": embedding")),
                   norm_eps=float(_need(_need(raw, "norm", where), "eps", where + ": norm")),
                   logit_softcap=float(raw.get("logit_softcap") or 0.0), layers=out)


def dokodra_plan(cfg: DokodraConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    norm = lambda tensor, prefix="": PartSpec(      # noqa: E731
        "rmsnorm", {"size": h, "eps": eps, "weight_offset": 1.0, "exact": True, "tensor": tensor}, prefix)
    layers, schedule = [], []
    cache_layer_of: dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "mamba2":
            mixer = PartSpec("ssd", {"hidden": h, "n_heads": m["heads"], "head_dim": m["vdim"], "state": m["state"],
                                     "groups": m["groups"], "conv": m["conv"], "norm_groups": m["norm_groups"], "eps": eps}, "mix.")
        else:
            mixer = PartSpec("latent_attention", {
                "hidden": h, "n_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"],
                "eps": eps, "q_rank": m.get("q_rank", 0) if layer["type"] == "latent_attention_2" else 0,
                "sink": layer["type"] == "latent_attention_2", "own_kv": m.get("kv_from") is None}, "mix.")
        mlp = layer["mlp"]
        ffn = None if mlp is None else PartSpec("glu_bounded", {
            "hidden": h, "intermediate": mlp["ff"], "limit": mlp["limit"], "alpha": FFN_ALPHA, "shift": FFN_SHIFT}, "mlp.")
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm"), norm1=norm("norm1"), mixer=mixer,
                                norm2=None if mlp is None else norm("norm2"), ffn=ffn))
        src = m.get("kv_from") if layer["type"] != "mamba2" else None
        if src is None:
            cache_layer_of[i] = len(cache_layer_of)
            schedule.append(LayerCall(i, cache_layer_of[i]))
        else:
            schedule.append(LayerCall(i, cache_layer_of[src], writes_cache=False))
    return ModelPlan(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": h, "scale": cfg.embedding_scale, "tensor": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("norm", "final."),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "softcap": cfg.logit_softcap, "tensor": "head"}),
        name_prefixes=("",),
    )
