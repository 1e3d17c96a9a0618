"""Vokusun: a decoder whose layers are listed one by one in config.json, each a block with a layer norm on
both sides of every sublayer around one of two mixers and, optionally, a gated feed-forward; a run of the
layers may be walked several times with the same weights.

config.json keys read: ``architecture``, ``width``, ``vocab``, ``norm.eps``, ``layers`` and ``loop``.

* per layer: ``type`` (``attention`` | ``latent_attention``), ``mixer`` (the mixer's sizes), ``mlp``
  (``{kind: dense, ff}`` or null).
* ``attention``: ``heads, kv_heads, dim, vdim, scale, rot.{base, dims, scaling.factor}, mask.{size, keep_first}``:
  grouped-query attention with biases on q and k, a unit-RMS norm per head on both (one weight for all heads),
  neighbouring pairs of the first ``rot.dims`` entries turned (angles divided by the scaling factor), values
  that are the keys as projected, and a window of ``mask.size`` that keeps the first ``mask.keep_first`` tokens.
* ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale, rot.{base, dims}``: attention through a
  normed latent with one rotated key part for all heads and a sigmoid gate per head.
* ``loop``: ``{start, stop, times}``: layers ``start .. stop - 1`` run ``times`` times in a row, every pass with a
  cache of its own; before each pass the stream is rewritten as ``W_in [x; x0] + step[t]`` (``x0``: the embedding
  output).

Every norm is a layer norm with weight and bias (``<name>`` and ``<name>.b``); the feed-forward's gate is the
tanh form of gelu.  Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step``,
``l<i>.{norm1, norm1b, norm2, norm2b}``, ``l<i>.mix.*``, ``l<i>.mlp.{gate, up, down}``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..config.model_config import ConfigError
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec, StreamCall

LAYER_TYPES = ("attention", "latent_attention")


def _need(d: Any, key: str, where: str) -> Any:
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"{where}: no '{key}'")
    return d[key]


@dataclass
class VokusunConfig:
    hidden_size: int
    vocab_size: int
    norm_eps: float
    layers: list[dict[str, Any]] = field(default_factory=list)
    #: (start, stop, times) of the looped run of layers, or None
    loop: tuple[int, int, int] | None = None
    architectures: list[str] = field(default_factory=lambda: ["Vokusun"])

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def run_order(self) -> list[tuple[int, int | None]]:
        """(layer, number of the pass that starts right before it, or None) for every layer run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order: list[tuple[int, int | None]] = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config") -> "VokusunConfig":
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
            rot = _need(m, "rot", at + ".mixer")
            for key in ("base", "dims"):
                _need(rot, key, at + ".mixer.rot")
            if kind == "attention":
                for key in ("heads", "kv_heads", "dim", "scale"):
                    _need(m, key, at + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{at}: kv_heads must divide heads")
                if m.get("vdim", m["dim"]) != m["dim"]:
                    raise ConfigError(f"{at}: the values are the keys, so vdim must equal dim")
                if rot["dims"] % 2 or rot["dims"] > m["dim"]:
                    raise ConfigError(f"{at}: rot.dims must be even and at most dim")
                mask = m.get("mask")
                if mask is not None:
                    if int(_need(mask, "size", at + ".mixer.mask")) <= 0 or int(mask.get("keep_first") or 0) < 0:
                        raise ConfigError(f"{at}: mask.size must be positive and mask.keep_first not negative")
                factor = (rot.get("scaling") or {}).get("factor", 1.0)
                if not float(factor) > 0:
                    raise ConfigError(f"{at}: rot.scaling.factor must be positive")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    _need(m, key, at + ".mixer")
                if rot["dims"] % 2 or rot["dims"] > m["rot_dim"] or m["rot_dim"] % 2 or m["kv_rank"] % 2:
                    raise ConfigError(f"{at}: kv_rank, rot_dim and rot.dims must be even, rot.dims at most rot_dim")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{at}: mlp.kind {mlp.get('kind')!r} is not supported (dense only)")
                _need(mlp, "ff", at + ".mlp")
            out.append({"type": kind, "mixer": dict(m), "mlp": dict(mlp) if mlp is not None else None})
        loop = raw.get("loop")
        run = None
        if loop is not None:
            start, stop, times = (int(_need(loop, k, where + ": loop")) for k in ("start", "stop", "times"))
            if not (0 <= start < stop <= len(out)) or times < 1:
                raise ConfigError(f"{where}: loop must name layers start < stop within the stack and times >= 1")
            run = (start, stop, times)
        return cls(hidden_size=int(_need(raw, "width", where)), vocab_size=int(_need(raw, "vocab", where)),
                   norm_eps=float(_need(_need(raw, "norm", where), "eps", where + ": norm")), layers=out, loop=run)


def vokusun_plan(cfg: VokusunConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    norm = lambda tensor, prefix="": PartSpec("layernorm", {"size": h, "eps": eps, "tensor": tensor}, prefix)   # noqa: E731
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        rot = m["rot"]
        if layer["type"] == "attention":
            mask = m.get("mask") or {}
            mixer = PartSpec("attention", {
                "hidden": h, "n_q_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"], "scale": m["scale"],
                "window": int(mask.get("size") or 0), "keep_first": int(mask.get("keep_first") or 0),
                "qk_bias": True, "qk_norm_eps": eps, "values_are_keys": True,
                "position": PartSpec("rope_pairs", {"head_dim": m["dim"], "theta": rot["base"], "rot_dim": rot["dims"],
                                                    "factor": float((rot.get("scaling") or {}).get("factor", 1.0))}),
                "names": {"q": "q", "k": "k", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "q_norm": "q.norm", "k_norm": "k.norm"},
            }, "mix.")
        else:
            mixer = PartSpec("latent_attention", {
                "hidden": h, "n_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "rot_base": rot["base"], "rot_dims": rot["dims"], "eps": eps,
                "gated": True}, "mix.")
        mlp = layer["mlp"]
        ffn = None if mlp is None else PartSpec("glu_bounded", {"hidden": h, "intermediate": mlp["ff"], "act": "gelu_tanh"}, "mlp.")
        block = PartSpec("sandwich", {"post1": norm("norm1b"), "post2": None if mlp is None else norm("norm2b")})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, norm1=norm("norm1"), mixer=mixer,
                                norm2=None if mlp is None else norm("norm2"), ffn=ffn))
    schedule: list[LayerCall | StreamCall] = []
    stream_ops = []
    if cfg.loop is not None:
        stream_ops.append(PartSpec("reentry", {"hidden": h, "passes": cfg.loop[2]}, "loop."))
    for run, (i, enters) in enumerate(cfg.run_order()):
        if enters is not None:
            schedule.append(StreamCall(0, enters))
        schedule.append(LayerCall(i, run))            # every layer run has a cache layer of its own
    return ModelPlan(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": h, "tensor": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("norm", "final."),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "tensor": "head"}),
        stream_ops=stream_ops, name_prefixes=("",),
    )
