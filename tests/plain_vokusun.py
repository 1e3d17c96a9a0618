"""A plain, slow Vokusun decoder on the CPU: the oracle of the tests.

One function per mechanism, in float64 tensors, with full score matrices and no cache.  It shares no
code with the engine: its own reading of the configuration, its own loops, its own masks.

Notation: ``x`` is the residual stream ``[T, width]``, ``h`` a sublayer's input, ``p`` a position, ``H`` the
query heads, ``G`` the key/value heads, ``d`` a head's query/key size.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w + b over the last axis."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w + b


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def turn_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int, factor: float = 1.0) -> torch.Tensor:
    """Neighbouring pairs (2i, 2i+1) of the first ``dims`` entries of the last axis turned by the angle
    ``p * base**(-2i/dims) / factor``; the rest passes.  ``x`` is ``[T, ..., d]``."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * i / dims) / factor
    ang = positions.to(F)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cs, sn = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cs - v * sn
    out[..., 1:dims:2] = v * cs + u * sn
    return out


def visible(T: int, size: int | None, keep_first: int = 0) -> torch.Tensor:
    """``[T, T]`` booleans: query i sees key j when j <= i and (no window, or i - j < size, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def softmax_rows(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    s = scores.masked_fill(~mask, float("-inf"))
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def window_attention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention whose values are the keys as projected: biases on q and k, a norm per head
    on q and k (one weight for all heads) before the turn, a window that keeps the first tokens."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, d)
    v = k                                                      # before norm and turn
    rot = m["rot"]
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    qn = turn_pairs(unit_rms(q, eps) * w["q.norm"], positions, rot["base"], rot["dims"], factor)
    kn = turn_pairs(unit_rms(k, eps) * w["k.norm"], positions, rot["base"], rot["dims"], factor)
    mask_cfg = m.get("mask") or {}
    mask = visible(T, mask_cfg.get("size"), mask_cfg.get("keep_first", 0))
    out = torch.zeros(T, H, d, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        p = softmax_rows((qn[:, hd] @ kn[:, g].T) * m["scale"], mask)
        out[:, hd] = p @ v[:, g]
    return out.reshape(T, H * d) @ w["o"].T


def latent_attention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    """Attention through a latent: per token a normed latent ``c`` from which every head's unrotated keys and
    values are made, and one turned key part shared by all heads; a sigmoid gate per head on the result."""
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    rot = m["rot"]
    q = (h @ w["q"].T).reshape(T, H, dn + dr)
    down = h @ w["dkv"].T
    c = unit_rms(down[:, :r], eps) * w["dkv.norm"]
    kr = turn_pairs(down[:, r:r + dr], positions, rot["base"], rot["dims"])
    qr = turn_pairs(q[:, :, dn:], positions, rot["base"], rot["dims"])
    kn = (c @ w["uk"].T).reshape(T, H, dn)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(h @ w["g"].T)
    mask = visible(T, None)
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        s = (q[:, hd, :dn] @ kn[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        out[:, hd] = softmax_rows(s, mask) @ v[:, hd]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w["o"].T


def dense_ffn(h: torch.Tensor, w: dict) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def run_order(config: dict) -> list[tuple[int, int | None]]:
    """(layer, pass to enter before it or None) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            out.append((i, t if i == loop["start"] else None))
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """Logits ``[T, vocab]`` of one sequence from position 0 (and the stream after every layer run)."""
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    ln = lambda x, name: layer_norm(x, tensors[name].to(F), tensors[name + ".b"].to(F), eps)   # noqa: E731
    x = tensors["embed"].to(F)[torch.tensor(tokens)]
    x0 = x.clone()
    after = []
    for i, enter in run_order(config):
        if enter is not None:
            x = torch.cat([x, x0], -1) @ tensors["loop.in"].to(F).T + tensors["loop.step"].to(F)[enter]
        layer = config["layers"][i]
        w = sub(tensors, f"l{i}.mix.")
        h = ln(x, f"l{i}.norm1")
        if layer["type"] == "attention":
            y = window_attention(h, w, layer["mixer"], eps, positions)
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, layer["mixer"], eps, positions)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + ln(y, f"l{i}.norm1b")
        if layer.get("mlp") is not None:
            y = dense_ffn(ln(x, f"l{i}.norm2"), sub(tensors, f"l{i}.mlp."))
            x = x + ln(y, f"l{i}.norm2b")
        after.append(x.clone())
    logits = ln(x, "final.norm") @ tensors["head"].to(F).T
    return (logits, torch.stack(after)) if return_layers else logits


# --- random models for the tests --------------------------------------------------------------

def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    W, V = config["width"], config["vocab"]
    out: dict[str, tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "head": (V, W)}
    if config.get("loop"):
        out["loop.in"] = (W, 2 * W)
        out["loop.step"] = (config["loop"]["times"], W)
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        norms = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer.get("mlp") is not None else [])
        for name in norms:
            out[p + name] = (W,)
            out[p + name + ".b"] = (W,)
        if layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,),
                        p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.o": (W, H * d)})
        else:
            H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (dn + dr), W), p + "mix.dkv": (r + dr, W), p + "mix.dkv.norm": (r,),
                        p + "mix.uk": (H * dn, r), p + "mix.uv": (H * dv, r), p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return out


def random_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Seeded weights, rounded to bfloat16 (so that both number formats of the engine see the same values)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if len(shape) == 2 and name != "loop.step":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
            if name.endswith((".mix.q", ".mix.k")):
                t = t * 2.0                                   # sharper scores: a wrong key shows
        elif name.endswith(".b") or name == "loop.step":
            t = 0.2 * torch.randn(shape, generator=gen)
        else:                                                 # norm weights
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        out[name] = t.to(torch.bfloat16)
    return out


def attention_layer(heads=4, kv_heads=2, dim=32, rot_dims=16, size=24, keep_first=3, factor=2.0, base=10000.0, ff=96,
                    scale=None) -> dict:
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5,
                      "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor}},
                      "mask": {"size": size, "keep_first": keep_first}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent_layer(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=32, base=10000.0, ff=96, scale=None) -> dict:
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def make_config(layers: list[dict], width=64, vocab=160, eps=1e-5, loop: dict | None = None) -> dict:
    cfg = {"architecture": "Vokusun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = loop
    return cfg
