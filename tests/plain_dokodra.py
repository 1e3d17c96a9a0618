"""A plain, slow Dokodra decoder on the CPU: the oracle of the tests.

One function per mechanism, written from the design's equations in float64 tensors, token by token
where a recurrence is involved and with full score matrices where attention is.  It shares no code
with the engine: its own reading of the configuration, its own loops, no cache (a layer that reads
another layer's latent simply gets that layer's tensors for the whole sequence).

Notation: ``h`` is a mixer's input ``[T, width]``, ``p`` a position, ``H`` the heads, ``dn`` / ``dr``
the unrotated / rotated query-key sizes per head, ``dv`` the value size, ``r`` the latent size.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norm of the design: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def turn_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotate neighbouring pairs (2i, 2i+1) of the first ``dims`` entries of the last axis by
    ``p * base**(-2i/dims)``; ``x`` is ``[T, ..., d]``, ``positions`` ``[T]``."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F)[:, None] * freq[None, :]                     # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cs, sn = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cs - v * sn
    out[..., 1:dims:2] = v * cs + u * sn
    return out


def latent_of(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor):
    """What a layer with a down-projection of its own keeps per token: the normed latent ``[T, r]``
    and the rotated key part ``[T, dr]`` that all heads share."""
    r, dr = m["kv_rank"], m["rot_dim"]
    down = h @ w["dkv"].T
    c = plain_norm(down[:, :r], w["dkv.norm"], eps)
    kr = turn_pairs(down[:, r:r + dr], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor,
                     c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """Attention through a latent: keys and values of every head are made from ``c``; one rotated key
    part ``kr`` serves all heads.  Covers both kinds: queries straight from ``h`` or through a normed
    latent of their own (``dq`` present), softmax with or without a per-head sink (``sink`` present)."""
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    if "dq" in w:
        q = plain_norm(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T
    else:
        q = h @ w["q"].T
    q = q.reshape(T, H, dn + dr)
    qn = q[:, :, :dn]
    qr = turn_pairs(q[:, :, dn:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ w["uk"].T).reshape(-1, H, dn)
    v = (c @ w["uv"].T).reshape(-1, H, dv)
    gate = torch.sigmoid(h @ w["g"].T)                                    # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        for hd in range(H):
            s = (kn[: t + 1, hd] @ qn[t, hd] + kr[: t + 1] @ qr[t, hd]) * m["scale"]
            top = s.max()
            if "sink" in w:
                top = torch.maximum(top, w["sink"][hd])
            e = torch.exp(s - top)
            den = e.sum()
            if "sink" in w:
                den = den + torch.exp(w["sink"][hd] - top)            # a term of the denominator only
            out[t, hd] = (e / den) @ v[: t + 1, hd]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w["o"].T


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def mamba2(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """The state-space mixer, one token after the other from a zero state."""
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    T = h.shape[0]
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F), xbc], 0)
    conv = torch.stack([(padded[t:t + taps] * w["conv"].T).sum(0) for t in range(T)]) + w["conv.b"]
    conv = silu(conv)
    x = conv[:, :inner].reshape(T, H, P)
    B = conv[:, inner:inner + G * N].reshape(T, G, N)
    C = conv[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + w["dt_bias"], threshold=1e9)
    S = torch.zeros(H, N, P, dtype=F)
    y = torch.zeros(T, H, P, dtype=F)
    per_group = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // per_group
            decay = torch.exp(-torch.exp(w["A_log"][hd]) * dt[t, hd])
            S[hd] = decay * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def dense_ffn(h: torch.Tensor, w: dict, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def sub(tensors: dict, prefix: str) -> dict:
    """The tensors below ``prefix`` with the prefix taken off, as float64."""
    return {k[len(prefix):]: v.to(F) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """Logits ``[T, vocab]`` of one sequence from position 0 (and the stream after every layer)."""
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = tensors["embed"].to(F)[torch.tensor(tokens)] * config["embedding"]["scale"]
    kept: dict[int, tuple] = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        m, kind = layer["mixer"], layer["type"]
        w = sub(tensors, f"l{i}.mix.")
        h = offset_norm(x, tensors[f"l{i}.norm1"].to(F), eps)
        if kind in ("latent_attention", "latent_attention_2"):
            if "kv_from" in m:
                c, kr = kept[m["kv_from"]]
            else:
                c, kr = kept[i] = latent_of(h, w, m, eps, positions)
            x = x + latent_attention(h, w, m, eps, positions, c, kr)
        elif kind == "mamba2":
            x = x + mamba2(h, w, m, eps)
        else:
            raise ValueError(f"unknown layer type {kind}")
        if layer.get("mlp") is not None:
            h = offset_norm(x, tensors[f"l{i}.norm2"].to(F), eps)
            x = x + dense_ffn(h, sub(tensors, f"l{i}.mlp."), layer["mlp"]["limit"])
        after.append(x.clone())
    h = offset_norm(x, tensors["final.norm"].to(F), eps)
    logits = h @ tensors["head"].to(F).T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits


# --- random models for the tests --------------------------------------------------------------

def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Names and shapes of a checkpoint of this configuration."""
    W, V = config["width"], config["vocab"]
    out: dict[str, tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out[p + "norm1"] = (W,)
        if layer["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            out.update({p + "mix.in": (2 * inner + 2 * G * N + H, W), p + "mix.conv": (ch, m["conv"]),
                        p + "mix.conv.b": (ch,), p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,),
                        p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
        else:
            H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            if layer["type"] == "latent_attention_2":
                out.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],),
                            p + "mix.uq": (H * (dn + dr), m["q_rank"]), p + "mix.sink": (H,)})
            else:
                out[p + "mix.q"] = (H * (dn + dr), W)
            if "kv_from" not in m:
                out.update({p + "mix.dkv": (r + dr, W), p + "mix.dkv.norm": (r,)})
            out.update({p + "mix.uk": (H * dn, r), p + "mix.uv": (H * dv, r), p + "mix.g": (H, W),
                        p + "mix.o": (W, H * dv)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out.update({p + "norm2": (W,), p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return out


def random_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Seeded weights, rounded to bfloat16 (so that both number formats of the engine see the same values)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[-1] if name[0] == "l" else name
        if len(shape) == 2 and not leaf.endswith("conv"):
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif leaf.endswith("conv"):
            t = torch.randn(shape, generator=gen) * 0.4
        elif leaf.endswith(("dkv.norm", "dq.norm", "mix.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif leaf.endswith("A_log"):
            t = torch.log(0.5 + 3.0 * torch.rand(shape, generator=gen))
        elif leaf.endswith("dt_bias"):
            t = torch.randn(shape, generator=gen) - 1.0
        elif leaf.endswith("D"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif leaf.endswith("sink"):
            t = torch.randn(shape, generator=gen)
        else:                                     # layer norms stored around zero, conv bias
            t = 0.2 * torch.randn(shape, generator=gen)
        out[name] = t.to(torch.bfloat16)
    return out
