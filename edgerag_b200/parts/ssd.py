"""A selective state-space mixer with a scalar decay per head (the "state-space duality" layer).

One input product gives, per token, ``z | x | B | C | dt`` (``inner = heads * head_dim``; B and C have
``groups * state`` entries, dt one per head).  ``x | B | C`` pass a short causal convolution per channel
and silu; then per head ``h`` of group ``g = h // (heads / groups)``, with ``dt = softplus(dt + dt_bias)``:

    S <- exp(-exp(A_log_h) * dt) * S + dt * outer(B_g, x_h)        S: [state, head_dim], float32
    y_h = S^T C_g + D_h * x_h

``y * silu(z)`` is normed to unit RMS in ``norm_groups`` equal pieces of the row, scaled by a weight, and
projected out.  Between steps a request keeps two records in its state slot: the last ``conv - 1`` inputs
of the convolution and ``S`` of every head; a new slot holds zeros, so a sequence starts from nothing,
and a portion of a prompt continues exactly where the one before it stopped.  The decay, the step size,
the state, ``y`` and the norm are float32 whatever the element type.
"""

from __future__ import annotations

import torch

from ..cache.manager import StateSpec
from ..ops import kernels
from .base import LayerCall, Mixer, WeightSpec, register_part


@register_part("mixer", "ssd")
class StateSpaceDuality(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, n_heads: int, head_dim: int, state: int, groups: int, conv: int, norm_groups: int,
                 eps: float, dtype: torch.dtype, device: torch.device) -> None:
        if n_heads % groups or (n_heads * head_dim) % norm_groups or conv < 1:
            raise ValueError("ssd: groups must divide the heads, norm_groups the inner width; conv >= 1")
        self.hidden, self.n_heads, self.head_dim, self.state, self.groups = hidden, n_heads, head_dim, state, groups
        self.taps, self.norm_groups, self.eps = conv, norm_groups, float(eps)
        self.dtype, self.device = dtype, device
        self.inner = n_heads * head_dim
        self.channels = self.inner + 2 * groups * state
        self.in_true = self.inner + self.channels + n_heads
        self.in_width = -(-self.in_true // 8) * 8
        self.w_in = self.w_conv = self.b_conv = self.w_o = None
        self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def cache_spec(self) -> list[StateSpec]:
        return [StateSpec("conv", (self.taps - 1, self.channels)),
                StateSpec("ssm", (self.n_heads, self.state, self.head_dim))]

    def weight_specs(self) -> list[WeightSpec]:
        H = self.n_heads
        return [WeightSpec("in", (self.in_true, self.hidden)), WeightSpec("conv", (self.channels, self.taps)),
                WeightSpec("conv.b", (self.channels,)), WeightSpec("dt_bias", (H,), "vector32"),
                WeightSpec("A_log", (H,), "vector32"), WeightSpec("D", (H,), "vector32"),
                WeightSpec("norm", (self.inner,), "vector32"), WeightSpec("o", (self.hidden, self.inner))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        cast = lambda t: t.to(device=self.device, dtype=self.dtype).contiguous()      # noqa: E731
        f32 = lambda t: t.to(device=self.device, dtype=torch.float32).contiguous()   # noqa: E731
        w_in = cast(tensors["in"])
        if self.in_width > self.in_true:
            pad = torch.zeros((self.in_width - self.in_true, self.hidden), dtype=self.dtype, device=self.device)
            w_in = torch.cat([w_in, pad], 0).contiguous()
        self.w_in = w_in
        self.w_conv, self.b_conv = cast(tensors["conv"]), cast(tensors["conv.b"])
        self.dt_bias, self.a_log, self.d_skip = f32(tensors["dt_bias"]), f32(tensors["A_log"]), f32(tensors["D"])
        self.norm_w = f32(tensors["norm"])
        self.w_o = cast(tensors["o"])

    def forward(self, x: torch.Tensor, ctx, call: LayerCall) -> torch.Tensor:
        n, inner = x.shape[0], self.inner
        proj = ctx.buf("ssd.proj", (n, self.in_width), self.dtype)
        kernels.linear(x, self.w_in, proj)
        conv_state = ctx.state("conv", call.cache_layer)
        xbc = ctx.buf("ssd.xbc", (n, self.channels), self.dtype)
        kernels.conv_silu(proj, inner, self.w_conv, self.b_conv, conv_state, ctx.seq_of_token, ctx.seq_starts,
                          ctx.state_slots, xbc)
        kernels.conv_state_update(proj, inner, conv_state, ctx.n_seqs, ctx.seq_starts, ctx.state_slots)
        y = ctx.buf("ssd.y", (n, inner), torch.float32)
        kernels.ssm_scan(xbc, proj, inner + self.channels, self.dt_bias, self.a_log, self.d_skip,
                         ctx.state("ssm", call.cache_layer), ctx.n_seqs, ctx.seq_starts, ctx.state_slots, y, self.groups)
        normed = ctx.buf("ssd.normed", (n, inner), self.dtype)
        kernels.gated_group_norm(y, self.norm_w, normed, self.eps, self.norm_groups, gate=proj[:, :inner])
        out = ctx.buf("mixer.out", (n, self.hidden), self.dtype)
        kernels.linear(normed, self.w_o, out)
        return out
