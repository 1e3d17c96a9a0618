"""Re-entry into a run of layers that is walked several times with the same weights.

Before each pass ``t`` over the run (the first too) the stream is rewritten from itself and the embedding
output ``x0`` of the step's tokens:

    x <- W_in [x ; x0] + step[t]

``W_in`` is ``[width, 2 width]`` (the stream's columns first), ``step`` one vector per pass.  The product runs
in the model's element type with float32 accumulation on the rounded stream; the sum with ``step[t]`` is
float32 and becomes the new stream.  ``x0`` is kept for the step in the right half of the product's input
buffer, written once after the embedding; each pass only rewrites the left half, in the same kernel that
adds (and, where a norm closes the sublayer, norms) the update still pending from the layer before.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import NormedUpdate, StreamCall, StreamOp, WeightSpec, register_part, settle_update


@register_part("stream", "reentry")
class ReEntry(StreamOp):
    graph_safe = True

    def __init__(self, hidden: int, passes: int, dtype: torch.dtype, device: torch.device, in_tensor: str = "in",
                 step_tensor: str = "step") -> None:
        self.hidden, self.passes = hidden, int(passes)
        self.dtype, self.device = dtype, device
        self.in_tensor, self.step_tensor = in_tensor, step_tensor
        self.w_in: torch.Tensor | None = None
        self.step: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.in_tensor, (self.hidden, 2 * self.hidden)),
                WeightSpec(self.step_tensor, (self.passes, self.hidden), kind="vector32")]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.w_in = tensors[self.in_tensor].to(device=self.device, dtype=self.dtype).contiguous()
        self.step = tensors[self.step_tensor].to(device=self.device, dtype=torch.float32).contiguous()

    def _pair(self, ctx) -> torch.Tensor:
        return ctx.buf("reentry.pair", (ctx.n_tokens, 2 * self.hidden), self.dtype)

    def begin(self, ctx, hidden: torch.Tensor) -> None:
        kernels.cast_rows(hidden, self._pair(ctx)[:, self.hidden:])

    def forward(self, hidden, delta, ctx, call: StreamCall):
        if not 0 <= call.index < self.passes:
            raise ValueError(f"re-entry {call.index} of {self.passes} passes")
        pair = self._pair(ctx)
        left = pair[:, : self.hidden]
        closing = delta.norm if isinstance(delta, NormedUpdate) else None
        if closing is not None and hasattr(closing, "add_normed_cast"):
            closing.add_normed_cast(hidden, delta.tensor, left)     # norm, add and cast in one kernel; the stream is rewritten below
        else:
            settle_update(hidden, delta, self.dtype)
            kernels.cast_rows(hidden, left)
        y = ctx.buf("reentry.out", (ctx.n_tokens, self.hidden), self.dtype)
        kernels.linear(pair, self.w_in, y)
        kernels.stream_set(hidden, y, self.step[call.index])
        return None
