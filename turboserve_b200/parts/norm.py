"""RMSNorm fused with the residual sum.

``out = gain * x * rsqrt(mean(x^2) + eps)`` with ``x = residual + delta`` taken in fp32, the
statistics in fp32 and one rounding to the activation dtype at the end. The reference rounds
the normalised value to the model dtype before the gain multiply
(``src/turboserve/engine/model/layers.py:202-208``); here the product is rounded once, which
is equal in float32 and at least as close to the exact value in bfloat16.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from .base import Norm, NormedUpdate, ParamSpec, pending_updates, register_norm


class RMSNorm(Norm):
    """``eps``; ``zero_centred`` (the stored weight lies around zero and the gain is ``1 + weight``,
    added once in float32 when the weights are bound); ``tensor`` (the weight's local name).

    ``delta`` may be one update, a pair of them (the two branches of a layer whose mixer and
    feed-forward run side by side), :class:`~turboserve_b200.parts.base.ScaledUpdates` (updates that enter the
    sum times a factor) or ``None``; ``shift`` a float32 vector that is added to every
    row as well. :meth:`forward_pair` norms the same sum with a second norm's gain in the same pass.
    """

    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.eps = float(spec["eps"])
        self.zero_centred = bool(spec.get("zero_centred", False))
        self.tensor = str(spec.get("tensor", "weight"))
        self.hidden_size = int(hidden_size)
        self.dtype = dtype
        self.gain: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.tensor, (self.hidden_size,), role="gain",
                          init="bias_normal" if self.zero_centred else "one_plus_normal")]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        weight = tensors[self.tensor]
        self.gain = (weight + 1.0).contiguous() if self.zero_centred else weight

    def scratch_per_token(self) -> int:
        return 0  # it writes into the block's buffer

    def forward(self, residual, delta, out, ctx, shift=None, rows_added=None):
        """``rows_added``: a float32 matrix, a row a token, that enters the sum as well."""
        if isinstance(delta, NormedUpdate) or rows_added is not None:
            n = ctx.batch.num_tokens
            if isinstance(delta, NormedUpdate):
                if shift is None:  # the pending update's own norm, the rows and this norm in one pass
                    kernels.norm_add_norm(residual, delta.update, delta.gain, delta.eps, rows_added, self.gain, self.eps, out, n)
                    return out
                kernels.norm_add_norm(residual, delta.update, delta.gain, delta.eps, rows_added, None, 0.0, None, n, out.dtype)
                delta = None
            elif shift is None and delta is None:
                kernels.norm_add_norm(residual, None, None, 0.0, rows_added, self.gain, self.eps, out, n)
                return out
            else:
                kernels.norm_add_norm(residual, None, None, 0.0, rows_added, None, 0.0, None, n, out.dtype)
        updates, mult = pending_updates(delta)
        if len(updates) <= 1 and shift is None and mult == 1.0:
            kernels.add_rmsnorm(residual, updates[0] if updates else None, self.gain, self.eps, out, None, ctx.batch.num_tokens)
        else:
            kernels.stream_norm(residual, updates, shift, self.gain, out, eps=self.eps, num_rows=ctx.batch.num_tokens, mult=mult)
        return out

    def forward_pair(self, residual, delta, other: "RMSNorm", out, out_other, ctx, shift=None):
        """Both norms of one sum: ``out`` with this norm's gain, ``out_other`` with ``other``'s (same ``eps``)."""
        if other.eps != self.eps:
            raise ValueError("forward_pair needs two norms with one eps")
        updates, mult = pending_updates(delta)
        kernels.stream_norm(residual, updates, shift, self.gain, out, other.gain, out_other, eps=self.eps,
                            num_rows=ctx.batch.num_tokens, mult=mult)
        return out, out_other

    def normed(self, update: torch.Tensor) -> NormedUpdate:
        """``update`` as a pending update that enters the stream through this norm."""
        return NormedUpdate(update, self.gain, self.eps)

    def forward_output(self, residual, update, mult: float, copy, ctx):
        """The norm behind a sublayer: ``residual += mult * norm(update)`` with this norm's gain, the statistics
        taken over ``update`` alone; ``copy`` (or ``None``) receives the new residual in the activation type."""
        kernels.norm_add(residual, update, self.gain, copy, self.eps, mult, ctx.batch.num_tokens)
        return copy

    def forward_rows(self, residual, delta, rows, num_rows, out, ctx):
        if isinstance(delta, NormedUpdate):
            kernels.norm_add_norm(residual, delta.update, delta.gain, delta.eps, None, self.gain, self.eps, out, num_rows, rows=rows)
            return out
        updates, mult = pending_updates(delta)
        if len(updates) <= 1 and mult == 1.0:
            kernels.add_rmsnorm(residual, updates[0] if updates else None, self.gain, self.eps, out, rows, num_rows)
        else:
            kernels.stream_norm(residual, updates, None, self.gain, out, eps=self.eps, rows=rows, num_rows=num_rows, mult=mult)
        return out


register_norm("rms_norm", RMSNorm)
