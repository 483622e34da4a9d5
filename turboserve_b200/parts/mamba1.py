"""The selective-scan mixer (Mamba): a state per channel and state index, with step sizes, ``B`` and ``C`` chosen by the input.

The input projection gives ``[x: inner | z: inner]`` per token. ``x`` passes a short causal convolution per channel
(``taps`` taps, the last one on the current token, with a bias) and silu. A low-rank projection of ``x`` gives
``[dt: dt_rank | B: N | C: N]``; ``dt`` is widened to one step size per channel. Then per channel ``c`` and state index
``n``, in float32,

    dt_c     = softplus(Wdt dt + dt_bias)_c
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,         A = -exp(A_log)        (S zero at a request's start)
    y_c      = sum_n S[c, n] C_n + D_c x_c

and ``y * silu(z)`` is projected back. A request keeps two states between steps: ``S`` in float32 and the last
``taps - 1`` inputs of the convolution.

Sizes are parameters: ``inner``, ``state``, ``dt_rank``, ``taps``; ``names`` maps the roles ``in conv conv_bias x dt dt_bias
a_log d out`` to the checkpoint's local tensor names.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, ParamSpec, StateNeed, register_mixer

DEFAULT_NAMES = {
    "in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "x": "x_proj.weight", "dt": "dt_proj.weight",
    "dt_bias": "dt_proj.bias", "a_log": "A_log", "d": "D", "out": "out_proj.weight",
}


class Mamba1Mixer(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("a state-space mixer has no pages another run could share")
        self.hidden_size = int(hidden_size)
        self.inner, self.state, self.rank = int(spec["inner"]), int(spec["state"]), int(spec["dt_rank"])
        self.taps = int(spec.get("taps", 4))
        if not 1 <= self.taps <= 16:
            raise ValueError(f"taps must be between 1 and 16, got {self.taps}")
        if not 1 <= self.state <= 512 or self.rank < 1 or self.inner < 1:
            raise ValueError(f"state must be between 1 and 512 and dt_rank positive, got {self.state} and {self.rank}")
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        self.low_width = self.rank + 2 * self.state
        for name in ("in_w", "conv_w", "conv_b", "x_w", "dt_w", "dt_bias", "a_log", "d_skip", "out_w"):
            setattr(self, name, None)

    def cache_need(self):
        recurrent = StateNeed((self.inner, self.state), torch.float32)
        if self.taps == 1:
            return recurrent
        return recurrent, StateNeed((self.taps - 1, self.inner), None)

    def scratch_per_token(self) -> int:
        # [x | z], the convolved x, [dt | B | C], the step sizes in float32 (two elements' worth), the gated rows, the output
        return 2 * self.inner + self.inner + self.low_width + 2 * self.inner + self.inner + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        return [
            ParamSpec(n["in"], (2 * self.inner, h)),
            ParamSpec(n["conv"], (self.inner, self.taps), role="gain", init="bias_normal"),
            ParamSpec(n["conv_bias"], (self.inner,), role="bias", init="bias_normal"),
            ParamSpec(n["x"], (self.low_width, self.inner)),
            ParamSpec(n["dt"], (self.inner, self.rank)),
            ParamSpec(n["dt_bias"], (self.inner,), role="bias", init="bias_normal"),
            ParamSpec(n["a_log"], (self.inner, self.state), role="gain", init="bias_normal"),
            ParamSpec(n["d"], (self.inner,), role="gain", init="one_plus_normal"),
            ParamSpec(n["out"], (h, self.inner)),
        ]

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        for attr, role in (("in_w", "in"), ("conv_w", "conv"), ("conv_b", "conv_bias"), ("x_w", "x"), ("dt_w", "dt"),
                           ("dt_bias", "dt_bias"), ("a_log", "a_log"), ("d_skip", "d"), ("out_w", "out")):
            setattr(self, attr, tensors[n[role]].contiguous())

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        projected = ctx.buffer("mamba1.in", (n, 2 * self.inner))
        linear(x, self.in_w, projected, None, n, ctx)
        convolved = ctx.buffer("mamba1.conv", (n, self.inner))
        tail = cache.states[1] if self.taps > 1 else projected.new_empty((1, 0, self.inner))
        kernels.causal_conv(projected, 0, self.conv_w, self.conv_b, tail, convolved, batch.seq_of_token, batch.query_start_loc,
                            batch.state_slots, n, batch.num_seqs, silu=True, status=ctx.status)
        low = ctx.buffer("mamba1.low", (n, self.low_width))
        linear(convolved, self.x_w, low, None, n, ctx)
        dt_raw = ctx.buffer("mamba1.dt", (n, self.inner), torch.float32)
        linear(low[:, :self.rank], self.dt_w, dt_raw, None, n, ctx)
        gated = ctx.buffer("mamba1.gated", (n, self.inner))
        kernels.selective_scan(convolved, dt_raw, self.dt_bias, low, self.rank, self.rank + self.state, self.a_log, self.d_skip,
                               projected[:, self.inner:], cache.states[0], gated, batch.query_start_loc, batch.state_slots,
                               batch.num_seqs, n)
        out = ctx.buffer("mamba1.out", (n, self.hidden_size))
        linear(gated, self.out_w, out, None, n, ctx)
        return out


register_mixer("mamba1", Mamba1Mixer)
