"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``, or with ``clamped_swish``
``down(g sigmoid(alpha g) (u + 1))`` for ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit, limit)``.

Gate and up projections are kept as one ``[2 * intermediate, hidden]`` matrix so the step runs
one product for both (the reference runs two, ``src/turboserve/engine/model/layers.py:412-440``);
the activation and the multiply are fp32 with one rounding: in the product's epilogue for small
bfloat16 batches, else in a kernel of their own (``ops.linear.gated_linear``).
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import gated_linear, interleave_gate_up, linear
from .base import FeedForward, ParamSpec, register_feed_forward


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(spec["intermediate_size"])
        self.activation = str(spec.get("activation", "silu"))
        if self.activation not in kernels.ACTIVATION_CODES:
            raise ValueError(f"activation {self.activation!r} is not implemented; known: {sorted(kernels.ACTIVATION_CODES)}")
        self.limit, self.alpha = float(spec.get("limit", 0.0)), float(spec.get("alpha", 1.702))
        """Constants of ``clamped_swish``: ``g sigmoid(alpha g) (u + 1)`` with ``g = min(gate, limit)`` and
        ``u = clamp(up, -limit, limit)``; other activations ignore them."""
        if self.activation == "clamped_swish" and not self.limit > 0.0:
            raise ValueError("the clamped activation needs a positive 'limit'")
        self.has_bias = bool(spec.get("bias", False))
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", **dict(spec.get("names") or {})}
        """The three matrices' local names in the checkpoint."""
        self.dtype = dtype
        self.gate_up: torch.Tensor | None = None
        self.gate_block = 0
        self.down: torch.Tensor | None = None
        self.gate_up_bias = None
        self.down_bias = None

    def param_specs(self) -> list[ParamSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = [
            ParamSpec(self.names["gate"], (i, h)),
            ParamSpec(self.names["up"], (i, h)),
            ParamSpec(self.names["down"], (h, i)),
        ]
        if self.has_bias:
            specs += [
                ParamSpec("gate_proj.bias", (i,), role="bias", init="bias_normal"),
                ParamSpec("up_proj.bias", (i,), role="bias", init="bias_normal"),
                ParamSpec("down_proj.bias", (h,), role="bias", init="bias_normal"),
            ]
        return specs

    def scratch_per_token(self) -> int:
        return 3 * self.intermediate_size + self.hidden_size  # gate and up, their product, the output

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gate_up, self.gate_block = interleave_gate_up(tensors[self.names["gate"]], tensors[self.names["up"]])
        self.down = tensors[self.names["down"]].contiguous()
        if self.has_bias:
            self.gate_up_bias, _ = interleave_gate_up(tensors["gate_proj.bias"], tensors["up_proj.bias"])
            self.down_bias = tensors["down_proj.bias"].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = ctx.batch.num_tokens
        hidden = ctx.buffer("mlp.hidden", (n, self.intermediate_size))
        gated_linear(x, self.gate_up, hidden, self.gate_up_bias, self.activation, self.gate_block, n, ctx,
                     limit=self.limit, alpha=self.alpha)
        out = ctx.buffer("mlp.out", (n, self.hidden_size))
        linear(hidden, self.down, out, self.down_bias, n, ctx)
        return out


class DenseMLP(FeedForward):
    """Ungated feed-forward: ``down(act(up(x)))``.

    ``intermediate_size``; ``activation`` (``relu2``: the square of relu, ``gelu_tanh``, ``silu``),
    applied in float32 and rounded once; ``up`` and ``down`` (the two matrices' local names).
    """

    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(spec["intermediate_size"])
        self.activation = str(spec.get("activation", "relu2"))
        if self.activation not in kernels.PLAIN_ACTIVATION_CODES:
            raise ValueError(f"activation {self.activation!r} is not implemented; known: {sorted(kernels.PLAIN_ACTIVATION_CODES)}")
        self.up_name = str(spec.get("up", "up_proj.weight"))
        self.down_name = str(spec.get("down", "down_proj.weight"))
        self.dtype = dtype
        self.up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [ParamSpec(self.up_name, (i, h)), ParamSpec(self.down_name, (h, i))]

    def scratch_per_token(self) -> int:
        return 2 * self.intermediate_size + self.hidden_size

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.up = tensors[self.up_name].contiguous()
        self.down = tensors[self.down_name].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = ctx.batch.num_tokens
        raised = ctx.buffer("dense_mlp.up", (n, self.intermediate_size))
        linear(x, self.up, raised, None, n, ctx)
        hidden = ctx.buffer("dense_mlp.hidden", (n, self.intermediate_size))
        kernels.activation(raised, hidden, self.activation, n)
        out = ctx.buffer("dense_mlp.out", (n, self.hidden_size))
        linear(hidden, self.down, out, None, n, ctx)
        return out


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("dense_mlp", DenseMLP)
