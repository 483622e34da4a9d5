"""Mixture of experts: a router chooses a few small gated feed-forwards per token.

Router logits ``z = Wr h`` in float32 (``Wr`` is kept in float32), scores ``s = softmax(z)`` over all experts.
The experts form ``groups`` equal groups of neighbours; a group's score is its largest ``s``, and only experts
of the ``keep`` best groups may be chosen. Of those the ``top`` with the largest ``s`` are chosen, with weights
``s / (sum of the chosen s + 1e-20)``. An expert is ``down(act(gate h) * (up h))`` without biases; the output is
the weighted sum of the chosen experts' outputs, plus a ``shared`` expert of the same form (its own
intermediate size) that runs for every token, if the layer has one.

Three ways through the experts. A step in which every request brings one token reads nothing back and is
replayed from CUDA graphs: with very few tokens every (token, chosen expert) pair streams that expert's rows
on its own (two kernels); with a batch of them one block puts the pairs in expert order and a block per
(expert, tile of features) streams the expert's rows once for up to eight of its tokens at a time. A step with
portions of prompts puts the pairs in expert order too, reads the experts' row counts back once, and runs each
expert's rows as one matrix product through :func:`~turboserve_b200.ops.linear.linear`; a kernel adds the
weighted rows up per token in a fixed order.

Options: ``score`` ``"sigmoid"`` scores every expert on its own, ``s = sigmoid(z)``; ``renormalize`` ``False`` uses the
chosen scores as weights as they are; ``weight_on`` ``"input"`` puts the weight on what the expert reads, ``sum
expert(w h)``, instead of on what it gives (an expert is not linear, so the two differ; since gate and up are,
``gate(w h) = w gate(h)`` and the factor enters on their sums in fp32 before the activation).

Parameters: ``experts``, ``top``, ``groups``, ``keep``, ``intermediate_size``, ``shared`` (intermediate size of
the shared expert, or ``None``), ``activation``, ``shared_activation`` (default: the experts'), ``score``,
``renormalize``, ``weight_on``; ``names``: ``router``, ``expert`` (a pattern with ``{index}``),
``shared`` (a prefix), and ``gate up down`` (the matrices' names behind those prefixes).
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import FeedForward, ParamSpec, register_feed_forward
from .mlp import GatedMLP

PAIRS_ALONE = 4
"""Up to this many (token, expert) pairs of a step of single tokens each stream their expert on their own (two launches);
more are put in expert order first (four launches), so that an expert many tokens chose is read once."""

DEFAULT_NAMES = {"router": "gate.weight", "expert": "experts.{index}.", "shared": "shared_expert.",
                 "gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str) -> None:
        self.hidden_size = int(hidden_size)
        self.experts, self.top = int(spec["experts"]), int(spec["top"])
        self.groups, self.keep = int(spec.get("groups", 1)), int(spec.get("keep", 1))
        self.ff = int(spec["intermediate_size"])
        self.activation = str(spec.get("activation", "silu"))
        if self.activation not in kernels.ACTIVATION_CODES or kernels.ACTIVATION_CODES[self.activation] > 2:  # the experts' kernels take act(gate) * up only
            raise ValueError(f"activation {self.activation!r} is not implemented; known: {sorted(kernels.ACTIVATION_CODES)}")
        if not 1 <= self.top <= min(self.experts, 32):
            raise ValueError(f"top must be between 1 and min(experts, 32), got {self.top} of {self.experts}")
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.experts} experts do not form {self.groups} equal groups of which {self.keep} are kept")
        if self.keep * (self.experts // self.groups) < self.top:
            raise ValueError("the kept groups hold fewer experts than are to be chosen")
        self.score = str(spec.get("score", "softmax"))
        self.renormalize = bool(spec.get("renormalize", True))
        self.weight_on = str(spec.get("weight_on", "output"))
        if self.score not in ("softmax", "sigmoid") or self.weight_on not in ("input", "output"):
            raise ValueError(f"scores are 'softmax' or 'sigmoid' and weights stand on 'input' or 'output', got {self.score!r}, {self.weight_on!r}")
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        shared = spec.get("shared")
        self.shared = None
        if shared:
            inner = {role: self.names["shared"] + self.names[role] for role in ("gate", "up", "down")}
            self.shared = GatedMLP(PartSpec("gated_mlp", dict(intermediate_size=int(shared), activation=str(spec.get("shared_activation") or self.activation), names=inner)),
                                   hidden_size, dtype, device)
        self.router: torch.Tensor | None = None
        self.gate_up: torch.Tensor | None = None  # [experts, 2 * ff, hidden]: an expert's gate rows, then its up rows
        self.down: torch.Tensor | None = None     # [experts, hidden, ff]

    def _expert(self, index: int, role: str) -> str:
        return self.names["expert"].format(index=index) + self.names[role]

    def param_specs(self) -> list[ParamSpec]:
        h, i = self.hidden_size, self.ff
        specs = [ParamSpec(self.names["router"], (self.experts, h), role="gain", init="normal")]
        for e in range(self.experts):
            specs += [ParamSpec(self._expert(e, "gate"), (i, h)), ParamSpec(self._expert(e, "up"), (i, h)),
                      ParamSpec(self._expert(e, "down"), (h, i))]
        if self.shared is not None:
            specs += self.shared.param_specs()
        return specs

    def scratch_per_token(self) -> int:
        own = self.top * (3 * self.ff + 2 * self.hidden_size) + self.hidden_size + 4 * self.top
        return own + (self.shared.scratch_per_token() if self.shared is not None else 0)

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.router = tensors[self.names["router"]].contiguous()
        self.gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], dim=0)
                                    for e in range(self.experts)]).contiguous()
        self.down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        batch = ctx.batch
        n, top = batch.num_tokens, self.top
        chosen = ctx.buffer("moe.chosen", (n, top), torch.int32)
        weights = ctx.buffer("moe.weights", (n, top), torch.float32)
        kernels.moe_route(x, self.router, chosen, weights, n, top, self.groups, self.keep, self.score, self.renormalize)
        # the weight stands on one side of an expert: on what it reads, or on what it gives
        w_in, w_out = (weights, None) if self.weight_on == "input" else (None, weights)
        always = self.shared.forward(x, ctx) if self.shared is not None else None
        out = ctx.buffer("moe.out", (n, self.hidden_size))
        pairs = n * top
        # every buffer of both ways is asked for in every step: the dry run that sizes the scratch before it is
        # frozen for graph capture is a step without requests, and must see what a portion of a prompt needs
        hidden = ctx.buffer("moe.hidden", (pairs, self.ff))
        counters = ctx.buffer("moe.counters", (3 * self.experts + 1,), torch.int32)
        place = ctx.buffer("moe.place", (pairs,), torch.int32)
        pair_of_row = ctx.buffer("moe.pair_of_row", (pairs,), torch.int32)
        rows = ctx.buffer("moe.rows", (pairs, self.hidden_size))
        both = ctx.buffer("moe.gate_up", (pairs, 2 * self.ff))
        moved = ctx.buffer("moe.rows_out", (pairs, self.hidden_size))
        if batch.max_query_len <= 1:
            if pairs <= PAIRS_ALONE or 8 * max(self.hidden_size, self.ff) * x.element_size() > kernels.MOE_EXPERT_ROWS_SMEM:
                kernels.moe_pair_gate_up(x, self.gate_up, chosen, hidden, n, top, self.activation, in_weights=w_in)
                kernels.moe_pair_down(hidden, self.down, chosen, w_out, always, out, n, top)
                return out
            # a batch of single tokens: an expert's rows are streamed once for all the tokens that chose it
            kernels.moe_sort(chosen, pairs, self.experts, counters, place, pair_of_row)
            kernels.moe_expert_rows(True, x, self.gate_up, counters, pair_of_row, hidden, top, self.activation, in_weights=w_in)
            kernels.moe_expert_rows(False, hidden, self.down, counters, pair_of_row, moved, top)
            kernels.moe_combine(moved, place, w_out, always, out, n, top)
            return out
        kernels.moe_sort(chosen, pairs, self.experts, counters, place, pair_of_row)
        kernels.moe_gather(x, pair_of_row, rows, pairs, top, in_weights=w_in)
        first = counters[self.experts: 2 * self.experts + 1].tolist()  # the one read-back: where each expert's rows start
        for e in range(self.experts):
            a, b = first[e], first[e + 1]
            if b > a:
                linear(rows[a:b], self.gate_up[e], both[a:b], None, b - a, ctx)
        kernels.act_mul(both, hidden, self.activation, pairs, block=0)
        for e in range(self.experts):
            a, b = first[e], first[e + 1]
            if b > a:
                linear(hidden[a:b], self.down[e], moved[a:b], None, b - a, ctx)
        kernels.moe_combine(moved, place, w_out, always, out, n, top)
        return out


register_feed_forward("routed_experts", RoutedExperts)
