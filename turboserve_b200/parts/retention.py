"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

Per token ``q = Wq h`` and ``k = Wk h`` (``heads x dim``), ``v = Wv h`` (``heads x vdim``), no biases. The first
``rot.dims`` elements of every head of ``q`` and ``k`` are rotated by the position (pairs ``(i, i + dims / 2)``,
frequencies from ``rot``: ``base``, ``dims``, optional ``scaling``); ``k`` is then multiplied by ``dim^-1/2``.
Per head, in float32, with the state zero at a request's start:

    S_t = decay_h S_{t-1} + k_t v_t^T,        o_t = S_t^T q_t

Each head's ``o`` is divided by its root mean square (``eps`` inside the root, no weight); the heads side by
side are multiplied by ``silu(Wg h)`` and projected by ``Wo``. A request keeps ``S`` of every head in float32
in its state slot (``[heads, vdim, dim]``); one kernel runs prompts, portions of them and single tokens.

Sizes and constants are parameters: ``heads``, ``dim``, ``vdim``, ``decay`` (one per head), ``rot``, ``eps``;
``names`` maps the roles ``q k v g o norm`` to the checkpoint's local tensor names.

The lightning-attention form is the same recurrence with other constants around it, each a parameter:
``activation`` (``"silu"``: q, k and v pass it as the scan reads them; then without a rotation), ``key_scale``
(what k is multiplied by; default ``dim^-1/2``), ``norm`` (``"heads"``: every head alone, ``"row"``: the heads side by
side as one row), ``norm_weight`` (a weight of ``heads * vdim`` values on the normed row) and ``gate`` (``"silu"`` or
``"sigmoid"``).
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, ParamSpec, StateNeed, register_mixer
from .rope import scaled_rotary_frequencies

DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight", "o": "o_proj.weight",
                 "norm": "norm.weight"}


class Retention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("a retention mixer has no pages another run could share")
        self.hidden_size = int(hidden_size)
        self.heads, self.dim, self.vdim = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        self.eps = float(spec["eps"])
        decay = [float(d) for d in spec["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"retention needs one decay per head: {len(decay)} for {self.heads} heads")
        if not 1 <= self.dim <= 256 or self.vdim < 1:
            raise ValueError(f"retention takes dim between 1 and 256, got {self.dim}")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        rot = dict(spec.get("rot") or {})
        self.rot = int(rot.get("dims", 0))
        if self.rot > self.dim or self.rot % 2:
            raise ValueError(f"the rotation covers {self.rot} of {self.dim} elements; it must be even and fit")
        if self.rot:
            freq, self.amplitude = scaled_rotary_frequencies(self.rot, float(rot["base"]), rot.get("scaling"))
            self.inv_freq = freq.to(device)
        else:
            self.inv_freq, self.amplitude = torch.zeros(0, dtype=torch.float32, device=device), 1.0
        self.activation = spec.get("activation") or None
        if self.activation not in (None, "silu") or (self.activation and self.rot):
            raise ValueError("retention's activation is 'silu' or none, and goes with no rotation")
        self.key_scale = float(spec.get("key_scale", self.dim ** -0.5))
        self.norm_over, self.gate = str(spec.get("norm", "heads")), str(spec.get("gate", "silu"))
        if self.norm_over not in ("heads", "row") or self.gate not in ("silu", "sigmoid"):
            raise ValueError("retention norms 'heads' or the 'row', and gates with 'silu' or 'sigmoid'")
        self.has_norm_weight = bool(spec.get("norm_weight", False))
        self.plain = self.norm_over == "heads" and self.gate == "silu" and not self.has_norm_weight
        self.norm_w: torch.Tensor | None = None
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.vdim
        self.proj_width = 2 * self.qk_width + 2 * self.v_width
        self.proj: torch.Tensor | None = None
        self.out_w: torch.Tensor | None = None
        self._scan_scratch: int | None = None

    @property
    def scan_scratch(self) -> int:
        """Floats per token the scan wants for the rotated q and k and the values in fp32."""
        if self._scan_scratch is None:
            self._scan_scratch = kernels.retention_scratch_per_token(self.heads, self.dim, self.vdim)
        return self._scan_scratch

    def cache_need(self) -> StateNeed:
        return StateNeed((self.heads, self.vdim, self.dim), torch.float32)

    def scratch_per_token(self) -> int:
        # the projection, o in float32 (two elements' worth), the normed and gated rows, the output
        # (the scan's own fp32 copies are counted by their widths, not asked of the library: no compiler is needed to size a pool)
        return self.proj_width + 3 * self.v_width + self.hidden_size + 2 * (4 * self.qk_width + 2 * self.v_width)

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        specs = [ParamSpec(n["q"], (self.qk_width, h)), ParamSpec(n["k"], (self.qk_width, h)), ParamSpec(n["v"], (self.v_width, h)),
                 ParamSpec(n["g"], (self.v_width, h)), ParamSpec(n["o"], (h, self.v_width))]
        if self.has_norm_weight:
            specs.append(ParamSpec(n["norm"], (self.v_width,), role="gain", init="one_plus_normal"))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], dim=0).contiguous()
        self.out_w = tensors[n["o"]].contiguous()
        if self.has_norm_weight:
            self.norm_w = tensors[n["norm"]].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        projected = ctx.buffer("retention.proj", (n, self.proj_width))
        linear(x, self.proj, projected, None, n, ctx)
        y = ctx.buffer("retention.y", (n, self.v_width), torch.float32)
        scratch = ctx.buffer("retention.scratch", (n * self.scan_scratch,), torch.float32)
        kernels.retention_scan(projected, 0, self.qk_width, 2 * self.qk_width, self.decay, self.inv_freq, self.rot,
                               self.amplitude, self.key_scale, batch.positions, batch.seq_of_token, batch.query_start_loc,
                               batch.state_slots, cache.states[0], y, scratch, n, batch.num_seqs, self.heads, self.dim, self.vdim,
                               activation=self.activation)
        gated = ctx.buffer("retention.gated", (n, self.v_width))
        gate = projected[:, 2 * self.qk_width + self.v_width:]
        if self.plain:
            kernels.head_norm_gate(y, gate, gated, n, self.heads, self.vdim, self.eps)
        elif self.norm_over == "heads":
            kernels.part_norm_gate(y, gate, gated, n, self.heads, self.vdim, self.eps, self.norm_w, self.gate)
        else:
            kernels.part_norm_gate(y, gate, gated, n, 1, self.v_width, self.eps, self.norm_w, self.gate)
        out = ctx.buffer("retention.out", (n, self.hidden_size))
        linear(gated, self.out_w, out, None, n, ctx)
        return out


register_mixer("retention", Retention)
