"""Time mixing with a decay the input chooses (the wkv recurrence), fed by blends with the previous token.

With ``h'`` the previous token's input (zeros before a request's first token), each of the five roles ``s`` in
``r k v g w`` reads its own blend ``m_s = h + (h' - h) * mu_s``. Then ``r = Wr m_r``, ``k = Wk m_k`` (``heads x dim``),
``v = Wv m_v`` (``heads x vdim``), ``gate = silu(Wg m_g)`` and, per head and key channel, in float32,

    w_t = exp(-exp(W2 tanh(W1 m_w) + w0))
    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t           (the bonus u counts for the current token alone)
    S_t = diag(w_t) S_{t-1} + k_t v_t^T                  (S is dim x vdim, zero at a request's start)

Each head's ``o`` is divided by its root mean square (``eps`` inside the root); the heads side by side are
multiplied by a weight, by the gate, and projected by ``Wo``. A request keeps two states: ``S`` of every head in
float32 and its last input row (in the activation type, as it was).

Sizes and constants are parameters: ``heads``, ``dim``, ``vdim`` (default ``dim``), ``decay_rank``, ``eps``; ``names`` maps
the roles ``mu_r mu_k mu_v mu_g mu_w r k v g w1 w2 w0 u norm o`` to the checkpoint's local tensor names.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, ParamSpec, StateNeed, register_mixer

DEFAULT_NAMES = {
    "mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k", "v": "v", "g": "g",
    "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "o": "o",
}
MIX_ORDER = ("r", "k", "v", "g", "w")


class WkvMixer(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("a recurrent mixer has no pages another run could share")
        self.hidden_size = int(hidden_size)
        self.heads, self.dim = int(spec["heads"]), int(spec["dim"])
        self.vdim = int(spec.get("vdim") or self.dim)
        self.rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        if not 1 <= self.dim <= 256 or self.vdim < 1 or self.rank < 1:
            raise ValueError(f"wkv takes dim between 1 and 256 and a positive rank, got {self.dim} and {self.rank}")
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.vdim
        self.proj_width = 2 * self.qk_width + 2 * self.v_width  # r | k | v | g
        for name in ("mu", "w_r", "w_k", "w_v", "w_g", "w1", "w2", "w0", "bonus", "norm_w", "out_w"):
            setattr(self, name, None)
        self._scan_scratch: int | None = None

    @property
    def scan_scratch(self) -> int:
        if self._scan_scratch is None:
            self._scan_scratch = kernels.chosen_decay_scratch_per_token(self.heads, self.dim, self.vdim)
        return self._scan_scratch

    def cache_need(self):
        return StateNeed((self.heads, self.vdim, self.dim), torch.float32), StateNeed((self.hidden_size,), None)

    def scratch_per_token(self) -> int:
        # the five blends, the projections, the low-rank decay rows, fp32 rows (two elements' worth each): the decays, o
        # and the scan's own copies; the gated rows and the output
        return (5 * self.hidden_size + self.proj_width + 2 * self.rank + 2 * self.qk_width + 3 * self.v_width + self.hidden_size
                + 2 * (6 * self.qk_width + 2 * self.v_width))

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        specs = [ParamSpec(n["mu_" + s], (h,), role="gain", init="bias_normal") for s in MIX_ORDER]
        specs += [ParamSpec(n["r"], (self.qk_width, h)), ParamSpec(n["k"], (self.qk_width, h)), ParamSpec(n["v"], (self.v_width, h)),
                  ParamSpec(n["g"], (self.v_width, h)), ParamSpec(n["w1"], (self.rank, h)), ParamSpec(n["w2"], (self.qk_width, self.rank)),
                  ParamSpec(n["w0"], (self.qk_width,), role="bias", init="bias_normal"),
                  ParamSpec(n["u"], (self.heads, self.dim), role="gain", init="bias_normal"),
                  ParamSpec(n["norm"], (self.v_width,), role="gain", init="one_plus_normal"),
                  ParamSpec(n["o"], (h, self.v_width))]
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.mu = torch.stack([tensors[n["mu_" + s]] for s in MIX_ORDER], dim=0).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = (tensors[n[s]].contiguous() for s in ("r", "k", "v", "g"))
        self.w1, self.w2 = tensors[n["w1"]].contiguous(), tensors[n["w2"]].contiguous()
        self.w0, self.bonus = tensors[n["w0"]].contiguous(), tensors[n["u"]].contiguous()
        self.norm_w, self.out_w = tensors[n["norm"]].contiguous(), tensors[n["o"]].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n, h = batch.num_tokens, self.hidden_size
        blends = ctx.buffer("wkv.blends", (n, 5 * h))
        kernels.shift_mix(x, self.mu, cache.states[1], blends, batch.positions, batch.seq_of_token, batch.query_start_loc,
                          batch.state_slots, n, batch.num_seqs)
        projected = ctx.buffer("wkv.proj", (n, self.proj_width))
        first = 0
        views = []
        for index, weight in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            view = projected[:, first:first + weight.shape[0]]
            linear(blends[:, index * h:(index + 1) * h], weight, view, None, n, ctx)
            views.append(view)
            first += weight.shape[0]
        low = ctx.buffer("wkv.low", (n, self.rank))
        linear(blends[:, 4 * h:], self.w1, low, None, n, ctx)
        bent = ctx.buffer("wkv.low_tanh", (n, self.rank))
        kernels.activation(low, bent, "tanh", n)
        decay_raw = ctx.buffer("wkv.decay", (n, self.qk_width), torch.float32)
        linear(bent, self.w2, decay_raw, None, n, ctx)
        y = ctx.buffer("wkv.y", (n, self.v_width), torch.float32)
        scratch = ctx.buffer("wkv.scratch", (n * self.scan_scratch,), torch.float32)
        kernels.chosen_decay_scan(views[0], views[1], views[2], self.bonus, decay_raw, self.w0, batch.positions,
                                  batch.seq_of_token, batch.query_start_loc, batch.state_slots, cache.states[0], y, scratch, n,
                                  batch.num_seqs, self.heads, self.dim, self.vdim)
        gated = ctx.buffer("wkv.gated", (n, self.v_width))
        kernels.part_norm_gate(y, views[3], gated, n, self.heads, self.vdim, self.eps, self.norm_w, "silu")
        out = ctx.buffer("wkv.out", (n, h))
        linear(gated, self.out_w, out, None, n, ctx)
        return out


register_mixer("wkv", WkvMixer)
