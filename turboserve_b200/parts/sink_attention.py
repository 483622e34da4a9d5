"""Grouped-query softmax attention with normed heads, capped scores and a sink in the denominator.

Per token ``q = Wq h`` (``heads x dim``), ``k = Wk h`` (``kv_heads x dim``), ``v = Wv h`` (``kv_heads x vdim``); query
head ``j`` reads key/value head ``j // (heads / kv_heads)``. Options, each a parameter:

* ``bias``: q, k and v each have a bias (added in float32 by the kernel that norms, rotates and appends);
* ``qk_norm``: every head of ``q`` and of ``k`` is divided by its root mean square over ``dim`` (``eps`` inside the
  root) and multiplied by a weight of ``dim`` values that all heads share (one for queries, one for keys), before
  the rotation;
* ``rot``: the first ``rot.dims`` elements of every head of ``q`` and ``k`` turn by ``position * base^(-2i / dims)``;
  pair ``i`` is elements ``(2i, 2i + 1)`` when ``rot.interleaved``, else ``(i, i + dims / 2)``; ``rot.scaling`` stretches the
  long waves (:func:`~turboserve_b200.parts.rope.rotary_frequencies`);
* ``softcap``: ``score = cap * tanh(scale * (q . k) / cap)``;
* ``sink``: the softmax's denominator is one larger, ``p_j = exp(s_j) / (1 + sum exp(s_j))``: a key that scores 0
  and has no value; with ``sink = "learned"`` every query head has a number ``b`` of its own in a tensor and the term is
  ``exp(b)`` (``b`` is neither scaled nor capped);
* ``window``: the keys seen, the query's own included (``None``: all up to its position).

Norm, rotation and the append of keys and values to the request's pages are one kernel in fp32; scores, the
softmax and its sums are fp32 in the attention kernel. bfloat16 steps with portions of prompts run the tiled
tensor-core kernel (``attention_capped_mma.cu``) when it takes the head sizes; steps of single tokens, float32 and
other sizes the kernel for every size (``attention_generic.cu``), which scores the query heads of a key head together
when a step has few tokens. ``names`` maps the roles ``q k v o q_norm k_norm q_bias k_bias v_bias sink`` to the
checkpoint's local tensor names.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, PagedKVNeed, ParamSpec, register_mixer
from .rope import rotary_frequencies

DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                 "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "q_bias": "q_proj.bias", "k_bias": "k_proj.bias",
                 "v_bias": "v_proj.bias", "sink": "sinks"}


class SinkAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("this attention keeps pages of its own")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads = int(spec["heads"]), int(spec["kv_heads"])
        self.dim, self.vdim = int(spec["dim"]), int(spec.get("vdim") or spec["dim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        if not 1 <= self.dim <= 256 or not 1 <= self.vdim <= 256:
            raise ValueError(f"dim and vdim must lie between 1 and 256, got {self.dim} and {self.vdim}")
        self.scale = float(spec.get("scale", self.dim ** -0.5))
        self.softcap = float(spec.get("softcap") or 0.0)
        self.sink = bool(spec.get("sink", False))
        self.learned_sink = spec.get("sink") == "learned"
        self.has_bias = bool(spec.get("bias", False))
        self.qk_norm = bool(spec.get("qk_norm", False))
        self.eps = float(spec.get("eps", 1e-6))
        window = spec.get("window")
        self.window = int(window) if window else None
        rot = dict(spec.get("rot") or {})
        self.rot = int(rot.get("dims", 0))
        self.interleaved = bool(rot.get("interleaved", False))
        if self.rot > self.dim or self.rot % 2:
            raise ValueError(f"the rotation covers {self.rot} of {self.dim} elements; it must be even and fit")
        self.inv_freq = None
        if self.rot:
            freq, amplitude = rotary_frequencies(self.rot, float(rot["base"]), rot.get("scaling"))
            if amplitude != 1.0:
                raise ValueError("this attention rotates without a factor on cos and sin")
            self.inv_freq = freq.to(device)
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        self.q_width, self.k_width, self.v_width = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.qkv_width = self.q_width + self.k_width + self.v_width
        self.qkv: torch.Tensor | None = None
        self.out_w: torch.Tensor | None = None
        self.q_gain: torch.Tensor | None = None
        self.k_gain: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.sink_values: torch.Tensor | None = None

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.kv_heads, self.dim, self.window, self.vdim)

    def scratch_per_token(self) -> int:
        return self.qkv_width + self.heads * self.vdim + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        specs = [ParamSpec(n["q"], (self.q_width, h)), ParamSpec(n["k"], (self.k_width, h)), ParamSpec(n["v"], (self.v_width, h))]
        if self.qk_norm:
            specs += [ParamSpec(n["q_norm"], (self.dim,), role="gain", init="one_plus_normal"),
                      ParamSpec(n["k_norm"], (self.dim,), role="gain", init="one_plus_normal")]
        if self.has_bias:
            specs += [ParamSpec(n["q_bias"], (self.q_width,), role="bias", init="bias_normal"),
                      ParamSpec(n["k_bias"], (self.k_width,), role="bias", init="bias_normal"),
                      ParamSpec(n["v_bias"], (self.v_width,), role="bias", init="bias_normal")]
        if self.learned_sink:
            specs.append(ParamSpec(n["sink"], (self.heads,), role="bias", init="bias_normal"))
        specs.append(ParamSpec(n["o"], (h, self.heads * self.vdim)))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.out_w = tensors[n["o"]].contiguous()
        if self.qk_norm:
            self.q_gain, self.k_gain = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()
        if self.has_bias:
            self.bias = torch.cat([tensors[n["q_bias"]], tensors[n["k_bias"]], tensors[n["v_bias"]]]).contiguous()
        if self.learned_sink:
            self.sink_values = tensors[n["sink"]].contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        table = batch.block_tables[cache.group]
        qkv = ctx.buffer("sink_attn.qkv", (n, self.qkv_width))
        linear(x, self.qkv, qkv, None, n, ctx)
        kernels.head_norm_rope_write(qkv, self.q_gain, self.k_gain, self.eps, batch.positions, batch.seq_of_token, table,
                                     cache.k_pages, cache.v_pages, n, self.heads, self.kv_heads, self.dim, self.vdim,
                                     self.inv_freq, self.rot, self.interleaved, cache.writes, ctx.status, bias=self.bias)
        attended = ctx.buffer("sink_attn.attended", (n, self.heads * self.vdim))
        if batch.max_query_len > 1 and kernels.paged_attention_capped_mma_takes(qkv.dtype, self.dim, self.vdim, self.scale):
            # portions of prompts in bfloat16: tiles of 64 positions on tensor cores
            kernels.paged_attention_capped_mma(qkv, attended, cache.k_pages, cache.v_pages, table, batch.query_start_loc,
                                               batch.context_lens, n, batch.num_seqs, self.heads, self.kv_heads, self.dim,
                                               self.vdim, self.window, self.scale, self.softcap, self.sink, ctx.status,
                                               sink_values=self.sink_values)
        else:
            kernels.paged_attention_capped(qkv, attended, cache.k_pages, cache.v_pages, table, batch.seq_of_token, batch.positions,
                                           n, self.heads, self.kv_heads, self.dim, self.vdim, self.window, self.scale,
                                           self.softcap, self.sink, ctx.status, sink_values=self.sink_values)
        out = ctx.buffer("sink_attn.out", (n, self.hidden_size))
        linear(attended, self.out_w, out, None, n, ctx)
        return out


register_mixer("sink_attention", SinkAttention)
