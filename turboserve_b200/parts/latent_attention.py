"""Latent attention: keys and values of all heads are made from one small latent per position.

Per token, with ``h`` the mixer's input: ``q = Wq h`` holds, head by head, ``dim`` plain and ``rot_dim``
rotated query elements. ``Wdkv h`` gives ``kv_rank + rot_dim`` numbers: the first ``kv_rank``, RMS-normed
with a weight, are the latent ``c``; the last ``rot_dim`` are one rotated key part ``r`` that all heads
share. A head's key is ``[Wuk_h c | r]``, its value ``Wuv_h c``; the score of key ``j`` is
``(q_plain . Wuk_h c_j + q_rot . r_j) * scale`` over the last ``window`` positions (itself included;
``None``: all), softmax, then the output projection on the heads' values side by side. Only ``c`` and ``r``
(after rotation) are cached: a page row is ``[c | r]``.

Keys and values are never formed. The query is carried into the latent space instead,
``q~ = Wuk_h^T q_plain``, so that a score is ``q~ . c_j + q_rot . r_j``, the softmax-weighted sum is taken
over the latents themselves and ``Wuv_h`` is applied to that sum: attention reads ``kv_rank + rot_dim``
numbers per key for all heads together, in prompts and in decoding alike.

Which code runs the attention itself: float32, single tokens, short portions and layers without a window
take the kernel for every size (``latent_attention.cu``: fp32 sums in one order, whatever the cut). In
bfloat16 a request that brings :data:`PORTION_MIN` tokens or more to a windowed layer is worked in stretches
of queries: the rows the stretch can see are gathered from the pages, the scores of all heads are one matrix
product (bfloat16 operands, float32 accumulation and result), a kernel takes the softmax under the mask in
float32 and rounds the weights to bfloat16, and a second product sums the latents.

The rotation acts on pairs ``(i, i + rot_dim / 2)`` with frequencies from ``rot`` (``base``, ``dims``, optional
``scaling``: see :func:`~turboserve_b200.parts.rope.rotary_frequencies`); ``scale`` is used as given. With
``rot.interleaved`` the checkpoint pairs neighbours ``(2i, 2i + 1)`` instead: the rows of ``Wq`` and ``Wdkv`` that make
the rotated parts are put in the other order once, when the weights are bound (a score is a sum over the rotated
elements, so the order they are kept in is free as long as queries and keys share it).

With ``gate`` a head's output is multiplied by ``sigmoid(Wg h)_head`` before the output projection (``Wg`` has one row
a head and reads the mixer's input; its rows ride in the fused projection, the sigmoid and the product are fp32 in
the kernel that applies ``Wuv``).

With ``shares_cache`` the mixer has no ``Wdkv`` and attends over the rows another run writes, with its own
queries, ``Wuk``, ``Wuv`` and window; ``cache_window`` is then the window the shared pages are kept for (the
largest of the runs that read them; ``None`` keeps everything).

Sizes and constants are parameters: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``window``,
``cache_window``, ``eps``, ``rot``, ``gate``; ``names`` maps the roles ``q dkv dkv_norm uk uv o g`` to the checkpoint's names.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from ..ops.linear import linear
from .base import Mixer, PagedKVNeed, ParamSpec, register_mixer
from .rope import rotary_frequencies

PORTION_MIN = 32
"""Tokens a request brings to a step from which its attention is worked as matrix products (bfloat16, windowed)."""

STRETCH_ELEMENTS = 1 << 24
"""Most scores (queries x heads x keys) of one stretch of queries."""


def matrix_product(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a @ b`` by the library: into ``out`` in its type, or as a new float32 matrix (fp32 accumulation in both)."""
    if out is None:
        return torch.mm(a, b, out_dtype=torch.float32)
    return torch.mm(a, b, out=out)


DEFAULT_NAMES = {"q": "q_proj.weight", "dkv": "kv_down_proj.weight", "dkv_norm": "kv_norm.weight",
                 "uk": "k_up_proj.weight", "uv": "v_up_proj.weight", "o": "o_proj.weight", "g": "gate_proj.weight"}
_UNSET = object()


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        self.hidden_size = int(hidden_size)
        self.heads, self.dim, self.rot_dim = int(spec["heads"]), int(spec["dim"]), int(spec["rot_dim"])
        self.vdim, self.rank = int(spec["vdim"]), int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        window = spec.get("window")
        self.window = int(window) if window else None
        kept = spec.get("cache_window", _UNSET)
        self.cache_window = self.window if kept is _UNSET else (int(kept) if kept else None)
        if self.cache_window is not None and (self.window is None or self.window > self.cache_window):
            raise ValueError("the window of a latent attention reaches beyond what its cache keeps")
        self.shares_cache = bool(shares_cache)
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        self.dtype = dtype
        rot = dict(spec.get("rot") or {})
        if self.heads < 1 or self.dim < 1 or self.vdim < 1 or not 1 <= self.rank <= 1024:
            raise ValueError("latent attention needs heads, dim, vdim >= 1 and a kv_rank between 1 and 1024")
        if self.rot_dim % 2 or self.rot_dim < 0 or (self.rot_dim and int(rot.get("dims", self.rot_dim)) != self.rot_dim):
            raise ValueError("rot_dim must be even and the rotation must cover all of it")
        if self.rot_dim:
            freq, self.amplitude = rotary_frequencies(self.rot_dim, float(rot["base"]), rot.get("scaling"))
            self.inv_freq = freq.to(device)
        else:
            self.inv_freq, self.amplitude = torch.zeros(0, dtype=torch.float32, device=device), 1.0
        self.q_head = self.dim + self.rot_dim
        self.q_width = self.heads * self.q_head
        self.row = self.rank + self.rot_dim
        self.interleaved = bool(rot.get("interleaved", False))
        self.gated = bool(spec.get("gate", False))
        self.gate_first = self.q_width + (0 if self.shares_cache else self.row)
        self.proj_width = self.gate_first + (self.heads if self.gated else 0)
        for name in ("proj", "norm_w", "uk_t", "uv", "out_w"):
            setattr(self, name, None)

    def cache_need(self) -> PagedKVNeed:
        # one row [c | r] per position, shared by all heads; the value of a key is the row's first kv_rank elements
        return PagedKVNeed(1, self.row, self.cache_window, value_dim=0)

    def scratch_per_token(self) -> int:
        return self.proj_width + self.heads * (self.row + self.rank) + self.heads * self.vdim + self.hidden_size

    def param_specs(self) -> list[ParamSpec]:
        n, h = self.names, self.hidden_size
        specs = [ParamSpec(n["q"], (self.q_width, h))]
        if not self.shares_cache:
            specs += [ParamSpec(n["dkv"], (self.row, h)), ParamSpec(n["dkv_norm"], (self.rank,), role="gain", init="one_plus_normal")]
        specs += [ParamSpec(n["uk"], (self.heads * self.dim, self.rank)), ParamSpec(n["uv"], (self.heads * self.vdim, self.rank))]
        if self.gated:
            specs.append(ParamSpec(n["g"], (self.heads, h)))
        specs.append(ParamSpec(n["o"], (h, self.heads * self.vdim)))
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        q_w = tensors[n["q"]]
        order = None
        if self.interleaved and self.rot_dim:  # pairs of neighbours become pairs half the part apart
            order = torch.cat([torch.arange(0, self.rot_dim, 2), torch.arange(1, self.rot_dim, 2)]).to(q_w.device)
            q_w = q_w.reshape(self.heads, self.q_head, -1)
            q_w = torch.cat([q_w[:, :self.dim], q_w[:, self.dim:][:, order]], dim=1).reshape(self.q_width, -1)
        stacked = [q_w]
        if not self.shares_cache:
            down = tensors[n["dkv"]]
            if order is not None:
                down = torch.cat([down[:self.rank], down[self.rank:][order]], dim=0)
            stacked.append(down)
            self.norm_w = tensors[n["dkv_norm"]].contiguous()
        if self.gated:
            stacked.append(tensors[n["g"]])
        self.proj = torch.cat(stacked, dim=0).contiguous()
        # [heads, rank, dim]: a head's rows are the columns of its Wuk, so that q~ = Wuk^T q_plain is a product by rows
        self.uk_t = tensors[n["uk"]].reshape(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].reshape(self.heads, self.vdim, self.rank).contiguous()
        self.out_w = tensors[n["o"]].contiguous()

    def _stretch(self) -> int:
        """Queries of one stretch of the matrix-product path, 0 where that path is never taken."""
        if self.dtype != torch.bfloat16 or self.window is None or self.row % 8 or self.rank % 8:
            return 0
        return max(16, min(512, STRETCH_ELEMENTS // (self.heads * (self.window + 512))))

    def _portions(self, carried, mixed, rows, weights, stretch, ctx, cache, table) -> None:
        """A step with long portions: those go stretch by stretch through two matrix products, the tokens of the
        other requests (runs of neighbours together) through the kernel."""
        batch = ctx.batch
        start = 0
        short_from = None

        def flush(upto: int) -> None:
            nonlocal short_from
            if short_from is not None and upto > short_from:
                a = short_from
                kernels.latent_attention(carried[a:upto], mixed[a:upto], cache.k_pages, table, batch.seq_of_token[a:upto],
                                         batch.positions[a:upto], upto - a, self.heads, self.rank, self.rot_dim, self.window,
                                         self.scale, ctx.status)
            short_from = None

        for index, (count, context) in enumerate(zip(batch.query_lens_host, batch.context_lens_host)):
            if count < PORTION_MIN:
                if short_from is None:
                    short_from = start
                start += count
                continue
            flush(start)
            first_position = context - count
            for offset in range(0, count, stretch):
                take = min(stretch, count - offset)
                a, position = start + offset, first_position + offset
                first_key = max(0, position - self.window + 1)
                num_keys = position + take - first_key
                padded = -(-num_keys // 8) * 8
                kernels.latent_gather(cache.k_pages, table[index], first_key, num_keys, rows, padded, ctx.status)
                scores = matrix_product(carried[a:a + take].view(take * self.heads, self.row), rows[:padded].t())
                share = weights[:take * self.heads * padded].view(take * self.heads, padded)
                kernels.latent_softmax(scores, share, self.heads, num_keys, position, first_key, self.window, self.scale)
                matrix_product(share, rows[:padded, :self.rank], out=mixed[a:a + take].view(take * self.heads, self.rank))
            start += count
        flush(start)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        batch = ctx.batch
        n = batch.num_tokens
        table = batch.block_tables[cache.group]
        projected = ctx.buffer("latent_attn.proj", (n, self.proj_width))
        linear(x, self.proj, projected, None, n, ctx)
        down = None if self.shares_cache else projected[:, self.q_width:self.gate_first]
        carried = ctx.buffer("latent_attn.q", (n, self.heads * self.row))  # per head [q~ | rotated part]
        kernels.latent_prepare(projected, down, self.norm_w, self.inv_freq, self.amplitude, batch.positions,
                               batch.seq_of_token, table, cache.k_pages, n, self.heads, self.dim, self.rot_dim, self.rank,
                               self.eps, ctx.status, packed=carried)
        kernels.head_linear(projected, self.q_head, self.uk_t, carried, self.row, n)
        mixed = ctx.buffer("latent_attn.mixed", (n, self.heads * self.rank))
        stretch = self._stretch()
        if stretch:  # asked for in every step, so that the dry run before the scratch is frozen sees them
            keys = -(-(self.window + stretch) // 8) * 8
            rows = ctx.buffer("latent_attn.rows", (keys, self.row))
            weights = ctx.buffer("latent_attn.weights", (stretch * self.heads * keys,))
        if stretch and batch.max_query_len >= PORTION_MIN:
            self._portions(carried, mixed, rows, weights, stretch, ctx, cache, table)
        else:
            kernels.latent_attention(carried, mixed, cache.k_pages, table, batch.seq_of_token, batch.positions, n, self.heads,
                                     self.rank, self.rot_dim, self.window, self.scale, ctx.status)
        values = ctx.buffer("latent_attn.values", (n, self.heads * self.vdim))
        kernels.head_linear(mixed, self.rank, self.uv, values, self.vdim, n,
                            gate=projected[:, self.gate_first:] if self.gated else None)
        out = ctx.buffer("latent_attn.out", (n, self.hidden_size))
        linear(values, self.out_w, out, None, n, ctx)
        return out


register_mixer("latent_attention", LatentAttention)
