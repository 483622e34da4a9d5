"""The Begovik design in float64, written from its equations alone: one function per mechanism.

Nothing here is shared with the package: no kernels, no parts, no cache. A sequence is computed
whole, position by position where the design is a recurrence, so it is slow and plain.

Notation: ``h`` [T, width] is a mixer's input, weights are stored ``[out, in]`` and applied as
``h @ W.T``; a mixer's weights arrive as a dict by their local names (``q``, ``left.q.norm``, ...).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_pairs(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """``x`` [T, heads, d]: elements (2i, 2i + 1), i < dims / 2, of every head turn by ``t * base^(-2i / dims)``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    tokens = x.shape[0]
    index = torch.arange(dims // 2, dtype=F64)
    angle = torch.arange(tokens, dtype=F64)[:, None] * base ** (-2.0 * index / dims)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def sink_attention(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """Causal softmax attention with normed and rotated queries and keys, capped scores, and a
    sink: an extra score of zero in the denominator that carries no value."""
    heads, kv_heads, dim, vdim = int(sizes["heads"]), int(sizes["kv_heads"]), int(sizes["dim"]), int(sizes["vdim"])
    tokens = h.shape[0]
    q = rms_norm((h @ w["q"].T).reshape(tokens, heads, dim), w["q.norm"], eps)
    k = rms_norm((h @ w["k"].T).reshape(tokens, kv_heads, dim), w["k.norm"], eps)
    v = (h @ w["v"].T).reshape(tokens, kv_heads, vdim)
    if sizes.get("rot") and int(sizes["rot"].get("dims", 0)):
        q, k = rotate_pairs(q, sizes["rot"]), rotate_pairs(k, sizes["rot"])
    per = heads // kv_heads
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * float(sizes["scale"])
    positions = torch.arange(tokens)
    weights = capped_sink_weights(scores, sizes.get("softcap"), positions[:, None] >= positions[None, :])
    return torch.einsum("hts,shv->thv", weights, v).reshape(tokens, heads * vdim) @ w["o"].T


def capped_sink_weights(scores: torch.Tensor, cap, seen: torch.Tensor) -> torch.Tensor:
    """``p_j = exp(s_j) / (1 + sum_i exp(s_i))`` over the keys that are ``seen``, with ``s = cap tanh(score / cap)``
    when there is a cap: the weights of a row add up to less than one, the rest is the sink's."""
    if cap:
        scores = float(cap) * torch.tanh(scores / float(cap))
    weights = torch.exp(scores).masked_fill(~seen, 0.0)
    return weights / (1.0 + weights.sum(dim=-1, keepdim=True))


def lightning_attention(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with silu on q, k and v; the heads side by
    side are normed together, gated by a sigmoid and projected."""
    heads, dim, vdim = int(sizes["heads"]), int(sizes["dim"]), int(sizes["vdim"])
    tokens = h.shape[0]
    q = silu(h @ w["q"].T).reshape(tokens, heads, dim)
    k = silu(h @ w["k"].T).reshape(tokens, heads, dim)
    v = silu(h @ w["v"].T).reshape(tokens, heads, vdim)
    decay = torch.tensor([float(d) for d in sizes["decay"]], dtype=F64)
    state = torch.zeros(heads, dim, vdim, dtype=F64)
    out = torch.zeros(tokens, heads, vdim, dtype=F64)
    for t in range(tokens):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    out = rms_norm(out.reshape(tokens, heads * vdim), w["norm"], eps)
    return (out * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def side_by_side(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """Both mixers read ``h``; each output is normed over the width, and the result is half their sum."""
    left = sink_attention(h, {n[5:]: t for n, t in w.items() if n.startswith("left.")}, sizes["left"], eps)
    right = lightning_attention(h, {n[6:]: t for n, t in w.items() if n.startswith("right.")}, sizes["right"], eps)
    return 0.5 * (rms_norm(left, w["left.out"], eps) + rms_norm(right, w["right.out"], eps))


def wkv(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """Time mixing with a decay per head and key channel that the input chooses, and a bonus for the current token."""
    heads, dim = int(sizes["heads"]), int(sizes["dim"])
    tokens = h.shape[0]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mixed(which: str) -> torch.Tensor:
        return h + (before - h) * w["mu." + which]

    r = (mixed("r") @ w["r"].T).reshape(tokens, heads, dim)
    k = (mixed("k") @ w["k"].T).reshape(tokens, heads, dim)
    v = (mixed("v") @ w["v"].T).reshape(tokens, heads, -1)
    gate = silu(mixed("g") @ w["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed("w") @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(tokens, heads, dim)
    bonus = w["u"].reshape(heads, dim)
    state = torch.zeros(heads, dim, v.shape[-1], dtype=F64)
    out = torch.zeros(tokens, heads, v.shape[-1], dtype=F64)
    for t in range(tokens):
        now = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state + bonus[:, :, None] * now, r[t])
        state = decay[t][:, :, None] * state + now
    out = rms_norm(out, None, eps).reshape(tokens, -1)
    return (out * w["norm"] * gate) @ w["o"].T


def mamba1(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """The selective scan: a state per channel and state index, step sizes and B, C chosen by the input."""
    inner, states, rank, taps = int(sizes["inner"]), int(sizes["state"]), int(sizes["dt_rank"]), int(sizes["conv"])
    tokens = h.shape[0]
    both = h @ w["in"].T
    x, z = both[:, :inner], both[:, inner:]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=F64), x], dim=0)
    conv = torch.zeros_like(x) + w["conv.b"]
    for j in range(taps):  # the last column multiplies the current token
        conv = conv + padded[j:j + tokens] * w["conv"][:, j]
    x = silu(conv)
    low = x @ w["x"].T
    dt = softplus(low[:, :rank] @ w["dt"].T + w["dt.b"])
    b, c = low[:, rank:rank + states], low[:, rank + states:rank + 2 * states]
    a = -torch.exp(w["A_log"])
    state = torch.zeros(inner, states, dtype=F64)
    y = torch.zeros(tokens, inner, dtype=F64)
    for t in range(tokens):
        state = torch.exp(dt[t][:, None] * a) * state + (dt[t] * x[t])[:, None] * b[t][None, :]
        y[t] = state @ c[t] + w["D"] * x[t]
    return (y * silu(z)) @ w["o"].T


def clamped_feed_forward(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


MIXERS = {"parallel": side_by_side, "wkv": wkv, "mamba1": mamba1}


def part(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t.to(F64) for name, t in weights.items() if name.startswith(prefix)}


def forward(config: dict, weights: dict, tokens: list[int], jitter: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Logits [T, vocab] and the stream after every layer [layers, T, width].

    ``jitter``: every sublayer's input and output is multiplied by ``1 + jitter * noise`` (unit normal noise per
    element): how far a position's logits move under relative errors of that size, as rounding to a short
    mantissa makes them."""
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    noise = torch.Generator().manual_seed(7)

    def shaken(t: torch.Tensor) -> torch.Tensor:
        return t * (1.0 + jitter * torch.randn(t.shape, generator=noise, dtype=F64)) if jitter else t

    x = weights["embed"].to(F64)[torch.tensor(tokens)] * float(config["embedding"]["scale"])
    after = []
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        update = shaken(MIXERS[layer["type"]](shaken(rms_norm(x, weights[name + "norm1"].to(F64), eps)), part(weights, name + "mix."),
                                              layer["mixer"], eps))
        if layer.get("mlp"):
            update = update + shaken(clamped_feed_forward(shaken(rms_norm(x, weights[name + "norm2"].to(F64), eps)),
                                                          part(weights, name + "mlp."), layer["mlp"]))
        x = x + mult * update
        after.append(x)
    final = rms_norm(x, weights["final.norm"].to(F64), eps)
    return final @ weights["head"].to(F64).T, torch.stack(after)


def logits_of(config: dict, weights: dict, tokens: list[int]) -> torch.Tensor:
    return forward(config, weights, tokens)[0]


def greedy(config: dict, weights: dict, prompt: list[int], count: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(logits_of(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


def read_model_folder(folder):
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))
