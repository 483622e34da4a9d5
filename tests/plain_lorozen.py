"""The Lorozen design in float64, written from its equations alone: one function per mechanism.

Nothing here is shared with the package: no kernels, no parts, no cache. A sequence is computed
whole, position by position where the design is a recurrence, so it is slow and plain.

Notation: ``h`` [T, width] is a sublayer's input, weights are stored ``[out, in]`` and applied as
``h @ W.T``; a sublayer's weights arrive as a dict by their local names (``q``, ``q.b``, ``mu.r``, ...).
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64

_SHAKE: list = []
"""While a shaken run is under way: ``[jitter, generator]``. :func:`made` then multiplies what a matrix product gives,
element by element, by ``1 + jitter * noise``: what arithmetic that rounds such results to that precision may do."""


def made(t: torch.Tensor) -> torch.Tensor:
    """The result of a matrix product (or a sublayer's input or output): itself, or shaken in a shaken run."""
    if not _SHAKE:
        return t
    return t * (1.0 + _SHAKE[0] * torch.randn(t.shape, generator=_SHAKE[1], dtype=F64))


def rms_norm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot: dict) -> torch.Tensor:
    """``f_i = base^(-2i / dims)``; with ``scaling`` the long waves are stretched: a wave longer than
    ``original / low`` turns ``factor`` times slower, one shorter than ``original / high`` is kept, and
    between them the two are blended by where ``original / wavelength`` lies between ``low`` and ``high``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[key]) for key in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(f.numel()):
        wave = 2.0 * math.pi / float(f[i])
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = f[i] / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def rotate(x: torch.Tensor, rot: dict | None, interleaved: bool, first_position: int = 0) -> torch.Tensor:
    """``x`` [T, heads, d]: the first ``dims`` elements of every head turn by ``position * f_i``; pair ``i`` is
    elements ``(2i, 2i + 1)`` when ``interleaved``, else ``(i, i + dims / 2)``; the rest pass unchanged."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    tokens = x.shape[0]
    angle = (first_position + torch.arange(tokens, dtype=F64))[:, None] * frequencies(rot)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    if interleaved:
        a, b = slice(0, dims, 2), slice(1, dims, 2)
    else:
        a, b = slice(0, dims // 2), slice(dims // 2, dims)
    out = x.clone()
    out[..., a] = x[..., a] * cos - x[..., b] * sin
    out[..., b] = x[..., b] * cos + x[..., a] * sin
    return out


def seen(tokens: int, window: int | None) -> torch.Tensor:
    """[T, T] bool: position ``i`` sees ``j`` with ``0 <= i - j < window`` (all before it without a window)."""
    back = torch.arange(tokens)[:, None] - torch.arange(tokens)[None, :]
    mask = back >= 0
    return mask if not window else mask & (back < int(window))


def window_of(sizes: dict) -> int | None:
    mask = sizes.get("mask") or {}
    return int(mask["size"]) if mask.get("size") else None


def attention(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """Grouped-query attention with biases, a rotation of split pairs, a window, and a learned sink per head:
    ``p_j = exp(s_j) / (exp(sink) + sum_i exp(s_i))``."""
    heads, kv_heads = int(sizes["heads"]), int(sizes.get("kv_heads") or sizes["heads"])
    dim, vdim = int(sizes["dim"]), int(sizes.get("vdim") or sizes["dim"])
    tokens = h.shape[0]
    q = made(h @ w["q"].T + w["q.b"]).reshape(tokens, heads, dim)
    k = made(h @ w["k"].T + w["k.b"]).reshape(tokens, kv_heads, dim)
    v = made(h @ w["v"].T + w["v.b"]).reshape(tokens, kv_heads, vdim)
    q, k = rotate(q, sizes.get("rot"), False), rotate(k, sizes.get("rot"), False)
    per = heads // kv_heads
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * float(sizes["scale"])
    scores = scores.masked_fill(~seen(tokens, window_of(sizes)), -math.inf)
    sink = w["sink"].reshape(heads, 1, 1).expand(heads, tokens, 1)
    weights = torch.softmax(torch.cat([scores, sink], dim=-1), dim=-1)[..., :tokens]
    return made(torch.einsum("hts,shv->thv", weights, v).reshape(tokens, heads * vdim)) @ w["o"].T


def latent_attention(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """Keys and values of all heads from one normed latent per position, one rotated key part for all heads
    (pairs of neighbours turn), a window, an ordinary softmax, and a sigmoid gate per head on the output."""
    heads, dim, rot_dim = int(sizes["heads"]), int(sizes["dim"]), int(sizes["rot_dim"])
    vdim, rank = int(sizes["vdim"]), int(sizes["kv_rank"])
    tokens = h.shape[0]
    q = made(h @ w["q"].T).reshape(tokens, heads, dim + rot_dim)
    down = made(h @ w["dkv"].T)
    latent = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    shared = rotate(down[:, None, rank:], sizes.get("rot"), True)[:, 0]
    q_plain, q_turned = q[..., :dim], rotate(q[..., dim:], sizes.get("rot"), True)
    keys = (latent @ w["uk"].T).reshape(tokens, heads, dim)
    values = (latent @ w["uv"].T).reshape(tokens, heads, vdim)
    scores = (torch.einsum("thd,shd->hts", q_plain, keys) + torch.einsum("thd,sd->hts", q_turned, shared)) * float(sizes["scale"])
    scores = scores.masked_fill(~seen(tokens, window_of(sizes)), -math.inf)
    mixed = torch.einsum("hts,shv->thv", torch.softmax(scores, dim=-1), values)
    gate = torch.sigmoid(made(h @ w["g"].T))  # [T, heads]
    return made((mixed * gate[:, :, None]).reshape(tokens, heads * vdim)) @ w["o"].T


def wkv(h: torch.Tensor, w: dict, sizes: dict, eps: float) -> torch.Tensor:
    """Time mixing: five blends with the token before, a decay per head and key channel that the input chooses,
    a bonus for the current token, a norm per head, a gate."""
    heads, dim = int(sizes["heads"]), int(sizes["dim"])
    tokens = h.shape[0]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    blend = {s: h + (before - h) * w["mu." + s] for s in "rkvgw"}
    r = made(blend["r"] @ w["r"].T).reshape(tokens, heads, dim)
    k = made(blend["k"] @ w["k"].T).reshape(tokens, heads, dim)
    v = made(blend["v"] @ w["v"].T).reshape(tokens, heads, dim)
    gate = silu(made(blend["g"] @ w["g"].T))
    decay = torch.exp(-torch.exp(made(torch.tanh(made(blend["w"] @ w["w1"].T))) @ w["w2"].T + w["w0"])).reshape(tokens, heads, dim)
    bonus = w["u"].reshape(heads, dim)
    state = torch.zeros(heads, dim, dim, dtype=h.dtype)  # [head, key channel, value channel]
    out = torch.zeros(tokens, heads, dim, dtype=h.dtype)
    for t in range(tokens):
        outer = k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state + bonus[:, :, None] * outer, r[t])
        state = decay[t, :, :, None] * state + outer
    out = rms_norm(out, None, eps).reshape(tokens, heads * dim) * w["norm"] * gate
    return made(out) @ w["o"].T


def gated(h: torch.Tensor, w: dict, prefix: str, act) -> torch.Tensor:
    return made(act(made(h @ w[prefix + "gate"].T)) * made(h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h: torch.Tensor, router: torch.Tensor, top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Scores are sigmoids of the router's logits; the ``top`` largest are chosen and used as they are."""
    scores = torch.sigmoid(h @ router.T)
    weights, chosen = torch.topk(scores, top, dim=-1)
    return chosen, weights


def mixture(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    """Every token goes through its chosen experts, scaled by the expert's score on the way IN, and through the
    shared expert."""
    chosen, weights = route(h, w["router"], int(mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weights[t]):
            out[t] += gated(s * h[t:t + 1], w, f"e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + gated(h, w, "shared.", silu)
    return out


def feed_forward(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return gated(h, w, "", gelu_tanh)
    return mixture(h, w, mlp)


MIXERS = {"attention": attention, "latent_attention": latent_attention, "wkv": wkv}


def part(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in weights.items() if name.startswith(prefix)}


def run_order(config: dict) -> list[tuple[int, bool]]:
    """(layer, whether the embedding's output is added right before it) for every layer run."""
    count = len(config["layers"])
    loop = config.get("loop") or {}
    start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
    if stop <= start:
        return [(i, False) for i in range(count)]
    order = [(i, False) for i in range(start)]
    for again in range(times):
        order += [(i, again > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, count)]


def forward(config: dict, weights: dict, tokens: list[int], jitter: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Logits [T, vocab] and the stream after every layer run [runs, T, width], both float64.

    With ``jitter`` the run is shaken: every sublayer's input and output and the result of every matrix product within
    one is multiplied, element by element, by ``1 + jitter * noise`` (standard normal noise from a fixed seed)."""
    if jitter:
        _SHAKE[:] = [float(jitter), torch.Generator().manual_seed(1234)]
    try:
        return _forward(config, weights, tokens)
    finally:
        _SHAKE.clear()


def _forward(config: dict, weights: dict, tokens: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    w = {name: t.to(F64) for name, t in weights.items()}
    eps = float(config["norm"]["eps"])
    embedded = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = embedded.clone()
    streams = []
    for index, again in run_order(config):
        layer = config["layers"][index]
        if again:
            x = x + embedded
        own = part(w, f"l{index}.")
        mixed = MIXERS[layer["type"]](made(rms_norm(x, own["norm1"], eps)), part(own, "mix."), layer["mixer"], eps)
        x = x + rms_norm(made(mixed), own["norm1b"], eps)
        if layer.get("mlp"):
            moved = feed_forward(made(rms_norm(x, own["norm2"], eps)), part(own, "mlp."), layer["mlp"])
            x = x + rms_norm(made(moved), own["norm2b"], eps)
        streams.append(x.clone())
    logits = made(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits, torch.stack(streams)


def logits_of(config: dict, weights: dict, tokens: list[int]) -> torch.Tensor:
    return forward(config, weights, tokens)[0]


def greedy(config: dict, weights: dict, prompt: list[int], count: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(torch.argmax(logits_of(config, weights, tokens)[-1])))
    return tokens[len(prompt):]


def read_model_folder(folder):
    """config.json and model.safetensors of a folder, read with nothing but the file format: eight bytes of
    length, that many of JSON (name -> dtype, shape, data_offsets), then the data."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    blob = (folder / "model.safetensors").read_bytes()
    (length,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + length])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16, "F64": torch.float64}
    weights = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        a, b = entry["data_offsets"]
        data = torch.frombuffer(bytearray(blob[8 + length + a:8 + length + b]), dtype=kinds[entry["dtype"]])
        weights[name] = data.reshape(entry["shape"]).clone()
    return config, weights
