"""Small Lorozen configurations for the tests, model folders made from them, and the comparison rule.

Five configurations that differ from one another in every size and option: attention with one, some and as many key
heads as query heads, head sizes from 10 to 64 with rotated parts of 2 elements up to the whole head, with and without
stretched frequencies, value rows narrower and wider than the keys, windows from 9 positions to none; latent attention
with ranks of 12 to 64 and rotated parts of 2 to 16 elements; wkv with one head and several; dense feed-forwards,
mixtures of 3 to 8 experts of which 1, 2 or all are chosen, with and without a shared expert, and layers without a
feed-forward; loops over the first layers, the last ones, all of them and none, run 1 to 3 times; widths that are no
multiple of 8; logits capped and not.

``sharpen`` rewrites a folder so that faults which random weights would hide show up: queries are scaled up until single
scores stand out in the softmax (a key at the far edge of a window then moves the output by a large part of it), the
sinks get values from -3 to 3 (so that in some heads the sink takes most of the weight and in others next to none), and
the wkv decays' offsets are so low that a state lost or mixed up hundreds of tokens earlier still shows in the output.

``steady_routing`` makes every router's choice a plain function of the token with wide margins, and
``steady_first_outputs`` keeps a wkv layer's output at a request's first token from hanging on the sign of a sum that
nearly cancels (see there): both are steps of the design that one rounding can turn round with nothing being wrong.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

ARCH = "Lorozen"


def attention(heads, kv_heads, dim, vdim, scale, window, base, dims, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    sizes = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot)
    if window:
        sizes["mask"] = {"size": window}
    return "attention", sizes


def latent(heads, dim, rot_dim, vdim, rank, scale, window, base):
    sizes = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale, rot={"base": base, "dims": rot_dim})
    if window:
        sizes["mask"] = {"size": window}
    return "latent_attention", sizes


def wkv(heads, dim, rank):
    return "wkv", dict(heads=heads, dim=dim, decay_rank=rank)


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind_and_mixer, mlp):
    return {"type": kind_and_mixer[0], "mixer": kind_and_mixer[1], "mlp": mlp}


def model(vocab, width, eps, layers, cap=None, loop=None):
    raw = {"architecture": ARCH, "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap:
        raw["logit_softcap"] = cap
    if loop:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


# a loop in the middle, run twice; every kind of mixer and feed-forward; key heads shared by two query heads
CASE_A = model(150, 96, 1e-5, [
    layer(attention(4, 2, 24, 20, 0.2, 40, 5000.0, 8, (8.0, 1.0, 4.0, 64)), moe(6, 2, 40, 56)),
    layer(wkv(3, 16, 8), dense(112)),
    layer(latent(3, 16, 8, 24, 40, 0.15, 33, 1000.0), moe(5, 1, 24, 16)),
    layer(attention(2, 2, 16, 16, 0.25, 17, 100.0, 16), None),
], cap=20.0, loop=(1, 3, 2))
# no loop, no cap, no windows in two layers; one key head for eight query heads; all experts chosen; no shared expert
CASE_B = model(140, 64, 1e-6, [
    layer(wkv(1, 64, 24), moe(4, 4, 16)),
    layer(attention(8, 1, 16, 8, 0.3, None, 1000.0, 4), dense(128)),
    layer(latent(2, 24, 2, 8, 16, 0.2, None, 50.0), None),
    layer(latent(4, 8, 16, 16, 24, 0.35, 9, 20000.0), moe(3, 1, 32, 8)),
])
# everything odd: a width that is no multiple of 8, head sizes of 10 and 7, a rank of 12, a loop over the last layers run
# three times
CASE_C = model(77, 100, 1e-6, [
    layer(wkv(5, 6, 3), dense(52)),
    layer(attention(3, 3, 10, 7, 0.4, 25, 50.0, 2, (2.0, 0.5, 3.0, 16)), moe(3, 3, 20, 12)),
    layer(latent(5, 6, 4, 10, 12, 0.3, 21, 300.0), dense(36)),
], cap=7.5, loop=(1, 3, 3))
# sizes of the tensor-core kernels: heads of 64 and 32, windows longer than a tile; a loop from the first layer on
CASE_D = model(260, 128, 1e-5, [
    layer(attention(8, 2, 64, 64, 0.11, 100, 10000.0, 32, (3.0, 1.0, 5.0, 128)), moe(8, 2, 64, 96)),
    layer(latent(4, 32, 16, 32, 64, 0.14, 70, 80000.0), dense(192)),
    layer(wkv(2, 64, 16), moe(8, 1, 32, 64)),
    layer(wkv(4, 32, 12), None),
    layer(attention(4, 4, 32, 48, 0.18, 130, 300.0, 12), dense(40)),
], cap=25.0, loop=(0, 2, 3))
# the whole model is the loop, run twice; a loop that runs once changes nothing
CASE_E = model(90, 72, 1e-5, [
    layer(latent(3, 8, 8, 8, 16, 0.25, 12, 100.0), moe(4, 2, 24, 24)),
    layer(attention(6, 3, 12, 12, 0.28, 11, 10.0, 12), dense(48)),
], cap=12.0, loop=(0, 2, 2))
CASES = {"A": (CASE_A, 51), "B": (CASE_B, 52), "C": (CASE_C, 53), "D": (CASE_D, 54), "E": (CASE_E, 55)}


def write_case(name: str, folder: Path, sharp: bool = False, steady: bool = False) -> Path:
    raw, seed = CASES[name]
    return write_raw(raw, seed, folder, sharp, steady)


def one_layer(kind_and_mixer, mlp=None, width=64, vocab=90, eps=1e-5, cap=None) -> dict:
    """A model of one layer around one mixer (and no feed-forward unless given): a mechanism alone."""
    return model(vocab, width, eps, [layer(kind_and_mixer, mlp)], cap=cap)


def write_raw(raw: dict, seed: int, folder: Path, sharp: bool = False, steady: bool = False) -> Path:
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.weights import write_random_model

    write_random_model(config_from_dict(raw), seed, folder, torch.bfloat16)
    written = read_config(folder)
    for entry in written["layers"]:  # a folder does not say how wide the decay's pair is: the tensors' shapes do
        entry["mixer"].pop("decay_rank", None)
    (Path(folder) / "config.json").write_text(json.dumps(written))
    steady_first_outputs(folder)
    if sharp:
        sharpen(folder)
    if steady:
        steady_routing(folder)
    return folder


def _rewrite(folder: Path, change) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(folder) / "model.safetensors"
    tensors = load_file(str(path))
    change(tensors)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path), metadata={"format": "pt"})


def steady_first_outputs(folder: Path) -> None:
    """Keep a wkv layer's output at a request's first token away from a coin toss.

    There the state is empty and a head gives ``(sum_k r_k u_k k_k) v``: one vector times a sum that, with random signs,
    nearly cancels for one token in a hundred. The norm behind the mixer brings the output to unit size however small it
    is, so whether such a sum comes out just above or just below zero (which one rounding to bfloat16 decides) turns
    the whole update round, with nothing being wrong. The folders of the tests therefore get receptance matrices that
    are the key matrices plus a part of their own, and positive bonuses: the sum is then mostly one of squares."""
    def change(tensors):
        for name in list(tensors):
            if name.endswith(".mix.r") and name[:-1] + "k" in tensors and name[:-1] + "u" in tensors:
                tensors[name] = (tensors[name[:-1] + "k"].float() + 0.5 * tensors[name].float()).to(torch.bfloat16)
                tensors[name[:-1] + "u"] = (0.5 + 4.0 * tensors[name[:-1] + "u"].float().abs()).to(torch.bfloat16)

    _rewrite(folder, change)


def sharpen(folder: Path) -> None:
    def change(tensors):
        for name in list(tensors):
            if name.endswith(".mix.q") or name.endswith(".mix.q.b") or name.endswith(".mix.uk"):
                tensors[name] = (tensors[name].float() * 4.0).to(torch.bfloat16)
            if name.endswith(".mix.sink"):
                heads = tensors[name].numel()
                tensors[name] = torch.linspace(-3.0, 3.0, heads).to(torch.bfloat16) if heads > 1 else torch.tensor([1.5], dtype=torch.bfloat16)
            if name.endswith(".mix.w0"):
                tensors[name] = (tensors[name].float() - 5.0).to(torch.bfloat16)

    _rewrite(folder, change)


def steady_routing(folder: Path) -> None:
    """Make every router's choice a plain function of the token, with wide margins.

    A choice among experts is a step function of the stream: where two scores nearly tie, rounding to bfloat16 takes
    the other expert and the logits of that position (and, through states and cached rows, of later ones) move by far
    more than any tolerance, with nothing being wrong. Comparisons in bfloat16 therefore run on folders rewritten here:
    the first ``tags`` elements of the stream carry a code of the token (a permutation of 1, 2, 3, ... per token); the
    norms behind the sublayers have weight zero there, so no sublayer ever adds to them (a further pass of a loop adds
    the code itself once more, which keeps its order); the norm before a mixture has weight one there, and every router
    reads expert ``e``'s logit from element ``e``. The norm divides all of them by one number, so the order of the
    scores is the code's, a step apart, whatever the rounding.
    """
    config = read_config(folder)
    tags = max([entry["mlp"]["router"]["experts"] for entry in config["layers"] if (entry.get("mlp") or {}).get("kind") == "moe"] or [0])
    if not tags:
        return

    def change(tensors):
        g = torch.Generator().manual_seed(99)
        code = torch.stack([torch.randperm(tags, generator=g) for _ in range(config["vocab"])]).float() + 1.0
        embed = tensors["embed"].float()
        embed[:, :tags] = code * 0.5
        tensors["embed"] = embed.to(torch.bfloat16)
        for name in list(tensors):
            if name.endswith(".norm1b") or name.endswith(".norm2b") or name.endswith(".norm2"):
                weight = tensors[name].float()
                weight[:tags] = 1.0 if name.endswith(".norm2") else 0.0
                tensors[name] = weight.to(torch.bfloat16)
            if name.endswith(".mlp.router"):
                router = torch.zeros_like(tensors[name].float())
                for e in range(router.shape[0]):
                    router[e, e] = 1.0
                tensors[name] = router.to(torch.bfloat16)

    _rewrite(folder, change)


def read_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


FP32_REL = 3e-5
"""float32 engine against the float64 plain implementation: root mean square of the difference of a
position's logits (their mean taken off) over the root mean square of the plain logits of the
request. Every sum of the engine is float32."""

BF16_REL = 0.1
"""The same in bfloat16: activations are rounded to 8 bits of mantissa between kernels; statistics, scores, states and
the residual stream are float32. Every sublayer's output is normed to unit size before it is added, so a rounding of
0.4 % in a small output weighs as much as in a large one, and a model runs up to fourteen such sublayers; the plain
implementation itself moves by 0.01 (median) to 0.15 (its touchiest positions) under one such rounding a sublayer. A fault of the cache, a state, a window or a sink moves a
position by 0.3 and more (``test_the_sharp_weights_do_make_single_keys_and_old_state_count``)."""


def relative_error(ours: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per position: rms over the vocabulary of (ours - ref), mean taken off, over the rms of ref."""
    diff = ours.double() - ref.double()
    diff = diff - diff.mean(-1, keepdim=True)
    centred = ref.double() - ref.double().mean(-1, keepdim=True)
    return diff.pow(2).mean(-1).sqrt() / centred.pow(2).mean().sqrt()


JITTER = {"bfloat16": 2.0 ** -8, "float32": 2.0 ** -20}
"""Relative noise on every sublayer's input and output in the plain implementation's shaken run: one rounding of
bfloat16's 8 bits; for float32 sixteen roundings of 24 bits (a sublayer is several kernels, each a sum of many terms)."""


def check(ours: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, slack: float = 1.0, shaken: torch.Tensor | None = None) -> None:
    """``shaken``: the plain logits under relative noise of ``JITTER``. Where they move far a position is touchy by the
    design itself (every sublayer's output is brought to unit size, however small it was; a softmax may hang on two
    scores that nearly tie) and gets three times that much more room."""
    assert ours.shape == ref.shape, f"{what}: shape {tuple(ours.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(ours).all(), f"{what}: non-finite logits"
    error = relative_error(ours, ref)
    bound = torch.full_like(error, (FP32_REL if dtype == "float32" else BF16_REL) * slack)
    if shaken is not None:
        bound = bound + 3.0 * relative_error(shaken, ref)
    over = error - bound
    worst = int(over.argmax())
    assert float(over.max()) <= 0.0, f"{what}: relative error {float(error[worst]):.3e} at position {worst} (bound {float(bound[worst]):.1e})"
