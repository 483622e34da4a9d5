"""Small Begovik configurations for the tests, model folders made from them, and the comparison rule.

Four configurations that differ from one another in every size and option: attention with one, some and as many
key heads as query heads, head sizes from 8 to 64 with rotated parts of 2 elements up to the whole head, value rows
narrower and wider than the keys, caps of 5 to 30, lightning heads of 6 to 128 elements, wkv with one head and
several and decay pairs of rank 3 to 24, selective scans with 3 to 32 states, step-size ranks of 1 to 8 and
convolutions of 1 to 4 taps, layers without a feed-forward, limits below and above 1, widths that are no multiple
of 8, and embedding scales and residual factors that are 1 and that are not.

``sharpen`` rewrites a folder so that faults which random weights would hide show up: the weights of the query norm
are scaled up until single scores stand out in the softmax (a key hundreds of positions back then moves the output
by a large part of it, and the sink's share changes from position to position), the lightning decays lie close to
1, the wkv decays' offsets are so low and the scan's step sizes so small that a state lost or mixed up hundreds of
tokens earlier still shows in the output.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def left(heads, kv_heads, dim, vdim, scale, softcap, base, dims):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap, rot={"base": base, "dims": dims})


def right(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def parallel(left_sizes, right_sizes):
    return "parallel", {"left": left_sizes, "right": right_sizes}


def wkv(heads, dim, rank):
    return "wkv", dict(heads=heads, dim=dim, decay_rank=rank)


def mamba1(inner, state, dt_rank, conv):
    return "mamba1", dict(inner=inner, state=state, dt_rank=dt_rank, conv=conv)


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(kind_and_mixer, mlp):
    return {"type": kind_and_mixer[0], "mixer": kind_and_mixer[1], "mlp": mlp}


CASE_A = {
    "architecture": "Begovik", "vocab": 190, "width": 96, "embedding": {"scale": 3.0}, "residual_mult": 0.7, "norm": {"eps": 1e-5},
    "layers": [
        layer(parallel(left(4, 2, 24, 20, 0.2, 30.0, 5000.0, 8), right(3, 16, 24, (0.9, 0.97, 0.995))), dense(112, 2.0)),
        layer(wkv(3, 16, 8), None),
        layer(mamba1(80, 12, 6, 4), dense(64, 0.5)),
        layer(parallel(left(2, 2, 16, 48, 0.25, 10.0, 100.0, 16), right(1, 8, 64, (0.98,))), dense(72, 1.5)),
    ],
}
# factors that are 1, one head, one key head for eight query heads, a layer order that starts with the scan
CASE_B = {
    "architecture": "Begovik", "vocab": 140, "width": 64, "embedding": {"scale": 1.0}, "residual_mult": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        layer(mamba1(64, 16, 8, 2), None),
        layer(wkv(1, 64, 24), dense(128, 1.0)),
        layer(parallel(left(8, 1, 8, 8, 0.3, 20.0, 1000.0, 4), right(2, 40, 10, (0.95, 0.99))), None),
        layer(mamba1(100, 5, 3, 3), dense(48, 3.0)),
    ],
}
# everything odd: widths that are no multiple of 8, a convolution of one tap, a rank of one
CASE_C = {
    "architecture": "Begovik", "vocab": 77, "width": 100, "embedding": {"scale": 0.6}, "residual_mult": 1.3, "norm": {"eps": 1e-6},
    "layers": [
        layer(wkv(5, 6, 3), dense(52, 0.8)),
        layer(parallel(left(3, 3, 10, 7, 0.4, 5.0, 50.0, 2), right(5, 6, 9, (0.9, 0.92, 0.94, 0.96, 0.98))), dense(36, 1.2)),
        layer(mamba1(36, 3, 1, 1), dense(20, 0.3)),
    ],
}
CASE_D = {
    "architecture": "Begovik", "vocab": 260, "width": 128, "embedding": {"scale": 7.5}, "residual_mult": 0.4, "norm": {"eps": 1e-5},
    "layers": [
        layer(parallel(left(8, 2, 64, 32, 0.125, 20.0, 10000.0, 32), right(4, 128, 32, (0.96, 0.98, 0.99, 0.999))), dense(192, 1.0)),
        layer(mamba1(256, 32, 8, 4), dense(96, 2.0)),
        layer(wkv(2, 64, 16), dense(64, 1.0)),
        layer(wkv(4, 32, 12), None),
        layer(parallel(left(4, 4, 32, 40, 0.18, 8.0, 300.0, 12), right(2, 24, 80, (0.97, 0.9925))), dense(40, 0.7)),
    ],
}
CASES = {"A": (CASE_A, 41), "B": (CASE_B, 42), "C": (CASE_C, 43), "D": (CASE_D, 44)}


def write_case(name: str, folder: Path, sharp: bool = False) -> Path:
    raw, seed = CASES[name]
    return write_raw(raw, seed, folder, sharp)


def one_layer(kind_and_mixer, mlp=None, width=64, vocab=90, scale=2.0, mult=0.8, eps=1e-5) -> dict:
    """A model of one layer around one mixer (and no feed-forward unless given): a mechanism alone."""
    return {"architecture": "Begovik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "residual_mult": mult,
            "norm": {"eps": eps}, "layers": [layer(kind_and_mixer, mlp)]}


def write_raw(raw: dict, seed: int, folder: Path, sharp: bool = False) -> Path:
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.weights import write_random_model

    if sharp:
        raw = json.loads(json.dumps(raw))
        for entry in raw["layers"]:
            if entry["type"] == "parallel":
                heads = entry["mixer"]["right"]["heads"]
                entry["mixer"]["right"]["decay"] = [1.0 - 0.004 / (i + 1) for i in range(heads)]
    write_random_model(config_from_dict(raw), seed, folder, torch.bfloat16)
    written = read_config(folder)
    for entry in written["layers"]:  # a folder does not say how wide the decay's pair is: the tensors' shapes do
        entry["mixer"].pop("decay_rank", None)
    (Path(folder) / "config.json").write_text(json.dumps(written))
    if sharp:
        sharpen(folder)
    return folder


def sharpen(folder: Path) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(folder) / "model.safetensors"
    tensors = load_file(str(path))
    for name in list(tensors):
        if name.endswith(".left.q.norm"):
            tensors[name] = (tensors[name].float() * 4.0).to(torch.bfloat16)
        if name.endswith(".mix.w0"):
            tensors[name] = (tensors[name].float() - 5.0).to(torch.bfloat16)
        if name.endswith(".mix.dt.b"):
            tensors[name] = (tensors[name].float() - 4.0).to(torch.bfloat16)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path), metadata={"format": "pt"})


def read_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


FP32_REL = 3e-5
"""float32 engine against the float64 plain implementation: root mean square of the difference of a
position's logits (their mean taken off) over the root mean square of the plain logits of the
request. Every sum of the engine is float32."""

BF16_REL = 0.06
"""The same in bfloat16: activations are rounded to 8 bits of mantissa between kernels; statistics, scores,
states and the residual stream are float32. A fault of the cache, a state or a slot moves a position by 0.3
and more (``test_the_sharp_weights_do_make_single_keys_and_old_state_count``)."""


def relative_error(ours: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per position: rms over the vocabulary of (ours - ref), mean taken off, over the rms of ref."""
    diff = ours.double() - ref.double()
    diff = diff - diff.mean(-1, keepdim=True)
    centred = ref.double() - ref.double().mean(-1, keepdim=True)
    return diff.pow(2).mean(-1).sqrt() / centred.pow(2).mean().sqrt()


JITTER = 2.0 ** -8
"""Relative noise on every sublayer's input and output in the plain implementation's shaken run (bfloat16 has 8 bits)."""


def check(ours: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, slack: float = 1.0, shaken: torch.Tensor | None = None) -> None:
    """``shaken``: the plain logits under relative noise of ``JITTER``. Where they move far a position is touchy by the
    design itself (a head's output of nearly no length brought to unit length, say) and gets that much more room."""
    assert ours.shape == ref.shape, f"{what}: shape {tuple(ours.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(ours).all(), f"{what}: non-finite logits"
    error = relative_error(ours, ref)
    bound = torch.full_like(error, (FP32_REL if dtype == "float32" else BF16_REL) * slack)
    if shaken is not None:
        bound = bound + 3.0 * relative_error(shaken, ref)
    over = error - bound
    worst = int(over.argmax())
    assert float(over.max()) <= 0.0, f"{what}: relative error {float(error[worst]):.3e} at position {worst} (bound {float(bound[worst]):.1e})"
