"""Typed configuration of the Begovik decoder, read from its ``config.json``.

Begovik is a small hybrid decoder. A layer's mixer and feed-forward read the same stream through two RMS norms and
enter it together: ``x += m * (mixer(norm1(x)) + ff(norm2(x)))`` with ``m = residual_mult``. The mixer is one of

* ``"parallel"``: two mixers side by side on the same input. Left: grouped-query softmax attention with an RMS norm
  per head on queries and keys, interleaved rotary positions on the first ``rot.dims`` elements, scores capped by a
  tanh and a sink in the softmax's denominator. Right: lightning attention (a decayed outer-product state per
  head, silu on q, k and v, the heads normed together, a sigmoid gate). Each output is RMS-normed over the width
  and the result is half their sum;
* ``"wkv"``: time mixing with a decay the input chooses and blends with the previous token;
* ``"mamba1"``: the selective scan with a short causal convolution.

The feed-forward is dense with clamped gate and up values: ``down(g sigmoid(1.702 g) (u + 1))``, ``g = min(gate, limit)``,
``u = clamp(up, -limit, limit)``; a layer may have none. The embedding is scaled; the head is a matrix of its own.

Keys of ``config.json``: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``residual_mult``, ``norm.eps`` and
``layers``: a list of ``{"type", "mixer", "mlp"}``. ``parallel``: ``left{heads kv_heads dim vdim scale softcap rot{base dims}}``,
``right{heads dim vdim decay[]}``; ``wkv``: ``heads dim``; ``mamba1``: ``inner state dt_rank conv``; ``mlp``: ``null`` or
``{"kind": "dense", "ff", "limit"}``. Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mlp.{gate,up,down}`` and ``l<i>.mix.*``: ``left.{q,k,v,o,q.norm,k.norm,out}``, ``right.{q,k,v,g,o,norm,out}``;
``mu.{r,k,v,g,w}``, ``r k v g w1 w2 w0 u norm o``; ``in conv conv.b x dt dt.b A_log D o``. The rank of the decay's low-rank
pair is not a key: it is the first size of ``w1`` (``decay_rank`` of the configuration object, filled in from the
checkpoint when a folder is loaded).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_spec import LayerSpec, ModelSpec, PartSpec, TensorNames

ARCHITECTURE = "Begovik"

SWISH_ALPHA = 1.702
"""The sigmoid's slope in the feed-forward's activation; the design fixes it."""

LEFT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}
RIGHT_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}
WKV_NAMES = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k", "v": "v", "g": "g",
             "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "o": "o"}
MAMBA1_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b", "a_log": "A_log",
                "d": "D", "out": "o"}
DENSE_NAMES = {"gate": "gate", "up": "up", "down": "down"}

MIXER_KEYS = {
    "wkv": ("heads", "dim"),
    "mamba1": ("inner", "state", "dt_rank", "conv"),
    "parallel": ("left", "right"),
}
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
RIGHT_KEYS = ("heads", "dim", "vdim", "decay")

DEFAULT_DECAY_RANK = 16
"""Rank of the decay's low-rank pair when nothing says otherwise (random weights without a checkpoint)."""


class BegovikConfigError(ValueError):
    """``config.json`` asks for something the design does not have."""


def _positive(value: Any, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) < 1:
        raise BegovikConfigError(f"{what} must be a positive integer, got {value!r}")
    return int(value)


@dataclass(frozen=True)
class BegovikConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    eps: float
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    max_position_embeddings: int = 1 << 20
    initializer_range: float = 0.05
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)
    architecture: str = ARCHITECTURE

    # the names the engine asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BegovikConfig":
        try:
            layers = data["layers"]
            vocab, width = _positive(data["vocab"], "vocab"), _positive(data["width"], "width")
            eps = float(data["norm"]["eps"])
        except (KeyError, TypeError) as exc:
            raise BegovikConfigError(f"config.json lacks {exc}") from None
        if not isinstance(layers, (list, tuple)) or not layers:
            raise BegovikConfigError("'layers' must be a non-empty list")
        checked = []
        for index, layer in enumerate(layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in MIXER_KEYS or not isinstance(mixer, Mapping):
                raise BegovikConfigError(f"layer {index}: unknown mixer type {kind!r}")
            for key in MIXER_KEYS[kind]:
                if key not in mixer:
                    raise BegovikConfigError(f"layer {index}: the {kind} mixer lacks {key!r}")
            if kind == "parallel":
                for side, keys in (("left", LEFT_KEYS), ("right", RIGHT_KEYS)):
                    for key in keys:
                        if key not in mixer[side]:
                            raise BegovikConfigError(f"layer {index}: the {side} mixer lacks {key!r}")
                left, right = mixer["left"], mixer["right"]
                if _positive(left["heads"], "heads") % _positive(left["kv_heads"], "kv_heads"):
                    raise BegovikConfigError(f"layer {index}: heads must be a multiple of kv_heads")
                if len(right["decay"]) != right["heads"]:
                    raise BegovikConfigError(f"layer {index}: {len(right['decay'])} decays for {right['heads']} heads")
                rot = left.get("rot")
                if rot and (int(rot.get("dims", 0)) % 2 or int(rot.get("dims", 0)) > left["dim"] or "base" not in rot):
                    raise BegovikConfigError(f"layer {index}: rot.dims must be even and at most dim, and rot needs a base")
            else:
                for key in MIXER_KEYS[kind]:
                    _positive(mixer[key], f"layer {index}: mixer.{key}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise BegovikConfigError(f"layer {index}: unknown feed-forward {mlp!r}")
                _positive(mlp.get("ff"), f"layer {index}: mlp.ff")
                if not float(mlp.get("limit", 0.0)) > 0.0:
                    raise BegovikConfigError(f"layer {index}: the feed-forward needs a positive 'limit'")
            checked.append(copy.deepcopy(dict(layer)))
        known = {"architecture", "architectures", "vocab", "width", "layers", "norm", "embedding", "residual_mult",
                 "max_position_embeddings", "initializer_range", "torch_dtype"}
        return cls(vocab=vocab, width=width, layers=tuple(checked), eps=eps,
                   embedding_scale=float((data.get("embedding") or {}).get("scale", 1.0)),
                   residual_mult=float(data.get("residual_mult", 1.0)),
                   max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)),
                   initializer_range=float(data.get("initializer_range", 0.05)),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        return {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
            "layers": copy.deepcopy([dict(layer) for layer in self.layers]), "norm": {"eps": self.eps},
            "max_position_embeddings": self.max_position_embeddings, "initializer_range": self.initializer_range,
        }

    def with_tensor_shapes(self, shapes: Mapping[str, tuple[int, ...]]) -> "BegovikConfig":
        """Sizes that only the checkpoint gives (the rank of a wkv layer's decay pair), filled in from its shapes."""
        layers = []
        for index, layer in enumerate(self.layers):
            layer = copy.deepcopy(dict(layer))
            shape = shapes.get(f"l{index}.mix.w1")
            if layer["type"] == "wkv" and shape is not None:
                layer["mixer"]["decay_rank"] = int(shape[0])
            layers.append(layer)
        return BegovikConfig(self.vocab, self.width, tuple(layers), self.eps, self.embedding_scale, self.residual_mult,
                             self.max_position_embeddings, self.initializer_range, self.extra)

    # -- translation ----------------------------------------------------------------------------

    def _mixer(self, layer: Mapping[str, Any]) -> PartSpec:
        sizes = layer["mixer"]
        if layer["type"] == "wkv":
            return PartSpec("wkv", dict(heads=sizes["heads"], dim=sizes["dim"], vdim=sizes.get("vdim"),
                                        decay_rank=sizes.get("decay_rank", DEFAULT_DECAY_RANK), eps=self.eps, names=WKV_NAMES))
        if layer["type"] == "mamba1":
            return PartSpec("mamba1", dict(inner=sizes["inner"], state=sizes["state"], dt_rank=sizes["dt_rank"], taps=sizes["conv"],
                                           names=MAMBA1_NAMES))
        left, right = sizes["left"], sizes["right"]
        rot = dict(left.get("rot") or {})
        if rot:
            rot["interleaved"] = True  # pairs (2i, 2i + 1)
        attention = PartSpec("sink_attention", dict(
            heads=left["heads"], kv_heads=left["kv_heads"], dim=left["dim"], vdim=left["vdim"], scale=left["scale"],
            softcap=left.get("softcap") or 0.0, sink=True, qk_norm=True, eps=self.eps, rot=rot, names=LEFT_NAMES))
        lightning = PartSpec("retention", dict(
            heads=right["heads"], dim=right["dim"], vdim=right["vdim"], decay=tuple(float(d) for d in right["decay"]),
            activation="silu", key_scale=1.0, norm="row", norm_weight=True, gate="sigmoid", eps=self.eps, names=RIGHT_NAMES))
        return PartSpec("side_by_side", dict(left=attention, right=lightning, eps=self.eps, weight_left=0.5, weight_right=0.5,
                                             left_prefix="left.", right_prefix="right.", left_norm="left.out", right_norm="right.out"))

    def to_model_spec(self) -> ModelSpec:
        layers, unused = [], []
        for index, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            feed_forward = ff_norm = None
            if mlp is None:
                unused.append(f"l{index}.norm2")  # a layer without a feed-forward has no use for a second norm
            else:
                feed_forward = PartSpec("gated_mlp", dict(intermediate_size=mlp["ff"], activation="clamped_swish", limit=mlp["limit"],
                                                          alpha=SWISH_ALPHA, names=DENSE_NAMES))
                ff_norm = PartSpec("rms_norm", dict(eps=self.eps, tensor="norm2"))
            layers.append(LayerSpec(
                mixer=self._mixer(layer), feed_forward=feed_forward,
                mixer_norm=PartSpec("rms_norm", dict(eps=self.eps, tensor="norm1")), feed_forward_norm=ff_norm,
                position=None, block="parallel", block_params=dict(residual_mult=self.residual_mult)))
        names = TensorNames(embedding="", head="", final_norm="final.", layer="l{index}.", mixer="mix.",
                            feed_forward="mlp.", mixer_norm="", feed_forward_norm="", prefix_rewrites=())
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            order=ModelSpec.sequential(len(layers)), final_norm=PartSpec("rms_norm", dict(eps=self.eps, tensor="norm")),
            embedding=PartSpec("table", dict(tensor="embed", scale=self.embedding_scale)),
            head=PartSpec("linear", dict(tensor="head")), tie_word_embeddings=False, names=names,
            optional_tensors=tuple(unused), eos_token_ids=(), max_position_embeddings=self.max_position_embeddings,
            init_std=self.initializer_range)
