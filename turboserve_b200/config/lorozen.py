"""Typed configuration of the Lorozen decoder, read from its ``config.json``.

Lorozen is a small decoder with norms on both sides of every sublayer: ``x += post1(mixer(pre1(x)))``, then
``x += post2(ff(pre2(x)))``, all four RMS norms with weights of their own. A layer's mixer is one of

* ``"attention"``: grouped-query softmax attention with biases on q, k and v, a rotation of the first ``rot.dims``
  elements of every head (pairs ``(i, i + dims / 2)``; ``rot.scaling`` stretches the long waves by their wavelength), a
  sliding window of ``mask.size`` positions and a learned sink per query head in the softmax's denominator;
* ``"latent_attention"``: keys and values of all heads made from one cached latent per position (``kv_rank`` numbers,
  RMS-normed) and one rotated key part the heads share (``rot_dim`` numbers, pairs of neighbours ``(2i, 2i + 1)``), a
  sliding window, an ordinary softmax, and a sigmoid gate per head on the output;
* ``"wkv"``: time mixing with a decay the input chooses and blends with the previous token.

The feed-forward is absent, dense and gated (``down(gelu_tanh(gate h) * up h)``), or a mixture of experts: sigmoid
scores, the ``top`` largest chosen and used as they are, the weight on the expert's INPUT (``sum expert(s h)``, experts
``down(silu(gate x) * up x)``), plus a shared expert of the same form for every token. A stretch of layers
(``loop``: ``start``, ``stop``, ``times``) runs several times in a row with the same weights, each pass with caches and
states of its own; before every pass but the first the embedding's output is added to the stream. The logits are bent
into ``(-logit_softcap, logit_softcap)`` by a tanh.

Keys of ``config.json``: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``, ``loop`` and ``layers``: a list of
``{"type", "mixer", "mlp"}``. ``attention``: ``heads kv_heads dim vdim scale mask{size} rot{base dims scaling{factor low high
original}}``; ``latent_attention``: ``heads dim rot_dim vdim kv_rank scale mask{size} rot{base dims}``; ``wkv``: ``heads dim``;
``mlp``: ``null``, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert"{ff}, "router"{experts top}, "shared"{ff}}``. Tensor
names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``l<i>.mix.*``
(``q q.b k k.b v v.b sink o``; ``q dkv dkv.norm uk uv g o``; ``mu.{r,k,v,g,w} r k v g w1 w2 w0 u norm o``) and ``l<i>.mlp.*``
(``gate up down``; ``router``, ``e<j>.{gate,up,down}``, ``shared.{gate,up,down}``). The rank of a wkv layer's decay pair is
not a key: it is the first size of ``w1`` (``decay_rank``, filled in from the checkpoint when a folder is loaded).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .model_spec import LayerRun, LayerSpec, ModelSpec, PartSpec, TensorNames

ARCHITECTURE = "Lorozen"

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "sink": "sink"}
LATENT_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g", "o": "o"}
WKV_NAMES = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "r": "r", "k": "k", "v": "v", "g": "g",
             "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm", "o": "o"}
DENSE_NAMES = {"gate": "gate", "up": "up", "down": "down"}
EXPERT_NAMES = {"router": "router", "expert": "e{index}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"}

MIXER_KEYS = {
    "attention": ("heads", "dim", "scale"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"),
    "wkv": ("heads", "dim"),
}

DEFAULT_DECAY_RANK = 16
"""Rank of the decay's low-rank pair when nothing says otherwise (random weights without a checkpoint)."""


class LorozenConfigError(ValueError):
    """``config.json`` asks for something the design does not have."""


def _positive(value: Any, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) < 1:
        raise LorozenConfigError(f"{what} must be a positive integer, got {value!r}")
    return int(value)


def _window(mixer: Mapping[str, Any]) -> int | None:
    size = (mixer.get("mask") or {}).get("size")
    return int(size) if size else None


@dataclass(frozen=True)
class LorozenConfig:
    vocab: int
    width: int
    layers: tuple[Mapping[str, Any], ...]
    eps: float
    logit_softcap: float = 0.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
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

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start and self.loop_times >= 1

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "LorozenConfig":
        try:
            layers = data["layers"]
            vocab, width = _positive(data["vocab"], "vocab"), _positive(data["width"], "width")
            eps = float(data["norm"]["eps"])
        except (KeyError, TypeError) as exc:
            raise LorozenConfigError(f"config.json lacks {exc}") from None
        if not isinstance(layers, (list, tuple)) or not layers:
            raise LorozenConfigError("'layers' must be a non-empty list")
        checked = []
        for index, layer in enumerate(layers):
            kind, mixer = layer.get("type"), layer.get("mixer")
            if kind not in MIXER_KEYS or not isinstance(mixer, Mapping):
                raise LorozenConfigError(f"layer {index}: unknown mixer type {kind!r}")
            for key in MIXER_KEYS[kind]:
                if key not in mixer:
                    raise LorozenConfigError(f"layer {index}: the {kind} mixer lacks {key!r}")
                if key != "scale":
                    _positive(mixer[key], f"layer {index}: mixer.{key}")
            if kind == "attention" and _positive(mixer["heads"], "heads") % _positive(mixer.get("kv_heads") or mixer["heads"], "kv_heads"):
                raise LorozenConfigError(f"layer {index}: heads must be a multiple of kv_heads")
            rot = mixer.get("rot")
            if kind != "wkv" and rot:
                dims, limit = int(rot.get("dims", 0)), int(mixer["rot_dim"] if kind == "latent_attention" else mixer["dim"])
                if dims % 2 or dims > limit or "base" not in rot or (kind == "latent_attention" and dims != limit):
                    raise LorozenConfigError(f"layer {index}: rot.dims must be even and fit the rotated part, and rot needs a base")
            if kind == "latent_attention" and not rot:
                raise LorozenConfigError(f"layer {index}: latent attention needs 'rot' for its rotated part")
            window = _window(mixer)
            if window is not None and window < 1:
                raise LorozenConfigError(f"layer {index}: mask.size must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
                    raise LorozenConfigError(f"layer {index}: unknown feed-forward {mlp!r}")
                if mlp["kind"] == "dense":
                    _positive(mlp.get("ff"), f"layer {index}: mlp.ff")
                else:
                    try:
                        experts = _positive(mlp["router"]["experts"], f"layer {index}: mlp.router.experts")
                        top = _positive(mlp["router"]["top"], f"layer {index}: mlp.router.top")
                        _positive(mlp["expert"]["ff"], f"layer {index}: mlp.expert.ff")
                        if mlp.get("shared"):
                            _positive(mlp["shared"]["ff"], f"layer {index}: mlp.shared.ff")
                    except (KeyError, TypeError) as exc:
                        raise LorozenConfigError(f"layer {index}: the mixture lacks {exc}") from None
                    if top > experts:
                        raise LorozenConfigError(f"layer {index}: {top} of {experts} experts cannot be chosen")
            checked.append(copy.deepcopy(dict(layer)))
        loop = data.get("loop") or {}
        start, stop, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
        if loop and not (0 <= start <= stop <= len(checked) and times >= 1):
            raise LorozenConfigError(f"loop {dict(loop)!r} does not fit {len(checked)} layers")
        cap = data.get("logit_softcap")
        if cap is not None and float(cap) < 0.0:
            raise LorozenConfigError("logit_softcap must be positive (or absent)")
        known = {"architecture", "architectures", "vocab", "width", "layers", "norm", "logit_softcap", "loop",
                 "max_position_embeddings", "initializer_range", "torch_dtype"}
        return cls(vocab=vocab, width=width, layers=tuple(checked), eps=eps, logit_softcap=float(cap or 0.0),
                   loop_start=start, loop_stop=stop, loop_times=times,
                   max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)),
                   initializer_range=float(data.get("initializer_range", 0.05)),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        out = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "layers": copy.deepcopy([dict(layer) for layer in self.layers]), "norm": {"eps": self.eps},
            "max_position_embeddings": self.max_position_embeddings, "initializer_range": self.initializer_range,
        }
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.has_loop:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    def with_tensor_shapes(self, shapes: Mapping[str, tuple[int, ...]]) -> "LorozenConfig":
        """Sizes that only the checkpoint gives (the rank of a wkv layer's decay pair), filled in from its shapes."""
        layers = []
        for index, layer in enumerate(self.layers):
            layer = copy.deepcopy(dict(layer))
            shape = shapes.get(f"l{index}.mix.w1")
            if layer["type"] == "wkv" and shape is not None:
                layer["mixer"]["decay_rank"] = int(shape[0])
            layers.append(layer)
        return LorozenConfig(self.vocab, self.width, tuple(layers), self.eps, self.logit_softcap, self.loop_start, self.loop_stop,
                             self.loop_times, self.max_position_embeddings, self.initializer_range, self.extra)

    # -- translation ----------------------------------------------------------------------------

    def run_order(self) -> tuple[LayerRun, ...]:
        """Every layer once, but the looped stretch ``times`` times in a row; each run owns its cache or state, and the
        first run of every pass but the first has the embedding's output added before it."""
        count = len(self.layers)
        if not self.has_loop:
            return ModelSpec.sequential(count)
        runs = [LayerRun(i) for i in range(self.loop_start)]
        for again in range(self.loop_times):
            for i in range(self.loop_start, self.loop_stop):
                runs.append(LayerRun(i, readds_embedding=again > 0 and i == self.loop_start))
        runs += [LayerRun(i) for i in range(self.loop_stop, count)]
        return tuple(runs)

    def _mixer(self, layer: Mapping[str, Any]) -> PartSpec:
        sizes = layer["mixer"]
        if layer["type"] == "wkv":
            return PartSpec("wkv", dict(heads=sizes["heads"], dim=sizes["dim"], vdim=sizes.get("vdim"),
                                        decay_rank=sizes.get("decay_rank", DEFAULT_DECAY_RANK), eps=self.eps, names=WKV_NAMES))
        rot = dict(sizes.get("rot") or {})
        if layer["type"] == "attention":
            if rot:
                rot["interleaved"] = False  # pairs (i, i + dims / 2)
            return PartSpec("sink_attention", dict(
                heads=sizes["heads"], kv_heads=sizes.get("kv_heads") or sizes["heads"], dim=sizes["dim"],
                vdim=sizes.get("vdim") or sizes["dim"], scale=sizes["scale"], softcap=0.0, sink="learned", bias=True, qk_norm=False,
                window=_window(sizes), eps=self.eps, rot=rot, names=ATTENTION_NAMES))
        rot["interleaved"] = True  # pairs (2i, 2i + 1)
        return PartSpec("latent_attention", dict(
            heads=sizes["heads"], dim=sizes["dim"], rot_dim=sizes["rot_dim"], vdim=sizes["vdim"], kv_rank=sizes["kv_rank"],
            scale=sizes["scale"], window=_window(sizes), eps=self.eps, rot=rot, gate=True, names=LATENT_NAMES))

    def _feed_forward(self, mlp: Mapping[str, Any]) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", dict(intermediate_size=mlp["ff"], activation="gelu_pytorch_tanh", names=DENSE_NAMES))
        shared = mlp.get("shared") or {}
        return PartSpec("routed_experts", dict(
            experts=mlp["router"]["experts"], top=mlp["router"]["top"], intermediate_size=mlp["expert"]["ff"],
            shared=shared.get("ff"), activation="silu", score="sigmoid", renormalize=False, weight_on="input", names=EXPERT_NAMES))

    def to_model_spec(self) -> ModelSpec:
        layers, unused = [], []

        def norm(tensor: str) -> PartSpec:
            return PartSpec("rms_norm", dict(eps=self.eps, tensor=tensor))

        for index, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            feed_forward = ff_norm = ff_out_norm = None
            if mlp is None:  # a layer without a feed-forward has no use for the norms around one
                unused += [f"l{index}.norm2", f"l{index}.norm2b"]
            else:
                feed_forward, ff_norm, ff_out_norm = self._feed_forward(mlp), norm("norm2"), norm("norm2b")
            layers.append(LayerSpec(
                mixer=self._mixer(layer), feed_forward=feed_forward, mixer_norm=norm("norm1"), feed_forward_norm=ff_norm,
                mixer_output_norm=norm("norm1b"), feed_forward_output_norm=ff_out_norm, position=None, block="both_sides_norm"))
        names = TensorNames(embedding="", head="", final_norm="final.", layer="l{index}.", mixer="mix.", feed_forward="mlp.",
                            mixer_norm="", feed_forward_norm="", mixer_output_norm="", feed_forward_output_norm="",
                            prefix_rewrites=())
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab, layers=tuple(layers),
            order=self.run_order(), final_norm=PartSpec("rms_norm", dict(eps=self.eps, tensor="norm")),
            embedding=PartSpec("table", dict(tensor="embed")),
            head=PartSpec("linear", dict(tensor="head", softcap=self.logit_softcap)), tie_word_embeddings=False, names=names,
            optional_tensors=tuple(unused), eos_token_ids=(), max_position_embeddings=self.max_position_embeddings,
            init_std=self.initializer_range)
