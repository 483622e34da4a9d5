"""Begovik without a GPU: its configuration, tensor names, cache plan, and the plain oracle's own properties."""

import json
import math

import pytest
import torch

import begovik_cases as C
import plain_begovik as P

F64 = torch.float64


def test_config_round_trip_and_registry(tmp_path):
    from turboserve_b200.config import BegovikConfig, config_from_dict, config_from_dir, registered_architectures

    assert "Begovik" in registered_architectures()
    for name, (raw, _) in C.CASES.items():
        config = config_from_dict(raw)
        assert isinstance(config, BegovikConfig) and config.architecture == "Begovik"
        assert config_from_dict(config.to_dict()) == config
        assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]
        assert config.embedding_scale == raw["embedding"]["scale"] and config.residual_mult == raw["residual_mult"]
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(raw))
        assert config_from_dir(tmp_path / name) == config


def test_bad_configurations_are_refused():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.begovik import BegovikConfigError

    def broken(change):
        raw = json.loads(json.dumps(C.CASE_A))
        change(raw)
        with pytest.raises(BegovikConfigError):
            config_from_dict(raw)

    broken(lambda raw: raw["layers"][0].update(type="convolution"))
    broken(lambda raw: raw["layers"][0].update(mlp={"kind": "sparse", "ff": 8}))
    broken(lambda raw: raw["layers"][0]["mlp"].pop("limit"))
    broken(lambda raw: raw["layers"][0]["mixer"]["left"].pop("scale"))
    broken(lambda raw: raw["layers"][0]["mixer"]["left"].update(kv_heads=3))          # four heads on three key heads
    broken(lambda raw: raw["layers"][0]["mixer"]["left"]["rot"].update(dims=7))       # an odd number of rotated elements
    broken(lambda raw: raw["layers"][0]["mixer"]["left"]["rot"].update(dims=26))      # more than the head has
    broken(lambda raw: raw["layers"][0]["mixer"]["right"].update(decay=[0.5]))        # one decay for three heads
    broken(lambda raw: raw["layers"][1]["mixer"].pop("dim"))
    broken(lambda raw: raw["layers"][2]["mixer"].update(state=0))
    broken(lambda raw: raw.pop("norm"))
    broken(lambda raw: raw.update(layers=[]))


def test_every_layer_is_a_parallel_block_of_the_parts_its_entry_names():
    from turboserve_b200.config import config_from_dict

    spec = config_from_dict(C.CASE_A).to_model_spec()
    assert [layer.mixer.kind for layer in spec.layers] == ["side_by_side", "wkv", "mamba1", "side_by_side"]
    assert all(layer.block == "parallel" and layer.block_params["residual_mult"] == 0.7 for layer in spec.layers)
    assert spec.layers[1].feed_forward is None and spec.layers[1].feed_forward_norm is None
    assert not spec.tie_word_embeddings and spec.embedding["scale"] == 3.0
    left, right = spec.layers[0].mixer["left"], spec.layers[0].mixer["right"]
    assert left.kind == "sink_attention" and left["sink"] and left["qk_norm"] and left["softcap"] == 30.0
    assert left["rot"] == {"base": 5000.0, "dims": 8, "interleaved": True} and left["scale"] == 0.2
    assert right.kind == "retention" and right["decay"] == (0.9, 0.97, 0.995) and right["activation"] == "silu"
    assert right["gate"] == "sigmoid" and right["norm"] == "row" and right["key_scale"] == 1.0
    ff = spec.layers[0].feed_forward
    assert ff["activation"] == "clamped_swish" and ff["limit"] == 2.0 and ff["alpha"] == 1.702
    assert spec.layers[2].mixer["taps"] == 4 and spec.layers[2].mixer["dt_rank"] == 6


def test_tensor_names_shapes_and_cache_plan():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.registry import lookup

    config = config_from_dict(C.CASE_A)
    model = lookup("Begovik").build_model(config, torch.float32, "cpu")
    shapes = {p.name: tuple(p.spec.shape) for p in model.named_params()}
    assert shapes["embed"] == (190, 96) and shapes["head"] == (190, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.left.q"] == (4 * 24, 96) and shapes["l0.mix.left.k"] == (2 * 24, 96) and shapes["l0.mix.left.v"] == (2 * 20, 96)
    assert shapes["l0.mix.left.q.norm"] == shapes["l0.mix.left.k.norm"] == (24,) and shapes["l0.mix.left.o"] == (96, 80)
    assert shapes["l0.mix.right.q"] == shapes["l0.mix.right.k"] == (48, 96)
    assert shapes["l0.mix.right.v"] == shapes["l0.mix.right.g"] == (72, 96) and shapes["l0.mix.right.norm"] == (72,)
    assert shapes["l0.mix.left.out"] == shapes["l0.mix.right.out"] == (96,) and shapes["l0.mix.right.o"] == (96, 72)
    assert shapes["l1.mix.mu.w"] == (96,) and shapes["l1.mix.w1"] == (8, 96) and shapes["l1.mix.w2"] == (48, 8)
    assert shapes["l1.mix.u"] == (3, 16) and shapes["l1.mix.w0"] == (48,) and shapes["l1.mix.norm"] == (48,)
    assert shapes["l2.mix.in"] == (160, 96) and shapes["l2.mix.conv"] == (80, 4) and shapes["l2.mix.conv.b"] == (80,)
    assert shapes["l2.mix.x"] == (6 + 24, 80) and shapes["l2.mix.dt"] == (80, 6) and shapes["l2.mix.A_log"] == (80, 12)
    assert shapes["l2.mix.D"] == (80,) and shapes["l2.mix.o"] == (96, 80)
    assert shapes["l0.mlp.gate"] == (112, 96) and shapes["l0.mlp.down"] == (96, 112)
    assert "l1.norm2" not in shapes and "l1.norm2" in model.optional_names() and "l1.norm1" in shapes
    plan = model.cache_plan()
    kinds = [run.kind for run in plan.runs]
    assert kinds.count("paged") == 2 and plan.windows == [None]  # both attentions see everything: one group of pages
    assert model.graph_safe
    states = [tuple(s.shape) for run in plan.runs for s in run.states]  # a run with pages may keep states beside them
    assert (3, 16, 16) in states and (96,) in states             # wkv: S of every head, the last input row
    assert (80, 12) in states and (3, 80) in states              # the scan: S, the convolution's last inputs
    assert (3, 24, 16) in states and (1, 64, 8) in states        # lightning attention beside both attentions
    assert plan.runs[0].need.head_dim == 24 and plan.runs[0].need.value_dim == 20 and plan.runs[3].need.value_dim == 48


def test_the_decay_rank_comes_from_the_checkpoint(tmp_path):
    """``config.json`` does not say how wide the decay's low-rank pair is: the shape of ``w1`` does."""
    from turboserve_b200.config import config_from_dir
    from turboserve_b200.weights import checkpoint_index

    folder = C.write_case("C", tmp_path / "c")
    raw = C.read_config(folder)
    for entry in raw["layers"]:
        entry["mixer"].pop("decay_rank", None)
    (folder / "config.json").write_text(json.dumps(raw))
    plain = config_from_dir(folder)
    assert "decay_rank" not in plain.layers[0]["mixer"]
    config = plain.with_tensor_shapes({name: tuple(entry[1]) for name, entry in checkpoint_index(folder).items()})
    assert config.layers[0]["mixer"]["decay_rank"] == 3
    assert config.to_model_spec().layers[0].mixer["decay_rank"] == 3


def test_the_oracle_is_causal_and_each_mechanism_does_what_its_equation_says():
    g = torch.Generator().manual_seed(0)
    eps = 1e-6
    # the sink: with all scores far below zero nothing is attended to; with one key at a high score the output is its value
    sizes = dict(heads=1, kv_heads=1, dim=4, vdim=3, scale=1.0, softcap=0.0, rot=None)
    w = {"q": torch.eye(4, dtype=F64), "k": torch.eye(4, dtype=F64), "v": torch.randn(3, 4, generator=g, dtype=F64),
         "q.norm": torch.ones(4, dtype=F64), "k.norm": torch.ones(4, dtype=F64), "o": torch.eye(3, dtype=F64)}
    h = torch.tensor([[1.0, 0, 0, 0], [-1.0, 0, 0, 0]], dtype=F64)
    out = P.sink_attention(h, w, sizes, eps)
    # position 0: one key of score 4 (unit-rms rows have length 2): p = e^4 / (1 + e^4)
    p = math.exp(4.0) / (1.0 + math.exp(4.0))
    assert torch.allclose(out[0], p * (h[0] @ w["v"].T), atol=1e-9)
    # position 1: scores -4 (key 0) and 4 (itself)
    a, b = math.exp(-4.0), math.exp(4.0)
    want = (a * (h[0] @ w["v"].T) + b * (h[1] @ w["v"].T)) / (1.0 + a + b)
    assert torch.allclose(out[1], want, atol=1e-9)
    # the cap: scores of 4 become cap * tanh(4 / cap)
    capped = P.sink_attention(h[:1], w, dict(sizes, softcap=2.0), eps)
    s = 2.0 * math.tanh(2.0)
    assert torch.allclose(capped[0], math.exp(s) / (1 + math.exp(s)) * (h[0] @ w["v"].T), atol=1e-9)
    # rotation: pairs (2i, 2i + 1), angle position * base^(-2i / dims); elements beyond dims pass
    x = torch.tensor([[[1.0, 0.0, 1.0, 0.0, 7.0]], [[1.0, 0.0, 1.0, 0.0, 7.0]]], dtype=F64)
    turned = P.rotate_pairs(x, {"base": 100.0, "dims": 4})
    assert torch.allclose(turned[0], x[0]) and turned[1, 0, 4] == 7.0
    assert torch.allclose(turned[1, 0, :4], torch.tensor([math.cos(1.0), math.sin(1.0), math.cos(0.1), math.sin(0.1)], dtype=F64))
    # lightning attention: o_t = sum_s decay^(t - s) (q_t . k_s) v_s, the current token with weight 1
    sizes = dict(heads=2, dim=3, vdim=2, decay=[0.5, 0.9])
    w = {k: torch.randn(n, 5, generator=g, dtype=F64) for k, n in (("q", 6), ("k", 6), ("v", 4), ("g", 4))}
    w.update(norm=torch.ones(4, dtype=F64), o=torch.eye(4, dtype=F64))
    h = torch.randn(7, 5, generator=g, dtype=F64)
    got = P.lightning_attention(h, w, sizes, eps)
    q, k, v = (P.silu(h @ w[s].T) for s in "qkv")
    raw = torch.zeros(7, 4, dtype=F64)
    for head, decay in enumerate(sizes["decay"]):
        for t in range(7):
            for s in range(t + 1):
                raw[t, 2 * head:2 * head + 2] += decay ** (t - s) * (q[t, 3 * head:3 * head + 3] @ k[s, 3 * head:3 * head + 3]) * v[s, 2 * head:2 * head + 2]
    assert torch.allclose(got, P.rms_norm(raw, None, eps) * torch.sigmoid(h @ w["g"].T), atol=1e-9)
    # the feed-forward: the gate is cut from above only, the other factor on both sides
    ff = {"gate": torch.tensor([[10.0], [-10.0]], dtype=F64), "up": torch.tensor([[10.0], [-10.0]], dtype=F64), "down": torch.eye(2, dtype=F64)}
    y = P.clamped_feed_forward(torch.ones(1, 1, dtype=F64), ff, {"limit": 2.0})
    assert torch.allclose(y[0], torch.tensor([2.0 / (1 + math.exp(-3.404)) * 3.0, -10.0 / (1 + math.exp(17.02)) * -1.0], dtype=F64))


def test_the_oracles_recurrences_written_as_sums_and_its_layers_are_causal(tmp_path):
    g = torch.Generator().manual_seed(1)
    eps = 1e-5
    # wkv written as a sum over earlier tokens: o_t = sum_{s<t} (prod_{s<j<t} w_j) (r_t*k_s) v_s + (r_t*u*k_t) v_t
    sizes = dict(heads=1, dim=3)
    w = {name: torch.randn(3, 4, generator=g, dtype=F64) for name in ("r", "k", "v", "g")}
    w.update({f"mu.{s}": torch.rand(4, generator=g, dtype=F64) for s in "rkvgw"})
    w.update(w1=torch.randn(2, 4, generator=g, dtype=F64), w2=torch.randn(3, 2, generator=g, dtype=F64), w0=torch.randn(3, generator=g, dtype=F64),
             u=torch.randn(1, 3, generator=g, dtype=F64), norm=torch.ones(3, dtype=F64), o=torch.eye(3, dtype=F64))
    h = torch.randn(6, 4, generator=g, dtype=F64)
    got = P.wkv(h, w, sizes, eps)
    before = torch.cat([torch.zeros(1, 4, dtype=F64), h[:-1]])
    mixed = {s: h + (before - h) * w[f"mu.{s}"] for s in "rkvgw"}
    r, k, v = (mixed[s] @ w[s].T for s in "rkv")
    decay = torch.exp(-torch.exp(torch.tanh(mixed["w"] @ w["w1"].T) @ w["w2"].T + w["w0"]))
    raw = torch.zeros(6, 3, dtype=F64)
    for t in range(6):
        raw[t] = ((r[t] * w["u"][0] * k[t]).sum()) * v[t]
        for s in range(t):
            between = torch.ones(3, dtype=F64)
            for j in range(s + 1, t):
                between = between * decay[j]
            raw[t] += (r[t] * between * k[s]).sum() * v[s]
    assert torch.allclose(got, P.rms_norm(raw, None, eps) * P.silu(mixed["g"] @ w["g"].T), atol=1e-9)
    assert torch.allclose(mixed["r"][0], h[0] * (1 - w["mu.r"]))  # before the first token there are zeros
    # the whole model: a position's logits do not depend on later tokens; the stream has one entry per layer
    folder = C.write_case("A", tmp_path / "a")
    config, weights = P.read_model_folder(folder)
    tokens = torch.randint(0, config["vocab"], (40,), generator=g).tolist()
    logits, layers = P.forward(config, weights, tokens)
    shorter, _ = P.forward(config, weights, tokens[:23])
    assert torch.allclose(logits[:23], shorter, atol=1e-9) and layers.shape == (4, 40, 96)
    # the convolution's last column is the current token's: with one tap nothing of the past enters before the scan
    sizes = dict(inner=2, state=1, dt_rank=1, conv=2)
    m = {"in": torch.randn(4, 3, generator=g, dtype=F64), "conv": torch.tensor([[0.0, 1.0], [0.0, 1.0]], dtype=F64),
         "conv.b": torch.zeros(2, dtype=F64), "x": torch.randn(3, 2, generator=g, dtype=F64), "dt": torch.randn(2, 1, generator=g, dtype=F64),
         "dt.b": torch.full((2,), -30.0, dtype=F64), "A_log": torch.zeros(2, 1, dtype=F64), "D": torch.tensor([2.0, 3.0], dtype=F64),
         "o": torch.eye(2, dtype=F64)}
    h = torch.randn(5, 3, generator=g, dtype=F64)
    both = h @ m["in"].T
    x, z = P.silu(both[:, :2]), both[:, 2:]
    assert torch.allclose(P.mamba1(h, m, sizes, eps), m["D"] * x * P.silu(z), atol=1e-9)  # step sizes of e^-30: only the skip is left
