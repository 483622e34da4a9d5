"""Lorozen without a GPU: its configuration, tensor names, run order, cache plan, and the plain oracle's own properties."""

import json
import math

import pytest
import torch

import lorozen_cases as C
import plain_lorozen as P

F64 = torch.float64


def test_config_round_trip_and_registry(tmp_path):
    from turboserve_b200.config import LorozenConfig, config_from_dict, config_from_dir, registered_architectures

    assert "Lorozen" in registered_architectures()
    for name, (raw, _) in C.CASES.items():
        config = config_from_dict(raw)
        assert isinstance(config, LorozenConfig) and config.architecture == "Lorozen"
        assert config_from_dict(config.to_dict()) == config
        assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]
        assert config.logit_softcap == float(raw.get("logit_softcap") or 0.0)
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(raw))
        assert config_from_dir(tmp_path / name) == config


def test_bad_configurations_are_refused():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.lorozen import LorozenConfigError

    def broken(change):
        raw = json.loads(json.dumps(C.CASE_A))
        change(raw)
        with pytest.raises(LorozenConfigError):
            config_from_dict(raw)

    broken(lambda raw: raw["layers"][0].update(type="convolution"))
    broken(lambda raw: raw["layers"][0].update(mlp={"kind": "sparse", "ff": 8}))
    broken(lambda raw: raw["layers"][1]["mlp"].pop("ff"))
    broken(lambda raw: raw["layers"][0]["mixer"].pop("scale"))
    broken(lambda raw: raw["layers"][0]["mixer"].update(kv_heads=3))              # four heads on three key heads
    broken(lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=7))           # an odd number of rotated elements
    broken(lambda raw: raw["layers"][0]["mixer"]["rot"].update(dims=26))          # more than the head has
    broken(lambda raw: raw["layers"][2]["mixer"]["rot"].update(dims=4))           # the rotated part is turned whole
    broken(lambda raw: raw["layers"][2]["mixer"].pop("kv_rank"))
    broken(lambda raw: raw["layers"][0]["mlp"]["router"].update(top=7))           # seven of six experts
    broken(lambda raw: raw["layers"][0]["mlp"].pop("expert"))
    broken(lambda raw: raw["layers"][1]["mixer"].pop("dim"))
    broken(lambda raw: raw["loop"].update(stop=9))
    broken(lambda raw: raw["loop"].update(times=0))
    broken(lambda raw: raw.pop("norm"))
    broken(lambda raw: raw.update(layers=[]))


def test_every_layer_has_norms_on_both_sides_and_the_parts_its_entry_names():
    from turboserve_b200.config import config_from_dict

    spec = config_from_dict(C.CASE_A).to_model_spec()
    assert [layer.mixer.kind for layer in spec.layers] == ["sink_attention", "wkv", "latent_attention", "sink_attention"]
    assert all(layer.block == "both_sides_norm" and layer.mixer_output_norm["tensor"] == "norm1b" for layer in spec.layers)
    assert spec.layers[3].feed_forward is None and spec.layers[3].feed_forward_norm is None and spec.layers[3].feed_forward_output_norm is None
    assert spec.layers[0].feed_forward_output_norm["tensor"] == "norm2b"
    assert not spec.tie_word_embeddings and spec.head["softcap"] == 20.0 and spec.head["tensor"] == "head"
    first = spec.layers[0].mixer
    assert first["sink"] == "learned" and first["bias"] and not first["qk_norm"] and first["window"] == 40 and first["scale"] == 0.2
    assert first["rot"] == {"base": 5000.0, "dims": 8, "interleaved": False,
                            "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    latent = spec.layers[2].mixer
    assert latent["gate"] and latent["rot"]["interleaved"] and latent["window"] == 33 and latent["kv_rank"] == 40
    experts = spec.layers[0].feed_forward
    assert experts.kind == "routed_experts" and experts["score"] == "sigmoid" and not experts["renormalize"]
    assert experts["weight_on"] == "input" and experts["shared"] == 56 and experts["top"] == 2 and experts["activation"] == "silu"
    assert spec.layers[1].feed_forward["activation"] == "gelu_pytorch_tanh"
    assert config_from_dict(C.CASE_B).to_model_spec().layers[1].mixer["window"] is None
    assert config_from_dict(C.CASE_B).to_model_spec().head["softcap"] == 0.0


def test_the_run_order_repeats_the_loop_and_marks_where_the_embedding_comes_back():
    from turboserve_b200.config import config_from_dict

    def order(raw):
        return [(run.layer, run.readds_embedding) for run in config_from_dict(raw).to_model_spec().order]

    assert order(C.CASE_A) == [(0, False), (1, False), (2, False), (1, True), (2, False), (3, False)]
    assert order(C.CASE_B) == [(0, False), (1, False), (2, False), (3, False)]
    assert order(C.CASE_C) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False)]
    assert order(C.CASE_E) == [(0, False), (1, False), (0, True), (1, False)]
    once = json.loads(json.dumps(C.CASE_A))
    once["loop"]["times"] = 1
    assert order(once) == [(i, False) for i in range(4)]
    for raw in (C.CASE_A, C.CASE_B, C.CASE_C, C.CASE_D, C.CASE_E, once):
        assert order(raw) == P.run_order(raw)
    # every run owns a cache or a state of its own
    spec = config_from_dict(C.CASE_C).to_model_spec()
    assert all(run.cache_from is None and run.shift is None for run in spec.order) and spec.stream_shifts is None


def test_tensor_names_shapes_and_cache_plan():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.registry import lookup

    config = config_from_dict(C.CASE_A)
    model = lookup("Lorozen").build_model(config, torch.float32, "cpu")
    shapes = {p.name: tuple(p.spec.shape) for p in model.named_params()}
    assert shapes["embed"] == (150, 96) and shapes["head"] == (150, 96) and shapes["final.norm"] == (96,)
    for index in range(4):
        assert shapes[f"l{index}.norm1"] == shapes[f"l{index}.norm1b"] == (96,)
    assert shapes["l0.norm2"] == shapes["l0.norm2b"] == (96,)
    assert "l3.norm2" not in shapes and "l3.norm2b" not in shapes and {"l3.norm2", "l3.norm2b"} <= model.optional_names()
    assert shapes["l0.mix.q"] == (4 * 24, 96) and shapes["l0.mix.k"] == (2 * 24, 96) and shapes["l0.mix.v"] == (2 * 20, 96)
    assert shapes["l0.mix.q.b"] == (96,) and shapes["l0.mix.k.b"] == (48,) and shapes["l0.mix.v.b"] == (40,)
    assert shapes["l0.mix.sink"] == (4,) and shapes["l0.mix.o"] == (96, 80)
    assert shapes["l2.mix.q"] == (3 * 24, 96) and shapes["l2.mix.dkv"] == (48, 96) and shapes["l2.mix.dkv.norm"] == (40,)
    assert shapes["l2.mix.uk"] == (48, 40) and shapes["l2.mix.uv"] == (72, 40) and shapes["l2.mix.g"] == (3, 96) and shapes["l2.mix.o"] == (96, 72)
    assert shapes["l1.mix.mu.w"] == (96,) and shapes["l1.mix.w1"] == (8, 96) and shapes["l1.mix.w2"] == (48, 8)
    assert shapes["l1.mix.u"] == (3, 16) and shapes["l1.mix.w0"] == (48,) and shapes["l1.mix.norm"] == (48,) and shapes["l1.mix.r"] == (48, 96)
    assert shapes["l1.mlp.gate"] == (112, 96) and shapes["l1.mlp.down"] == (96, 112)
    assert shapes["l0.mlp.router"] == (6, 96) and shapes["l0.mlp.e5.gate"] == (40, 96) and shapes["l0.mlp.e0.down"] == (96, 40)
    assert shapes["l0.mlp.shared.up"] == (56, 96) and "l0.mlp.e6.gate" not in shapes
    assert not any(name.startswith("l0.mlp.shared") for name in {p.name for p in lookup("Lorozen").build_model(
        config_from_dict(C.CASE_B), torch.float32, "cpu").named_params()})
    plan = model.cache_plan()
    assert len(plan.runs) == 6 and [run.kind for run in plan.runs] == ["paged", "state", "paged", "state", "paged", "paged"]
    assert sorted(plan.windows) == [17, 33, 40]                   # a group of pages per window
    assert plan.runs[0].need.head_dim == 24 and plan.runs[0].need.value_dim == 20 and plan.runs[0].need.window == 40
    assert plan.runs[2].need.num_kv_heads == 1 and plan.runs[2].need.head_dim == 48 and plan.runs[2].need.value_dim == 0
    assert plan.runs[2].group == plan.runs[4].group and plan.runs[1].owner != plan.runs[3].owner  # two passes, two caches
    states = [tuple(s.shape) for run in plan.runs for s in run.states]
    assert states.count((3, 16, 16)) == 2 and states.count((96,)) == 2   # wkv: S of every head and the last input row, per pass
    assert model.graph_safe


def test_the_decay_rank_comes_from_the_checkpoint(tmp_path):
    """``config.json`` does not say how wide the decay's low-rank pair is: the shape of ``w1`` does."""
    from turboserve_b200.config import config_from_dir
    from turboserve_b200.weights import checkpoint_index

    folder = C.write_case("C", tmp_path / "c")
    plain = config_from_dir(folder)
    assert "decay_rank" not in plain.layers[0]["mixer"]
    config = plain.with_tensor_shapes({name: tuple(entry[1]) for name, entry in checkpoint_index(folder).items()})
    assert config.layers[0]["mixer"]["decay_rank"] == 3
    assert config.to_model_spec().layers[0].mixer["decay_rank"] == 3


def test_stretched_frequencies_against_the_plain_ones():
    from turboserve_b200.parts.rope import rotary_frequencies, wavelength_scaled_frequencies

    for dims, base, scaling in ((8, 5000.0, (8.0, 1.0, 4.0, 64)), (32, 10000.0, (3.0, 1.0, 5.0, 128)), (2, 50.0, (2.0, 0.5, 3.0, 16)),
                                (64, 500000.0, (8.0, 1.0, 4.0, 8192)), (16, 100.0, None)):
        rot = {"base": base, "dims": dims}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
        ours, amplitude = rotary_frequencies(dims, base, rot.get("scaling"))
        assert amplitude == 1.0 and torch.allclose(ours.double(), P.frequencies(rot), rtol=1e-6, atol=0.0)
        assert torch.equal(ours, wavelength_scaled_frequencies(dims, base, rot.get("scaling")))
    # the three branches are all met: kept, slowed by the whole factor, and in between
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 128}}
    ratio = P.frequencies(rot) / P.frequencies({"base": 10000.0, "dims": 32})
    assert float(ratio[0]) == 1.0 and abs(float(ratio[-1]) - 0.2) < 1e-12 and ((ratio > 0.21) & (ratio < 0.99)).any()


def test_the_oracle_does_what_each_equation_says():
    g = torch.Generator().manual_seed(0)
    eps = 1e-6
    # the learned sink: exp(sink) joins the denominator, unscaled, with no value; a window of 2 drops the first key at position 2
    sizes = dict(heads=1, kv_heads=1, dim=4, vdim=3, scale=0.5, mask={"size": 2}, rot=None)
    w = {"q": torch.eye(4, dtype=F64), "k": torch.eye(4, dtype=F64), "v": torch.randn(3, 4, generator=g, dtype=F64),
         "q.b": torch.zeros(4, dtype=F64), "k.b": torch.zeros(4, dtype=F64), "v.b": torch.tensor([1.0, 2.0, 3.0], dtype=F64),
         "sink": torch.tensor([0.7], dtype=F64), "o": torch.eye(3, dtype=F64)}
    h = torch.tensor([[2.0, 0, 0, 0], [-2.0, 0, 0, 0], [0, 2.0, 0, 0]], dtype=F64)
    out = P.attention(h, w, sizes, eps)
    values = h @ w["v"].T + w["v.b"]
    sink = math.exp(0.7)
    assert torch.allclose(out[0], math.exp(2.0) / (sink + math.exp(2.0)) * values[0], atol=1e-12)
    a, b = math.exp(-2.0), math.exp(2.0)
    assert torch.allclose(out[1], (a * values[0] + b * values[1]) / (sink + a + b), atol=1e-12)
    a, b = math.exp(0.0), math.exp(2.0)  # position 2 sees positions 1 and 2 only
    assert torch.allclose(out[2], (a * values[1] + b * values[2]) / (sink + a + b), atol=1e-12)
    # biases enter before the rotation and the scores
    w2 = dict(w, **{"q.b": torch.tensor([0.0, 1.0, 0, 0], dtype=F64)})
    assert not torch.allclose(P.attention(h, w2, sizes, eps)[2], out[2])
    # rotation of split pairs (i, i + dims / 2), the rest passes; of neighbours (2i, 2i + 1)
    x = torch.tensor([[[1.0, 1.0, 0.0, 0.0, 7.0]], [[1.0, 1.0, 0.0, 0.0, 7.0]]], dtype=F64)
    turned = P.rotate(x, {"base": 100.0, "dims": 4}, False)
    assert torch.allclose(turned[0], x[0]) and turned[1, 0, 4] == 7.0
    assert torch.allclose(turned[1, 0, :4], torch.tensor([math.cos(1.0), math.cos(0.1), math.sin(1.0), math.sin(0.1)], dtype=F64))
    y = torch.tensor([[[1.0, 0.0, 1.0, 0.0]], [[1.0, 0.0, 1.0, 0.0]]], dtype=F64)
    assert torch.allclose(P.rotate(y, {"base": 100.0, "dims": 4}, True)[1, 0],
                          torch.tensor([math.cos(1.0), math.sin(1.0), math.cos(0.1), math.sin(0.1)], dtype=F64))
    # experts: sigmoid scores as they are, on the way in; with top = 1 of 2 the larger logit's expert alone
    mlp = {"kind": "moe", "expert": {"ff": 2}, "router": {"experts": 2, "top": 1}}
    e = {"router": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64)}
    for j in range(2):
        e.update({f"e{j}.gate": torch.randn(2, 2, generator=g, dtype=F64), f"e{j}.up": torch.randn(2, 2, generator=g, dtype=F64),
                  f"e{j}.down": torch.randn(2, 2, generator=g, dtype=F64)})
    hh = torch.tensor([[0.3, 1.2], [0.9, -0.4]], dtype=F64)
    got = P.mixture(hh, e, mlp)
    for t, j in ((0, 1), (1, 0)):
        s = 1.0 / (1.0 + math.exp(-float(hh[t, j])))
        x = s * hh[t]
        assert torch.allclose(got[t], (P.silu(x @ e[f"e{j}.gate"].T) * (x @ e[f"e{j}.up"].T)) @ e[f"e{j}.down"].T, atol=1e-12)
    both = P.mixture(hh, e, dict(mlp, router={"experts": 2, "top": 2}))
    assert not torch.allclose(both, got)
    # the dense feed-forward uses the tanh form of gelu
    z = torch.tensor([0.5, -1.5], dtype=F64)
    assert torch.allclose(P.gelu_tanh(z), 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))


def test_the_oracles_latent_attention_and_wkv_written_out(tmp_path):
    g = torch.Generator().manual_seed(1)
    eps = 1e-5
    # latent attention with explicit keys and values per head, and the gate on the head's output
    sizes = dict(heads=2, dim=3, rot_dim=2, vdim=2, kv_rank=4, scale=0.4, mask={"size": 3}, rot={"base": 10.0, "dims": 2})
    w = {"q": torch.randn(10, 5, generator=g, dtype=F64), "dkv": torch.randn(6, 5, generator=g, dtype=F64),
         "dkv.norm": torch.rand(4, generator=g, dtype=F64) + 0.5, "uk": torch.randn(6, 4, generator=g, dtype=F64),
         "uv": torch.randn(4, 4, generator=g, dtype=F64), "g": torch.randn(2, 5, generator=g, dtype=F64), "o": torch.eye(4, dtype=F64)}
    h = torch.randn(6, 5, generator=g, dtype=F64)
    got = P.latent_attention(h, w, sizes, eps)
    down = h @ w["dkv"].T
    c = P.rms_norm(down[:, :4], w["dkv.norm"], eps)

    def turn(pair, t):
        angle = float(t)  # one pair: frequency base^0 = 1
        return torch.stack([pair[0] * math.cos(angle) - pair[1] * math.sin(angle), pair[1] * math.cos(angle) + pair[0] * math.sin(angle)])

    want = torch.zeros(6, 4, dtype=F64)
    for head in range(2):
        for t in range(6):
            q = (h[t] @ w["q"].T)[5 * head:5 * head + 5]
            scores = []
            for s in range(max(0, t - 2), t + 1):
                key = torch.cat([w["uk"][3 * head:3 * head + 3] @ c[s], turn(down[s, 4:], s)])
                scores.append(0.4 * (torch.cat([q[:3], turn(q[3:], t)]) @ key))
            p = torch.softmax(torch.stack(scores), dim=0)
            value = sum(p[i] * (w["uv"][2 * head:2 * head + 2] @ c[s]) for i, s in enumerate(range(max(0, t - 2), t + 1)))
            want[t, 2 * head:2 * head + 2] = value * torch.sigmoid(h[t] @ w["g"][head])
    assert torch.allclose(got, want, atol=1e-10)
    # wkv written as a sum over earlier tokens: o_t = sum_{s<t} (prod_{s<j<t} w_j) (r_t*k_s) v_s + (r_t*u*k_t) v_t
    sizes = dict(heads=1, dim=3)
    w = {name: torch.randn(3, 4, generator=g, dtype=F64) for name in ("r", "k", "v", "g")}
    w.update({f"mu.{s}": torch.rand(4, generator=g, dtype=F64) for s in "rkvgw"})
    w.update(w1=torch.randn(2, 4, generator=g, dtype=F64), w2=torch.randn(3, 2, generator=g, dtype=F64), w0=torch.randn(3, generator=g, dtype=F64),
             u=torch.randn(1, 3, generator=g, dtype=F64), norm=torch.rand(3, generator=g, dtype=F64), o=torch.eye(3, dtype=F64))
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
    assert torch.allclose(got, P.rms_norm(raw, None, eps) * w["norm"] * P.silu(mixed["g"] @ w["g"].T), atol=1e-9)


def test_the_whole_oracle_is_causal_loops_and_caps(tmp_path):
    g = torch.Generator().manual_seed(2)
    folder = C.write_case("A", tmp_path / "a")
    config, weights = P.read_model_folder(folder)
    tokens = torch.randint(0, config["vocab"], (60,), generator=g).tolist()
    logits, layers = P.forward(config, weights, tokens)
    shorter, _ = P.forward(config, weights, tokens[:23])
    assert torch.allclose(logits[:23], shorter, atol=1e-9) and layers.shape == (6, 60, 96)
    assert float(logits.abs().max()) < 20.0
    # a token beyond every window and without a recurrent layer between cannot be seen: one layer of attention, window 17
    one = C.one_layer(C.attention(2, 2, 16, 16, 0.25, 17, 100.0, 16))
    folder = C.write_raw(one, 3, tmp_path / "one")
    config, weights = P.read_model_folder(folder)
    tokens = [t % config["vocab"] for t in tokens]
    base = P.logits_of(config, weights, tokens[:40])
    for place, moves in ((39 - 17, False), (39 - 16, True)):
        changed = list(tokens[:40])
        changed[place] = (changed[place] + 1) % config["vocab"]
        assert (not torch.allclose(P.logits_of(config, weights, changed)[-1], base[-1], atol=1e-12)) == moves, place
    # a loop that runs twice is not the layers written twice: the embedding comes back before the second pass
    raw = json.loads(json.dumps(C.CASE_E))
    folder = C.write_raw(raw, 5, tmp_path / "e")
    config, weights = P.read_model_folder(folder)
    looped, streams = P.forward(config, weights, tokens[:20])
    embedded = weights["embed"].to(F64)[torch.tensor(tokens[:20])]
    unrolled = dict(config, loop=None, layers=config["layers"] * 2)
    twice = {name.replace("l0.", "l2.").replace("l1.", "l3."): t for name, t in weights.items() if name[:3] in ("l0.", "l1.")}
    plain_twice, streams_twice = P.forward(unrolled, {**weights, **twice}, tokens[:20])
    assert torch.allclose(streams[1], streams_twice[1]) and not torch.allclose(looped, plain_twice)
    assert streams.shape[0] == 4
    # what the second pass starts from is the first pass's stream plus the embedding's output
    config_once = dict(config, loop={"start": 0, "stop": 2, "times": 1})
    _, once = P.forward(config_once, weights, tokens[:20])
    assert torch.allclose(once[1], streams[1]) and embedded.shape == (20, 72)


def test_the_command_line_writes_random_weights_and_plans_the_cache(tmp_path):
    from safetensors import safe_open
    from typer.testing import CliRunner

    from turboserve_b200.cli import app

    runner = CliRunner()
    config = tmp_path / "config.json"
    config.write_text(json.dumps(C.CASE_A))
    out = tmp_path / "model"
    result = runner.invoke(app, ["engine", "random-weights", "--config", str(config), "--out", str(out), "--seed", "7"])
    assert result.exit_code == 0, result.stdout
    written = json.loads((out / "config.json").read_text())
    assert written["architecture"] == "Lorozen" and written["loop"] == C.CASE_A["loop"] and written["logit_softcap"] == 20.0
    with safe_open(str(out / "model.safetensors"), "pt") as f:
        names = set(f.keys())
        assert {"embed", "head", "final.norm", "l0.mix.sink", "l0.mix.q.b", "l0.norm1b", "l2.mix.g", "l1.mix.w0", "l0.mlp.e5.down"} <= names
        assert f.get_tensor("l0.mix.sink").dtype == torch.bfloat16
    result = runner.invoke(app, ["engine", "kv-size", "-m", str(out), "--total-memory-gib", "1", "--block-size", "16",
                                 "--max-num-seqs", "4", "--max-model-len", "256", "--dtype", "bfloat16"])
    assert result.exit_code == 0, result.stdout
    assert json.loads(result.stdout)["num_blocks"] >= 4
