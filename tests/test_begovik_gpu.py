"""Begovik through the engine against the plain implementation (``plain_begovik``).

Kernels alone on made-up inputs, every mixer alone as a model of one layer, then whole models through the replay
loop (whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with pages and state slots
used again), then greedy generation through ``LLMEngine`` and its scheduler.
"""

import math

import pytest
import torch

import begovik_cases as C
import plain_begovik as P
import traces

pytestmark = pytest.mark.gpu

_folders: dict = {}
_references: dict = {}


class _Folders(dict):
    """Model folders by ``(case, sharp)``, written when first asked for."""

    def __init__(self, factory):
        super().__init__()
        self.factory = factory

    def __missing__(self, key):
        name, sharp = key[0], key[1]
        self[key] = C.write_case(name, self.factory.mktemp(f"begovik_{name}_{int(sharp)}"), sharp)
        return self[key]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    global _folders
    if not isinstance(_folders, _Folders):
        _folders = _Folders(tmp_path_factory)
    return _folders


def reference(folder, requests, jitter=0.0):
    config, weights = P.read_model_folder(folder)
    out = {}
    for rid, tokens in requests.items():
        key = (str(folder), tuple(tokens), jitter)
        if key not in _references:
            _references[key] = P.forward(config, weights, tokens, jitter)[0]
        out[rid] = _references[key]
    return out


def run_and_check(folder, dtype, builder, lengths, page_size=16, slack=1.0, **kwargs):
    from turboserve_b200.replay import Replayer

    config = C.read_config(folder)
    requests = traces.make_requests(config["vocab"], lengths, seed=11)
    steps, max_tokens = builder(requests, **kwargs)
    replayer = Replayer(folder, dtype, max_tokens, page_size=page_size)
    got = traces.collect(requests, steps, traces.replay(replayer, steps))
    ref = reference(folder, requests)
    shaken = reference(folder, requests, C.JITTER) if dtype == "bfloat16" else None
    for rid in requests:
        C.check(got[rid], ref[rid], dtype, f"{dtype} {builder.__name__} {rid}", slack, shaken[rid] if shaken else None)
    replayer.manager.check_invariants()
    assert replayer.manager.free_pages() == [g.num_pages for g in replayer.manager.groups]
    return replayer, got


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------

def _paged(rows, page_size, order):
    """``rows`` [T, heads, d] laid into pages in the order ``order`` (a page of the pool per logical page)."""
    tokens, heads, d = rows.shape
    pages = torch.zeros(max(order) + 1, page_size, heads, d, dtype=rows.dtype)
    for t in range(tokens):
        pages[order[t // page_size], t % page_size] = rows[t]
    return pages.cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, cap, sink, page_size", [
    (4, 2, 24, 20, 30.0, True, 16), (8, 1, 8, 8, 5.0, True, 8), (3, 3, 10, 7, 0.0, True, 4), (2, 2, 64, 128, 12.0, False, 32),
    (8, 2, 128, 128, 50.0, True, 16), (4, 1, 64, 64, 0.0, True, 16), (6, 6, 40, 3, 8.0, True, 16)])
def test_attention_with_a_cap_and_a_sink(dtype, heads, kv_heads, dim, vdim, cap, sink, page_size):
    """A prompt's portion and single tokens over keys in scattered pages. One key far back, the keys on both sides of
    every page border near the end and the first key of all are made to stand out for some query; other rows score
    far below zero, so that the sink takes most of their weight."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * dim + vdim)
    tokens, scale = 300, 0.37
    q = torch.randn(tokens, heads, dim, generator=g) * 0.3
    k = torch.randn(tokens, kv_heads, dim, generator=g) * 0.3
    v = torch.randn(tokens, kv_heads, vdim, generator=g)
    per = heads // kv_heads
    marks = {299: 7, 298: 0, 297: 299 - page_size, 296: 299 - page_size + 1, 295: 295 - 255, 250: 250, 200: 3}
    common = torch.randn(dim, generator=g)
    common = common / common.norm()
    for query, key in marks.items():  # query `query` looks for key `key` with every head
        direction = torch.randn(dim, generator=g)
        direction = direction - (direction @ common) * common  # (the marked keys stay as unloved as the others below)
        direction = direction / direction.norm()
        k[key] = k[key] + 6.0 * direction
        q[query] = q[query] + 6.0 * direction
    k = k + 2.0 * common
    q[100:120] = q[100:120] - 14.0 * common  # rows that like nothing they see
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scores = torch.einsum("thd,shd->hts", q.double(), k.double().repeat_interleave(per, dim=1)) * scale
    seen = torch.arange(tokens)[:, None] >= torch.arange(tokens)[None, :]
    if sink:
        weights = P.capped_sink_weights(scores, cap, seen)
    else:
        capped = cap * torch.tanh(scores / cap) if cap else scores
        weights = torch.softmax(capped.masked_fill(~seen, -math.inf), dim=-1)
    want = torch.einsum("hts,shv->thv", weights, v.double().repeat_interleave(per, dim=1)).reshape(tokens, heads * vdim)
    if sink:
        assert float(weights.sum(-1).min()) < 0.5 < float(weights.sum(-1).max())  # the sink counts, and not everywhere

    num_pages = -(-tokens // page_size)
    order = torch.randperm(num_pages + 3, generator=g)[:num_pages].tolist()
    k_pages, v_pages = _paged(k, page_size, order), _paged(v, page_size, order)
    table = _i32([order])
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2

    def run(first, count):
        out = torch.zeros(count, heads * vdim + 5, dtype=dtype, device="cuda")
        kernels.paged_attention_capped(q[first:first + count].reshape(count, heads * dim).cuda(), out, k_pages, v_pages, table,
                                       _i32([0] * count), _i32(list(range(first, first + count))), count, heads, kv_heads, dim, vdim,
                                       None, scale, cap, sink)
        return out[:, :heads * vdim].cpu().double()

    whole = run(0, tokens)
    assert (whole - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    tail = torch.cat([run(t, 1) for t in range(290, 300)])
    assert (tail - want[290:]).abs().max() <= tol * max(1.0, float(want.abs().max()))
    if dtype == torch.float32:
        assert torch.equal(tail, whole[290:])  # one order of every sum, alone or in a portion
    portion = run(180, 120)
    assert (portion - want[180:]).abs().max() <= tol * max(1.0, float(want.abs().max()))
    if not kernels.paged_attention_capped_mma_takes(dtype, dim, vdim, scale):
        return

    # the tiled kernel: a whole prompt; then the end of the same request beside another request's first portion
    def tiled(parts):
        rows = torch.cat([q[first:first + count] for first, count in parts]).reshape(-1, heads * dim).cuda()
        starts = [0]
        for _, count in parts:
            starts.append(starts[-1] + count)
        out = torch.zeros(starts[-1], heads * vdim + 8, dtype=dtype, device="cuda")
        kernels.paged_attention_capped_mma(rows, out, k_pages, v_pages, _i32([order] * len(parts)), _i32(starts),
                                           _i32([first + count for first, count in parts]), starts[-1], len(parts), heads,
                                           kv_heads, dim, vdim, None, scale, cap, sink)
        return out[:, :heads * vdim].cpu().double()

    bound = 2e-2 * max(1.0, float(want.abs().max()))
    assert (tiled([(0, tokens)]) - want).abs().max() <= bound
    both = tiled([(180, 120), (0, 70)])
    assert (both[:120] - want[180:]).abs().max() <= bound and (both[120:] - want[:70]).abs().max() <= bound
    assert torch.equal(tiled([(0, tokens)])[180:], both[:120])  # the same bits however the request is cut
    assert torch.equal(tiled([(299, 1)]), both[119:120])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_normed_rows_mixed_and_the_clamped_gate(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(5)
    n, hidden = 19, 100
    a, b = (torch.randn(n, hidden, generator=g) * 3.0).to(dtype), (torch.randn(n, hidden, generator=g) * 0.01).to(dtype)
    ga, gb = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    out = torch.empty(n, hidden, dtype=dtype, device="cuda")
    kernels.norm_pair_mix(a.cuda(), b.cuda(), ga.cuda(), gb.cuda(), out, n, 1e-5, 0.5, 0.25)
    want = 0.5 * P.rms_norm(a.double(), ga.double(), 1e-5) + 0.25 * P.rms_norm(b.double(), gb.double(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    # g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(1.702 g) (u + 1): values on both sides of the limit
    inter, limit = 36, 0.75
    gate_up = (torch.randn(n, 2 * inter, generator=g) * 1.5).to(dtype)
    out = torch.empty(n, inter, dtype=dtype, device="cuda")
    kernels.act_mul(gate_up.cuda(), out, "clamped_swish", n, limit=limit, alpha=1.702)
    gate, up = gate_up[:, :inter].double().clamp(max=limit), gate_up[:, inter:].double().clamp(-limit, limit)
    assert float(gate_up[:, :inter].max()) > limit and float(gate_up[:, inter:].min()) < -limit
    assert torch.allclose(out.cpu().double(), gate * torch.sigmoid(1.702 * gate) * (up + 1.0), atol=tol, rtol=tol)


ALONE = {
    "attention beside lightning": C.parallel(C.left(4, 2, 24, 20, 0.2, 30.0, 5000.0, 8), C.right(3, 16, 24, (0.9, 0.97, 0.995))),
    "one key head, whole head rotated": C.parallel(C.left(8, 1, 16, 8, 0.3, 20.0, 1000.0, 16), C.right(1, 40, 10, (0.99,))),
    "wide heads": C.parallel(C.left(2, 2, 128, 128, 0.09, 15.0, 10000.0, 64), C.right(2, 128, 64, (0.96, 0.999))),
    "wkv": C.wkv(3, 16, 8),
    "wkv one head": C.wkv(1, 64, 2),
    "wkv odd": C.wkv(5, 6, 3),
    "scan": C.mamba1(80, 12, 6, 4),
    "scan one tap": C.mamba1(36, 3, 1, 1),
    "scan many states": C.mamba1(48, 40, 4, 2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mixer_alone_as_a_model_of_one_layer(tmp_path, which, dtype):
    """Whole, token by token, and in portions: the mixer with nothing but the embedding before it and the head after."""
    folder = C.write_raw(C.one_layer(ALONE[which]), 7, tmp_path / "m")
    run_and_check(folder, dtype, traces.whole, [70, 9])
    run_and_check(folder, dtype, traces.tail_one_by_one, [70], tail=40, page_size=8)
    run_and_check(folder, dtype, traces.changing_portions, [70], sizes=(3, 2, 17, 1, 2, 30))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_feed_forward_alone_beside_a_small_mixer(tmp_path, dtype):
    for limit in (0.2, 1.0, 6.0):
        folder = C.write_raw(C.one_layer(C.wkv(1, 8, 2), C.dense(88, limit), width=72), 9, tmp_path / f"f{limit}")
        run_and_check(folder, dtype, traces.whole, [50])


# ---------------------------------------------------------------------------------------------
# whole models through the replay loop
# ---------------------------------------------------------------------------------------------

LENGTHS = {"A": [1, 7, 33, 100, 150], "B": [5, 40, 129, 70], "C": [3, 64, 130, 200], "D": [2, 9, 61, 140]}
MIXED_LENGTHS = [33, 100, 20, 150, 64, 7, 90, 129, 48, 5, 77, 130]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(folders, name, dtype):
    run_and_check(folders[name, False], dtype, traces.whole, LENGTHS[name])


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_stream_after_every_layer(folders, name):
    """The float32 residual stream after every layer: the first layer that differs names the mechanism."""
    from turboserve_b200.parts.block import ParallelBlock
    from turboserve_b200.replay import Replayer

    folder = folders[name, False]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [45], seed=3)["r0"]
    _, want = P.forward(config, weights, tokens)
    replayer = Replayer(folder, "float32", 64)
    mult = float(config["residual_mult"])
    got = []
    original = ParallelBlock.forward

    def recording(self, residual, pending, ctx, cache, shift=None):
        # a block hands its updates on to the next norm: the stream after it is the residual it got, plus what was
        # pending then, plus its own updates
        out = original(self, residual, pending, ctx, cache, shift)
        n = ctx.batch.num_tokens
        updates = getattr(out, "updates", None) or (out if isinstance(out, tuple) else (out,))
        got.append(residual[:n].cpu().double() + mult * sum(u[:n].cpu().double() for u in updates))
        return out

    ParallelBlock.forward = recording
    try:
        replayer.step([{"id": "a", "tokens": tokens, "want": []}], ["a"])
    finally:
        ParallelBlock.forward = original
    assert len(got) == len(want) == len(config["layers"])
    for index, (ours, ref) in enumerate(zip(got, want)):
        assert (ours - ref).abs().max() <= 3e-5 * max(1.0, float(ref.abs().max())), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompt_then_token_by_token(folders, name, dtype):
    run_and_check(folders[name, False], dtype, traces.tail_one_by_one, LENGTHS[name], tail=80)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size_down_to_two_tokens(folders, name, dtype):
    run_and_check(folders[name, False], dtype, traces.changing_portions, LENGTHS[name])
    run_and_check(folders[name, False], dtype, traces.changing_portions, LENGTHS[name][-2:], sizes=(2, 2, 3, 2, 1, 2), page_size=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("page_size", [16, 8])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, dtype, page_size):
    """Twelve requests, four live at a time, unequal portions beside single tokens: four state slots and a pool
    that holds the live requests only, so every slot and page goes to several requests."""
    replayer, _ = run_and_check(folders[name, False], dtype, traces.mixed, MIXED_LENGTHS, page_size=page_size, seed=3)
    assert replayer.manager.slots.num_slots == 4
    for pool, group in zip(replayer.manager.pools, replayer.manager.groups):
        assert pool.num_allocations > group.num_pages


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_sharp_scores_and_slow_decay_in_float32(folders, name):
    """Weights under which single keys stand out and the states remember hundreds of tokens: keys far back and at
    page borders, the sink's changing share, carried state; in prompts, in portions, token by token, in mixed batches."""
    folder = folders[name, True]
    lengths = [400, 170]
    run_and_check(folder, "float32", traces.whole, lengths, slack=2.5)
    run_and_check(folder, "float32", traces.tail_one_by_one, lengths, tail=90, slack=2.5)
    run_and_check(folder, "float32", traces.changing_portions, lengths, page_size=8, slack=2.5)
    run_and_check(folder, "float32", traces.mixed, [170, 60, 200, 33, 90, 120], seed=8, slack=2.5)


@pytest.mark.parametrize("name", ["A", "D"])
def test_sharp_scores_in_bfloat16_token_by_token(folders, name):
    run_and_check(folders[name, True], "bfloat16", traces.tail_one_by_one, [300], tail=100, slack=3.0)
    run_and_check(folders[name, True], "bfloat16", traces.mixed, [170, 60, 200, 33, 90], seed=8, slack=3.0)


def test_the_sharp_weights_do_make_single_keys_and_old_state_count(folders):
    """Under the sharpened weights a late position's logits move by far more than the tolerance when the first token
    of all, or a token 250 positions back, is another one."""
    folder = folders["A", True]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [300], seed=2)["r0"]
    base = P.logits_of(config, weights, tokens)[-1:]
    for place in (0, 49):
        changed = list(tokens)
        changed[place] = (changed[place] + 1) % config["vocab"]
        other = P.logits_of(config, weights, changed)[-1:]
        assert float(C.relative_error(other, base).max()) > 20 * C.FP32_REL, place


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_single_tokens_do_not_depend_on_the_batch_at_all(folders, name):
    """Decoded through other pages: a single token's float32 logits are the same bits (every sum has one order)."""
    folder = folders[name, False]
    _, a = run_and_check(folder, "float32", traces.tail_one_by_one, [90, 60, 41], tail=30)
    _, b = run_and_check(folder, "float32", traces.tail_one_by_one, [90, 60, 41], tail=30, page_size=8)
    for rid in a:
        assert torch.equal(a[rid][-29:], b[rid][-29:]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    """Positions 0, 1, 2 one by one and two at once: an empty state, zeros before the first token, a lone key beside the sink."""
    from turboserve_b200.replay import Replayer

    for name in C.CASES:
        folder = folders[name, False]
        config, weights = P.read_model_folder(folder)
        tokens = [5, 9, 2]
        ref = P.logits_of(config, weights, tokens)
        replayer = Replayer(folder, dtype, 64)
        rows = [replayer.step([{"id": "x", "tokens": [t], "want": [0]}], []) for t in tokens]
        C.check(torch.cat(rows), ref, dtype, f"{name} first tokens")
        replayer.step([], ["x"])
        both = replayer.step([{"id": "y", "tokens": tokens[:2], "want": [0, 1]}], ["y"])
        C.check(both, ref[:2], dtype, f"{name} first two tokens")


def test_a_slot_that_is_used_again_starts_empty(folders):
    """A request that follows another in the same state slot gets what it gets alone (float32, same bits)."""
    from turboserve_b200.replay import Replayer

    folder = folders["A", True]
    config = C.read_config(folder)
    requests = traces.make_requests(config["vocab"], [70, 40], seed=9)
    replayer = Replayer(folder, "float32", 128, state_slots=1)
    first = replayer.step([{"id": "a", "tokens": requests["r0"], "want": [69]}], ["a"])
    second = replayer.step([{"id": "b", "tokens": requests["r1"], "want": list(range(40))}], ["b"])
    alone = Replayer(folder, "float32", 128, state_slots=1).step([{"id": "b", "tokens": requests["r1"], "want": list(range(40))}], ["b"])
    assert first is not None and torch.equal(second, alone)


def test_long_decoding(folders):
    """600 tokens one by one after a short prompt: every state is carried 600 steps, the attention reads 40 pages."""
    run_and_check(folders["A", True], "float32", traces.tail_one_by_one, [620], tail=600, slack=2.5, page_size=16)
    run_and_check(folders["D", False], "bfloat16", traces.tail_one_by_one, [420], tail=400, slack=1.5, page_size=16)


# ---------------------------------------------------------------------------------------------
# generation through the engine's own entry point and scheduler
# ---------------------------------------------------------------------------------------------


def engine_for(folder, dtype, **scheduler):
    from turboserve_b200 import EngineConfig, LLMEngine, SchedulerConfig

    defaults = dict(max_num_seqs=4, max_num_batched_tokens=256, block_size=16, num_blocks=64)
    defaults.update(scheduler)
    return LLMEngine(EngineConfig(model=str(folder), dtype=dtype, scheduler=SchedulerConfig(**defaults)))


def check_greedy_path(config, weights, prompt, generated, dtype):
    """Every generated token is the plain argmax given the tokens before it (in bfloat16: or a token
    whose plain logit lies within the bfloat16 tolerance of the best)."""
    logits = P.logits_of(config, weights, prompt + generated)
    spread = float((logits - logits.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    slack = (C.FP32_REL if dtype == "float32" else C.BF16_REL) * spread * 4
    for i, token in enumerate(generated):
        row = logits[len(prompt) + i - 1]
        best = int(row.argmax())
        assert token == best or row[best] - row[token] <= slack, (i, token, best, float(row[best] - row[token]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, lengths, new", [("A", [1, 7, 33, 100, 60, 12], 40), ("B", [5, 40, 129], 30), ("C", [3, 70], 24)])
def test_greedy_generation_through_the_engine(folders, name, lengths, new, dtype):
    from turboserve_b200 import SamplingParams

    folder = folders[name, False]
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in lengths]
    with engine_for(folder, dtype) as engine:
        outputs = engine.generate(prompts, SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True))
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    for prompt, out in zip(prompts, outputs):
        assert out.finished and out.output_tokens == new and out.prompt_tokens == len(prompt)
        check_greedy_path(config, weights, prompt, out.token_ids, dtype)
    if dtype == "float32":
        assert outputs[1].token_ids[:6] == P.greedy(config, weights, prompts[1], 6)


def test_small_budget_and_few_pages_change_no_token(folders):
    """Prompts cut by a token budget of 16, and a pool too small for everyone (requests are preempted, their state
    slots zeroed and their prompts computed again): every token still follows the plain logits in float32."""
    from turboserve_b200 import SamplingParams

    folder = folders["A", False]
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in [5, 40, 129, 33, 64, 18]]
    sampling = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    with engine_for(folder, "float32", max_num_batched_tokens=16) as engine:
        chunked = engine.generate(prompts, sampling)
    with engine_for(folder, "float32", max_num_batched_tokens=64, num_blocks=14) as engine:
        tight = engine.generate(prompts, sampling)
        stats = engine.stats()
        engine.scheduler.check_invariants()
    assert stats["num_preemptions"] > 0
    for prompt, a, b in zip(prompts, chunked, tight):
        check_greedy_path(config, weights, prompt, a.token_ids, "float32")
        check_greedy_path(config, weights, prompt, b.token_ids, "float32")


def test_bfloat16_with_steps_launched_ahead_and_preemption_together(folders):
    from turboserve_b200 import SamplingParams

    folder = folders["D", False]
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in [5, 40, 129, 33, 64, 18, 90]]
    sampling = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
    with engine_for(folder, "bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_blocks=22) as engine:
        outputs = engine.generate(prompts, sampling)
        stats = engine.stats()
        engine.scheduler.check_invariants()
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    assert stats["num_preemptions"] > 0
    for prompt, out in zip(prompts, outputs):
        assert out.output_tokens == 40
        check_greedy_path(config, weights, prompt, out.token_ids, "bfloat16")
