"""Lorozen through the engine against the plain implementation (``plain_lorozen``).

Kernels alone on made-up inputs, every mixer and feed-forward alone as a model of one layer, then whole models through
the replay loop (whole prompts, the stream after every layer, token-by-token decoding, portions down to two tokens,
mixed batches with pages and state slots used again), then greedy generation through ``LLMEngine`` and its scheduler.
"""

import json
import math

import pytest
import torch

import lorozen_cases as C
import plain_lorozen as P
import traces

pytestmark = pytest.mark.gpu

_folders: dict = {}
_references: dict = {}


class _Folders(dict):
    """Model folders by ``(case, sharp)`` or ``(case, sharp, dtype)``, written when first asked for. A bfloat16
    comparison gets the folder whose routers are steady (``lorozen_cases.steady_routing``)."""

    def __init__(self, factory):
        super().__init__()
        self.factory = factory

    def __missing__(self, key):
        name, sharp = key[0], key[1]
        steady = len(key) > 2 and key[2] == "bfloat16"
        self[key] = C.write_case(name, self.factory.mktemp(f"lorozen_{name}_{int(sharp)}_{int(steady)}"), sharp, steady)
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
    ref, shaken = reference(folder, requests), reference(folder, requests, C.JITTER[dtype])
    for rid in requests:
        C.check(got[rid], ref[rid], dtype, f"{dtype} {builder.__name__} {rid}", slack, shaken[rid])
    replayer.manager.check_invariants()
    assert replayer.manager.free_pages() == [g.num_pages for g in replayer.manager.groups]
    return replayer, got


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def _context(query_lens, dtype, starts=None, slots=None, tables=None):
    """A step context for parts that are run alone: one request per entry of ``query_lens``."""
    from turboserve_b200.engine.batch import RequestSlice, StepContext, Workspace, build_step_batch

    starts = starts or [0] * len(query_lens)
    slots = slots or list(range(len(query_lens)))
    tables = tables or [[0]] * len(query_lens)
    slices = [RequestSlice(token_ids=[0] * n, start_position=s, block_tables=[list(t)], state_slot=slot)
              for n, s, slot, t in zip(query_lens, starts, slots, tables)]
    batch = build_step_batch(slices, 1, "cuda")
    return StepContext(batch=batch, workspace=Workspace("cuda"), dtype=dtype, device=torch.device("cuda"),
                       status=torch.zeros(1, dtype=torch.int32, device="cuda"))


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [100, 192, 1000])
def test_the_norm_behind_one_sublayer_and_before_the_next_in_one_kernel(dtype, hidden):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(hidden)
    n = 23
    res = torch.randn(n, hidden, generator=g) * 3.0
    update = (torch.randn(n, hidden, generator=g) * 0.02).to(dtype)   # a small output counts as much as a large one
    extra = torch.randn(n, hidden, generator=g)
    post, pre = 1 + 0.3 * torch.randn(hidden, generator=g), 1 + 0.3 * torch.randn(hidden, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for with_update, with_extra, with_out in ((True, False, True), (True, True, True), (False, True, True), (False, False, True),
                                              (True, False, False), (False, True, False)):
        want = res.double()
        if with_update:
            want = want + P.rms_norm(update.double(), post.double(), 1e-5)
        if with_extra:
            want = want + extra.double()
        residual = res.cuda()
        out = torch.zeros(n, hidden, dtype=dtype, device="cuda") if with_out else None
        kernels.norm_add_norm(residual, update.cuda() if with_update else None, post.cuda() if with_update else None, 1e-5,
                              extra.cuda() if with_extra else None, pre.cuda() if with_out else None, 1e-6, out, n, dtype)
        assert torch.allclose(residual.cpu().double(), want, atol=2e-6, rtol=1e-6)
        if with_out:
            assert torch.allclose(out.cpu().double(), P.rms_norm(want, pre.double(), 1e-6), atol=tol, rtol=tol)
    # chosen rows alone (the final norm): the residual stays as it is
    rows = [5, 0, 22, 7]
    residual = res.cuda()
    out = torch.zeros(len(rows), hidden, dtype=dtype, device="cuda")
    kernels.norm_add_norm(residual, update.cuda(), post.cuda(), 1e-5, None, pre.cuda(), 1e-6, out, len(rows), rows=_i32(rows))
    want = P.rms_norm(res.double() + P.rms_norm(update.double(), post.double(), 1e-5), pre.double(), 1e-6)[rows]
    assert torch.equal(residual.cpu(), res) and torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


def test_capped_logits():
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(3)
    logits = torch.randn(7, 333, generator=g) * 40.0
    data = logits.cuda()
    kernels.softcap_rows(data, 22.0, 5)
    assert torch.allclose(data[:5].cpu().double(), 22.0 * torch.tanh(logits[:5].double() / 22.0), atol=1e-5)
    assert torch.equal(data[5:].cpu(), logits[5:]) and float(data[:5].abs().max()) <= 22.0


def _paged(rows, page_size, order):
    """``rows`` [T, heads, d] laid into pages in the order ``order`` (a page of the pool per logical page)."""
    tokens, heads, d = rows.shape
    pages = torch.zeros(max(order) + 1, page_size, heads, d, dtype=rows.dtype)
    for t in range(tokens):
        pages[order[t // page_size], t % page_size] = rows[t]
    return pages.cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, page_size", [
    (4, 2, 24, 20, 40, 16), (8, 1, 16, 8, 130, 8), (3, 3, 10, 7, 9, 4), (8, 2, 64, 64, 100, 16), (2, 2, 128, 128, 64, 32), (4, 4, 32, 48, None, 16)])
def test_attention_with_a_learned_sink_and_a_window(dtype, heads, kv_heads, dim, vdim, window, page_size):
    """A prompt's portion and single tokens over keys in scattered pages. For some queries the key at the far edge of
    the window, the one just outside it, the keys on both sides of a page border and the first key of all are made to
    stand out; other rows score far below their head's sink, which then takes most of their weight. Heads have sinks
    from -3 to 4."""
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(heads * dim + vdim)
    tokens, scale = 300, 0.37
    reach = window or tokens
    q = torch.randn(tokens, heads, dim, generator=g) * 0.3
    k = torch.randn(tokens, kv_heads, dim, generator=g) * 0.3
    v = torch.randn(tokens, kv_heads, vdim, generator=g)
    sinks = torch.linspace(-3.0, 4.0, heads)
    per = heads // kv_heads
    # query -> key: the window's last key, the first one outside it (must not count), page borders, the first key of all
    marks = {299: max(0, 299 - reach + 1), 298: max(0, 298 - reach), 297: 299 - page_size, 296: 299 - page_size + 1, 250: 250,
             min(reach - 1, 200): 0, 150: max(0, 150 - reach + 1)}
    common = torch.randn(dim, generator=g)
    common = common / common.norm()
    for query, key in marks.items():
        direction = torch.randn(dim, generator=g)
        direction = direction - (direction @ common) * common
        direction = direction / direction.norm()
        k[key] = k[key] + 6.0 * direction
        q[query] = q[query] + 6.0 * direction
    k = k + 2.0 * common
    q[100:120] = q[100:120] - 14.0 * common  # rows that like nothing they see
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scores = torch.einsum("thd,shd->hts", q.double(), k.double().repeat_interleave(per, dim=1)) * scale
    scores = scores.masked_fill(~P.seen(tokens, window), -math.inf)
    column = sinks.double().reshape(heads, 1, 1).expand(heads, tokens, 1)
    weights = torch.softmax(torch.cat([scores, column], dim=-1), dim=-1)[..., :tokens]
    want = torch.einsum("hts,shv->thv", weights, v.double().repeat_interleave(per, dim=1)).reshape(tokens, heads * vdim)
    assert float(weights.sum(-1).min()) < 0.3 and float(weights.sum(-1).max()) > 0.7  # the sink counts, and not everywhere
    if window:
        assert float(weights[:, 299, 299 - reach + 1].max()) > 0.3  # the key at the window's far edge decides position 299

    num_pages = -(-tokens // page_size)
    order = torch.randperm(num_pages + 3, generator=g)[:num_pages].tolist()
    k_pages, v_pages = _paged(k, page_size, order), _paged(v, page_size, order)
    table = _i32([order])
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    bound = tol * max(1.0, float(want.abs().max()))

    def run(first, count):
        out = torch.zeros(count, heads * vdim + 5, dtype=dtype, device="cuda")
        kernels.paged_attention_capped(q[first:first + count].reshape(count, heads * dim).cuda(), out, k_pages, v_pages, table,
                                       _i32([0] * count), _i32(list(range(first, first + count))), count, heads, kv_heads, dim, vdim,
                                       window, scale, 0.0, True, sink_values=sinks.cuda())
        return out[:, :heads * vdim].cpu().double()

    whole = run(0, tokens)
    assert (whole - want).abs().max() <= bound
    tail = torch.cat([run(t, 1) for t in range(290, 300)])
    assert (tail - want[290:]).abs().max() <= bound
    if dtype == torch.float32:
        assert torch.equal(tail, whole[290:])  # one order of every sum, alone or in a portion
    assert (run(180, 120) - want[180:]).abs().max() <= bound
    # without the heads' own numbers the sink scores 0: another result
    out = torch.zeros(tokens, heads * vdim, dtype=dtype, device="cuda")
    kernels.paged_attention_capped(q.reshape(tokens, heads * dim).cuda(), out, k_pages, v_pages, table, _i32([0] * tokens),
                                   _i32(list(range(tokens))), tokens, heads, kv_heads, dim, vdim, window, scale, 0.0, True)
    assert (out.cpu().double() - want).abs().max() > 10 * bound
    if not kernels.paged_attention_capped_mma_takes(dtype, dim, vdim, scale):
        return

    def tiled(parts):
        rows = torch.cat([q[first:first + count] for first, count in parts]).reshape(-1, heads * dim).cuda()
        starts = [0]
        for _, count in parts:
            starts.append(starts[-1] + count)
        out = torch.zeros(starts[-1], heads * vdim + 8, dtype=dtype, device="cuda")
        kernels.paged_attention_capped_mma(rows, out, k_pages, v_pages, _i32([order] * len(parts)), _i32(starts),
                                           _i32([first + count for first, count in parts]), starts[-1], len(parts), heads,
                                           kv_heads, dim, vdim, window, scale, 0.0, True, sink_values=sinks.cuda())
        return out[:, :heads * vdim].cpu().double()

    bound = 2e-2 * max(1.0, float(want.abs().max()))
    assert (tiled([(0, tokens)]) - want).abs().max() <= bound
    both = tiled([(180, 120), (0, 70)])
    assert (both[:120] - want[180:]).abs().max() <= bound and (both[120:] - want[:70]).abs().max() <= bound
    assert (tiled([(297, 3)]) - want[297:]).abs().max() <= bound and (tiled([(299, 1)]) - want[299:]).abs().max() <= bound


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_biases_enter_before_the_rotation_and_reach_the_pages(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(8)
    heads, kv_heads, dim, vdim, rot, page_size, n = 3, 1, 12, 5, 8, 4, 9
    width = (heads + kv_heads) * dim + kv_heads * vdim
    qkv = torch.randn(n, width, generator=g).to(dtype)
    bias = torch.randn(width, generator=g)
    freq = torch.tensor([1.0, 0.3, 0.05, 0.001])
    positions = list(range(20, 20 + n))
    k_pages = torch.zeros(8, page_size, kv_heads, dim, dtype=dtype, device="cuda")
    v_pages = torch.zeros(8, page_size, kv_heads, vdim, dtype=dtype, device="cuda")
    table = _i32([[3, 1, 4, 0, 5, 7, 2, 6]])
    work = qkv.cuda()
    kernels.head_norm_rope_write(work, None, None, 1e-6, _i32(positions), _i32([0] * n), table, k_pages, v_pages, n, heads, kv_heads,
                                 dim, vdim, freq.cuda(), rot, False, True, None, bias=bias.cuda())
    full = qkv.double() + bias.double()
    angle = torch.tensor(positions, dtype=torch.float64)[:, None] * freq.double()[None, :]

    def turned(x):  # [n, heads, dim]
        out = x.clone()
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2] = a * torch.cos(angle)[:, None] - b * torch.sin(angle)[:, None]
        out[..., rot // 2:rot] = b * torch.cos(angle)[:, None] + a * torch.sin(angle)[:, None]
        return out

    tol = 1e-5 if dtype == torch.float32 else 3e-2
    want_q = turned(full[:, :heads * dim].reshape(n, heads, dim))
    assert torch.allclose(work[:, :heads * dim].cpu().double().reshape(n, heads, dim), want_q, atol=tol, rtol=tol)
    want_k = turned(full[:, heads * dim:(heads + kv_heads) * dim].reshape(n, kv_heads, dim))
    order = table[0].tolist()
    for i, p in enumerate(positions):
        assert torch.allclose(k_pages[order[p // page_size], p % page_size].cpu().double(), want_k[i], atol=tol, rtol=tol)
        assert torch.allclose(v_pages[order[p // page_size], p % page_size, 0].cpu().double(), full[i, -vdim:], atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_heads_outputs_through_its_gate(dtype):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(4)
    n, heads, rank, vdim = 70, 5, 24, 10
    x = torch.randn(n, heads * rank, generator=g).to(dtype)
    w = (torch.randn(heads, vdim, rank, generator=g) * 0.3).to(dtype)
    wide = (torch.randn(n, 11 + heads, generator=g) * 2.0).to(dtype)  # the gate's numbers lie at the end of wider rows
    out = torch.zeros(n, heads * vdim, dtype=dtype, device="cuda")
    kernels.head_linear(x.cuda(), rank, w.cuda(), out, vdim, n, gate=wide.cuda()[:, 11:])
    want = torch.einsum("thr,hvr->thv", x.double().reshape(n, heads, rank), w.double()) * torch.sigmoid(wide[:, 11:].double())[:, :, None]
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double().reshape(n, heads, vdim), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("experts, top", [(8, 2), (6, 1), (4, 4), (12, 3), (64, 6)])
def test_router_with_sigmoid_scores_used_as_they_are(experts, top):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(experts)
    n, width = 300, 72
    h = torch.randn(n, width, generator=g).bfloat16()
    router = torch.randn(experts, width, generator=g) * 0.3
    want_ids, want_weights = P.route(h.double(), router.double(), top)
    for dtype in (torch.bfloat16, torch.float32):
        chosen = torch.zeros(n, top, dtype=torch.int32, device="cuda")
        weights = torch.zeros(n, top, device="cuda")
        kernels.moe_route(h.to(dtype).cuda(), router.cuda(), chosen, weights, n, top, 1, 1, "sigmoid", False)
        assert torch.equal(chosen.cpu().long(), want_ids)
        assert torch.allclose(weights.cpu().double(), want_weights, atol=2e-6, rtol=1e-5)
    assert float(want_weights.sum(-1).max()) > 1.0 or top == 1  # not a distribution: nothing is renormalized


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, ff, shared, width", [(8, 2, 48, 32, 96), (6, 1, 40, None, 100), (4, 4, 24, None, 64), (12, 3, 32, 64, 128)])
def test_experts_weighted_on_the_way_in(dtype, experts, top, ff, shared, width):
    """The same rows as a step of single tokens (pairs in expert order, an expert streamed once for its tokens), as one portion
    of a prompt (one product per expert), mixed, and as a step of very few single tokens (every pair streams its expert):
    all against the plain mixture, whose experts read the token times the score."""
    from turboserve_b200.config.lorozen import EXPERT_NAMES
    from turboserve_b200.config.model_spec import PartSpec
    from turboserve_b200.parts.base import FEED_FORWARDS

    g = torch.Generator().manual_seed(ff)
    n = 57
    spec = PartSpec("routed_experts", dict(experts=experts, top=top, intermediate_size=ff, shared=shared, score="sigmoid",
                                           renormalize=False, weight_on="input", names=EXPERT_NAMES))
    part = FEED_FORWARDS.get("routed_experts")(spec, width, dtype, "cuda")
    weights = {}
    for p in part.param_specs():
        std = 0.1 if p.name == "router" else 0.15  # logits of about one: scores well inside (0, 1)
        weights[p.name] = (torch.randn(p.shape, generator=g) * std).bfloat16()
    part.bind({p.name: weights[p.name].to("cuda", p.device_dtype(dtype)) for p in part.param_specs()})
    x = torch.randn(n, width, generator=g).to(dtype)
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    plain = {k: v.double() for k, v in weights.items()}
    want = P.mixture(x.double(), plain, mlp)
    # the weight on the way out is another function: the test would see the difference
    chosen, scores = P.route(x.double(), plain["router"], top)
    other = torch.zeros_like(want)
    for t in range(n):
        for e, s in zip(chosen[t].tolist(), scores[t]):
            other[t] += s * P.gated(x[t:t + 1].double(), plain, f"e{e}.", P.silu)[0]
    if shared:
        other = other + P.gated(x.double(), plain, "shared.", P.silu)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    scale = float(want.abs().max())
    assert (other - want).abs().max() > 3 * tol * scale
    for query_lens in ([1] * n, [n], [20, 1, 36]):
        out = part.forward(x.cuda(), _context(query_lens, dtype))
        assert (out.cpu().double() - want).abs().max() <= tol * scale, query_lens
    few = max(1, 4 // top)  # so few single tokens that every pair streams its expert alone
    out = part.forward(x[:few].cuda(), _context([1] * few, dtype))
    assert (out.cpu().double() - want[:few]).abs().max() <= tol * scale


# ---------------------------------------------------------------------------------------------
# every mechanism alone as a model of one layer
# ---------------------------------------------------------------------------------------------

ALONE = {
    "attention": (C.attention(4, 2, 24, 20, 0.2, 40, 5000.0, 8, (8.0, 1.0, 4.0, 64)), None),
    "attention one key head, whole head rotated, short window": (C.attention(8, 1, 16, 8, 0.3, 9, 1000.0, 16), None),
    "attention wide heads": (C.attention(2, 2, 128, 128, 0.09, 64, 10000.0, 64, (6.0, 1.0, 3.0, 32)), None),
    "attention no window": (C.attention(3, 3, 10, 7, 0.4, None, 50.0, 2), None),
    "latent": (C.latent(3, 16, 8, 24, 40, 0.15, 33, 1000.0), None),
    "latent short window": (C.latent(4, 8, 16, 16, 24, 0.35, 9, 20000.0), None),
    "latent odd": (C.latent(5, 6, 4, 10, 12, 0.3, 21, 300.0), None),
    "latent no window": (C.latent(2, 24, 2, 8, 16, 0.2, None, 50.0), None),
    "wkv": (C.wkv(3, 16, 8), None),
    "wkv one head": (C.wkv(1, 64, 2), None),
    "wkv odd": (C.wkv(5, 6, 3), None),
    "dense": (C.wkv(1, 8, 2), C.dense(88)),
    "experts": (C.wkv(1, 8, 2), C.moe(6, 2, 40, 56)),
    "experts all chosen, none shared": (C.wkv(1, 8, 2), C.moe(3, 3, 24)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mechanism_alone_as_a_model_of_one_layer(tmp_path, which, dtype):
    """Whole, token by token past the window, and in portions: with nothing but the embedding before and the head after."""
    mixer, mlp = ALONE[which]
    folder = C.write_raw(C.one_layer(mixer, mlp, cap=15.0 if "odd" in which else None), 7, tmp_path / "m",
                         steady=dtype == "bfloat16" and mlp is not None and mlp["kind"] == "moe")
    run_and_check(folder, dtype, traces.whole, [70, 9])
    run_and_check(folder, dtype, traces.tail_one_by_one, [70], tail=40, page_size=8)
    run_and_check(folder, dtype, traces.changing_portions, [70], sizes=(3, 2, 17, 1, 2, 30))


# ---------------------------------------------------------------------------------------------
# whole models through the replay loop
# ---------------------------------------------------------------------------------------------

LENGTHS = {"A": [1, 7, 33, 100, 150], "B": [5, 40, 129, 70], "C": [3, 64, 130, 200], "D": [2, 9, 61, 170], "E": [4, 90, 31]}
MIXED_LENGTHS = [33, 100, 20, 150, 64, 7, 90, 129, 48, 5, 77, 130]
NAMES = sorted(C.CASES)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(folders, name, dtype):
    run_and_check(folders[name, False, dtype], dtype, traces.whole, LENGTHS[name])


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(folders, name):
    """The float32 residual stream after every layer run: the first run that differs names the mechanism."""
    from turboserve_b200.parts.block import BothSidesNormBlock
    from turboserve_b200.replay import Replayer

    folder = folders[name, False]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [45], seed=3)["r0"]
    _, want = P.forward(config, weights, tokens)
    replayer = Replayer(folder, "float32", 64)
    got = []
    original = BothSidesNormBlock.forward

    def recording(self, residual, pending, ctx, cache, **extras):
        # a block leaves its last sublayer's output pending with its norm: the stream after the block is the residual
        # plus that output normed
        out = original(self, residual, pending, ctx, cache, **extras)
        n = ctx.batch.num_tokens
        update = out.update[:n].cpu().double()
        got.append(residual[:n].cpu().double() + P.rms_norm(update, out.gain.cpu().double(), out.eps))
        return out

    BothSidesNormBlock.forward = recording
    try:
        replayer.step([{"id": "a", "tokens": tokens, "want": []}], ["a"])
    finally:
        BothSidesNormBlock.forward = original
    assert len(got) == len(want) == len(P.run_order(config))
    for index, (ours, ref) in enumerate(zip(got, want)):
        assert (ours - ref).abs().max() <= 3e-5 * max(1.0, float(ref.abs().max())), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(folders, name, dtype):
    """The windows (9 to 130 positions) pass over decoded tokens: the tail is longer than every one of them."""
    run_and_check(folders[name, False, dtype], dtype, traces.tail_one_by_one, LENGTHS[name], tail=140 if name == "D" else 80)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_changing_size_down_to_two_tokens(folders, name, dtype):
    folder = folders[name, False, dtype]
    run_and_check(folder, dtype, traces.changing_portions, LENGTHS[name])
    run_and_check(folder, dtype, traces.changing_portions, LENGTHS[name][-2:], sizes=(2, 2, 3, 2, 1, 2), page_size=8)
    run_and_check(folder, dtype, traces.changing_portions, LENGTHS[name][-1:], sizes=(40, 33, 64, 35, 70), page_size=32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("page_size", [16, 8])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name, dtype, page_size):
    """Twelve requests, four live at a time, unequal portions beside single tokens: four state slots and a pool
    that holds the live requests only, so every slot and page goes to several requests."""
    replayer, _ = run_and_check(folders[name, False, dtype], dtype, traces.mixed, MIXED_LENGTHS, page_size=page_size, seed=3)
    assert replayer.manager.slots.num_slots == 4
    for pool, group in zip(replayer.manager.pools, replayer.manager.groups):
        assert pool.num_allocations > group.num_pages


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_sharp_scores_sinks_and_slow_decay_in_float32(folders, name):
    """Weights under which single keys stand out, the sinks take from nearly nothing to most of the weight and the states
    remember hundreds of tokens: a window's edge, page borders, carried state; in prompts, in portions, token by token,
    in mixed batches."""
    folder = folders[name, True]
    lengths = [400, 170]
    run_and_check(folder, "float32", traces.whole, lengths, slack=2.5)
    run_and_check(folder, "float32", traces.tail_one_by_one, lengths, tail=150, slack=2.5)
    run_and_check(folder, "float32", traces.changing_portions, lengths, page_size=8, slack=2.5)
    run_and_check(folder, "float32", traces.mixed, [170, 60, 200, 33, 90, 120], seed=8, slack=2.5)


@pytest.mark.parametrize("name", ["A", "D"])
def test_sharp_scores_in_bfloat16_token_by_token(folders, name):
    run_and_check(folders[name, True, "bfloat16"], "bfloat16", traces.tail_one_by_one, [300], tail=150, slack=2.0)
    run_and_check(folders[name, True, "bfloat16"], "bfloat16", traces.mixed, [170, 60, 200, 33, 90], seed=8, slack=2.0)


def test_the_sharp_weights_do_make_single_keys_and_old_state_count(folders):
    """Under the sharpened weights a late position's logits move by far more than the tolerance when the first token of
    all (which only a recurrent state still holds), or the token at the far edge of the shortest window, is another one."""
    folder = folders["A", True]
    config, weights = P.read_model_folder(folder)
    tokens = traces.make_requests(config["vocab"], [300], seed=2)["r0"]
    base = P.logits_of(config, weights, tokens)[-1:]
    for place in (0, 299 - 16):
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
        folder = folders[name, False, dtype]
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
    """A request that follows another in the same state slot and pages gets what it gets alone (float32, same bits)."""
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
    """600 tokens one by one after a short prompt: every state is carried 600 steps, every window moves over 40 pages."""
    run_and_check(folders["A", True], "float32", traces.tail_one_by_one, [620], tail=600, slack=2.5, page_size=16)
    run_and_check(folders["D", False, "bfloat16"], "bfloat16", traces.tail_one_by_one, [420], tail=400, slack=1.5, page_size=16)


def test_other_constants_than_any_case(tmp_path):
    """A loop that runs once, a cap of 1, a scale of 1, a window of one position (a token sees itself and the sink), a
    factor of 1 in the stretched frequencies, one expert of one."""
    raw = C.model(50, 48, 1e-3, [
        C.layer(C.attention(2, 1, 8, 8, 1.0, 1, 7.0, 8, (1.0, 1.0, 2.0, 8)), C.moe(1, 1, 16, 8)),
        C.layer(C.latent(1, 8, 8, 8, 8, 1.0, 1, 7.0), C.dense(8)),
        C.layer(C.wkv(1, 8, 1), None),
    ], cap=1.0, loop=(1, 2, 1))
    folder = C.write_raw(raw, 12, tmp_path / "m")
    for dtype in ("float32", "bfloat16"):
        run_and_check(folder, dtype, traces.whole, [40, 3])
        run_and_check(folder, dtype, traces.tail_one_by_one, [40], tail=20)
        run_and_check(folder, dtype, traces.changing_portions, [40], sizes=(2, 5, 1, 2))


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
@pytest.mark.parametrize("name, lengths, new", [("A", [1, 7, 33, 100, 60, 12], 40), ("B", [5, 40, 129], 30), ("C", [3, 70], 24), ("E", [20, 2], 30)])
def test_greedy_generation_through_the_engine(folders, name, lengths, new, dtype):
    from turboserve_b200 import SamplingParams

    folder = folders[name, False, dtype]
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


def test_generation_with_a_small_budget_preemption_and_steps_launched_ahead(folders):
    """A token budget that cuts prompts into portions, a pool so small that requests are preempted and computed again,
    decode steps replayed from graphs and launched ahead: the tokens are the plain greedy ones all the same."""
    from turboserve_b200 import SamplingParams

    folder = folders["A", False]
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in (50, 21, 70, 9)]
    with engine_for(folder, "float32", max_num_batched_tokens=24, num_blocks=14) as engine:
        outputs = engine.generate(prompts, SamplingParams(max_tokens=36, temperature=0.0, ignore_eos=True))
        assert engine.cache.free_pages() == [g.num_pages for g in engine.cache.groups]
    for prompt, out in zip(prompts, outputs):
        assert out.finished and out.output_tokens == 36
        check_greedy_path(config, weights, prompt, out.token_ids, "float32")


def test_the_command_line_serves_a_folder(folders, tmp_path):
    """``bin/trace_run`` as a process on a folder of this design: the logits of one step, as the file format says."""
    import subprocess
    import sys
    from pathlib import Path

    folder = folders["E", False]
    config, weights = P.read_model_folder(folder)
    tokens = [3, 14, 15, 9, 2, 6]
    step = {"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [0, 5]}], "end": ["a"]}
    runner = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    done = subprocess.run([sys.executable, str(runner), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "out"),
                           "--max-tokens", "64"], input=json.dumps(step) + "\n", capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and "done 0" in done.stdout, done.stderr[-2000:]
    got = torch.frombuffer(bytearray((tmp_path / "out" / "0.f32").read_bytes()), dtype=torch.float32).reshape(2, config["vocab"])
    C.check(got, P.logits_of(config, weights, tokens)[[0, 5]], "float32", "trace_run")


def test_generate_from_the_command_line_with_the_engines_sampler(folders):
    """``engine generate`` on a folder of this design: greedy tokens are the plain ones, and sampling with a seed, a
    temperature, top-p, a repetition penalty and log-probabilities runs through the same step."""
    from typer.testing import CliRunner

    from turboserve_b200.cli import app

    runner = CliRunner()
    folder = folders["E", False]
    config, weights = P.read_model_folder(folder)
    prompt = [5, 17, 3, 60, 2]
    result = runner.invoke(app, ["engine", "generate", "-m", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "6",
                                 "--ignore-eos", "--num-blocks", "32", "--dtype", "float32", "--temperature", "0"])
    assert result.exit_code == 0, result.stdout
    line = next(line for line in result.stdout.splitlines() if line.startswith("output "))
    assert json.loads(line.split(": ", 1)[1]) == P.greedy(config, weights, prompt, 6)
    result = runner.invoke(app, ["engine", "generate", "-m", str(folder), "--prompt-ids", "5,17,3,5,17,3", "--max-tokens", "8", "--ignore-eos",
                                 "--num-blocks", "32", "--temperature", "0.8", "--top-p", "0.9", "--seed", "3", "--repetition-penalty", "1.3",
                                 "--logprobs"])
    assert result.exit_code == 0, result.stdout
    values = [float(v) for v in next(line for line in result.stdout.splitlines() if line.strip().startswith("logprobs:")).split(":", 1)[1].split()]
    assert len(values) == 8 and all(v <= 0.0 for v in values)
