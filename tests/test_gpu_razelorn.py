"""The Razelorn decoder in the engine against the plain implementation (``plain_razelorn.py``, float64): each mechanism
alone, whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, pages and slots used
again, keys far away, at page borders and just inside and outside a window under a sharp softmax, the first tokens,
long decoding, several shapes, and greedy generation through the entry point."""

import math

import pytest
import torch

import helpers as H
import plain_razelorn as plain
import razelorn_cases as R

pytestmark = pytest.mark.gpu
DTYPES = [pytest.param(torch.float32, id="f32"), pytest.param(torch.bfloat16, id="bf16")]


def has_experts(cfg) -> bool:
    return any(layer["mlp"] is not None and layer["mlp"]["kind"] == "moe" for layer in cfg["layers"])


def share_for(cfg, dtype) -> float:
    # bfloat16 with routed experts: the router reads rows that are a percent off the float64 ones, and a close call
    # among the experts may fall the other way; such a token, and little else, is then far off
    return 0.85 if dtype == torch.bfloat16 and has_experts(cfg) else 1.0


def case(tmp_path, name, seed, sharp=None):
    cfg = R.CONFIGS[name] if sharp is None else R.sharpen(R.CONFIGS[name], sharp)
    W = R.weights_for(cfg, seed)
    return cfg, W, R.write_model(str(tmp_path), cfg, W)


def requests_for(cfg, lengths, seed):
    return {f"r{i}": H.random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ---- kernels alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [54, 88, 1032, 4104])
def test_layer_norm_with_one_and_two_addends_and_for_chosen_rows(dtype, width):
    from llm_pipeline_b200.ops import kernels
    torch.manual_seed(width)
    dev, T = "cuda", 7
    residual = torch.randn(T, width) * 3 + 1.5                     # a mean well away from zero
    a, b = torch.randn(T, width).to(dtype).float(), torch.randn(T, width)
    w, bias = (1 + 0.3 * torch.randn(width)).to(dtype).float(), (0.3 * torch.randn(width)).to(dtype).float()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for first, second in ((None, None), (a, None), (a, b)):
        res = residual.clone().to(dev)
        out = torch.empty(T, width, device=dev, dtype=dtype)
        kernels.add_layernorm(res, first.to(dev).to(dtype) if first is not None else None, second.to(dev) if second is not None else None,
                              w.to(dev).to(dtype), bias.to(dev).to(dtype), 1e-5, out)
        x = residual.double() + (first.double() if first is not None else 0) + (second.double() if second is not None else 0)
        assert (res.cpu().double() - x).abs().max() < 1e-5
        assert (out.float().cpu().double() - plain.layer_norm(x, w.double(), bias.double(), 1e-5)).abs().max() < tol
        rows = torch.tensor([T - 1, 0, 3], dtype=torch.int32, device=dev)
        res2 = residual.clone().to(dev)
        some = torch.empty(3, width, device=dev, dtype=dtype)
        kernels.add_layernorm(res2, first.to(dev).to(dtype) if first is not None else None, second.to(dev) if second is not None else None,
                              w.to(dev).to(dtype), bias.to(dev).to(dtype), 1e-5, some, rows=rows)
        assert torch.equal(some, out[rows.long()]) and torch.equal(res2.cpu(), residual)


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_kernels_alone(dtype):
    from llm_pipeline_b200.ops import kernels
    torch.manual_seed(1)
    dev = "cuda"
    for shape in ((5, 104), (3, 37)):
        z = (torch.randn(*shape) * 2).to(dtype)
        out = torch.empty(*shape, device=dev, dtype=dtype)
        kernels.relu_squared(z.to(dev), out)
        want = torch.relu(z.double()) ** 2
        assert ((out.float().cpu().double() - want).abs() <= (1e-6 if dtype == torch.float32 else 2.0 ** -8) * want + 1e-6).all()
        acc, x, s = torch.randn(*shape), torch.randn(*shape).to(dtype), torch.rand(shape[0])
        got = kernels.add_scaled_rows(acc.clone().to(dev), x.to(dev), s.to(dev))
        assert (got.cpu().double() - (acc.double() + s.double()[:, None] * x.double())).abs().max() < 1e-5
    table = torch.randn(20, 56).to(dtype)
    ids = torch.tensor([3, 19, 0, 3], dtype=torch.int32)
    out = torch.empty(4, 56, device=dev)
    kernels.embedding(ids.to(dev), table.to(dev), out, 2.5)
    assert (out.cpu().double() - table[ids.long()].double() * 2.5).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N", [6, 45])
def test_router_and_experts_alone(dtype, N):
    """Softmax scores over experts and identity experts, the choice by score plus correction, gated SiLU experts whose
    weight scales the output, identity experts, the shared expert's gate: a few rows (a warp per entry) and many (grouped
    products in bfloat16)."""
    from llm_pipeline_b200.ops import kernels
    torch.manual_seed(2)
    dev, D, E, I, F, top = "cuda", 56, 5, 2, 24, 3
    W = {"f.router": torch.randn(E + I, D) / 3, "f.correction": torch.randn(E + I) * 0.1, "f.shared.sg": torch.randn(1, D) / 3}
    for e in range(E):
        W[f"f.e{e}.gate"], W[f"f.e{e}.up"], W[f"f.e{e}.down"] = torch.randn(F, D) / 3, torch.randn(F, D) / 3, torch.randn(D, F) / 4
    W = {k: v.to(torch.bfloat16).double() for k, v in W.items()}
    h = torch.randn(N, D).to(torch.bfloat16).double()
    ids = torch.empty(N, top, dtype=torch.int32, device=dev)
    wts = torch.empty(N, top, device=dev)
    gate = torch.empty(N, device=dev)
    router = torch.cat([W["f.router"], W["f.shared.sg"]]).float().to(dev)
    kernels.route_topk(h.to(dev).to(dtype), router, top, ids, wts, softmax=True, correction=W["f.correction"].float().to(dev), gate=gate)
    chosen, weights = plain.route(h, W, "f", top)
    assert torch.equal(ids.cpu().long(), chosen)                     # float32 logits of identical inputs: no close call here
    assert (ids.cpu() >= E).any() and (ids.cpu() < E).any()          # identity experts and real ones were chosen
    without = torch.topk(torch.softmax(h @ W["f.router"].T, -1), top).indices
    assert not torch.equal(without, chosen)                          # and the correction changed a choice
    assert (wts.cpu().double() - weights).abs().max() < 1e-6
    assert (gate.cpu().double() - torch.sigmoid(h @ W["f.shared.sg"].T)[:, 0]).abs().max() < 1e-6
    gu = torch.stack([torch.cat([W[f"f.e{e}.gate"], W[f"f.e{e}.up"]]) for e in range(E)]).to(dev).to(dtype)
    down = torch.stack([W[f"f.e{e}.down"] for e in range(E)]).to(dev).to(dtype)
    out = torch.empty(N, D, device=dev)
    kernels.routed_experts(h.to(dev).to(dtype), gu, down, ids, wts, 0.0, out, "silu", I)
    want = plain.expert_ff(h, W, "f", {"router": {"experts": E, "identity": I, "top": top}})
    assert (out.cpu().double() - want).abs().max() < (1e-4 if dtype == torch.float32 else 5e-2)


def _attention_case(dtype, H_, G, d, dv, window, n, page, seed, plant=None, rot=0):
    """Queries, keys and values as they enter the scores, written into shuffled pages; (engine output, plain output)."""
    from llm_pipeline_b200.ops import kernels
    gen = torch.Generator().manual_seed(seed)
    dev = "cuda"
    q = torch.randn(n, H_, 2, d, generator=gen)
    k = torch.randn(n, G, 2, d, generator=gen)
    v = torch.randn(n, G, dv, generator=gen)
    if plant is not None:
        plant(q, k, v)
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    pages_n = -(-n // page)
    order = torch.randperm(pages_n + 3, generator=gen)[:pages_n]     # the request's pages lie anywhere in the pool
    pages = torch.full((pages_n + 3, G, page, 2 * d + dv), 7.0)      # other pages hold garbage
    for t in range(n):
        pages[order[t // page], :, t % page] = torch.cat([k[t].reshape(G, 2 * d), v[t]], dim=-1)
    table = order.to(torch.int32).view(1, -1).to(dev)
    positions = torch.arange(n, dtype=torch.int32, device=dev)
    scale, lam, diff, eps = 1.0 / math.sqrt(d), 0.7, 0.3, 1e-5
    want = plain.two_map_attention(q.double(), k.double(), v.double(), torch.arange(n), window, scale, lam, diff, eps)
    qd = q.reshape(n, -1).to(dev).to(dtype).contiguous()
    pd = pages.to(dev).to(dtype)
    out = torch.empty(n, H_ * dv, device=dev, dtype=dtype)
    args = (H_, G, d, dv, window or 0, scale, lam, eps, 1.0 - diff)
    kernels.diff_attention(qd, pd, table, torch.zeros(n, dtype=torch.int32, device=dev), positions, out, *args)
    results = {"general": out.float().cpu()}
    if kernels.diff_mma_supports(dtype, d, dv, page):
        per = kernels.diff_mma_tokens_per_tile(H_, G)
        tiles = torch.arange(0, n, per, dtype=torch.int32, device=dev)
        q_start = torch.tensor([0, n], dtype=torch.int32, device=dev)
        ctx_len = torch.tensor([n], dtype=torch.int32, device=dev)
        for segments in (0, -(-n // kernels.DIFF_SEGMENT_KEYS)):
            out2 = torch.empty_like(out)
            kernels.diff_attention_mma(qd, pd, table, q_start, ctx_len, positions, torch.zeros_like(tiles), tiles, out2, *args, segments=segments)
            results[f"tensor cores, {segments} segments"] = out2.float().cpu()
        # a step of single tokens: the last 40 tokens as 40 requests that share the pages, each with one new token; the
        # four warps of a block then share a key tile
        last = 40
        rows = torch.arange(n - last, n, device=dev)
        out3 = torch.empty(last, H_ * dv, device=dev, dtype=dtype)
        ones = torch.arange(last + 1, dtype=torch.int32, device=dev)
        kernels.diff_attention_mma(qd[rows].contiguous(), pd, table.expand(last, -1).contiguous(), ones, (rows + 1).to(torch.int32),
                                   positions[rows].contiguous(), torch.arange(last, dtype=torch.int32, device=dev),
                                   torch.zeros(last, dtype=torch.int32, device=dev), out3, *args,
                                   segments=-(-n // kernels.DIFF_SEGMENT_KEYS), split=True)
        results["tensor cores, single tokens"] = torch.cat([want[:n - last].float(), out3.float().cpu()])
    return results, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 32, 24), (3, 3, 12, 20, 9), (6, 1, 48, 48, None), (2, 2, 128, 64, 300), (32, 2, 16, 16, 70),
                                   (1, 1, 64, 128, 64), (40, 1, 16, 32, None)], ids=str)
def test_attention_kernels_alone(dtype, sizes):
    """Both maps, grouped heads (also more of them on a key/value head than a tile's 16 rows a token), values of another
    width than keys, windows below, at and above a tile of keys, over shuffled pages: the general kernel in both types, the
    tensor-core kernel whole, in key segments and for single tokens in bfloat16."""
    H_, G, d, dv, window = sizes
    results, want = _attention_case(dtype, H_, G, d, dv, window, n=330, page=16, seed=3)
    assert dtype != torch.bfloat16 or d % 16 or len(results) == 4
    for name, got in results.items():
        assert (got.double() - want).abs().max() < (2e-4 if dtype == torch.float32 else 4e-2), name


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [5, 16, 64, 65, 100])
def test_a_key_just_outside_the_window_is_not_seen_and_the_one_just_inside_is(dtype, window):
    """Map 1's keys are orthogonal to each other over any stretch of 128 tokens, and every query points at the key
    `window` tokens back (the first outside its window) and, less, at the key window - 1 back (the last inside): a window
    that is one too long puts all weight on the outside key, one that is one too short loses the key that holds most of it."""
    H_, G, d, dv, n = 2, 1, 128, 32, 300

    def plant(q, k, v):
        basis = torch.linalg.qr(torch.randn(d, d, generator=torch.Generator().manual_seed(9)))[0]
        direction = basis[torch.arange(n) % d]
        k[:, 0, 0] = direction * 6
        for t in range(n):
            q[t, :, 0] = 0.0
            if t - window >= 0:
                q[t, :, 0] += direction[t - window] * 30
            if t - window + 1 >= 0:
                q[t, :, 0] += direction[t - window + 1] * 12

    results, want = _attention_case(dtype, H_, G, d, dv, window, n, page=16, seed=4, plant=plant)
    for other in (window + 1, window - 1):
        wrong, _ = _attention_case(dtype, H_, G, d, dv, other, n, page=16, seed=4, plant=plant)
        assert (wrong["general"].double() - want).abs().max() > 0.1    # the premise: one key more or fewer changes the answer
    for name, got in results.items():
        assert (got.double() - want).abs().max() < (2e-4 if dtype == torch.float32 else 4e-2), name


@pytest.mark.parametrize("dtype", DTYPES)
def test_projection_norm_rotation_and_cache_rows_alone(dtype):
    """The kernel after the q/k/v product against the plain norm and rotation: rotated parts of all, some and none of a
    key, with rescaled frequencies, positions far from zero, rows written into the right place of the pages."""
    from llm_pipeline_b200.ops import kernels
    from llm_pipeline_b200.parts.position import RotaryPositions
    torch.manual_seed(5)
    dev, n, page = "cuda", 11, 4
    for H_, G, d, dv, rot in ((3, 1, 24, 40, 8), (4, 2, 16, 16, 16), (2, 2, 40, 8, 0)):
        qkv = torch.randn(n, 2 * d * (H_ + G) + G * dv).to(dtype).float()
        qw, kw = (1 + 0.3 * torch.randn(d)).to(dtype).float(), (1 + 0.3 * torch.randn(d)).to(dtype).float()
        positions = torch.arange(1000, 1000 + n)
        q = plain.rms(qkv[:, :2 * d * H_].double().view(n, H_, 2, d), 1e-5) * qw.double()
        k = plain.rms(qkv[:, 2 * d * H_:2 * d * (H_ + G)].double().view(n, G, 2, d), 1e-5) * kw.double()
        cos = sin = None
        if rot:
            freq = plain.rotary_frequencies(rot, 500.0, R.SCALING)
            q, k = plain.rotate_half(q, positions, freq), plain.rotate_half(k, positions, freq)
            part = RotaryPositions("", rot, 500.0, frequency_scaling=R.SCALING)
            cos, sin = torch.empty(n, rot // 2, device=dev), torch.empty(n, rot // 2, device=dev)
            kernels.rope_tables(positions.to(torch.int32).to(dev), part._inv_freq_cpu.to(dev), 1.0, cos, sin)
        pages = torch.zeros(6, G, page, 2 * d + dv, device=dev, dtype=dtype)
        slots = torch.tensor([(5 - t // page) * page + t % page for t in range(n)], dtype=torch.int32, device=dev)
        x = qkv.to(dev).to(dtype)
        kernels.diff_qkv_post(x, H_, G, d, dv, qw.to(dev).to(dtype), kw.to(dev).to(dtype), 1e-5, cos, sin, rot, slots, pages)
        tol = 2e-4 if dtype == torch.float32 else 4e-2               # float32 angles at positions around 1000
        assert (x[:, :2 * d * H_].float().cpu().double() - q.reshape(n, -1)).abs().max() < tol
        for t in range(n):
            row = pages[5 - t // page, :, t % page].float().cpu().double()
            assert (row[:, :2 * d] - k[t].reshape(G, 2 * d)).abs().max() < tol
            assert torch.equal(row[:, 2 * d:].float(), qkv[t, 2 * d * (H_ + G):].view(G, dv))


# ---- each mixer and feed-forward alone in a model of one layer ---------------------------------------------------------
ONE_LAYER = {
    "attention": R.config([R.attention(4, 2, 16, 24, None, window=11, rot_dims=8, scaling=R.SCALING)], width=40, vocab=61),
    "dense": R.config([R.attention(1, 1, 16, 16, R.dense(72))], width=40, vocab=61),
    "experts": R.config([R.attention(1, 1, 16, 16, R.moe(5, 2, 24, identity=2, shared=32))], width=40, vocab=61),
    "experts_plain": R.config([R.attention(1, 1, 16, 16, R.moe(4, 1, 24))], width=40, vocab=61),
}


@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_alone(tmp_path, name):
    cfg = ONE_LAYER[name]
    W = R.weights_for(cfg, 11)
    folder = R.write_model(str(tmp_path), cfg, W)
    requests = requests_for(cfg, [1, 2, 33, 70], 50)
    want = R.oracle(cfg, W, requests)
    runner = H.make_runner(folder, torch.float32, page_size=8, num_pages=24, max_request_tokens=96, max_requests=2)
    R.assert_matches(H.replay(runner, H.cut_whole(requests)), want, torch.float32, f"{name}, whole")
    R.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 5, 1, 16))), want, torch.float32, f"{name}, portions")


# ---- whole models --------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(R.CONFIGS))
def test_prefill_decoding_portions_and_batches(tmp_path, name, dtype):
    cfg, W, folder = case(tmp_path, name, 3)
    requests = requests_for(cfg, [1, 2, 3, 19, 64, 65, 150], 100)
    want = R.oracle(cfg, W, requests)
    share = share_for(cfg, dtype)
    page = 8
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=2 * (-(-150 // page)) + 6, max_request_tokens=160, max_requests=4)
    R.assert_matches(H.replay(runner, H.cut_whole(requests)), want, dtype, f"{name}: whole prompts", share)
    R.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=40)), want, dtype, f"{name}: last tokens one by one", share)
    R.assert_matches(H.replay(runner, H.cut_portions(requests, (1,))), want, dtype, f"{name}: token by token", share)
    R.assert_matches(H.replay(runner, H.cut_portions(requests, (2, 7, 3, 64, 2, 33))), want, dtype, f"{name}: portions", share)
    # unequal requests side by side, four live at most, so the slots and pages of finished ones go to later ones
    got = H.replay(runner, H.cut_mixed(requests, (2, 5, 16, 3, 31), max_live=4, decode_tail=9))
    R.assert_matches(got, want, dtype, f"{name}: mixed batches", share)
    assert runner.cache.num_live == 0 and runner.cache.pages_reused > 0


def test_the_same_logits_alone_and_in_a_batch(tmp_path):
    """float32: a request's logits beside others, or cut into portions, are those it has alone, to rounding of sums."""
    cfg, W, folder = case(tmp_path, "mixed", 4)
    requests = requests_for(cfg, [5, 40, 77, 130], 200)
    runner = H.make_runner(folder, torch.float32, page_size=16, num_pages=24, max_request_tokens=144, max_requests=4)
    alone = H.replay(runner, H.cut_whole(requests))
    mixed = H.replay(runner, H.cut_mixed(requests, (3, 2, 17), max_live=4, decode_tail=5))
    for rid in requests:
        assert (alone[rid] - mixed[rid]).abs().max() < 2e-4, rid


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "no_window"])
def test_far_keys_page_borders_window_edges_and_first_tokens_under_a_sharp_softmax(tmp_path, name, dtype):
    """Score scales raised so that a map's softmax sits on one or two keys, often hundreds of tokens back (or at the far
    end of a window): a key that is lost, off by one, read from another request's page or taken from outside a window
    changes the logits by its whole value. Prompts as long as many pages, positions around every page border, decoded
    alone and inside portions; windowed layers give their first pages back while the request lives."""
    cfg, W, folder = case(tmp_path, name, 5, sharp=6.0)
    page = 16
    requests = requests_for(cfg, [4 * page, 4 * page + 1, 330, 17], 300)
    want = R.oracle(cfg, W, requests)
    if name == "no_window":
        # the premise: in the oracle itself the far keys matter (dropping the first 3 pages changes the late logits a lot)
        late = plain.forward(cfg, {k: v.double() for k, v in W.items()}, requests["r2"][3 * page:]).float()
        assert R.row_errors(late[-40:], want["r2"][-40:]).median() > 0.1
    runner = H.make_runner(folder, dtype, page_size=page, num_pages=2 * 21 + 4, max_request_tokens=336, max_requests=4)
    share = min(share_for(cfg, dtype), 1.0 if dtype == torch.float32 else 0.95)   # bfloat16 scores of spread 6 move a near-tie of two keys
    R.assert_matches(H.replay(runner, H.cut_whole(requests)), want, dtype, "sharp: whole", share)
    R.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=3 * page + 2)), want, dtype, "sharp: decoding across borders", share)
    R.assert_matches(H.replay(runner, H.cut_portions(requests, (page - 1, 2, page + 1, 2 * page, 3))), want, dtype, "sharp: portions", share)
    R.assert_matches(H.replay(runner, H.cut_mixed(requests, (page, 2, page + 1), max_live=3, decode_tail=page + 3)), want, dtype, "sharp: mixed", share)


def test_few_rows_over_long_contexts_take_key_segments(tmp_path):
    """Contexts of several segments of keys without a window, sharp softmax, bfloat16: decoding steps and short portions
    cut the keys into segments with blocks of their own, whose sums a second kernel adds; positions around segment borders."""
    from llm_pipeline_b200.ops import kernels
    dtype = torch.bfloat16
    cfg, W, folder = case(tmp_path, "no_window", 8, sharp=5.0)
    seg = kernels.DIFF_SEGMENT_KEYS
    requests = requests_for(cfg, [2 * seg + 40, 3 * seg + 2, 70], 700)
    want = R.oracle(cfg, W, requests)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=120, max_request_tokens=3 * seg + 16, max_requests=3)
    used = []
    launch = kernels.diff_attention_mma

    def counting(*args, **kwargs):
        used.append(kwargs.get("segments", 0))
        return launch(*args, **kwargs)

    kernels.diff_attention_mma = counting
    try:
        share = 0.85
        R.assert_matches(H.replay(runner, H.cut_tail_one_by_one(requests, tail=seg + 70)), want, dtype, "segments: decoding", share)
        R.assert_matches(H.replay(runner, H.cut_portions(requests, (seg - 3, 2, 5, seg + 7, 3))), want, dtype, "segments: portions", share)
        R.assert_matches(H.replay(runner, H.cut_mixed(requests, (seg, 2, 9), max_live=3, decode_tail=40)), want, dtype, "segments: mixed", share)
    finally:
        kernels.diff_attention_mma = launch
    assert any(n > 1 for n in used) and any(n == 0 for n in used), "both forms of the tensor-core kernel should have run"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_through_replayed_graphs(tmp_path, dtype):
    """Two requests decode side by side for 220 steps, far past every window and over many pages that windowed layers
    give back on the way: from the third step on a captured graph is replayed."""
    cfg, W, folder = case(tmp_path, "mixed", 6)
    requests = requests_for(cfg, [260, 231], 400)
    want = R.oracle(cfg, W, requests)
    runner = H.make_runner(folder, dtype, page_size=16, num_pages=40, max_request_tokens=272, max_requests=2)
    from llm_pipeline_b200.engine import StepEntry
    rows = {rid: [] for rid in requests}
    out = runner.step([StepEntry(rid, toks[:11], list(range(11))) for rid, toks in requests.items()])
    for k, rid in enumerate(requests):
        rows[rid].append(out[11 * k:11 * (k + 1)].float().cpu())
    for t in range(11, 231):
        out = runner.step([StepEntry(rid, [toks[t]], [0]) for rid, toks in requests.items()])
        for k, rid in enumerate(requests):
            rows[rid].append(out[k:k + 1].float().cpu())
    assert runner.graph_replays > 200
    for rid in requests:
        R.assert_matches({rid: torch.cat(rows[rid])}, {rid: want[rid][:231]}, dtype, f"long decoding of {rid}", share_for(cfg, dtype))


def test_decoding_through_graphs_across_the_length_where_key_segments_begin(tmp_path):
    """bfloat16 without a window: a request decodes from below two segments of keys to above them. The first step of a
    shape runs eagerly with its real length (no segments yet), the captured step is sized for the longest context its
    block tables can hold (segments): what the segments need must exist before the capture."""
    from llm_pipeline_b200.engine import StepEntry
    from llm_pipeline_b200.ops import kernels
    cfg, W, folder = case(tmp_path, "no_window", 9, sharp=4.0)
    first = 2 * kernels.DIFF_SEGMENT_KEYS - 40
    requests = requests_for(cfg, [first + 80], 800)
    want = R.oracle(cfg, W, requests)
    runner = H.make_runner(folder, torch.bfloat16, page_size=16, num_pages=48, max_request_tokens=768, max_requests=2)
    toks = requests["r0"]
    rows = [runner.step([StepEntry("r0", toks[:first], list(range(first)))]).float().cpu()]
    for t in range(first, len(toks)):
        rows.append(runner.step([StepEntry("r0", [toks[t]], [0])]).float().cpu())
    assert runner.graph_replays > 60
    R.assert_matches({"r0": torch.cat(rows)}, want, torch.bfloat16, "decoding across the first segment border", 0.85)


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    from llm_pipeline_b200.inference import InferenceConfig, InferenceEngine
    cfg, W, folder = case(tmp_path, "mixed" if dtype == torch.float32 else "shared_weights", 7)
    engine = InferenceEngine(InferenceConfig(model_path=folder, dtype=dtype, block_size=8, num_blocks=64, max_sequence_length=128,
                                             max_batch_size=4, max_num_batched_tokens=32))
    prompts = [H.random_tokens(cfg["vocab"], n, 600 + n) for n in (1, 7, 30, 45, 12)]       # five requests for four slots
    got = engine.generate(prompts, max_tokens=10, temperature=0.0)
    W64 = {k: v.double() for k, v in W.items()}
    checked = 0
    for prompt, tokens in zip(prompts, got):
        ids = list(prompt)
        for token in tokens:
            logits = plain.forward(cfg, W64, ids)[-1]
            top2 = torch.topk(logits, 2).values
            if dtype == torch.bfloat16 and float(top2[0] - top2[1]) < 0.15:
                break                                                   # a near tie: the two sequences may part here
            assert token == int(logits.argmax()), (len(prompt), len(ids) - len(prompt))
            ids.append(token)
            checked += 1
    assert checked >= (50 if dtype == torch.float32 else 20)
    assert engine.engine.cache.num_live == 0
    info = engine.get_model_info()
    assert info["vocab_size"] == cfg["vocab"] and info["num_layers"] == len(cfg["layers"]) and info["total_parameters"] > 0
