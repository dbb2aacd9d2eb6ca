"""Tulipel on the GPU against the plain implementation: every mechanism alone (with inputs made so that a
fault shows), then whole models under every way of cutting the work, through the step function, the
trace replay program and the scheduler."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import plain_tulipel as plain
import tulipel_helpers as th

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 4e-2}       # on logits of order one (the test models' mixers are scaled up)


def bf16_exact(array):
    """Values that bfloat16 holds exactly, as float32."""
    return torch.from_numpy(np.asarray(array, dtype=np.float32)).to(torch.bfloat16).float()


# =============================================================================== mechanisms alone
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_polynorm(out_dtype):
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(0)
    z = torch.from_numpy(rng.normal(0, 1.3, size=(5, 77)).astype(np.float32))
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    out = torch.empty(5, 77, dtype=DTYPES[out_dtype], device=DEV)
    kernels.polynorm(z.to(DEV), out, coef.to(DEV), 1e-5)
    want = plain.polynorm(z.double().numpy(), coef.double().numpy(), 1e-5)
    assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-5 if out_dtype == "float32" else 2e-2)
    # the three terms are normalised separately: doubling z leaves N(z), N(z^2), N(z^3) where they were
    kernels.polynorm((2 * z).to(DEV), out, coef.to(DEV), 1e-12)
    again = torch.empty_like(out)
    kernels.polynorm(z.to(DEV), again, coef.to(DEV), 1e-12)
    assert np.abs(out.float().cpu().numpy() - again.float().cpu().numpy()).max() <= (1e-5 if out_dtype == "float32" else 2e-2)


def test_sum_norm_and_scale_cast():
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.normal(0, 2.0, size=(7, 62)).astype(np.float32)).to(DEV)
    w = torch.from_numpy(rng.normal(0, 0.2, size=62).astype(np.float32))
    y, h = torch.empty_like(x), torch.empty(7, 62, dtype=torch.bfloat16, device=DEV)
    kernels.scale_cast(x, y, h, 1.7)
    assert torch.equal(y, 1.7 * x) and torch.equal(h, x.to(torch.bfloat16))
    out, y2 = torch.empty_like(x), torch.empty_like(x)
    kernels.sum_norm(y, (1.0 + w).to(DEV), out, 1e-6, y2=y2, h=h, alpha=0.5)
    want = plain.norm_around_zero(y.double().cpu().numpy(), w.double().numpy(), 1e-6)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-6
    assert torch.equal(y2, 0.5 * out) and torch.equal(h, out.to(torch.bfloat16))
    kernels.sum_norm(y, (1.0 + w).to(DEV), y, 1e-6)               # in place
    assert torch.equal(y, out)


def test_depth_average_and_softcap():
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(2)
    results = [rng.normal(size=(4, 10)).astype(np.float32) for _ in range(4)]
    weights = [rng.normal(size=n + 2).astype(np.float32) for n in range(3)]
    history = torch.full((4, 4, 10), float("nan"), device=DEV)
    history[0] = torch.from_numpy(results[0])
    for n in range(3):
        x = torch.from_numpy(results[n + 1]).to(DEV)
        kernels.depth_average(history, x, torch.from_numpy(weights[n]).to(DEV), n)
        want = sum(float(weights[n][j]) * results[j].astype(np.float64) for j in range(n + 2))
        assert np.abs(x.cpu().numpy() - want).max() <= 1e-5
        assert torch.equal(history[n + 1].cpu(), torch.from_numpy(results[n + 1]))    # the result itself is kept, not the average
    # the norm, the average and the next layer's readers in one launch give what the three steps give
    for width in (12, 10):                     # rows that allow 16-byte accesses, and rows that do not
        y = torch.from_numpy(rng.normal(0, 2, size=(4, width)).astype(np.float32)).to(DEV)
        gain = torch.from_numpy(rng.normal(1, 0.2, size=width).astype(np.float32)).to(DEV)
        w = torch.from_numpy(rng.normal(size=4).astype(np.float32)).to(DEV)
        base = torch.from_numpy(rng.normal(size=(4, 4, width)).astype(np.float32)).to(DEV)
        one, two = base.clone(), base.clone()
        x1, y1, h1 = torch.empty_like(y), torch.empty_like(y), torch.empty(4, width, dtype=torch.bfloat16, device=DEV)
        kernels.sum_norm(y, gain, x1, 1e-5, y2=y1, h=h1, alpha=1.5, history=one, weights=w, n=2)
        x2, y2, h2 = torch.empty_like(y), torch.empty_like(y), torch.empty(4, width, dtype=torch.bfloat16, device=DEV)
        kernels.sum_norm(y, gain, x2, 1e-5)
        kernels.depth_average(two, x2, w, 2)
        kernels.scale_cast(x2, y2, h2, 1.5)
        assert torch.equal(one, two) and torch.equal(x1, x2) and torch.equal(y1, y2) and torch.equal(h1, h2)
    logits = torch.from_numpy(rng.normal(0, 20, size=(3, 17)).astype(np.float32)).to(DEV)
    want = plain.softcap(logits.double().cpu().numpy(), 7.5)
    kernels.softcap(logits, 7.5)
    assert np.abs(logits.cpu().numpy() - want).max() <= 1e-5 and float(logits.abs().max()) <= 7.5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_headwise_gemm(dtype):
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(3)
    heads, n, k, rows, gap = 3, 13, 22, 70, 5
    a = bf16_exact(rng.normal(size=(rows, heads * (k + gap))))
    w = bf16_exact(rng.normal(size=(heads, n, k)))
    out = torch.zeros(rows, heads * (n + 2), dtype=DTYPES[dtype], device=DEV)
    kernels.headwise_gemm(a.to(DTYPES[dtype]).to(DEV), w.to(DTYPES[dtype]).to(DEV), out, heads, k + gap, n + 2)
    got = out.float().cpu().numpy().reshape(rows, heads, n + 2)
    want = np.einsum("thk,hnk->thn", a.numpy().reshape(rows, heads, k + gap)[:, :, :k].astype(np.float64), w.numpy().astype(np.float64))
    assert np.abs(got[:, :, :n] - want).max() <= (1e-4 if dtype == "float32" else 0.1)
    assert np.all(got[:, :, n:] == 0)


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rows_appended_and_query_tails(dtype, interleaved):
    """The cached row (normed latent, rotated shared key part) and the rotated tail of every query head, with
    fewer rotated elements than the rotated width, at positions on both sides of page borders."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.rope import InterleavedRotary, ScaledHalfSplitRotary
    rng = np.random.default_rng(4)
    rank, rot, dims, heads, dim, page = 20, 10, 6, 3, 4, 4
    rot_cfg = {"base": 300.0, "dims": dims}
    if not interleaved:
        rot_cfg["scaling"] = {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}
    cls = InterleavedRotary if interleaved else ScaledHalfSplitRotary
    part = cls("", dims=dims, theta=300.0, max_positions=64, scaling=rot_cfg.get("scaling"))
    cos, sin = part.rotary_tables(SimpleNamespace(device=torch.device(DEV)))
    positions = [0, 1, 3, 4, 7, 8, 30, 31, 32]
    pages = [5, 2, 7, 0, 9, 1, 8, 3, 6]                                  # logical page i lives in pages[i]
    table = torch.tensor([[-1] * 9, pages], dtype=torch.int32, device=DEV)
    src = torch.from_numpy(rng.normal(0, 2, size=(len(positions), rank + rot + 3)).astype(np.float32))
    weight = torch.from_numpy(rng.normal(1, 0.3, size=rank).astype(np.float32))
    cache = torch.zeros(10, 1, page, rank + rot, dtype=DTYPES[dtype], device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    seq = torch.ones(len(positions), dtype=torch.int32, device=DEV)
    kernels.latent_kv_append(src.to(DEV)[:, :rank + rot + 3], weight.to(DEV), pos, seq, table, cos, sin, interleaved, cache, rank,
                             1e-5, status)
    tol = 1e-5 if dtype == "float32" else 3e-2
    latent = plain.norm_plain(src[:, :rank].double().numpy(), weight.double().numpy(), 1e-5)
    shared = plain.rotate(src[:, rank:rank + rot].double().numpy(), positions, rot_cfg, interleaved)
    for i, p in enumerate(positions):
        row = cache[pages[p // page], 0, p % page].float().cpu().numpy()
        assert np.abs(row[:rank] - latent[i]).max() <= tol and np.abs(row[rank:] - shared[i]).max() <= tol, (i, p)
    assert np.allclose(shared[:, dims:], src[:, rank + dims:rank + rot].numpy())          # beyond the rotated elements: unchanged
    assert int((cache.float().abs().sum(-1) > 0).sum()) == len(positions)                # nothing else was written
    q = bf16_exact(rng.normal(size=(len(positions), heads * (dim + rot))))
    qlat = torch.zeros(len(positions), heads * (rank + rot), dtype=DTYPES[dtype], device=DEV)
    kernels.latent_query_tail(q.to(DTYPES[dtype]).to(DEV), qlat, pos, cos, sin, interleaved, heads, dim, rot, rank, status)
    got = qlat.float().cpu().numpy().reshape(len(positions), heads, rank + rot)
    want = plain.rotate(q.numpy().reshape(len(positions), heads, dim + rot)[:, :, dim:].astype(np.float64), positions, rot_cfg, interleaved)
    assert np.abs(got[:, :, rank:] - want).max() <= tol and np.all(got[:, :, :rank] == 0)
    assert int(status.item()) == 0


def _paged_rows(rows_by_request, page, width, dtype, rng):
    """Scatter requests' rows [n, width] over shuffled pages; (cache, table)."""
    counts = [-(-len(r) // page) for r in rows_by_request]
    order = rng.permutation(sum(counts) + 3)
    cache = torch.full((len(order), 1, page, width), float("nan"), dtype=dtype)
    table = np.full((len(rows_by_request), max(counts)), -1, dtype=np.int32)
    at = 0
    for i, rows in enumerate(rows_by_request):
        for j in range(counts[i]):
            table[i, j] = order[at]
            chunk = rows[j * page:(j + 1) * page]
            cache[order[at], 0, :len(chunk)] = torch.from_numpy(chunk).to(dtype)
            at += 1
    return cache.to(DEV), torch.from_numpy(table).to(DEV)


def _attend_plain(q, rows, rank, scale, sink):
    scores = (q @ rows.T) * scale
    top = max(scores.max(), sink) if sink is not None else scores.max()
    e = np.exp(scores - top)
    return (e @ rows[:, :rank]) / (e.sum() + (math.exp(sink - top) if sink is not None else 0.0))


@pytest.mark.parametrize("page", [16, 8])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(3, 48, 16), (5, 20, 6), (16, 128, 32), (20, 64, 16), (6, 160, 16), (4, 320, 32), (16, 512, 64), (2, 640, 32)])
def test_latent_attention_kernels(dtype, page, shape):
    """Prompt portions and single decode tokens in one batch over shuffled pages, against a direct softmax (shapes:
    heads, latent, rotated width; latents of one, two and more blocks of value columns).
    One far key (position 2 of a long context) is made to stand out for one query, a key just beyond the
    causal limit is made huge (it must not be seen), and one head's sink dominates its softmax."""
    from sprout_lm_b200 import kernels
    heads, rank, rot = shape
    width, scale = rank + rot, 0.3
    rng = np.random.default_rng(heads)
    contexts = [700, 129, 1, 37]                      # tokens held after the step
    new = [1, 5, 1, 37]                               # of which this step brings the last ones
    rows = [bf16_exact(rng.normal(0, 0.5, size=(n, width))).numpy() for n in contexts]
    direction = bf16_exact(rng.normal(size=width)).numpy()
    rows[0][2] = bf16_exact(direction * 1.5).numpy()                      # the far key
    rows[3][20] = bf16_exact(direction * 40).numpy()                      # position 20 of request 3: queries before it must not see it
    sink = bf16_exact(rng.normal(0, 1, size=heads)).numpy()
    sink[1] = 30.0                                    # head 1: the sink takes nearly all the weight
    q_rows, positions, seq_of = [], [], []
    for r, (n, m) in enumerate(zip(contexts, new)):
        for p in range(n - m, n):
            q_rows.append(bf16_exact(rng.normal(0, 0.5, size=(heads, width))).numpy())
            positions.append(p)
            seq_of.append(r)
    q_rows[0][0] = bf16_exact(direction * 3).numpy()                      # request 0's decode token, head 0, asks for the far key
    q = torch.from_numpy(np.stack(q_rows)).reshape(len(positions), heads * width)
    cache, table = _paged_rows(rows, page, width, DTYPES[dtype], rng)
    starts = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    ctx = SimpleNamespace(seq_of_token=torch.tensor(seq_of, dtype=torch.int32, device=DEV),
                          positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                          q_start=torch.from_numpy(starts).to(DEV), context_lens=torch.tensor(contexts, dtype=torch.int32, device=DEV),
                          max_q_len=max(new), max_context=max(contexts), planned_context=0, num_seqs=len(contexts),
                          num_tokens=len(positions))
    view = SimpleNamespace(k=cache, v=None, block_table=table, page_tokens=page, write=False)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for label, sinks in (("sink", sink), ("no sink", None)):
        out = torch.empty(len(positions), heads * rank, dtype=DTYPES[dtype], device=DEV)
        kernels.latent_attention(q.to(DTYPES[dtype]).to(DEV), view, ctx, None if sinks is None else torch.from_numpy(sinks).to(DEV),
                                 out, heads, rank, scale, status)
        got = out.float().cpu().numpy().reshape(len(positions), heads, rank)
        for t, (p, r) in enumerate(zip(positions, seq_of)):
            for h in range(heads):
                want = _attend_plain(q_rows[t][h].astype(np.float64), rows[r][:p + 1].astype(np.float64), rank, scale,
                                     None if sinks is None else float(sinks[h]))
                err = np.abs(got[t, h] - want).max()
                reach = max(1.0, float(np.abs(rows[r][:p + 1, :rank]).max()))       # the output is a weighted mean of these values
                assert np.isfinite(err) and err <= tol * reach, (label, "token", t, "position", p, "request", r, "head", h, err)
        if sinks is not None:
            calm = [t for t, r in enumerate(seq_of) if r != 3]                      # (request 3 holds the huge key)
            assert np.abs(got[calm, 1]).max() < 1e-6                                # the sink has no value: head 1 outputs nearly nothing
        far = got[0, 0] / rows[0][2][:rank]
        assert np.nanmedian(far) > 0.9                                              # the far key carries head 0 of the decode token
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(6, 32, 16), (20, 144, 16), (16, 512, 64), (3, 640, 32)])
def test_decode_only_batches_of_many_lengths(dtype, shape):
    """One token per request (the decode kernels' case): contexts of 1 key, around page and 128-key borders, and long;
    latents of one, two and more blocks of value columns, more heads than one row group."""
    from sprout_lm_b200 import kernels
    (heads, rank, rot), page, scale = shape, 16, 0.2
    width = rank + rot
    rng = np.random.default_rng(9)
    contexts = [1, 2, 15, 16, 17, 127, 128, 129, 255, 256, 257, 1000, 1537]
    rows = [bf16_exact(rng.normal(0, 0.6, size=(n, width))).numpy() for n in contexts]
    sink = bf16_exact(rng.normal(0, 1, size=heads)).numpy()
    q_rows = bf16_exact(rng.normal(0, 0.6, size=(len(contexts), heads, width))).numpy()
    cache, table = _paged_rows(rows, page, width, DTYPES[dtype], rng)
    ctx = SimpleNamespace(seq_of_token=torch.arange(len(contexts), dtype=torch.int32, device=DEV),
                          positions=torch.tensor([n - 1 for n in contexts], dtype=torch.int32, device=DEV),
                          q_start=torch.arange(len(contexts) + 1, dtype=torch.int32, device=DEV),
                          context_lens=torch.tensor(contexts, dtype=torch.int32, device=DEV), max_q_len=1, max_context=max(contexts),
                          planned_context=0, num_seqs=len(contexts), num_tokens=len(contexts))
    view = SimpleNamespace(k=cache, v=None, block_table=table, page_tokens=page, write=False)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(len(contexts), heads * rank, dtype=DTYPES[dtype], device=DEV)
    kernels.latent_attention(torch.from_numpy(q_rows).reshape(len(contexts), -1).to(DTYPES[dtype]).to(DEV), view, ctx,
                             torch.from_numpy(sink).to(DEV), out, heads, rank, scale, status)
    got = out.float().cpu().numpy().reshape(len(contexts), heads, rank)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for r, n in enumerate(contexts):
        for h in range(heads):
            want = _attend_plain(q_rows[r, h].astype(np.float64), rows[r].astype(np.float64), rank, scale, float(sink[h]))
            assert np.abs(got[r, h] - want).max() <= tol, (n, h)
    assert int(status.item()) == 0


# =============================================================================== whole models
@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("tulipel")
    return {name: th.make_model_dir(base, name) for name in th.CONFIGS}


def make_requests(name, seed, lengths):
    vocab = th.CONFIGS[name][0]["vocab"]
    rng = np.random.default_rng(seed)
    return {f"r{i}": helpers.random_tokens(rng, n, vocab) for i, n in enumerate(lengths)}


def make_runner(model_dir, dtype, pages, page_tokens, requests=8):
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.models import load_model
    model = load_model(model_dir, dtype=DTYPES[dtype])
    return ModelRunner(model, num_pages=pages, page_tokens=page_tokens, max_requests=requests, prefix_caching=False)


def test_layers_one_by_one(model_dirs):
    """The stream after every layer (after the depth average) in 32-bit, so that a fault names its layer."""
    from sprout_lm_b200.engine.batch import StepEntry
    for name, directory in model_dirs.items():
        config, tensors = th.plain_model(directory)
        tokens = make_requests(name, 1, [21])["r0"]
        runner = make_runner(directory, "float32", 8, th.CONFIGS[name][2])
        seen = []
        stream = runner.model.stream
        original, original_fused = stream.after, stream.norm_after
        stream.after = lambda carry, n, x: (original(carry, n, x), seen.append(x.clone()))
        stream.norm_after = lambda carry, n, y, gain, eps, x, **more: (original_fused(carry, n, y, gain, eps, x, **more),
                                                                         seen.append(x.clone()))
        seq = runner.new_sequence()
        assert runner.reserve(seq, len(tokens))
        runner.step([StepEntry(seq, tokens, [0])])
        want, _ = plain.hidden_states(config, tensors, tokens)
        assert len(seen) == len(want)
        for i, (got, expected) in enumerate(zip(seen, want)):
            assert np.abs(got.cpu().numpy() - expected).max() <= 2e-5 * max(1.0, np.abs(expected).max()), (name, "layer", i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_all_cuttings_in_process(model_dirs, name, dtype):
    """Whole, tail decoded token by token (80 tokens), portions down to two tokens, mixed batches with
    pages used again: against the plain implementation, and in 32-bit bitwise equal to one another."""
    page = th.CONFIGS[name][2]
    requests = make_requests(name, 11, [5, 17, 33, 70, 150, 1])
    rng = np.random.default_rng(5)
    plans = {
        "whole": helpers.plan_whole(requests),
        "tail": helpers.plan_tail_decode(requests, tail=80),
        "portions": helpers.plan_portions(requests),
        "mixed": helpers.plan_mixed(requests, rng),
    }
    results = {}
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = make_runner(model_dirs[name], dtype, budget // page, page, requests=4)
        got = results[label] = helpers.run_plan_in_process(runner, plan)
        assert len(got) == sum(len(t) for t in requests.values())
        th.compare(model_dirs[name], requests, got, TOL[dtype], f"{name}/{dtype}/{label}", page)
        runner.manager.check_invariants()
        assert len(runner.manager.pools[0].free) == runner.manager.pools[0].num_pages        # every page came back
    if dtype == "float32":
        for label in ("tail", "portions", "mixed"):
            for place, row in results["whole"].items():
                assert np.array_equal(row, results[label][place]), f"{name}: {label} differs from whole at {place}"


def test_long_context_crosses_many_pages(model_dirs):
    """A prompt of several hundred tokens in uneven portions with a decoded tail, bfloat16 and 32-bit."""
    name = "Q"
    requests = make_requests(name, 21, [530])
    plan = helpers.plan_portions(requests, sizes=(130, 2, 127, 3, 64, 100, 2, 1, 1, 1, 97, 1, 1))
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(model_dirs[name], dtype, 70, 8)
        got = helpers.run_plan_in_process(runner, plan)
        th.compare(model_dirs[name], requests, got, TOL[dtype], f"long/{dtype}", 8)


def test_trace_replay_program(model_dirs, tmp_path):
    """bin/trace_run picks the model class by config.json and replays a mixed plan."""
    name = "P"
    requests = make_requests(name, 13, [9, 40, 70, 23])
    plan = helpers.plan_mixed(requests, np.random.default_rng(2))
    budget = helpers.live_token_budget(plan, requests)
    vocab = th.CONFIGS[name][0]["vocab"]
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_with_trace_run(model_dirs[name], dtype, plan, tmp_path / dtype, budget, vocab=vocab)
        th.compare(model_dirs[name], requests, got, TOL[dtype], f"trace/{dtype}", 16)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_scheduler(model_dirs, name):
    """generate(): continuous batching, chunked prefill and captured decode steps; in 32-bit the tokens are the
    plain implementation's, in bfloat16 every token is within bfloat16's reach of the plain choice."""
    from sprout_lm_b200 import generate, load_model
    config, tensors = th.plain_model(model_dirs[name])
    rng = np.random.default_rng(7)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (3, 19, 44)]
    new_tokens = 12
    for dtype in ("float32", "bfloat16"):
        model = load_model(model_dirs[name], dtype=dtype)
        results = generate(model, prompts, max_new_tokens=new_tokens, ignore_eos=True)
        for prompt, result in zip(prompts, results):
            assert len(result["output"]) == new_tokens
            if dtype == "float32":
                assert result["output"] == plain.greedy(config, tensors, prompt, new_tokens)
                continue
            history = list(prompt)
            for token in result["output"]:
                row = plain.logits(config, tensors, history)[-1]
                assert row[token] >= row.max() - 2 * TOL["bfloat16"], (name, len(history), token)
                history.append(token)


def test_scheduler_under_page_pressure(model_dirs):
    """A pool smaller than the requests together: preemption and recomputation give the same greedy tokens."""
    from sprout_lm_b200 import EngineOptions, generate, load_model
    name = "P"
    config, tensors = th.plain_model(model_dirs[name])
    rng = np.random.default_rng(8)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (30, 41, 26, 35)]
    model = load_model(model_dirs[name], dtype="float32")
    options = EngineOptions(block_size=8, num_blocks=14, max_sequences=4, max_batch_tokens=24, prefill_chunk_size=7)
    results = generate(model, prompts, max_new_tokens=10, ignore_eos=True, options=options)
    for prompt, result in zip(prompts, results):
        assert result["output"] == plain.greedy(config, tensors, prompt, 10)
