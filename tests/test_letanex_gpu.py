"""Letanex on the GPU against the plain implementation: every mechanism alone (with inputs made so that a fault
shows), then whole models under every way of cutting the work, through the step function, the trace replay program
and the scheduler."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers
import letanex_helpers as lh
import plain_letanex as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 4e-2}       # root mean square over the vocabulary, on logits of order one


def rounded(array, dtype):
    """float32 values that ``dtype`` holds exactly."""
    return torch.from_numpy(np.asarray(array, dtype=np.float32)).to(DTYPES[dtype]).float()


def dev(array, dtype=None):
    t = array if isinstance(array, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(array))
    return (t.to(DTYPES[dtype]) if dtype else t).to(DEV)


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


# =============================================================================== mechanisms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layernorm_and_norm_add(dtype):
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(0)
    tol = 2e-6 if dtype == "float32" else 2e-2
    for width in (72, 257, 1030, 256, 768, 2048):                             # a block per row, and (the last three) a warp per row
        x = (rng.normal(3.0, 2.0, size=(6, width))).astype(np.float32)        # a mean far from zero: the deviations matter
        w, wb, w2 = (rng.normal(1.0, 0.3, size=width).astype(np.float32) for _ in range(3))
        out = torch.empty(6, width, dtype=DTYPES[dtype], device=DEV)
        kernels.layernorm(dev(x), dev(w), out, 1e-5)
        want = plain.layer_norm(x.astype(np.float64), w, 1e-5)
        assert np.abs(out.float().cpu().numpy() - want).max() <= tol * 4
        picked = torch.empty(2, width, dtype=DTYPES[dtype], device=DEV)
        kernels.layernorm(dev(x), dev(w), picked, 1e-5, rows=ints([4, 1]))
        assert torch.equal(picked, out[[4, 1]])
        y = rng.normal(-1.0, 4.0, size=(6, width)).astype(np.float32)
        stream, h = dev(x.copy()), torch.empty(6, width, dtype=DTYPES[dtype], device=DEV)
        kernels.norm_add(dev(y), dev(wb), stream, 1e-5, next_gain=dev(w2), h=h)
        summed = x.astype(np.float64) + plain.layer_norm(y.astype(np.float64), wb, 1e-5)
        assert np.abs(stream.cpu().numpy() - summed).max() <= 4e-6
        assert np.abs(h.float().cpu().numpy() - plain.layer_norm(summed, w2, 1e-5)).max() <= tol * 4
        alone = dev(x.copy())
        kernels.norm_add(dev(y), dev(wb), alone, 1e-5)
        assert torch.equal(alone, stream)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_activations(dtype):
    from sprout_lm_b200 import kernels
    rng = np.random.default_rng(1)
    tol = 2e-6 if dtype == "float32" else 1.5e-2
    z = rounded(rng.normal(0, 2.0, size=(5, 37)), dtype)
    out = torch.empty(5, 37, dtype=DTYPES[dtype], device=DEV)
    kernels.relu2(dev(z, dtype), out)
    assert np.abs(out.float().cpu().numpy() - np.maximum(z.numpy().astype(np.float64), 0) ** 2).max() <= tol * 8
    gate_up = rounded(rng.normal(0, 2.0, size=(5, 2 * 19)), dtype)            # values on both sides of every limit
    act = torch.empty(5, 19, dtype=DTYPES[dtype], device=DEV)
    kernels.glu_clamped(dev(gate_up, dtype), act, 1.5, 1.702)
    g = np.minimum(gate_up.numpy()[:, :19].astype(np.float64), 1.5)
    u = np.clip(gate_up.numpy()[:, 19:].astype(np.float64), -1.5, 1.5)
    assert np.abs(act.float().cpu().numpy() - g * plain.sigmoid(1.702 * g) * (u + 1)).max() <= tol * 4
    o = rng.normal(0, 3.0, size=(5, 44)).astype(np.float32)
    gain = rng.normal(1.0, 0.3, size=44).astype(np.float32)
    rows = rounded(rng.normal(0, 1.5, size=(5, 100)), dtype)                  # the gate is a view into wider rows
    gated = torch.empty(5, 44, dtype=DTYPES[dtype], device=DEV)
    kernels.gated_rmsnorm(dev(o), dev(gain), dev(rows, dtype)[:, 56:], gated, 1e-6)
    want = plain.rms(o.astype(np.float64), 1e-6) * gain * plain.sigmoid(rows.numpy()[:, 56:].astype(np.float64))
    assert np.abs(gated.float().cpu().numpy() - want).max() <= tol * 4


def _fill_cache(kernels, dtype, contexts, G, maps, dim, vdim, page, cos, sin, rng, keys=None, values=None):
    """Append every request's keys and values through the kernel, into shuffled pages.  Returns the cache view, the
    unrotated keys [r][S, G, maps, dim] and values [r][S, G, vdim] as the dtype holds them."""
    pages_per = [-(-n // page) for n in contexts]
    total = sum(pages_per) + 3
    order = rng.permutation(total)[:sum(pages_per)]
    table = np.full((len(contexts), max(pages_per)), -1, dtype=np.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = order[at:at + n]
        at += n
    k_cache = torch.full((total, G, page, maps * dim), float("nan"), dtype=DTYPES[dtype], device=DEV)
    v_cache = torch.full((total, G, page, vdim), float("nan"), dtype=DTYPES[dtype], device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    all_k, all_v = [], []
    for r, n in enumerate(contexts):
        k = rounded(rng.normal(0, 1.0, size=(n, G, maps, dim)), dtype) if keys is None else rounded(keys[r], dtype)
        v = rounded(rng.normal(0, 1.0, size=(n, G, vdim)), dtype) if values is None else rounded(values[r], dtype)
        all_k.append(k.numpy().astype(np.float64))
        all_v.append(v.numpy().astype(np.float64))
        rows = torch.cat([torch.zeros(n, 1 * maps * dim), k.reshape(n, -1), v.reshape(n, -1)], dim=1)
        kernels.rope_maps_append(dev(rows, dtype), ints(range(n)), ints([r] * n), dev(table), cos, sin, k_cache, v_cache,
                                 maps, G, maps, dim, vdim, page, True, status)
    assert int(status.item()) == 0
    view = SimpleNamespace(k=k_cache, v=v_cache, block_table=dev(table), page_tokens=page, write=False)
    return view, all_k, all_v, status


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(6, 2, 16, 24, 8, 16), (3, 3, 8, 8, 4, 8), (2, 1, 12, 40, 12, 16), (8, 4, 32, 64, 16, 16),
                                   (8, 2, 64, 128, 32, 16), (3, 1, 16, 32, 8, 8), (2, 2, 128, 128, 64, 32), (2, 1, 8, 300, 4, 16)])
def test_two_map_attention_over_pages(dtype, sizes):
    """Rotation, append and attention together: contexts on both sides of page and 128-key borders, a portion of
    queries and single queries, pages in shuffled order."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.rope import LinearScaledRotary
    H, G, dim, vdim, rot, page = sizes
    rng = np.random.default_rng(sum(sizes))
    rot_spec = {"base": 300.0, "dims": rot, "scaling": {"factor": 2.0}}
    cos, sin = LinearScaledRotary("", rot, 300.0, 1024, 2.0).rotary_tables(SimpleNamespace(device=DEV))
    contexts = [1, 2, page - 1, page, page + 1, 127, 128, 129, 257, 300]
    view, keys, values, status = _fill_cache(kernels, dtype, contexts, G, 2, dim, vdim, page, cos, sin, rng)
    scale, lam, eps, out_scale = 0.3, 0.37, 1e-5, 0.6
    tol = 3e-5 if dtype == "float32" else 3e-2
    # the last few positions of every request are the step's queries: single tokens, short portions and long ones
    wanted = [min(n, 5) for n in contexts]
    wanted[0], wanted[-2], wanted[-1] = 1, 40, 100
    q_rows, positions, seqs = [], [], []
    for r, n in enumerate(contexts):
        for p in range(n - wanted[r], n):
            positions.append(p)
            seqs.append(r)
    q = rounded(rng.normal(0, 1.0, size=(len(positions), H, 2, dim)), dtype)
    rows = dev(q.reshape(len(positions), -1), dtype)
    kernels.rope_maps_append(rows, ints(positions), ints(seqs), view.block_table, cos, sin, None, None, H * 2, G, 2, dim, vdim,
                             page, False, status)
    starts = np.concatenate([[0], np.cumsum(wanted)])
    ctx = SimpleNamespace(positions=ints(positions), seq_of_token=ints(seqs), q_start=ints(starts), max_q_len=max(wanted))
    out = torch.empty(len(positions), H * vdim, dtype=DTYPES[dtype], device=DEV)
    kernels.multimap_attention(rows, view, ctx, out, H, G, 2, dim, vdim, scale, lam, eps, out_scale, status)
    got = out.float().cpu().numpy().reshape(len(positions), H, vdim)
    # the same with single tokens only (every request's last position): the step a decoding batch makes, in which
    # the bfloat16 kernel divides a request's keys among several CTAs (some of which find no keys in the short requests)
    last = [int(starts[r + 1]) - 1 for r in range(len(contexts))]
    single = SimpleNamespace(positions=ints([positions[i] for i in last]), seq_of_token=ints(range(len(contexts))),
                             q_start=ints(range(len(contexts) + 1)), max_q_len=1, max_context=max(contexts))
    out1 = torch.empty(len(contexts), H * vdim, dtype=DTYPES[dtype], device=DEV)
    kernels.multimap_attention(rows[last].contiguous(), view, single, out1, H, G, 2, dim, vdim, scale, lam, eps, out_scale, status)
    got1 = out1.float().cpu().numpy().reshape(len(contexts), H, vdim)
    assert int(status.item()) == 0
    at = 0
    for r, n in enumerate(contexts):
        count = wanted[r]
        pos = list(range(n - count, n))
        qr = plain.rotate(q[at:at + count].numpy().astype(np.float64).reshape(count, H * 2, dim), pos, rot_spec).reshape(count, H, 2, dim)
        kr = plain.rotate(keys[r].reshape(n, G * 2, dim), list(range(n)), rot_spec).reshape(n, G, 2, dim)
        want = plain.differential_heads(qr, kr, values[r], pos, scale, lam, eps, out_scale)
        assert np.abs(got[at:at + count] - want).max() <= tol, (n, np.abs(got[at:at + count] - want).max())
        assert np.abs(got1[r] - want[-1]).max() <= tol, (n, "single token", np.abs(got1[r] - want[-1]).max())
        at += count


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dims", [(16, 24), (32, 64)])
def test_attention_finds_a_far_key_and_ignores_the_future(dtype, dims):
    """One key among 700, far back, is the only one map 0 of one head scores high: the head's output must be that
    key's value.  A huge key one position after the query must not be seen.  With one map, the plain softmax."""
    from sprout_lm_b200 import kernels
    (dim, vdim), H, G, page, n = dims, 2, 1, 16, 700
    rng = np.random.default_rng(9)
    keys = rng.normal(0, 0.1, size=(n, G, 2, dim))
    values = rng.normal(0, 1.0, size=(n, G, vdim))
    far, query_at = 3, n - 2
    keys[far, 0, 0, :] = 0.0
    keys[far, 0, 0, 5] = 8.0                       # map 0 of the only key/value head
    keys[query_at + 1, 0, :, :] = 50.0             # the future: a key that would take everything
    view, k, v, status = _fill_cache(kernels, dtype, [n], G, 2, dim, vdim, page, None, None, rng, keys=[keys], values=[values])
    q = np.zeros((1, H, 2, dim))
    q[0, 0, 0, 5] = 8.0                            # head 0, map 0 asks for the far key; the other maps are uniform
    ctx = SimpleNamespace(positions=ints([query_at]), seq_of_token=ints([0]), q_start=ints([0, 1]), max_q_len=1, max_context=n)
    out = torch.empty(1, H * vdim, dtype=DTYPES[dtype], device=DEV)
    kernels.multimap_attention(dev(q.reshape(1, -1).astype(np.float32), dtype), view, ctx, out, H, G, 2, dim, vdim, 1.0, 0.0, 0.0, 1.0, status)
    got = out.float().cpu().numpy().reshape(H, vdim)
    want = plain.differential_heads(q, k[0], v[0], [query_at], 1.0, 0.0, 1e-30, 1.0)
    mean_value = v[0][:query_at + 1, 0].mean(axis=0)
    tol = 1e-4 if dtype == "float32" else 2e-2
    assert np.abs(got[0] - v[0][far, 0]).max() <= tol            # lambda 0, no norm: map 0 alone
    assert np.abs(got[1] - mean_value).max() <= tol              # uniform scores: the mean of the visible values
    assert np.abs(want[0, 0] * np.sqrt((v[0][far, 0] ** 2).mean()) - v[0][far, 0]).max() <= 1e-6
    # with lambda, norm and scale: the two maps' difference
    kernels.multimap_attention(dev(q.reshape(1, -1).astype(np.float32), dtype), view, ctx, out, H, G, 2, dim, vdim, 1.0, 0.5, 1e-6, 0.25, status)
    want = plain.differential_heads(q, k[0], v[0], [query_at], 1.0, 0.5, 1e-6, 0.25)
    assert np.abs(out.float().cpu().numpy().reshape(H, vdim) - want[0]).max() <= tol * 2
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(3, 8, 20, (0.9, 0.5, 0.99)), (1, 24, 8, (1.0,)), (4, 32, 64, (0.6, 0.9, 0.95, 0.998)), (2, 16, 130, (0.8, 0.97)),
                                   (2, 64, 40, (0.95, 1.0)), (1, 128, 64, (0.999,)), (3, 64, 128, (0.5, 0.9, 0.99))])
def test_decay_scan_carries_state(dtype, sizes):
    """Whole against portions against token by token; slots given back and used again; a decay of exactly 1."""
    from sprout_lm_b200 import kernels
    heads, dim, vdim, decay = sizes
    rng = np.random.default_rng(heads + dim)
    lengths = [70, 1, 33, 150]
    width = heads * (2 * dim + vdim)
    raw = [rounded(rng.normal(0, 1.0, size=(n, width + 8)), dtype) for n in lengths]      # rows wider than q | k | v
    state = torch.full((3, heads, dim, vdim), float("nan"), device=DEV)
    decay_t = dev(np.asarray(decay, dtype=np.float32))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # token by token everything is float32 on inputs the rows' type holds exactly; 64 tokens at a time the decayed
    # scores are rounded to bfloat16 for the value product (the portions of 8 tokens and more of bfloat16 rows)
    tol = 1e-2 if dtype == "bfloat16" and dim in (64, 128) else 2e-4

    def activated(rows):
        act = plain.silu(rows.numpy().astype(np.float64))
        return rounded(act, dtype).numpy().astype(np.float64)       # the kernel rounds the activation to the rows' type

    def oracle(rows):
        a = activated(rows)
        n = a.shape[0]
        q = a[:, :heads * dim].reshape(n, heads, dim)
        k = a[:, heads * dim:2 * heads * dim].reshape(n, heads, dim)
        v = a[:, 2 * heads * dim:width].reshape(n, heads, vdim)
        return plain.decay_recurrence(q, k, v, decay)

    def run(batch):
        """batch: [(slot, rows)] -> outputs per entry"""
        rows = torch.cat([r for _, r in batch])
        starts = np.concatenate([[0], np.cumsum([r.shape[0] for _, r in batch])])
        out = torch.empty(rows.shape[0], heads * vdim, device=DEV)
        ctx = SimpleNamespace(q_start=ints(starts), max_q_len=max(r.shape[0] for _, r in batch))
        view = SimpleNamespace(buffer=state, slots=ints([s for s, _ in batch]))
        kernels.decay_attention(dev(rows, dtype), ctx, view, decay_t, out, heads, dim, vdim, True, status)
        got = out.cpu().numpy()
        return [got[starts[i]:starts[i + 1]] for i in range(len(batch))]

    wants = [oracle(r) for r in raw]
    scale = max(1.0, max(np.abs(w[0]).max() for w in wants))
    # requests 0 and 1 whole, in one batch, in slots 2 and 0
    state[2].zero_(); state[0].zero_()
    got = run([(2, raw[0]), (0, raw[1])])
    for i in (0, 1):
        assert np.abs(got[i].reshape(-1, heads, vdim) - wants[i][0]).max() <= tol * scale
    assert np.abs(state[2].cpu().numpy() - wants[0][1]).max() <= tol * scale
    # slot 2 is used again (zeroed by its new owner) by request 2 in portions, beside request 3 token by token in slot 1
    state[2].zero_(); state[1].zero_()
    cuts = [0, 2, 9, 10, 33]
    pieces = {2: [], 3: []}
    for step in range(150):
        batch = []
        if step + 1 < len(cuts):
            batch.append((2, raw[2][cuts[step]:cuts[step + 1]]))
        batch.append((1, raw[3][step:step + 1]))
        got = run(batch)
        if len(batch) == 2:
            pieces[2].append(got[0])
        pieces[3].append(got[-1])
    for i in (2, 3):
        assert np.abs(np.concatenate(pieces[i]).reshape(-1, heads, vdim) - wants[i][0]).max() <= tol * scale, i
    assert np.abs(state[1].cpu().numpy() - wants[3][1]).max() <= tol * scale
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(5, 2, 2, 24, 1.0, True), (3, 0, 1, 16, 0.5, False), (4, 3, 5, 8, 2.5, True), (8, 3, 3, 40, 1.25, False),
                                   (6, 1, 3, 12, 1.2, True), (3, 2, 2, 200, 1.0, False)])
def test_routed_experts_part(dtype, sizes):
    """The whole routed feed-forward against the oracle: choice by score + correction, weights without it, identity
    experts, a single expert per token, nearly all experts per token, with and without a shared expert."""
    from sprout_lm_b200.parts import Runtime, WeightSource, build_part
    from sprout_lm_b200.config.specs import PartSpec
    experts, identity, top, ff, limit, shared = sizes
    width, tokens = 40, 37
    rng = np.random.default_rng(experts * 10 + top)
    weights = {"m.router": rng.normal(0, 0.6, size=(experts + identity, width)), "m.correction": rng.normal(0, 0.2, size=experts + identity)}
    for e in range(experts):
        weights[f"m.e{e}.gate"] = rng.normal(0, 0.4, size=(ff, width))
        weights[f"m.e{e}.up"] = rng.normal(0, 0.4, size=(ff, width))
        weights[f"m.e{e}.down"] = rng.normal(0, 0.2, size=(width, ff))
    if shared:
        weights.update({"m.shared.gate": rng.normal(0, 0.4, size=(12, width)), "m.shared.up": rng.normal(0, 0.4, size=(12, width)),
                        "m.shared.down": rng.normal(0, 0.2, size=(width, 12))})
    stored = {k: rounded(v, "bfloat16") for k, v in weights.items()}
    weights = {k: v.numpy().astype(np.float64) for k, v in stored.items()}
    mlp = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "scale": 1.3},
           "expert": {"ff": ff, "limit": limit}, "shared": {"ff": 12, "limit": 0.8} if shared else None}
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": width, "experts": experts, "identity": identity, "top": top, "scale": 1.3, "expert_ff": ff,
        "expert_limit": limit, "shared_ff": 12 if shared else None, "shared_limit": 0.8 if shared else None}), "m.")
    runtime = Runtime(DEV, DTYPES[dtype])
    part.load(WeightSource(lambda name: stored[name], runtime))
    h = rounded(rng.normal(0, 1.0, size=(tokens, width)), dtype)
    # no close calls: drop tokens whose top-th and next choices are nearly equal
    s = plain.softmax(h.numpy().astype(np.float64) @ weights["m.router"].T) + weights["m.correction"]
    ordered = -np.sort(-s, axis=1)
    keep = np.ones(tokens, dtype=bool) if top == experts + identity else (ordered[:, top - 1] - ordered[:, top]) > 1e-3
    assert keep.sum() > tokens // 2
    x = rng.normal(0, 1.0, size=(tokens, width)).astype(np.float32)
    stream = dev(x.copy())
    part.forward(dev(h, dtype), stream, None)
    want = x + plain.mixture_ff(h.numpy().astype(np.float64), weights, "m.", mlp)
    err = np.abs(stream.cpu().numpy() - want)[keep].max()
    assert err <= (3e-5 if dtype == "float32" else 4e-2), err
    if identity:                                    # some token did take an identity expert, or the case shows nothing
        chosen, _ = plain.route(h.numpy().astype(np.float64), weights, "m.", mlp["router"])
        assert (chosen >= experts).any()
    # a handful of tokens (the step a decoding batch makes): the bfloat16 path has a kernel of its own for it
    few = dev(x[:5].copy())
    part.forward(dev(h[:5], dtype), few, None)
    err = np.abs(few.cpu().numpy() - want[:5])[keep[:5]].max() if keep[:5].any() else 0.0
    assert err <= (3e-5 if dtype == "float32" else 4e-2), ("few tokens", err)
    # a second call: the counters were left clean
    again = dev(x.copy())
    part.forward(dev(h, dtype), again, None)
    assert torch.equal(again, stream)
    assert int(runtime.status.item()) == 0


# =============================================================================== whole models
@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("letanex")
    return {name: lh.make_model_dir(base, name) for name in lh.CONFIGS}


def make_requests(name, seed, lengths):
    vocab = lh.CONFIGS[name][0]["vocab"]
    rng = np.random.default_rng(seed)
    return {f"r{i}": helpers.random_tokens(rng, n, vocab) for i, n in enumerate(lengths)}


def make_runner(model_dir, dtype, pages, page_tokens, requests=4):
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.models import load_model
    model = load_model(model_dir, dtype=DTYPES[dtype])
    return ModelRunner(model, num_pages=pages, page_tokens=page_tokens, max_requests=requests, prefix_caching=False)


def test_layers_one_by_one(model_dirs):
    """The stream after every layer in 32-bit, so that a fault names its layer."""
    from sprout_lm_b200.engine.batch import StepEntry
    for name, directory in model_dirs.items():
        config, tensors = lh.plain_model(directory)
        tokens = make_requests(name, 1, [21])["r0"]
        runner = make_runner(directory, "float32", 8, lh.CONFIGS[name][2])
        seen = []
        for block in runner.model.blocks:
            def wrapped(x, *args, _inner=block.forward, **more):
                _inner(x, *args, **more)
                seen.append(x.clone())
            block.forward = wrapped
        seq = runner.new_sequence()
        assert runner.reserve(seq, len(tokens))
        runner.step([StepEntry(seq, tokens, [0])])
        _, want = plain.forward(config, tensors, tokens, return_layers=True)
        assert len(seen) == len(want)
        for i, (got, expected) in enumerate(zip(seen, want)):
            assert np.abs(got.cpu().numpy() - expected).max() <= 2e-5 * max(1.0, np.abs(expected).max()), (name, "layer", i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_all_cuttings_in_process(model_dirs, name, dtype):
    """Whole, tail decoded token by token (80 tokens), portions down to two tokens, mixed batches with pages and
    state slots used again: against the plain implementation, and in 32-bit bitwise equal to one another."""
    page = lh.CONFIGS[name][2]
    requests = make_requests(name, 11, [5, 17, 33, 70, 150, 1, 40])
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
        worst = lh.compare(model_dirs[name], requests, got, TOL[dtype], f"{name}/{dtype}/{label}", page, outliers=0.25 if dtype == "bfloat16" else 0.0)
        print(f"{name}/{dtype}/{label}: worst difference {worst:.2e}")
        runner.manager.check_invariants()
        assert len(runner.manager.pools[0].free) == runner.manager.pools[0].num_pages        # every page came back
        assert len(runner.manager._free_state) == 4                                           # and every state slot
    if dtype == "float32":
        for label in ("tail", "portions", "mixed"):
            for place, row in results["whole"].items():
                assert np.array_equal(row, results[label][place]), f"{name}: {label} differs from whole at {place}"


def test_long_context_crosses_many_pages(model_dirs):
    """A prompt of several hundred tokens in uneven portions with a decoded tail, bfloat16 and 32-bit: the slow
    decay's state and the far keys reach across all of it."""
    name = "Q"
    requests = make_requests(name, 21, [530])
    plan = helpers.plan_portions(requests, sizes=(130, 2, 127, 3, 64, 100, 2, 1, 1, 1, 97, 1, 1))
    for dtype in ("float32", "bfloat16"):
        runner = make_runner(model_dirs[name], dtype, 70, 8)
        got = helpers.run_plan_in_process(runner, plan)
        lh.compare(model_dirs[name], requests, got, TOL[dtype], f"long/{dtype}", 8, outliers=0.25 if dtype == "bfloat16" else 0.0)


def test_a_lost_state_or_wrong_slot_shows(model_dirs):
    """The test models are made so that the recurrent state matters: the same tokens after another prefix give
    other logits, by far more than the bar."""
    name = "P"
    tokens = make_requests(name, 31, [60])["r0"]
    full = lh.plain_logits(model_dirs[name], tokens)
    tail_alone = lh.plain_logits(model_dirs[name], tokens[30:])
    assert np.sqrt(np.mean((full[-1] - tail_alone[-1]) ** 2)) > 5 * TOL["bfloat16"]


def test_trace_replay_program(model_dirs, tmp_path):
    """bin/trace_run picks the model class by config.json and replays a mixed plan with four state slots."""
    name = "P"
    requests = make_requests(name, 13, [9, 40, 70, 23, 31, 12])
    plan = helpers.plan_mixed(requests, np.random.default_rng(2))
    budget = helpers.live_token_budget(plan, requests)
    vocab = lh.CONFIGS[name][0]["vocab"]
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_with_trace_run(model_dirs[name], dtype, plan, tmp_path / dtype, budget, vocab=vocab)
        lh.compare(model_dirs[name], requests, got, TOL[dtype], f"trace/{dtype}", 16, outliers=0.25 if dtype == "bfloat16" else 0.0)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_scheduler(model_dirs, name):
    """generate(): continuous batching, chunked prefill and captured decode steps; in 32-bit the tokens are the
    plain implementation's, in bfloat16 every token is within bfloat16's reach of the plain choice."""
    from sprout_lm_b200 import generate, load_model
    config, tensors = lh.plain_model(model_dirs[name])
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
                assert row[token] >= row.max() - 4 * TOL["bfloat16"], (name, len(history), token)
                history.append(token)


def test_scheduler_under_page_pressure(model_dirs):
    """A pool smaller than the requests together: a preempted request gives its state slot back and recomputes its
    state from the start; the greedy tokens stay the plain implementation's."""
    from sprout_lm_b200 import EngineOptions, generate, load_model
    name = "P"
    config, tensors = lh.plain_model(model_dirs[name])
    rng = np.random.default_rng(8)
    prompts = [helpers.random_tokens(rng, n, config["vocab"]) for n in (30, 41, 26, 35)]
    model = load_model(model_dirs[name], dtype="float32")
    options = EngineOptions(block_size=8, num_blocks=14, max_sequences=4, max_batch_tokens=24, prefill_chunk_size=7)
    results = generate(model, prompts, max_new_tokens=10, ignore_eos=True, options=options)
    for prompt, result in zip(prompts, results):
        assert result["output"] == plain.greedy(config, tensors, prompt, 10)
