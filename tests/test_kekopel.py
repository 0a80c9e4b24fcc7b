"""Kekopel in the ragged engine against the plain evaluation in ``kekopel_oracle.py`` (float64, whole sequences, no cache):
every mechanism alone, prefill against token-by-token decoding, prompt portions down to two tokens, unequal batches,
reuse of cache pages and state slots, keys far back, at page borders and on both sides of the window's edge, the first
tokens, long decoding, odd sizes, and greedy generation through the scheduler.  Runs on the PyTorch branch of every op
without a GPU; ``test_kekopel_gpu.py`` runs the same cases on the CUDA kernels."""
import copy

import pytest
import torch

import kekopel_oracle as O
from shuffle_exchange_b200.inference.v2.config_v2 import RaggedInferenceEngineConfig
from shuffle_exchange_b200.inference.v2.engine_factory import build_engine_from_state_dict
from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
from shuffle_exchange_b200.inference.v2.ragged.ragged_manager import DSStateManagerConfig
from shuffle_exchange_b200.inference.v2.scheduler import generate
from shuffle_exchange_b200.ops import moe_ops

DEV = "cuda" if torch.cuda.is_available() else "cpu"

LATENT = {"type": "latent_attention",
          "mixer": {"dim": 8, "heads": 3, "kv_rank": 20, "mask": {"size": 7}, "q_rank": 12,
                    "rot": {"base": 500.0, "dims": 4}, "rot_dim": 4, "scale": 0.3, "vdim": 12},
          "mlp": {"ff": 40, "kind": "dense"}}
MLSTM = {"type": "mlstm", "mixer": {"dim": 8, "gate_cap": 6.0, "heads": 2, "vdim": 12},
         "mlp": {"expert": {"ff": 16}, "kind": "moe", "router": {"experts": 5, "top": 2}}}


def make_cfg(layers, width=24, vocab=53, taps=3, eps=1e-5):
    return {"architecture": "Kekopel", "canon": {"taps": taps}, "layers": copy.deepcopy(layers), "norm": {"eps": eps},
            "vocab": vocab, "width": width}


MIXED = make_cfg([LATENT, MLSTM, dict(MLSTM, mlp=None), dict(LATENT, mlp=MLSTM["mlp"])])


def make_engine(cfg, W, dtype=torch.float32, blocks=64, block_size=4, max_live=4, max_tokens=256):
    sm = DSStateManagerConfig(max_tracked_sequences=max_live, max_ragged_sequence_count=max_live,
                              max_ragged_batch_size=max_tokens, max_context=blocks * block_size, num_kv_blocks=blocks)
    return build_engine_from_state_dict(cfg, W, RaggedInferenceEngineConfig(state_manager=sm, kv_block_size=block_size),
                                        dtype=dtype)


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def feed(engine, uid, toks, sizes):
    """Give ``toks`` to the engine in portions of the given sizes (cycled); returns the logits of every token."""
    out, lo, i = [], 0, 0
    while lo < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - lo)
        i += 1
        out.append(engine.put([uid], [torch.tensor(toks[lo: lo + n])], logit_positions=[list(range(n))]))
        lo += n
    return torch.cat(out).double().cpu()


def close(got, want, tol=2e-4):
    """Difference with the mean over the vocabulary taken off, relative to the spread of the expected logits."""
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std()
    assert err.max() < tol, f"worst row {int(err.argmax())}: {float(err.max()):.3e}"


@pytest.fixture(scope="module")
def mixed():
    W = O.random_weights(MIXED, seed=4)
    toks = tokens(41, MIXED["vocab"], 5)
    return W, toks, O.forward(toks, W, MIXED)[0]


# ------------------------------------------------------------------------------------------------ single mechanisms
@pytest.mark.parametrize("layer", [LATENT, MLSTM, dict(LATENT, mlp=None), dict(MLSTM, mlp=LATENT["mlp"]),
                                   dict(LATENT, mixer=dict(LATENT["mixer"], mask=None))],
                         ids=["latent_dense", "mlstm_experts", "latent_alone", "mlstm_dense", "latent_causal"])
def test_one_layer_of_each_kind(layer):
    cfg = make_cfg([layer])
    W = O.random_weights(cfg, seed=1)
    toks = tokens(23, cfg["vocab"], 2)
    want, _ = O.forward(toks, W, cfg)
    eng = make_engine(cfg, W)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [3, 1, 2]), want)


def test_stream_after_every_layer(mixed):
    W, toks, _ = mixed
    _, handed = O.forward(toks, W, MIXED)
    eng = make_engine(MIXED, W)
    eng.model().layer_outputs = []
    feed(eng, 1, toks, [len(toks)])
    for got, want in zip(eng.model().layer_outputs, handed):
        assert torch.allclose(got.double().cpu(), want, atol=2e-4, rtol=1e-4)


def test_input_filter_carries_inputs_across_calls():
    g = torch.Generator().manual_seed(3)
    C, taps, T = 10, 4, 11
    x = torch.randn(T, C, generator=g)
    w = torch.randn(C, taps, generator=g)
    want = O.input_filter(x.double(), w.double())
    state = torch.full((3, taps - 1, C), 7.0, device=DEV)           # what a previous owner of the slot left
    got, lo = [], 0
    for n in (1, 1, 2, 7):                                           # portions shorter than the filter first
        info = torch.tensor([[0, n, lo, 2]], dtype=torch.int32, device=DEV)
        xs = x[lo: lo + n].to(DEV).contiguous()
        t2s = torch.zeros(n, dtype=torch.int32, device=DEV)
        got.append(M.conv_residual(xs, w.to(DEV), state, info, t2s, torch.float32).cpu())
        M.conv_state_update(xs, state, info)
        lo += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-5)
    assert torch.all(state[:2] == 7.0)


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_input_filter_over_several_sequences(taps):
    g = torch.Generator().manual_seed(taps)
    C, lens = 12, (9, 1, 4)
    xs = [torch.randn(n, C, generator=g) for n in lens]
    w = torch.randn(C, taps, generator=g)
    want = torch.cat([O.input_filter(x.double(), w.double()) for x in xs])
    state = torch.zeros(4, taps - 1, C, device=DEV)
    info, row = [], 0
    for s, n in enumerate(lens):
        info.append([row, n, 0, 3 - s])
        row += n
    t2s = torch.tensor(sum(([s] * n for s, n in enumerate(lens)), []), dtype=torch.int32, device=DEV)
    got = M.conv_residual(torch.cat(xs).to(DEV), w.to(DEV), state, torch.tensor(info, dtype=torch.int32, device=DEV), t2s,
                          torch.float32)
    assert torch.allclose(got.double().cpu(), want, atol=1e-5)


def test_post_norm_with_one_gain_scale_and_stream_mixture():
    g = torch.Generator().manual_seed(7)
    T, Wd, n_prev = 5, 18, 3
    x, y = torch.randn(T, Wd, generator=g), torch.randn(T, Wd, generator=g) * 3
    stack = torch.randn(n_prev + 1, T, Wd, generator=g)
    gain, ls, mixw = torch.tensor([1.3]), torch.randn(Wd, generator=g), torch.randn(n_prev + 1, generator=g)
    v = x.double() + ls.double() * (O.rms(y.double(), 1e-3) * 1.3)
    mixed_want = sum(mixw[j].double() * stack[j].double() for j in range(n_prev)) + mixw[n_prev].double() * v
    st, mo = stack.to(DEV).contiguous(), torch.empty(T, Wd, device=DEV)
    M.post_norm_mix(x.to(DEV), y.to(DEV), gain.to(DEV), ls.to(DEV), st[n_prev], 1e-3, st, n_prev, mixw.to(DEV), mo)
    assert torch.allclose(st[n_prev].double().cpu(), v, atol=1e-5)
    assert torch.allclose(mo.double().cpu(), mixed_want, atol=1e-5)
    rows = torch.tensor([4, 0], dtype=torch.int32, device=DEV)
    fin = M.rms_scale_rows(st[n_prev], rows, gain.to(DEV), 1e-3, torch.float32)
    assert torch.allclose(fin.double().cpu(), (O.rms(v, 1e-3) * 1.3)[[4, 0]], atol=1e-5)


@pytest.mark.parametrize("rot,n_rot", [(8, 8), (6, 4), (4, 0)])
def test_latent_cache_rows_and_rotated_queries(rot, n_rot):
    """Positions far from 0, pages in shuffled order: the cached row is [normalised latent | rotated shared key part],
    the query [its latent-space part | its rotated part]; channels past the rotated ones pass unchanged."""
    g = torch.Generator().manual_seed(rot)
    T, H, d, r, bs, base = 6, 3, 5, 7, 4, 300.0
    pos = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32) + 1000
    q = torch.randn(T, H * (d + rot), generator=g)
    q_abs = torch.randn(H, T, r, generator=g).transpose(0, 1)
    kv = torch.randn(T, r + rot, generator=g)
    wn = torch.randn(r, generator=g)
    inv = torch.tensor([base ** (-2.0 * i / max(n_rot, 1)) for i in range(n_rot // 2)], dtype=torch.float32)
    n_pages = 1006 // bs + 1
    tables = torch.randperm(n_pages, generator=g).to(torch.int32)[None].contiguous()
    cache = torch.zeros(n_pages, bs, 1, r + rot, device=DEV)
    t2s = torch.zeros(T, dtype=torch.int32, device=DEV)
    out = M.latent_qk_prepare(q.to(DEV), q_abs.to(DEV), kv.to(DEV), wn.to(DEV), inv.to(DEV), cache, t2s, pos.to(DEV),
                              tables.to(DEV), H, d, rot, 1e-4).cpu().double()
    want_c = O.rms(kv[:, :r].double(), 1e-4) * wn.double()
    want_k = O.rotate_pairs(kv[:, r:].double(), pos.tolist(), n_rot, base)
    want_q = O.rotate_pairs(q.view(T, H, d + rot)[..., d:].double(), pos.tolist(), n_rot, base)
    for t in range(T):
        p = int(pos[t])
        row = cache[int(tables[0, p // bs]), p % bs, 0].cpu().double()
        assert torch.allclose(row[:r], want_c[t], atol=1e-5) and torch.allclose(row[r:], want_k[t], atol=2e-4)
    assert torch.allclose(out[..., :r], q_abs.double(), atol=1e-6)
    assert torch.allclose(out[..., r:], want_q, atol=2e-4)


def _attend_latent(q, rows, sink, scale, window, block_size, dv, pos0=0, tiled=True):
    """Attention in the latent space: queries at positions pos0.. over cached rows 0.. laid out in shuffled pages; the
    values are the first ``dv`` channels of the rows."""
    Tk, d = rows.shape
    Tq, Hq, _ = q.shape
    n_pages = (Tk + block_size - 1) // block_size
    order = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(5))[:n_pages]
    cache = torch.zeros(n_pages + 3, block_size, 1, d)
    for j in range(Tk):
        cache[order[j // block_size], j % block_size, 0] = rows[j]
    tables = order.to(torch.int32)[None].contiguous()
    pos = torch.arange(pos0, pos0 + Tq, dtype=torch.int32)
    atoms, n_long = None, 0
    if tiled and 16 < Tq <= 128 and d % 4 == 0 and dv % 4 == 0:      # a prompt portion: the tiled kernel where there is one
        atoms, n_long = torch.tensor([[0, 0, Tq, pos0, 0, pos0 + Tq]], dtype=torch.int32, device=DEV), 1
    parts = []
    for c0 in range(0, dv, 256):                  # one pass holds at most 256 value channels
        n = min(256, dv - c0)
        out = M.sink_attention(q.to(DEV).contiguous(), cache.to(DEV), None, None if sink is None else sink.to(DEV),
                               torch.zeros(Tq, dtype=torch.int32, device=DEV), pos.to(DEV), tables.to(DEV), scale, 0,
                               torch.float32, atoms if dv <= 256 else None, n_long if dv <= 256 else 0, window=window,
                               value_cols=n, value_col0=c0)
        parts.append(out.cpu().view(Tq, Hq, n))
    return torch.cat(parts, dim=2)


@pytest.mark.parametrize("window,block_size,T", [(6, 4, 40), (8, 8, 40), (17, 16, 40), (1, 4, 12), (257, 16, 300), (0, 4, 40)])
def test_attention_sees_exactly_its_window(window, block_size, T):
    """Row j of the cache is [one-hot of j | score channel], so a query's output IS its attention weights.  The oldest key
    inside the window and the newest one outside get scores far above the rest: the inside one must take nearly all the
    weight and the outside one none -- also hundreds of positions back and where the edge falls on a page border --
    for rows of a prompt and for single decode tokens."""
    dv = (T + 3) // 4 * 4
    d = dv + 4
    for i in sorted({0, 1, window - 1, window, window + 1, 2 * window, 23, T - 1}):
        if i < 0 or i >= T:
            continue
        lo = max(0, i - window + 1) if window else 0
        rows = torch.zeros(T, d)
        rows[:, :T] = torch.eye(T)
        rows[:, dv] = 1.0
        rows[lo, dv] = 30.0                       # oldest key the query may see
        if lo > 0:
            rows[lo - 1, dv] = 60.0               # newest key it may not see, with a larger score
        q = torch.zeros(T, 2, d)
        q[:, :, dv] = 1.0
        first = max(0, i - 100)                   # as a row of a prompt portion of at most 101 rows
        whole = _attend_latent(q[first: i + 1], rows, None, 1.0, window, block_size, dv, pos0=first)[i - first]
        alone = _attend_latent(q[i: i + 1], rows, None, 1.0, window, block_size, dv, pos0=i)[0]
        for w in (whole, alone):
            assert torch.allclose(w.sum(-1), torch.ones(2), atol=1e-5)
            assert w[:, :lo].abs().sum() == 0 and w[:, i + 1:].abs().sum() == 0
            assert w[0, lo] > 0.99 or i == lo


def test_sink_takes_its_share_of_the_weight():
    """Equal scores on n keys and a sink logit of log(n): the keys share half of the weight; without the sink all of it;
    with a huge sink logit nearly nothing is left."""
    T, dv = 8, 8
    rows = torch.zeros(T, dv + 4)
    rows[:, :T] = torch.eye(T)
    q = torch.zeros(T, 3, dv + 4)
    sink = torch.tensor([float(torch.log(torch.tensor(8.0))), 50.0, -50.0])
    for q_rows, pos0 in ((q, 0), (q[7:8], 7)):
        w = _attend_latent(q_rows, rows, sink, 1.0, 0, 4, dv, pos0=pos0)[-1]
        assert torch.allclose(w[0], torch.full((dv,), 1.0 / 16), atol=1e-6)
        assert w[1].abs().max() < 1e-12 and torch.allclose(w[2], torch.full((dv,), 1.0 / 8), atol=1e-6)
    w = _attend_latent(q[7:8], rows, None, 1.0, 0, 4, dv, pos0=7)[0]
    assert torch.allclose(w, torch.full((3, dv), 1.0 / 8), atol=1e-6)


@pytest.mark.parametrize("dv", [20, 300])
def test_wide_latents_and_column_ranges(dv):
    """Value channels beyond what one pass holds are taken in column ranges of the cached rows."""
    g = torch.Generator().manual_seed(dv)
    T, H, d = 9, 2, dv + 8
    rows, q = torch.randn(T, d, generator=g), torch.randn(T, H, d, generator=g)
    s = torch.einsum("ihd,jd->hij", q.double(), rows.double()) * 0.2
    w = O.windowed_sink_softmax(s, torch.tensor([0.5, -0.5]).double(), 5)
    want = torch.einsum("hij,jd->ihd", w, rows[:, :dv].double())
    cache = rows.view(3, 3, 1, d).to(DEV).contiguous()
    tables = torch.tensor([[0, 1, 2]], dtype=torch.int32, device=DEV)
    zeros, pos = torch.zeros(T, dtype=torch.int32, device=DEV), torch.arange(T, dtype=torch.int32, device=DEV)
    parts = []
    for c0 in range(0, dv, 256):
        n = min(256, dv - c0)
        parts.append(M.sink_attention(q.to(DEV), cache, None, torch.tensor([0.5, -0.5], device=DEV), zeros, pos, tables, 0.2,
                                      0, torch.float32, window=5, value_cols=n, value_col0=c0).view(T, H, n))
    assert torch.allclose(torch.cat(parts, 2).double().cpu(), want, atol=1e-5)


def _mlstm_ops(proj, bias_i, bias_f, norm_w, H, n, dv, cap, eps, cuts):
    """The kernels of the matrix-memory LSTM in the order the mixer runs them, in portions."""
    S = torch.full((2, H, dv + 1, n), 3.0, device=DEV)
    mst = torch.full((2, H), -9.0, device=DEV)
    g0 = 2 * H * n + H * dv
    i0 = g0 + H * dv
    out, lo = [], 0
    for c in cuts:
        info = torch.tensor([[0, c, lo, 1]], dtype=torch.int32, device=DEV)
        p = proj[lo: lo + c].to(DEV).contiguous()
        decay, beta, mt = M.mlstm_gate_scan(p[:, i0: i0 + H], p[:, i0 + H: i0 + 2 * H], bias_i.to(DEV), bias_f.to(DEV), cap,
                                            mst, info)
        x = M.mlstm_prepare(p, H, n, dv, n ** -0.5)
        o = M.linear_recurrence(x[:, H * n: 2 * H * n], x[:, : H * n], x[:, 2 * H * n:], decay, beta, None, S, info, H, H, n,
                                dv + 1, False)
        out.append(M.mlstm_output(o, mt, p[:, g0: g0 + H * dv], norm_w.to(DEV), H, dv, eps, torch.float32).cpu())
        lo += c
    return torch.cat(out).double()


@pytest.mark.parametrize("H,n,dv,scale", [(2, 8, 12, 1.0), (3, 5, 7, 6.0), (1, 32, 4, 0.05)],
                         ids=["plain", "gates_at_their_cap", "tiny_inputs_floor_of_the_normaliser"])
def test_mlstm_mechanism(H, n, dv, scale):
    """Against the plain recurrence with explicit matrix, normaliser and running maximum (which starts at 0): gate
    pre-activations far past the cap, inputs so small that exp(-m) is the denominator, portions of 1, 2 and 40 tokens
    (more than one warp's scan), a state slot that holds another sequence's leftovers."""
    g = torch.Generator().manual_seed(n)
    T, width, cap, eps = 75, 10, 4.0, 1e-5
    h = torch.randn(T, width, generator=g)
    p = {k: torch.randn(rows, width, generator=g) * s for k, rows, s in
         (("q", H * n, scale), ("k", H * n, scale), ("v", H * dv, 1.0), ("g", H * dv, 1.0), ("i", H, 3 * scale),
          ("f", H, 3 * scale))}
    p["i.b"], p["f.b"] = torch.randn(H, generator=g) - 2, torch.randn(H, generator=g) + 1
    p["norm"], p["o"] = torch.randn(H * dv, generator=g), torch.eye(H * dv)
    m = {"heads": H, "dim": n, "vdim": dv, "gate_cap": cap}
    want = O.mlstm(h.double(), {k: v.double() for k, v in p.items()}, m, eps)
    proj = h @ torch.cat([p[k] for k in ("q", "k", "v", "g", "i", "f")]).T
    for cuts in ([T], [1, 1, 2, 40, 31]):
        got = _mlstm_ops(proj, p["i.b"], p["f.b"], p["norm"], H, n, dv, cap, eps, cuts)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())


@pytest.mark.parametrize("E,K", [(5, 2), (4, 4), (9, 1), (40, 3)])
def test_sigmoid_routing_scales_the_experts_input(E, K):
    g = torch.Generator().manual_seed(E)
    T, Hd = 13, 12
    logits, x = torch.randn(T, E, generator=g) * 2, torch.randn(T, Hd, generator=g)
    scores, assign, offsets, counts = moe_ops.top_k_gating(logits.to(DEV), K, renormalize=False, score_function="sigmoid")
    want_s, want_e = torch.topk(torch.sigmoid(logits), K, dim=-1)
    assert torch.equal(assign.cpu().long(), want_e) and torch.allclose(scores.cpu(), want_s, atol=1e-6)
    assert torch.equal(counts.cpu().long(), torch.bincount(want_e.reshape(-1), minlength=E))
    rows, cumsum, slots = moe_ops.moe_scatter_scaled(x.to(DEV), scores, assign, offsets, counts)
    ends = cumsum.cpu().tolist()
    for t in range(T):
        for k in range(K):
            s, e = int(slots[t, k]), int(assign[t, k])
            assert (ends[e - 1] if e else 0) <= s < ends[e]
            assert torch.allclose(rows[s].cpu(), x[t] * want_s[t, k], atol=1e-6)
    assert sorted(slots.cpu().reshape(-1).tolist()) == list(range(T * K))


# ------------------------------------------------------------------------------------------------ cache, state, batches
def test_prefill_equals_token_by_token_decoding(mixed):
    W, toks, want = mixed
    eng = make_engine(MIXED, W)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [1]), want)


@pytest.mark.parametrize("sizes", [[2], [3, 5], [7, 1, 1, 2], [16, 2, 9], [40, 1]])
def test_prompt_portions(mixed, sizes):
    W, toks, want = mixed
    eng = make_engine(MIXED, W)
    close(feed(eng, 1, toks, sizes), want)


def test_unequal_requests_in_one_batch_equal_each_alone():
    W = O.random_weights(MIXED, seed=9)
    reqs = {u: tokens(n, MIXED["vocab"], 10 + u) for u, n in ((1, 19), (2, 3), (3, 31), (4, 8))}
    want = {u: O.forward(t, W, MIXED)[0] for u, t in reqs.items()}
    eng = make_engine(MIXED, W)
    at = {u: 0 for u in reqs}
    got = {u: [] for u in reqs}
    plan = [{1: 5, 3: 2}, {1: 1, 2: 3, 3: 9, 4: 2}, {1: 13, 3: 1, 4: 1}, {3: 1, 4: 5}, {3: 18}]   # 2 is left out, 1 ends
    for step in plan:
        uids = list(step)
        toks = [torch.tensor(reqs[u][at[u]: at[u] + n]) for u, n in step.items()]
        out = eng.put(uids, toks, logit_positions=[list(range(n)) for n in step.values()]).double().cpu()
        k = 0
        for u, n in step.items():
            got[u].append(out[k: k + n])
            k, at[u] = k + n, at[u] + n
    for u in reqs:
        assert at[u] == len(reqs[u])
        close(torch.cat(got[u]), want[u])


def test_pages_and_state_slots_are_reused():
    """As many pages as the longest request and its neighbour need, two state slots: every later request gets pages and
    a slot that an earlier one filled, in another order, and must come out as if alone."""
    W = O.random_weights(MIXED, seed=3)
    eng = make_engine(MIXED, W, blocks=10, block_size=4, max_live=2)
    for i in range(4):
        toks = tokens(20 + 3 * i, MIXED["vocab"], 20 + i)
        other = tokens(6, MIXED["vocab"], 40 + i)
        eng.put([100 + i], [torch.tensor(other)])                 # a neighbour that holds the other slot and two pages
        got = feed(eng, i, toks, [7, 1, 2])
        close(got, O.forward(toks, W, MIXED)[0])
        eng.flush(i)
        eng.flush(100 + i)
        assert eng.free_blocks == 10


def test_a_far_key_inside_the_window_decides_the_logits():
    """One latent layer, window of 130 over pages of 8, key up-projection scaled up so that the softmax is peaked: single
    keys up to 129 positions back carry most of a query's weight, and the step at which such a key leaves the window
    changes the logits; prompt rows, portions and decode tokens must all follow the plain evaluation."""
    layer = dict(LATENT, mixer=dict(LATENT["mixer"], mask={"size": 130}, scale=1.5), mlp=None)
    cfg = make_cfg([layer], vocab=31)
    W = O.random_weights(cfg, seed=21)
    W["l0.mix.uk"] = W["l0.mix.uk"] * 3
    toks = tokens(150, cfg["vocab"], 22)
    want = O.forward(toks, W, cfg)[0]
    eng = make_engine(cfg, W, block_size=8, blocks=64, max_tokens=160)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [125] + [1] * 25), want)
    close(feed(eng, 3, toks, [64, 64, 3, 2]), want)


def test_long_decoding(mixed):
    W, _, _ = mixed
    toks = tokens(150, MIXED["vocab"], 6)
    want = O.forward(toks, W, MIXED)[0]
    eng = make_engine(MIXED, W)
    close(feed(eng, 1, toks, [9] + [1] * 200), want)


ODD = [
    make_cfg([dict(LATENT, mixer={"dim": 5, "heads": 1, "kv_rank": 9, "mask": {"size": 1}, "q_rank": 7,
                                  "rot": {"base": 77.0, "dims": 6}, "rot_dim": 6, "scale": 1.7, "vdim": 3},
                   mlp={"expert": {"ff": 7}, "kind": "moe", "router": {"experts": 3, "top": 3}}),
              dict(MLSTM, mixer={"dim": 3, "gate_cap": 15.0, "heads": 5, "vdim": 2}, mlp={"ff": 11, "kind": "dense"})],
             width=10, vocab=17, taps=1, eps=1e-3),
    make_cfg([dict(MLSTM, mixer={"dim": 33, "gate_cap": 2.0, "heads": 1, "vdim": 40},
                   mlp={"expert": {"ff": 64}, "kind": "moe", "router": {"experts": 2, "top": 1}}),
              dict(LATENT, mixer={"dim": 16, "heads": 8, "kv_rank": 8, "mask": {"size": 100}, "q_rank": 40,
                                  "rot": {"base": 1e6, "dims": 2}, "rot_dim": 2, "scale": 0.25, "vdim": 4}, mlp=None)],
             width=64, vocab=29, taps=6),
    make_cfg([dict(LATENT, mixer={"dim": 4, "heads": 2, "kv_rank": 24, "mask": {"size": 5}, "q_rank": 4,
                                  "rot": {"base": 10.0, "dims": 4}, "rot_dim": 8, "scale": 0.5, "vdim": 6},
                   mlp={"ff": 8, "kind": "dense"})] * 3, width=8, vocab=11, taps=2),
    make_cfg([dict(MLSTM, mlp=None), MLSTM], width=16, vocab=23),
]


@pytest.mark.parametrize("cfg", ODD, ids=["no_multiples_of_8_window_of_one_all_experts", "one_head_long_filter_window_past_prompt",
                                          "same_layer_three_times_part_of_the_channels_turn", "no_attention_layer_no_cache"])
def test_other_sizes(cfg):
    W = O.random_weights(cfg, seed=8)
    toks = tokens(21, cfg["vocab"], 9)
    want = O.forward(toks, W, cfg)[0]
    eng = make_engine(cfg, W, block_size=8)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [4, 1, 2]), want)


def test_configuration_is_read_into_the_layer_specs():
    from shuffle_exchange_b200.inference.v2.checkpoint.huggingface_engine import PlainModelConfig
    from shuffle_exchange_b200.inference.v2.model_implementations.kekopel import KekopelPolicy
    spec = KekopelPolicy(PlainModelConfig(MIXED)).spec(PlainModelConfig(MIXED))
    assert [L.kind for L in spec.layers] == ["latent_attention", "mlstm", "mlstm", "latent_attention"]
    a, b, c, d = spec.layers
    assert (a.window, a.kv_rank, a.q_rank, a.rot_dim, a.rot_dims, a.rot_base, a.attn_scale) == (7, 20, 12, 4, 4, 500.0, 0.3)
    assert (a.ff_kind, a.ff_dim, a.ff_activation) == ("biased", 40, "relu_sq")
    assert (b.ff_kind, b.ff_dim, b.n_experts, b.top_k, b.moe_score, b.moe_weight_input) == ("moe", 16, 5, 2, "sigmoid", True)
    assert c.ff_dim == 0 and b.gate_cap == 6.0
    assert spec.block_form == "post_scaled" and spec.input_conv_taps == 3 and spec.depth_mix


def test_bf16_serving_stays_near_the_exact_evaluation(mixed):
    W, toks, want = mixed
    eng = make_engine(MIXED, W, dtype=torch.bfloat16)
    whole = feed(eng, 1, toks, [len(toks)])
    parts = feed(eng, 2, toks, [5, 1, 2])
    close(whole, want, tol=0.08)
    close(parts, want, tol=0.08)


# ------------------------------------------------------------------------------------------------ generation
def test_greedy_generation_through_the_scheduler():
    W = O.random_weights(MIXED, seed=12)
    prompts = [tokens(n, MIXED["vocab"], 30 + n) for n in (5, 17, 2, 9, 12)]          # five requests, four may be live
    eng = make_engine(MIXED, W, blocks=40, block_size=4, max_live=4, max_tokens=16)
    got = generate(eng, prompts, max_new_tokens=6, max_batch_tokens=16, max_prompt_portion=7)
    for p, out in zip(prompts, got):
        seq = list(p)
        for tok in out:
            logits = O.forward(seq, W, MIXED)[0][-1]
            top2 = logits.topk(2).values
            if top2[0] - top2[1] > 1e-3:                       # a near tie may go either way in 32-bit
                assert tok == int(logits.argmax())
            seq.append(tok)
        assert len(out) == 6
    assert eng.free_blocks == 40 and eng._state_manager.n_tracked_sequences == 0


def test_command_line_generation_from_a_checkpoint_folder(tmp_path):
    """``config.json`` + ``model.safetensors`` (bf16) on disk, ``bin/sxb_generate`` picks the model class by the
    configuration, loads the tensors by their checkpoint names and continues two prompts greedily."""
    import json
    import os
    import struct
    import subprocess
    import sys
    W = O.random_weights(MIXED, seed=14)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(MIXED, f)
    meta, blobs, off = {}, [], 0
    for name, t in W.items():
        b = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        meta[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    header = json.dumps(meta).encode()
    with open(tmp_path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"".join(blobs))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompts = [[5, 17, 3], [9, 9, 1, 2, 3, 4, 5, 6, 7]]
    cmd = [sys.executable, os.path.join(root, "bin", "sxb_generate"), "--model", str(tmp_path), "--max-new-tokens", "4",
           "--dtype", "float32"]
    for p in prompts:
        cmd += ["--prompt", ",".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    assert [x["prompt"] for x in lines] == prompts
    for p, x in zip(prompts, lines):
        seq = list(p)
        for tok in x["generated"]:
            logits = O.forward(seq, W, MIXED)[0][-1]
            top2 = logits.topk(2).values
            if top2[0] - top2[1] > 1e-3:
                assert tok == int(logits.argmax())
            seq.append(tok)
        assert len(x["generated"]) == 4
