"""Fomalix in the ragged engine against the plain evaluation in ``fomalix_oracle.py`` (float64, whole sequences, no cache):
every mixer alone, prefill against token-by-token decoding, prompt portions down to two tokens, unequal batches, reuse
of KV pages and state slots, keys at chunk and page borders, the first tokens, long decoding, odd sizes, and greedy
generation through the scheduler.  Runs on the PyTorch branch of every op without a GPU; ``test_fomalix_gpu.py`` runs
the same cases on the CUDA kernels."""
import copy
import math

import pytest
import torch

import fomalix_oracle as O
from shuffle_exchange_b200.inference.v2.config_v2 import RaggedInferenceEngineConfig
from shuffle_exchange_b200.inference.v2.engine_factory import build_engine_from_state_dict
from shuffle_exchange_b200.inference.v2.kernels import mixer_ops as M
from shuffle_exchange_b200.inference.v2.ragged.ragged_manager import DSStateManagerConfig
from shuffle_exchange_b200.inference.v2.sampling import SamplingParams, sample
from shuffle_exchange_b200.inference.v2.scheduler import RaggedScheduler, generate

DEV = "cuda" if torch.cuda.is_available() else "cpu"

DELTA = {"type": "delta", "mixer": {"conv": 3, "dim": 8, "heads": 4, "kv_heads": 2, "vdim": 12}, "mlp": None}
SSD = {"type": "mamba2", "mixer": {"conv": 5, "groups": 2, "heads": 4, "norm_groups": 2, "state": 8, "vdim": 6},
       "mlp": None}
ATTN = {"type": "attention", "mixer": {"dim": 16, "heads": 4, "kv_heads": 2, "mask": {"size": 6}, "scale": 0.3,
                                       "vdim": 8}, "mlp": {"ff": 40, "kind": "dense"}}


def make_cfg(layers, width=48, vocab=61, loop=None, scale=2.0, eps=1e-5):
    cfg = {"architecture": "Fomalix", "embedding": {"scale": scale}, "layers": copy.deepcopy(layers),
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


MIXED = make_cfg([DELTA, ATTN, SSD, dict(ATTN, mlp=None)], loop=(1, 3, 2))


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


# ------------------------------------------------------------------------------------------------ single mechanisms
@pytest.mark.parametrize("layer", [DELTA, SSD, ATTN, dict(ATTN, mixer=dict(ATTN["mixer"], mask=None))],
                         ids=["delta", "mamba2", "attention_chunked", "attention_causal"])
def test_one_layer_of_each_kind(layer):
    cfg = make_cfg([layer])
    W = O.random_weights(cfg, seed=1)
    toks = tokens(23, cfg["vocab"], 2)
    want, _ = O.forward(toks, W, cfg)
    eng = make_engine(cfg, W)
    close(feed(eng, 1, toks, [len(toks)]), want)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(6, 2, 12, 8), (8, 2, 16, 20), (8, 1, 8, 136), (5, 5, 24, 132)],
                         ids=["group_of_3", "group_of_4", "group_of_8_wide_values", "no_sharing_wide_values"])
def test_attention_head_groupings(heads, kv_heads, dim, vdim):
    """Every way the kernels take the query heads of a key/value head together, and value heads on both sides of 128;
    a whole prompt, portions that start inside a chunk, and single tokens."""
    layer = dict(ATTN, mixer={"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": 21}, "scale": dim ** -0.5,
                              "vdim": vdim})
    cfg = make_cfg([layer], width=40)
    W = O.random_weights(cfg, seed=heads)
    toks = tokens(50, cfg["vocab"], 3)
    want, _ = O.forward(toks, W, cfg)
    eng = make_engine(cfg, W, block_size=8)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [19, 17, 5] + [1] * 9), want)


def test_short_conv_carries_inputs_across_calls():
    g = torch.Generator().manual_seed(3)
    C, taps, T = 10, 4, 9
    x = torch.randn(T, C, generator=g)
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = O.silu(O.short_conv(x.double(), w.double(), b.double()))
    state = torch.full((3, taps - 1, C), 7.0, device=DEV)          # garbage of a previous owner of the slot
    got, lo = [], 0
    for n in (1, 1, 2, 5):                                          # portions shorter than the filter first
        info = torch.tensor([[0, n, lo, 2]], dtype=torch.int32, device=DEV)
        xs = x[lo: lo + n].to(DEV)
        t2s = torch.zeros(n, dtype=torch.int32, device=DEV)
        got.append(M.conv_silu(xs, w.to(DEV), b.to(DEV), state, info, t2s).cpu())
        M.conv_state_update(xs, state, info)
        lo += n
    assert torch.allclose(torch.cat(got).double(), want, atol=1e-5)
    assert torch.all(state[:2] == 7.0)


@pytest.mark.parametrize("taps", [2, 3, 4, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_short_conv_over_channel_groups_of_8_and_several_sequences(taps, dtype):
    """Channel counts and pitches that are multiples of 8 (16-byte loads), three sequences of unequal portions in each
    batch, portions longer than the kernel's row groups, the input a column slice of a wider matrix."""
    g = torch.Generator().manual_seed(taps)
    C, lens = 24, (229, 3, 11)
    xs = [torch.randn(n, C, generator=g).to(dtype) for n in lens]
    w, b = torch.randn(C, taps, generator=g).to(dtype), torch.randn(C, generator=g).to(dtype)
    want = [O.silu(O.short_conv(x.double(), w.double(), b.double())) for x in xs]
    state = torch.full((4, taps - 1, C), -5.0, device=DEV, dtype=dtype)
    cuts = ([17, 201, 11], [2, 1], [1, 9, 1])                       # per sequence; batch i holds every i-th portion
    at, got = [0, 0, 0], [[], [], []]
    for i in range(3):
        rows, info, t2s = [], [], []
        for q in range(3):
            if i >= len(cuts[q]):
                continue
            n = cuts[q][i]
            info.append([sum(r.shape[0] for r in rows), n, at[q], q + 1])
            t2s += [len(info) - 1] * n
            rows.append(xs[q][at[q]: at[q] + n])
            at[q] += n
        wide = torch.zeros(len(t2s), 8 + C + 8, dtype=dtype)
        wide[:, 8: 8 + C] = torch.cat(rows)
        xin = wide.to(DEV)[:, 8: 8 + C]
        info_t = torch.tensor(info, dtype=torch.int32, device=DEV)
        out = M.conv_silu(xin, w.to(DEV), b.to(DEV), state, info_t, torch.tensor(t2s, dtype=torch.int32, device=DEV)).cpu()
        M.conv_state_update(xin, state, info_t)
        for k, row in enumerate(info):
            got[row[3] - 1].append(out[row[0]: row[0] + row[1]])
    for q in range(3):
        assert torch.allclose(torch.cat(got[q]).double(), want[q], atol=1e-5)
    assert torch.all(state[0] == -5.0)


def _attend(q, k, v, sink, scale, chunk, block_size, pos0=0):
    """Run the attention op for queries at positions pos0.. over keys 0.. laid out in shuffled pages."""
    Tk, G, d = k.shape
    Tq, Hq, _ = q.shape
    dv = v.shape[2]
    n_pages = (Tk + block_size - 1) // block_size
    order = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(5))[:n_pages]
    kc = torch.zeros(n_pages + 3, block_size, G, d)
    vc = torch.zeros(n_pages + 3, block_size, G, dv)
    for j in range(Tk):
        kc[order[j // block_size], j % block_size] = k[j]
        vc[order[j // block_size], j % block_size] = v[j]
    tables = order.to(torch.int32)[None].contiguous()
    pos = torch.arange(pos0, pos0 + Tq, dtype=torch.int32)
    atoms, n_long = None, 0
    if 16 < Tq <= 128 and d % 4 == 0 and dv % 4 == 0:         # a prompt portion: the tiled kernel where there is one
        atoms, n_long = torch.tensor([[0, 0, Tq, pos0, 0, pos0 + Tq]], dtype=torch.int32, device=DEV), 1
    out = M.sink_attention(q.to(DEV).contiguous(), kc.to(DEV), vc.to(DEV), None if sink is None else sink.to(DEV),
                           torch.zeros(Tq, dtype=torch.int32, device=DEV), pos.to(DEV), tables.to(DEV), scale, chunk,
                           torch.float32, atoms, n_long)
    return out.cpu().view(Tq, Hq, dv)


@pytest.mark.parametrize("chunk,block_size", [(6, 4), (8, 8), (5, 16), (0, 4)])
def test_attention_sees_exactly_its_chunk(chunk, block_size):
    """Value j is the one-hot of j, so the output of a query IS its attention weights.  One key just inside and one just
    outside each query's chunk get a score far above the rest: the inside one must take nearly all the weight, the
    outside one none, also where the edge falls on a page border, for whole prompts and for single decode tokens."""
    T, d = 40, 8
    k = torch.zeros(T, 1, d)
    k[:, 0, 0] = 1.0
    v = torch.eye(T).view(T, 1, T)
    for i in (0, 1, chunk - 1, chunk, chunk + 1, 2 * chunk, 23, 39):
        if i < 0 or i >= T:
            continue
        lo = (i // chunk) * chunk if chunk else 0
        kk = k.clone()
        kk[lo, 0, 0] = 30.0                       # first key the query may see
        if lo > 0:
            kk[lo - 1, 0, 0] = 60.0               # last key it may not see, with a larger score
        q = torch.zeros(T, 2, d)
        q[:, :, 0] = 1.0
        whole = _attend(q[: i + 1], kk, v, None, 1.0, chunk, block_size)[i]           # as a row of a prompt
        alone = _attend(q[i: i + 1], kk, v, None, 1.0, chunk, block_size, pos0=i)[0]   # as a decode token
        for w in (whole, alone):
            assert torch.allclose(w.sum(-1), torch.ones(2), atol=1e-5)
            assert w[:, :lo].abs().sum() == 0 and w[:, i + 1:].abs().sum() == 0
            assert w[0, lo] > 0.99 or i == lo
        assert torch.allclose(whole, alone, atol=1e-6)


def test_attention_sink_takes_weight_but_gives_no_value():
    T, d = 9, 4
    g = torch.Generator().manual_seed(7)
    q, k, v = torch.randn(T, 2, d, generator=g), torch.randn(T, 1, d, generator=g), torch.randn(T, 1, 3, generator=g)
    sink = torch.tensor([-1.0, 2.5])
    got = _attend(q, k, v, sink, 0.7, 0, 4)
    for h in range(2):
        for i in range(T):
            s = (k[: i + 1, 0] @ q[i, h]) * 0.7
            e = torch.exp(s - s.max())
            want = (e[:, None] * v[: i + 1, 0]).sum(0) / (e.sum() + math.exp(float(sink[h] - s.max())))
            assert torch.allclose(got[i, h], want, atol=1e-5)
    without = _attend(q, k, v, None, 0.7, 0, 4)
    assert (without - got).abs().max() > 1e-2


def test_recurrence_op_matches_its_equations_and_ignores_a_used_slot():
    g = torch.Generator().manual_seed(11)
    T, H, G, n, dv = 13, 4, 2, 5, 7
    kv, qv = torch.randn(T, G * n, generator=g), torch.randn(T, G * n, generator=g)
    val = torch.randn(T, H * dv, generator=g)
    decay, beta = torch.rand(T, H, generator=g), torch.rand(T, H, generator=g)
    skip = torch.randn(H, generator=g)
    for delta in (True, False):
        want = torch.zeros(T, H, dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(n, dv, dtype=torch.float64)
            kk, qq = kv.view(T, G, n)[:, h // (H // G)].double(), qv.view(T, G, n)[:, h // (H // G)].double()
            for t in range(T):
                S = decay[t, h].double() * S
                v = val.view(T, H, dv)[t, h].double()
                u = beta[t, h].double() * ((v - S.T @ kk[t]) if delta else v)
                S = S + torch.outer(kk[t], u)
                want[t, h] = S.T @ qq[t] + (0 if delta else skip[h].double() * v)
        state = torch.full((2, H, dv, n), 3.0, device=DEV)       # left by a finished sequence
        got, lo = [], 0
        for rows in (4, 1, 8):
            info = torch.tensor([[0, rows, lo, 1]], dtype=torch.int32, device=DEV)
            sl = slice(lo, lo + rows)
            got.append(M.linear_recurrence(kv[sl].to(DEV), qv[sl].to(DEV), val[sl].to(DEV), decay[sl].to(DEV),
                                           beta[sl].to(DEV), None if delta else skip.to(DEV), state, info, H, G, n, dv,
                                           delta).cpu())
            lo += rows
        assert torch.allclose(torch.cat(got).double().view(T, H, dv), want, atol=1e-4)
        assert torch.all(state[0] == 3.0)


@pytest.mark.parametrize("n,dv,portions", [(128, 24, (19, 18)), (130, 20, (37,)), (64, 17, (8, 16, 9)), (40, 33, (33,))])
def test_recurrence_op_over_many_rows_and_wide_states(n, dv, portions):
    """Rows beyond one staging group of the kernel, state sizes on both sides of its register layouts' limits."""
    g = torch.Generator().manual_seed(n + dv)
    T, H, G = sum(portions), 3, 1
    kv = torch.randn(T, G * n, generator=g) / n ** 0.5
    qv = torch.randn(T, G * n, generator=g) / n ** 0.5
    val = torch.randn(T, H * dv, generator=g)
    decay, beta = torch.rand(T, H, generator=g) * 0.2 + 0.8, torch.rand(T, H, generator=g)
    for delta in (True, False):
        want = torch.zeros(T, H, dv, dtype=torch.float64)
        for h in range(H):
            S = torch.zeros(n, dv, dtype=torch.float64)
            for t in range(T):
                S = decay[t, h].double() * S
                v = val.view(T, H, dv)[t, h].double()
                u = beta[t, h].double() * ((v - S.T @ kv[t].double()) if delta else v)
                S = S + torch.outer(kv[t].double(), u)
                want[t, h] = S.T @ qv[t].double()
        state = torch.full((1, H, dv, n), -2.0, device=DEV)
        got, lo = [], 0
        for rows in portions:
            info = torch.tensor([[0, rows, lo, 0]], dtype=torch.int32, device=DEV)
            sl = slice(lo, lo + rows)
            got.append(M.linear_recurrence(kv[sl].to(DEV), qv[sl].to(DEV), val[sl].to(DEV), decay[sl].to(DEV),
                                           beta[sl].to(DEV), None, state, info, H, G, n, dv, delta).cpu())
            lo += rows
        assert torch.allclose(torch.cat(got).double().view(T, H, dv), want, atol=2e-4)


def test_far_token_reaches_the_end_through_the_recurrent_state():
    """A delta-rule layer with decay ~1 keeps what an early token wrote: changing token 2 of a long prompt must change
    the last logits by the amount the plain evaluation says, after decoding through many steps."""
    cfg = make_cfg([DELTA])
    W = O.random_weights(cfg, seed=4)
    W["l0.mix.A_log"] = torch.full_like(W["l0.mix.A_log"], -9.0)            # decay = exp(-e^-9 * softplus(.)) ~ 1
    a = tokens(70, cfg["vocab"], 5)
    b = list(a)
    b[2] = (a[2] + 1) % cfg["vocab"]
    wa, wb = O.forward(a, W, cfg)[0][-1], O.forward(b, W, cfg)[0][-1]
    assert (wa - wb).abs().max() > 1e-3
    eng = make_engine(cfg, W)
    ga = feed(eng, 1, a, [40, 1])[-1]
    eng.flush(1)
    gb = feed(eng, 2, b, [40, 1])[-1]
    close(ga[None], wa[None])
    close(gb[None], wb[None])
    assert torch.allclose(ga - gb, wa - wb, atol=1e-4)


# ------------------------------------------------------------------------------------------------ whole model
@pytest.fixture(scope="module")
def mixed():
    W = O.random_weights(MIXED, seed=0)
    toks = tokens(45, MIXED["vocab"], 1)
    return W, toks, O.forward(toks, W, MIXED)[0]


def test_prefill_equals_token_by_token_decoding(mixed):
    W, toks, want = mixed
    eng = make_engine(MIXED, W)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [1]), want)


@pytest.mark.parametrize("sizes", [[2], [3, 2, 7, 1, 1, 11], [6, 6, 6], [5, 4]], ids=str)
def test_prompt_portions(mixed, sizes):
    W, toks, want = mixed
    close(feed(make_engine(MIXED, W), 1, toks, sizes), want)


def test_first_tokens_one_at_a_time(mixed):
    W, toks, want = mixed
    eng = make_engine(MIXED, W)
    close(feed(eng, 1, toks[:7], [1]), want[:7])


def test_unequal_requests_in_one_batch_equal_each_alone():
    W = O.random_weights(MIXED, seed=2)
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
    """As many pages as the longest request and its neighbour need, two state slots: every later request gets pages and a slot that an earlier
    one filled, in another order, and must come out as if alone."""
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


def test_long_decoding(mixed):
    W, _, _ = mixed
    toks = tokens(150, MIXED["vocab"], 6)
    want = O.forward(toks, W, MIXED)[0]
    eng = make_engine(MIXED, W)
    close(feed(eng, 1, toks, [9] + [1] * 200), want)


ODD = [
    make_cfg([dict(DELTA, mixer={"conv": 2, "dim": 5, "heads": 3, "kv_heads": 3, "vdim": 7}, mlp={"ff": 17, "kind": "dense"}),
              dict(SSD, mixer={"conv": 4, "groups": 1, "heads": 3, "norm_groups": 3, "state": 9, "vdim": 5})],
             width=30, vocab=37, loop=(0, 2, 3), scale=0.5, eps=1e-3),
    make_cfg([dict(ATTN, mixer={"dim": 6, "heads": 6, "kv_heads": 1, "mask": {"size": 1}, "scale": 1.7, "vdim": 10}),
              dict(SSD, mixer={"conv": 1, "groups": 4, "heads": 4, "norm_groups": 1, "state": 3, "vdim": 9}),
              dict(DELTA, mixer={"conv": 6, "dim": 33, "heads": 2, "kv_heads": 1, "vdim": 4})],
             width=20, vocab=16, loop=(1, 2, 2), scale=1.0),
    make_cfg([dict(ATTN, mixer={"dim": 4, "heads": 2, "kv_heads": 2, "mask": {"size": 100}, "scale": 0.5, "vdim": 4},
                   mlp=None)], width=8, vocab=11),
]


@pytest.mark.parametrize("cfg", ODD, ids=["no_multiples_of_8", "one_wide_chunks_and_groups", "chunk_longer_than_prompt"])
def test_other_sizes(cfg):
    W = O.random_weights(cfg, seed=8)
    toks = tokens(21, cfg["vocab"], 9)
    want = O.forward(toks, W, cfg)[0]
    eng = make_engine(cfg, W, block_size=8)
    close(feed(eng, 1, toks, [len(toks)]), want)
    close(feed(eng, 2, toks, [4, 1, 2]), want)


def test_layer_order_with_a_repeated_span():
    cfg = make_cfg([DELTA, SSD, ATTN, DELTA], loop=(1, 3, 3))
    assert [i for i, _ in O.layer_runs(cfg)] == [0, 1, 2, 1, 2, 1, 2, 3]
    from shuffle_exchange_b200.inference.v2.checkpoint.huggingface_engine import PlainModelConfig
    from shuffle_exchange_b200.inference.v2.model_implementations.fomalix import FomalixPolicy
    spec = FomalixPolicy(PlainModelConfig(cfg)).spec(PlainModelConfig(cfg))
    assert spec.runs() == O.layer_runs(cfg)


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


def test_scheduler_mixes_prompt_portions_with_decode_tokens():
    W = O.random_weights(MIXED, seed=13)
    eng = make_engine(MIXED, W, blocks=40, block_size=4, max_live=4, max_tokens=8)
    sched = RaggedScheduler(eng, max_batch_tokens=8)
    sched.add_request(1, tokens(3, MIXED["vocab"], 1), 5)
    sched.add_request(2, tokens(20, MIXED["vocab"], 2), 2)
    first = sched.step()                                   # request 1 whole (3 tokens) + 5 tokens of request 2
    assert list(first) == [1]
    assert sched._live[2].fed == 5
    second = sched.step()                                  # 1 decode token + 7 more prompt tokens
    assert list(second) == [1] and sched._live[2].fed == 12
    out = sched.run()
    assert len(out[1]) == 5 and len(out[2]) == 2


def test_sampling_modes():
    logits = torch.tensor([[0.0, 3.0, 1.0, 2.9]])
    assert int(sample(logits)[0]) == 1
    g = torch.Generator().manual_seed(0)
    picks = {int(sample(logits, SamplingParams(temperature=1.0, top_k=2), g)[0]) for _ in range(50)}
    assert picks == {1, 3}
    picks = {int(sample(logits, SamplingParams(temperature=1.0, top_p=0.3), g)[0]) for _ in range(20)}
    assert picks == {1}
