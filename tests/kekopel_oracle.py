"""Plain, slow evaluation of a Kekopel model for the tests: one function per mechanism, whole sequences only, no cache,
no batching, float64 by default.  Nothing here is imported by the package, and nothing of the package is imported here.

Notation: ``h`` [T, width] is what a sublayer reads, ``p`` a dict of that layer's tensors by their names after
``l<i>.mix.`` / ``l<i>.mlp.``, ``m`` the layer's ``mixer`` (or ``mlp``) entry of the configuration.
"""
import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def input_filter(x, w):
    """x + y with y[t, c] = sum_j w[c, j] x[t - (taps - 1) + j, c], zeros before the start."""
    T, _ = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return x + y


def rotate_pairs(x, positions, n_rot, base):
    """x [T, ..., n]: the pairs (2i, 2i+1), i < n_rot / 2, turned by the angle position * base^(-2i / n_rot)."""
    out = x.clone()
    for t, pos in enumerate(positions):
        for i in range(n_rot // 2):
            a = float(pos) * base ** (-2.0 * i / n_rot)
            u, v = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * math.cos(a) - v * math.sin(a)
            out[t, ..., 2 * i + 1] = v * math.cos(a) + u * math.sin(a)
    return out


def windowed_sink_softmax(scores, sink, window):
    """scores [H, T, T] (query, key): weights over the keys j with 0 <= i - j < window (all j <= i if window is None); the
    denominator also holds exp(sink[h]), which has no key."""
    H, T, _ = scores.shape
    w = torch.zeros_like(scores)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        s = scores[:, i, lo: i + 1]
        mx = torch.maximum(s.max(-1).values, sink)
        e = torch.exp(s - mx[:, None])
        w[:, i, lo: i + 1] = e / (e.sum(-1) + torch.exp(sink - mx))[:, None]
    return w


def latent_attention(h, p, m, eps):
    T = h.shape[0]
    H, d, rot, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    n_rot, base = m["rot"]["dims"], m["rot"]["base"]
    pos = list(range(T))
    cq = rms(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).view(T, H, d + rot)
    down = h @ p["dkv"].T
    c = rms(down[:, :r], eps) * p["dkv.norm"]
    k_shared = rotate_pairs(down[:, r:], pos, n_rot, base)                  # [T, rot], the same for every head
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, n_rot, base)
    k_plain = (c @ p["uk"].T).view(T, H, d)
    v = (c @ p["uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_shared)) * m["scale"]
    size = (m.get("mask") or {}).get("size")
    w = windowed_sink_softmax(scores, p["sink"], size)
    return torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * dv) @ p["o"].T


def mlstm(h, p, m, eps):
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ p["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ p["k"].T).view(T, H, d)
    v = (h @ p["v"].T).view(T, H, dv)
    log_i = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        z = torch.zeros(d, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new = torch.maximum(log_f[t, hh] + mx, log_i[t, hh])
            keep, take = torch.exp(log_f[t, hh] + mx - new), torch.exp(log_i[t, hh] - new)
            S = keep * S + take * torch.outer(k[t, hh], v[t, hh])
            z = keep * z + take * k[t, hh]
            mx = new
            den = torch.maximum((z @ q[t, hh]).abs(), torch.exp(-mx)) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    o = rms(out, eps).reshape(T, H * dv) * p["norm"] * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def dense_ff(h, p):
    return (torch.relu(h @ p["up"].T + p["up.b"]) ** 2) @ p["down"].T + p["down.b"]


def expert_ff(h, p, mlp):
    """Every token goes to the ``top`` experts with the largest sigmoid(router logit); the score multiplies what the
    expert READS; the experts' outputs are summed as they are."""
    top = mlp["router"]["top"]
    score = torch.sigmoid(h @ p["router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(score[t], top).indices.tolist():
            x = score[t, e] * h[t]
            out[t] += (silu(p[f"e{e}.gate"] @ x) * (p[f"e{e}.up"] @ x)) @ p[f"e{e}.down"].T
    return out


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(tokens, W, cfg, dtype=torch.float64):
    """-> (logits [T, vocab], [the stream every layer hands on])."""
    W = {k: v.to(dtype) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    results, handed = [x], []
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        mixer = latent_attention if L["type"] == "latent_attention" else mlstm
        y = mixer(input_filter(x, W[pre + "canon1"]), sub(W, pre + "mix."), L["mixer"], eps)
        x = x + W[pre + "ls1"] * (rms(y, eps) * W[pre + "norm1"])
        if L.get("mlp") is not None:
            h = input_filter(x, W[pre + "canon2"])
            y = dense_ff(h, sub(W, pre + "mlp.")) if L["mlp"]["kind"] == "dense" else expert_ff(h, sub(W, pre + "mlp."), L["mlp"])
            x = x + W[pre + "ls2"] * (rms(y, eps) * W[pre + "norm2"])
        results.append(x)
        x = sum(W[pre + "dwa"][j] * results[j] for j in range(i + 2))
        handed.append(x)
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T, handed


def random_weights(cfg, seed=0):
    """bf16-representable fp32 tensors under the checkpoint's names."""
    g = torch.Generator().manual_seed(seed)
    W, width = {}, cfg["width"]
    taps = cfg["canon"]["taps"]

    def rnd(*shape, scale=1.0, shift=0.0):
        return (torch.randn(tuple(shape), generator=g) * scale + shift).to(torch.bfloat16).float()

    def lin(out, inp, gain=1.0):
        return rnd(out, inp, scale=gain / math.sqrt(inp))

    W["embed"] = rnd(cfg["vocab"], width)
    W["head"] = lin(cfg["vocab"], width)
    W["final.norm"] = rnd(scale=0.1, shift=1.0)
    for i, L in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", L["mixer"]
        W[pre + "norm1"], W[pre + "ls1"] = rnd(scale=0.1, shift=1.0), rnd(width, scale=0.2, shift=0.6)
        W[pre + "canon1"] = rnd(width, taps, scale=0.4)
        dwa = rnd(i + 2, scale=0.15)
        dwa[-1] += 0.8
        W[pre + "dwa"] = dwa.to(torch.bfloat16).float()
        if L["type"] == "latent_attention":
            H, d, rot, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            W[pre + "mix.dq"], W[pre + "mix.dq.norm"] = lin(qr, width), rnd(qr, scale=0.1, shift=1.0)
            W[pre + "mix.uq"] = lin(H * (d + rot), qr, 2.0)
            W[pre + "mix.dkv"], W[pre + "mix.dkv.norm"] = lin(r + rot, width, 1.5), rnd(r, scale=0.1, shift=1.0)
            W[pre + "mix.uk"], W[pre + "mix.uv"] = lin(H * d, r, 2.0), lin(H * dv, r)
            W[pre + "mix.sink"] = rnd(H)
            W[pre + "mix.o"] = lin(width, H * dv)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            W[pre + "mix.q"], W[pre + "mix.k"] = lin(H * d, width, 2.0), lin(H * d, width, 2.0)
            W[pre + "mix.v"], W[pre + "mix.g"] = lin(H * dv, width), lin(H * dv, width)
            W[pre + "mix.i"], W[pre + "mix.i.b"] = lin(H, width, 3.0), rnd(H, scale=2.0, shift=-2.0)
            W[pre + "mix.f"], W[pre + "mix.f.b"] = lin(H, width, 3.0), rnd(H, scale=2.0, shift=2.0)
            W[pre + "mix.norm"] = rnd(H * dv, scale=0.1, shift=1.0)
            W[pre + "mix.o"] = lin(width, H * dv)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        W[pre + "norm2"], W[pre + "ls2"] = rnd(scale=0.1, shift=1.0), rnd(width, scale=0.2, shift=0.6)
        W[pre + "canon2"] = rnd(width, taps, scale=0.4)
        if mlp["kind"] == "dense":
            W[pre + "mlp.up"], W[pre + "mlp.up.b"] = lin(mlp["ff"], width), rnd(mlp["ff"], scale=0.3)
            W[pre + "mlp.down"], W[pre + "mlp.down.b"] = lin(width, mlp["ff"]), rnd(width, scale=0.3)
        else:
            F = mlp["expert"]["ff"]
            W[pre + "mlp.router"] = lin(mlp["router"]["experts"], width, 3.0)
            for e in range(mlp["router"]["experts"]):
                W[pre + f"mlp.e{e}.gate"], W[pre + f"mlp.e{e}.up"] = lin(F, width), lin(F, width)
                W[pre + f"mlp.e{e}.down"] = lin(width, F)
    return W
