"""Plain, slow evaluation of a Fomalix model for the tests: one function per mechanism, whole sequences only, no cache,
no batching, float64 by default.  Nothing here is imported by the package, and nothing of the package is imported here.

Notation: ``h`` [T, width] is a sublayer's input, ``p`` a dict of that layer's tensors by their names after
``l<i>.mix.`` / ``l<i>.mlp.``, ``m`` the layer's ``mixer`` entry of the configuration.
"""
import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def position_vector(positions, width, dtype):
    out = torch.zeros(len(positions), width, dtype=dtype)
    for r, p in enumerate(positions):
        for c in range(width):
            i = c // 2
            ang = float(p) * 10000.0 ** (-2.0 * i / width)
            out[r, c] = math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return out


def short_conv(x, w, b=None):
    """Causal per-channel filter: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c], zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            if t - j >= 0:
                y[t] += w[:, taps - 1 - j] * x[t - j]
    if b is not None:
        y = y + b
    return y


def attention(h, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).view(T, H, d)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, d)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, dv)
    q, k = rms(q, eps), rms(k, eps)
    size = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if size is None or j // size == i // size]
            s = torch.stack([(q[i, hh] * k[j, g]).sum() * m["scale"] for j in js])
            mx = torch.maximum(s.max(), p["sink"][hh])
            e = torch.exp(s - mx)
            den = e.sum() + torch.exp(p["sink"][hh] - mx)
            for n, j in enumerate(js):
                out[i, hh] += e[n] / den * v[j, g]
    return out.reshape(T, H * dv) @ p["o"].T


def gated_delta(h, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ p["q"].T, p["q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ p["k"].T, p["k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ p["v"].T, p["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                            # [T, H]
    decay = torch.exp(-torch.exp(p["A_log"]) * softplus(h @ p["a"].T + p["dt_bias"]))
    gate = silu(h @ p["g"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = rms(out, eps) * p["norm"] * gate
    return out.reshape(T, H * dv) @ p["o"].T


def mamba2(h, p, m, eps):
    T = h.shape[0]
    H, dv, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * dv
    proj = h @ p["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, p["conv"], p["conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + p["dt_bias"])
    y = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-torch.exp(p["A_log"][hh]) * dt[t, hh]) * S + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + p["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    y = rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T


def dense_ff(h, p):
    return (gelu_tanh(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


MIXERS = {"attention": attention, "delta": gated_delta, "mamba2": mamba2}


def layer_runs(cfg):
    """[(layer index, starts a repeated pass)] in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, False) for i in range(loop["start"])]
    for rep in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, rep > 0 and i == loop["start"]))
    runs += [(i, False) for i in range(loop["stop"], n)]
    return runs


def forward(tokens, W, cfg, dtype=torch.float64):
    """-> (logits [T, vocab], residual stream after every layer run [runs, T, width])."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x + position_vector(range(T), cfg["width"], dtype)
    x0 = x.clone()
    trace = []
    for li, again in layer_runs(cfg):
        L = cfg["layers"][li]
        if again:
            x = x + x0
        pre = f"l{li}."
        p = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mix.")}
        y = MIXERS[L["type"]](rms(x, eps) * W[pre + "norm1"], p, L["mixer"], eps)
        x = x + rms(y, eps) * W[pre + "norm1b"]
        if L.get("mlp") is not None:
            p = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mlp.")}
            y = dense_ff(rms(x, eps) * W[pre + "norm2"], p)
            x = x + rms(y, eps) * W[pre + "norm2b"]
        trace.append(x.clone())
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T
    return logits, torch.stack(trace)


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Random tensors with the names and shapes the configuration implies."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    width = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(n, lo, hi):
        return (torch.rand(n, generator=g) * (hi - lo) + lo).to(dtype)

    W["embed"] = (torch.randn(cfg["vocab"], width, generator=g) * 0.5).to(dtype)
    W["head"] = mat(cfg["vocab"], width)
    W["final.norm"] = vec(width, 0.5, 1.5)
    for i, L in enumerate(cfg["layers"]):
        m, pre = L["mixer"], f"l{i}."
        W[pre + "norm1"], W[pre + "norm1b"] = vec(width, 0.5, 1.5), vec(width, 0.5, 1.5)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, o in (("q", H * d), ("k", G * d), ("v", G * dv)):
                W[pre + "mix." + n] = mat(o, width, 2.0)
                W[pre + "mix." + n + ".b"] = vec(o, -0.3, 0.3)
            W[pre + "mix.sink"] = vec(H, -1.0, 2.0)
            W[pre + "mix.o"] = mat(width, H * dv)
        elif L["type"] == "delta":
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, o in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[pre + "mix." + n] = mat(o, width, 2.0)
                W[pre + "mix." + n + ".conv"] = vec(o * taps, -0.6, 0.6).view(o, taps)
            W[pre + "mix.b"], W[pre + "mix.a"] = mat(H, width, 2.0), mat(H, width, 2.0)
            W[pre + "mix.A_log"], W[pre + "mix.dt_bias"] = vec(H, -2.0, 0.5), vec(H, -1.0, 1.0)
            W[pre + "mix.norm"] = vec(dv, 0.5, 1.5)
            W[pre + "mix.g"], W[pre + "mix.o"] = mat(H * dv, width, 2.0), mat(width, H * dv)
        elif L["type"] == "mamba2":
            H, dv, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * dv, H * dv + 2 * G * N
            W[pre + "mix.in"] = mat(2 * inner + 2 * G * N + H, width, 2.0)
            W[pre + "mix.conv"] = vec(ch * taps, -0.6, 0.6).view(ch, taps)
            W[pre + "mix.conv.b"] = vec(ch, -0.2, 0.2)
            W[pre + "mix.dt_bias"], W[pre + "mix.A_log"] = vec(H, -1.0, 1.0), vec(H, -2.0, 0.5)
            W[pre + "mix.D"], W[pre + "mix.norm"] = vec(H, 0.5, 1.5), vec(inner, 0.5, 1.5)
            W[pre + "mix.o"] = mat(width, inner)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            ff = L["mlp"]["ff"]
            W[pre + "norm2"], W[pre + "norm2b"] = vec(width, 0.5, 1.5), vec(width, 0.5, 1.5)
            W[pre + "mlp.gate"], W[pre + "mlp.up"] = mat(ff, width, 2.0), mat(ff, width, 2.0)
            W[pre + "mlp.down"] = mat(width, ff)
    return W
