"""Python entry points of the ragged-batch kernels for hybrid layer stacks (``csrc/seq_mixers.cu``): fp32 residual
stream with pre- and post-norms, chunk-local attention with a sink logit, short causal convolutions with carried inputs,
and the linear recurrences of the gated delta rule and of state-space duality.

As in ``ragged_ops``, every wrapper has a PyTorch branch with identical semantics (CPU execution and test oracle of the
kernels); CUDA tensors always take the kernel.  ``seq_info`` is int32 ``[n_seqs, 4]`` = (first row of the sequence in
the batch, rows, tokens already seen, state slot); activations are bf16 or fp32 (``x.dtype``), everything the norms,
softmax and recurrences touch is fp32.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ....native import lib as _lib

_lib.register({
    "sxb_embed_sinusoid": "pppp" "ii" "ff" "i" "p",
    "sxb_resid_norm_step": "pppppp" "l" "i" "f" "i" "p",
    "sxb_qk_norm_append": "p" "l" "ppppppp" "iiiiiii" "f" "ii" "p",
    "sxb_sink_attention": "pppppppp" "iiiiiii" "f" "ii" "p",
    "sxb_sink_attention_atoms": "pppppp" "ii" "p" "iiiiii" "f" "ii" "p",
    "sxb_conv_silu": "p" "l" "pppppp" "iii" "i" "p",
    "sxb_conv_state_update": "p" "l" "pp" "iii" "i" "p",
    "sxb_unit_norm_heads": "p" "l" "iii" "ff" "i" "p",
    "sxb_recurrence_gates": "pp" "l" "pppp" "iii" "i" "p",
    "sxb_linear_recurrence": "pp" "l" "p" "l" "pppppp" "iiiiii" "p",
    "sxb_group_norm_gate": "pp" "l" "p" "i" "p" "iii" "f" "i" "i" "p",
    "sxb_gated_act_rows": "pp" "l" "ii" "i" "p",
})

_ACTS = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3}


def _dt(t: torch.Tensor) -> int:
    return _lib.dtype_code(t.dtype)


def _rows(t: torch.Tensor) -> torch.Tensor:
    """2-D view with unit inner stride (row pitch may exceed the width: column slices of a fused projection)."""
    if t.stride(-1) != 1:
        raise ValueError("expected unit inner stride")
    return t


# ------------------------------------------------------------------------------------------------ embedding
def embed_sinusoid(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, scale: float,
                   base: float = 10000.0) -> torch.Tensor:
    """fp32 ``[T, width]``: ``table[ids] * scale + p`` with ``p[2i] = sin(pos * base^(-2i/width))``, ``p[2i+1] = cos``."""
    T, W = ids.numel(), table.shape[1]
    if table.is_cuda:
        out = torch.empty(T, W, dtype=torch.float32, device=table.device)
        _lib.call("sxb_embed_sinusoid", ids.data_ptr(), positions.data_ptr(), table.data_ptr(), out.data_ptr(), T, W,
                  float(scale), float(base), _dt(table), _lib.stream_ptr())
        return out
    i = torch.arange(W, device=table.device) // 2
    freq = torch.exp2(-(2.0 * i.float() / W) * math.log2(base))
    ang = positions.float()[:, None] * freq[None, :]
    pe = torch.where(torch.arange(W, device=table.device) % 2 == 1, ang.cos(), ang.sin())
    return table[ids.long()].float() * scale + pe


# ------------------------------------------------------------------------------------------------ residual + norms
def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def resid_norm_step(resid: torch.Tensor, y: Optional[torch.Tensor], w_post: Optional[torch.Tensor],
                    extra: Optional[torch.Tensor], w_pre: Optional[torch.Tensor], eps: float,
                    out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """In place on the fp32 residual ``[T, W]``: ``+= rms_norm(y) * w_post`` (if ``y``), ``+= extra`` (if given); returns
    ``rms_norm(residual) * w_pre`` in ``out_dtype`` (None without ``w_pre``).  One pass per row."""
    T, W = resid.shape
    if resid.is_cuda:
        out = torch.empty(T, W, dtype=out_dtype, device=resid.device) if w_pre is not None else None
        code = _lib.dtype_code(out_dtype)
        _lib.call("sxb_resid_norm_step", resid.data_ptr(), _lib.ptr(y), _lib.ptr(w_post), _lib.ptr(extra),
                  _lib.ptr(w_pre), _lib.ptr(out), T, W, float(eps), code, _lib.stream_ptr())
        return out
    if y is not None:
        resid += _rms(y.float(), eps) * w_post.float()
    if extra is not None:
        resid += extra
    if w_pre is None:
        return None
    return (_rms(resid, eps) * w_pre.float()).to(out_dtype)


# ------------------------------------------------------------------------------------------------ attention
def qk_norm_append(qkv: torch.Tensor, bias: Optional[torch.Tensor], kcache: torch.Tensor, vcache: torch.Tensor,
                   tok_seq: torch.Tensor, tok_pos: torch.Tensor, tables: torch.Tensor, Hq: int, G: int, d: int, dv: int,
                   eps: float, normalize: bool = True) -> torch.Tensor:
    """``qkv`` ``[T, Hq*d + G*d + G*dv]`` (+ ``bias``): q and k heads are divided by their root mean square (fp32), q is
    returned as fp32 ``[T, Hq, d]``, k and v are written to the paged caches ``[pages, block, G, d]`` /
    ``[pages, block, G, dv]`` at every token's (sequence, position)."""
    T = qkv.shape[0]
    bs = kcache.shape[1]
    if qkv.is_cuda:
        q = torch.empty(T, Hq, d, dtype=torch.float32, device=qkv.device)
        _lib.call("sxb_qk_norm_append", _rows(qkv).data_ptr(), qkv.stride(0), _lib.ptr(bias), q.data_ptr(),
                  kcache.data_ptr(), vcache.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), tables.data_ptr(), T,
                  tables.shape[1], bs, Hq, G, d, dv, float(eps), int(normalize), _dt(qkv), _lib.stream_ptr())
        return q
    x = qkv[:, : (Hq + G) * d + G * dv].float() + (bias.float() if bias is not None else 0.0)
    q = x[:, : Hq * d].reshape(T, Hq, d)
    k = x[:, Hq * d: (Hq + G) * d].reshape(T, G, d)
    v = x[:, (Hq + G) * d:].reshape(T, G, dv)
    if normalize:
        q, k = _rms(q, eps), _rms(k, eps)
    page = tables[tok_seq.long(), (tok_pos // bs).long()].long()
    off = (tok_pos % bs).long()
    kcache[page, off] = k.to(kcache.dtype)
    vcache[page, off] = v.to(vcache.dtype)
    return q.contiguous()


SHORT_ATOM = 16          # atoms of at most this many queries run one warp per (query, head)


def tiles_supported(d: int, dv: int) -> bool:
    return d % 4 == 0 and dv % 4 == 0 and d <= 256 and dv <= 256


def sink_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, sink: Optional[torch.Tensor],
                   tok_seq: torch.Tensor, tok_pos: torch.Tensor, tables: torch.Tensor, scale: float, chunk: int,
                   out_dtype: torch.dtype, atoms: Optional[torch.Tensor] = None, n_long: int = 0) -> torch.Tensor:
    """Softmax attention of each token (fp32 ``q`` ``[T, Hq, d]``) over the cached keys ``lo..pos`` of its sequence,
    ``lo`` = first position of the token's chunk of ``chunk`` positions (0: plain causal).  ``sink`` (fp32 ``[Hq]``)
    adds ``exp(sink[h])`` to the denominator.  Returns ``[T, Hq * dv]``.

    With the batch's attention ``atoms`` (longest first) of which the first ``n_long`` hold more than
    :data:`SHORT_ATOM` queries, those run the tiled kernel (64 queries per CTA, K/V tiles shared by them) and the rest
    one warp per (query, head); without atoms every token takes the latter."""
    T, Hq, d = q.shape
    bs, G, dv = kcache.shape[1], kcache.shape[2], vcache.shape[3]
    if q.is_cuda:
        if kcache.dtype != out_dtype or vcache.dtype != out_dtype:
            raise ValueError("the caches and the output share one activation dtype")
        out = torch.empty(T, Hq * dv, dtype=out_dtype, device=q.device)
        if atoms is not None and n_long > 0 and tiles_supported(d, dv):
            _lib.call("sxb_sink_attention_atoms", q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), _lib.ptr(sink),
                      out.data_ptr(), atoms.data_ptr(), atoms.shape[0], int(n_long), tables.data_ptr(), tables.shape[1],
                      bs, Hq, G, d, dv, float(scale), int(chunk), _lib.dtype_code(out_dtype), _lib.stream_ptr())
            return out
        _lib.call("sxb_sink_attention", q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), _lib.ptr(sink),
                  out.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), tables.data_ptr(), T, tables.shape[1], bs, Hq,
                  G, d, dv, float(scale), int(chunk), _lib.dtype_code(out_dtype), _lib.stream_ptr())
        return out
    out = torch.empty(T, Hq, dv, dtype=torch.float32)
    rep = Hq // G
    for t in range(T):
        pos = int(tok_pos[t])
        lo = (pos // chunk) * chunk if chunk > 0 else 0
        js = torch.arange(lo, pos + 1)
        page = tables[int(tok_seq[t]), (js // bs)].long()
        k = kcache[page, js % bs].float().repeat_interleave(rep, dim=1)      # [n, Hq, d]
        v = vcache[page, js % bs].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", q[t], k) * scale
        if sink is not None:
            s = torch.cat([s, sink.float()[:, None]], dim=1)
        p = torch.softmax(s, dim=-1)[:, : js.numel()]
        out[t] = torch.einsum("hn,nhd->hd", p, v)
    return out.reshape(T, Hq * dv).to(out_dtype)


# ------------------------------------------------------------------------------------------------ short convolution
def conv_silu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              seq_info: torch.Tensor, tok_seq: torch.Tensor) -> torch.Tensor:
    """Short causal per-channel filter + SiLU over the rows ``x`` ``[T, C]`` of a ragged batch; ``w`` ``[C, taps]`` (last
    column multiplies the current token), inputs before this batch's rows come from ``state`` ``[slots, taps-1, C]``,
    inputs before a sequence's start are zero.  Returns fp32 ``[T, C]``; call :func:`conv_state_update` afterwards."""
    T, C = x.shape
    taps = w.shape[1]
    if x.is_cuda:
        out = torch.empty(T, C, dtype=torch.float32, device=x.device)
        _lib.call("sxb_conv_silu", _rows(x).data_ptr(), x.stride(0), w.data_ptr(), _lib.ptr(bias), state.data_ptr(),
                  seq_info.data_ptr(), tok_seq.data_ptr(), out.data_ptr(), T, C, taps, _dt(x), _lib.stream_ptr())
        return out
    out = torch.empty(T, C, dtype=torch.float32)
    wf = w.float()
    for first, n, seen, slot in seq_info.tolist():
        hist = state[slot].float() if seen > 0 else torch.zeros(taps - 1, C)
        if 0 < seen < taps - 1:
            hist = hist.clone()
            hist[: taps - 1 - seen] = 0
        full = torch.cat([hist, x[first: first + n].float()], dim=0)
        acc = torch.zeros(n, C)
        for j in range(taps):
            acc += wf[:, taps - 1 - j] * full[taps - 1 - j: taps - 1 - j + n]
        if bias is not None:
            acc += bias.float()
        out[first: first + n] = torch.nn.functional.silu(acc)
    return out


def conv_state_update(x: torch.Tensor, state: torch.Tensor, seq_info: torch.Tensor) -> None:
    """Every sequence's slot of ``state`` ``[slots, taps-1, C]`` becomes the last ``taps-1`` rows of (its carried inputs
    followed by this batch's rows of ``x``)."""
    keep = state.shape[1]
    if keep == 0:
        return
    C = x.shape[1]
    if x.is_cuda:
        _lib.call("sxb_conv_state_update", _rows(x).data_ptr(), x.stride(0), state.data_ptr(), seq_info.data_ptr(),
                  seq_info.shape[0], C, keep + 1, _dt(x), _lib.stream_ptr())
        return
    for first, n, seen, slot in seq_info.tolist():
        hist = state[slot] if seen > 0 else torch.zeros_like(state[slot])
        if 0 < seen < keep:
            hist = hist.clone()
            hist[: keep - seen] = 0
        state[slot] = torch.cat([hist, x[first: first + n].to(state.dtype)], dim=0)[-keep:]


def unit_norm_heads(x: torch.Tensor, col0: int, n_heads: int, dim: int, mult: float, eps: float) -> None:
    """In place on fp32 rows: each head ``x[:, col0 + h*dim : col0 + (h+1)*dim]`` becomes ``x * mult / sqrt(sum x^2 + eps)``."""
    T = x.shape[0]
    if x.is_cuda:
        _lib.call("sxb_unit_norm_heads", _rows(x).data_ptr(), x.stride(0), col0, n_heads, dim, float(mult), float(eps), T,
                  _lib.stream_ptr())
        return
    v = x[:, col0: col0 + n_heads * dim].reshape(T, n_heads, dim)
    x[:, col0: col0 + n_heads * dim] = (v * mult / torch.sqrt(v.pow(2).sum(-1, keepdim=True) + eps)).reshape(T, -1)


def recurrence_gates(a_raw: torch.Tensor, b_raw: Optional[torch.Tensor], A_log: torch.Tensor, dt_bias: torch.Tensor,
                     mode: str):
    """fp32 ``(decay, beta)`` ``[T, H]`` of a linear recurrence from raw projections ``[T, H]`` (column slices allowed).
    ``"delta"``: ``beta = sigmoid(b_raw)``, ``decay = exp(-exp(A_log) * softplus(a_raw + dt_bias))``.
    ``"ssd"``: ``dt = softplus(a_raw + dt_bias)``, ``beta = dt``, ``decay = exp(-exp(A_log) * dt)``."""
    T, H = a_raw.shape
    if a_raw.is_cuda:
        decay = torch.empty(T, H, dtype=torch.float32, device=a_raw.device)
        beta = torch.empty_like(decay)
        b = a_raw if b_raw is None else b_raw
        if b.stride(0) != a_raw.stride(0):
            raise ValueError("a_raw and b_raw must share their row pitch")
        _lib.call("sxb_recurrence_gates", _rows(a_raw).data_ptr(), _rows(b).data_ptr(), a_raw.stride(0),
                  A_log.data_ptr(), dt_bias.data_ptr(), decay.data_ptr(), beta.data_ptr(), H, T,
                  0 if mode == "delta" else 1, _dt(a_raw), _lib.stream_ptr())
        return decay, beta
    dt = torch.nn.functional.softplus(a_raw.float() + dt_bias.float(), threshold=30.0)
    decay = torch.exp(-torch.exp(A_log.float()) * dt)
    beta = torch.sigmoid(b_raw.float()) if mode == "delta" else dt
    return decay, beta


def linear_recurrence(kvec: torch.Tensor, qvec: torch.Tensor, val: torch.Tensor, decay: torch.Tensor,
                      beta: torch.Tensor, skip: Optional[torch.Tensor], state: torch.Tensor, seq_info: torch.Tensor,
                      H: int, G: int, n: int, dv: int, delta: bool) -> torch.Tensor:
    """Per sequence and head, rows in order: ``S <- decay S``; ``u = beta (v - S^T k)`` (``delta``) or ``beta v``;
    ``S <- S + k u^T``; ``o = S^T q (+ skip[h] v)``.  ``kvec`` / ``qvec`` fp32 ``[T, G*n]`` and ``val`` fp32
    ``[T, H*dv]`` may be column slices (``kvec`` and ``qvec`` with one row pitch); ``state`` fp32 ``[slots, H, dv, n]`` is
    read (zero for a sequence that has seen no token) and written back.  Returns fp32 ``[T, H*dv]``."""
    T = val.shape[0]
    if val.is_cuda:
        if kvec.stride(0) != qvec.stride(0):
            raise ValueError("kvec and qvec must share their row pitch")
        out = torch.empty(T, H * dv, dtype=torch.float32, device=val.device)
        _lib.call("sxb_linear_recurrence", _rows(kvec).data_ptr(), _rows(qvec).data_ptr(), kvec.stride(0),
                  _rows(val).data_ptr(), val.stride(0), decay.data_ptr(), beta.data_ptr(), _lib.ptr(skip),
                  state.data_ptr(), out.data_ptr(), seq_info.data_ptr(), seq_info.shape[0], H, G, n, dv, int(delta),
                  _lib.stream_ptr())
        return out
    out = torch.empty(T, H, dv, dtype=torch.float32)
    rep = H // G
    for first, rows, seen, slot in seq_info.tolist():
        S = state[slot].clone() if seen > 0 else torch.zeros_like(state[slot])           # [H, dv, n]
        for t in range(first, first + rows):
            k = kvec[t].reshape(G, n).repeat_interleave(rep, dim=0)                      # [H, n]
            q = qvec[t].reshape(G, n).repeat_interleave(rep, dim=0)
            v = val[t].reshape(H, dv)
            S = S * decay[t][:, None, None]
            u = beta[t][:, None] * ((v - torch.einsum("hvn,hn->hv", S, k)) if delta else v)
            S = S + u[:, :, None] * k[:, None, :]
            o = torch.einsum("hvn,hn->hv", S, q)
            if skip is not None:
                o = o + skip.float()[:, None] * v
            out[t] = o
        state[slot] = S
    return out.reshape(T, H * dv)


def group_norm_gate(y: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, group_size: int, eps: float,
                    gate_first: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """RMS norm over groups of ``group_size`` channels of fp32 ``y`` ``[T, C]`` with a SiLU gate ``[T, C]`` (column slice
    allowed) and a weight that repeats along the row.  ``gate_first``: ``norm(y * silu(gate)) * w``; else
    ``norm(y) * w * silu(gate)``."""
    T, C = y.shape
    if y.is_cuda:
        out = torch.empty(T, C, dtype=out_dtype, device=y.device)
        _lib.call("sxb_group_norm_gate", y.data_ptr(), _rows(gate).data_ptr(), gate.stride(0), w.data_ptr(), w.numel(),
                  out.data_ptr(), T, C, group_size, float(eps), int(gate_first), _lib.dtype_code(out_dtype),
                  _lib.stream_ptr())
        return out
    sg = torch.nn.functional.silu(gate.float())
    wf = w.float().repeat(C // w.numel())
    z = y * sg if gate_first else y
    z = _rms(z.reshape(T, C // group_size, group_size), eps).reshape(T, C) * wf
    return (z if gate_first else z * sg).to(out_dtype)


def gated_act_rows(x: torch.Tensor, act: str = "gelu") -> torch.Tensor:
    """``act(x[:, :F]) * x[:, F:]`` for rows of any width, bf16 or fp32 (``gelu`` is the tanh form)."""
    T, F2 = x.shape
    Fh = F2 // 2
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty(T, Fh, dtype=x.dtype, device=x.device)
        _lib.call("sxb_gated_act_rows", x.data_ptr(), out.data_ptr(), T, Fh, _ACTS[act], _dt(x), _lib.stream_ptr())
        return out
    g, u = x[:, :Fh].float(), x[:, Fh:].float()
    a = {"gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "silu": torch.nn.functional.silu,
         "relu": torch.relu, "identity": lambda t: t}[act](g)
    return (a * u).to(x.dtype)
