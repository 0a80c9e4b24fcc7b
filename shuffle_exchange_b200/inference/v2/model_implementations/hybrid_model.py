"""Ragged-batch model for hybrid layer stacks: every layer names its own token mixer — attention over the paged cache, a
gated-delta-rule recurrence or a state-space-duality recurrence — and may or may not have a feed-forward; a span of
layers can be executed several times in a row with the same weights, every execution with its own cache or state.

The stack is data (:class:`HybridSpec`), as :class:`~.inference_transformer_base.ArchSpec` is for the uniform
transformer family; per-architecture policies (``fomalix/policy.py``) fill it from a checkpoint's configuration and fuse
the checkpoint's tensors into the projection layouts the mixer modules declare.

Numerics: the residual stream, norms, softmax, recurrences and their gates are fp32; projections, short convolutions'
inputs, the KV cache and the sublayer outputs use ``spec.dtype`` (bf16 when serving; fp32 evaluates everything in
32-bit, matrix products included).  Per layer execution: ``x += post_norm(mixer(pre_norm(x)))`` then, if the layer has a
feed-forward, ``x += post_norm(ff(pre_norm(x)))``; closing one sublayer and opening the next is one kernel
(``fp32_sandwich_rms``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ....ops import functional as F
from ..config_v2 import RaggedInferenceEngineConfig
from ..inference_utils import ActivationType, DtypeEnum, NormTypeEnum, ceil_div
from ..kernels import mixer_ops as M
from ..modules import heuristics
from ..modules.configs import (DSEmbeddingsConfig, DSLinearConfig, DSNormConfig, DSRecurrentMixerConfig,
                               DSSelfAttentionConfig, MaskingType, PositionalEmbeddingType)
from ..ragged.kv_cache import KVCacheConfig
from ..ragged.state_pool import StatePoolConfig
from .inference_transformer_base import DSInferenceModelBase, LayerWeights


@dataclass
class HybridLayerSpec:
    kind: str                                   # "attention" | "delta" | "ssd"
    n_heads: int
    n_heads_kv: int                             # key/value heads (attention), key/query heads (delta), groups (ssd)
    key_dim: int                                # query/key head size, or state size per group (ssd)
    value_dim: int
    attn_scale: float = 1.0
    chunk_size: int = 0                         # attention: 0 = plain causal, else chunk-local
    qk_unit_rms: bool = False
    sink: bool = False
    qkv_bias: bool = False
    conv_taps: int = 1
    norm_groups: int = 1
    ff_dim: int = 0                             # 0: the layer has no feed-forward
    ff_activation: str = "gelu"


@dataclass
class HybridSpec:
    vocab_size: int
    model_dim: int
    layers: List[HybridLayerSpec]
    norm_eps: float = 1e-5
    embed_scale: float = 1.0
    sinusoid_base: Optional[float] = 10000.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    dtype: torch.dtype = torch.bfloat16
    max_seq_len: int = 1 << 20

    def runs(self) -> List[Tuple[int, bool]]:
        """[(layer index, whether a repeated pass starts here)] in execution order: the layers before the span once,
        the span ``loop_times`` times, the rest once."""
        out = [(i, False) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            out += [(i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, False) for i in range(self.loop_stop, len(self.layers))]


def pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Zero rows up to a multiple of 8 outputs, so that a fused projection of any width stays on the tensor-core GEMM."""
    extra = (-w.shape[0]) % multiple
    if extra == 0:
        return w.contiguous()
    return torch.cat([w, w.new_zeros(extra, *w.shape[1:])], dim=0).contiguous()


class DSHybridModel(DSInferenceModelBase):
    """``weights``: ``{"embed", "final_norm_w", "unembed", "layers": [LayerWeights]}``; a layer has ``norm1``, ``norm1b``
    (+ ``norm2``, ``norm2b``, ``w_gate_up`` ``[2F, W]``, ``w_down`` with a feed-forward), ``w_in`` (the mixer's fused
    projection, rows in the order of the mixer module's ``projection layout``), ``wo``, and per kind: attention ``b_in``,
    ``sink`` (fp32); delta ``conv_w``, ``A_log``, ``dt_bias`` (fp32), ``norm``; ssd ``conv_w``, ``conv_b``, ``A_log``,
    ``dt_bias``, ``D`` (fp32), ``norm``."""

    def __init__(self, spec: HybridSpec, weights: Dict, engine_config: RaggedInferenceEngineConfig, state_manager=None,
                 base_mp_group=None) -> None:
        super().__init__()
        if base_mp_group is not None:
            import torch.distributed as dist
            if dist.get_world_size(base_mp_group) > 1:
                raise NotImplementedError("hybrid stacks run on one tensor-parallel rank")
        self.spec = spec
        self.weights = weights
        self._engine_config = engine_config or RaggedInferenceEngineConfig()
        self.state_manager = state_manager
        self.tp_rank, self.tp_size = 0, 1
        self.flattened_params = self.flattened_param_metadata = None
        if spec.dtype == torch.float32:
            torch.backends.cuda.matmul.allow_tf32 = False          # exact evaluation: no reduced-precision products
            torch.backends.cudnn.allow_tf32 = False
        self._runs = spec.runs()
        # which cache / state entries every execution of a layer uses
        self._cache_of_run: Dict[int, int] = {}
        self._state_of_run: Dict[int, Tuple[int, int]] = {}
        self._build_modules()

    # ------------------------------------------------------------------------------------------ construction
    def _build_modules(self) -> None:
        s, ec = self.spec, self._engine_config
        sm = ec.state_manager
        dt, mt = DtypeEnum(s.dtype), sm.max_ragged_batch_size
        self.embed = heuristics.instantiate_embed(DSEmbeddingsConfig(
            max_tokens=mt, residual_dtype=DtypeEnum.fp32, embedding_dim=s.model_dim, scale=s.embed_scale,
            sinusoid_base=s.sinusoid_base), ec)
        self.norm = heuristics.instantiate_sandwich_norm(DSNormConfig(
            max_tokens=mt, type=NormTypeEnum.RMSNorm, channels=s.model_dim, residual_dtype=DtypeEnum.fp32,
            input_dtype=dt, output_dtype=dt, eps=s.norm_eps), ec)
        self.linear = heuristics.instantiate_linear(DSLinearConfig(
            max_tokens=mt, in_channels=s.model_dim, out_channels=s.model_dim, input_dtype=dt, output_dtype=dt), ec)
        self.mixers = []
        for L in s.layers:
            if L.kind == "attention":
                mod = heuristics.instantiate_attention(DSSelfAttentionConfig(
                    max_tokens=mt, n_heads_q=L.n_heads, n_heads_kv=L.n_heads_kv, head_size=L.key_dim,
                    v_head_size=L.value_dim, max_sequences=sm.max_ragged_sequence_count, scale_factor=L.attn_scale,
                    input_dtype=dt, output_dtype=dt,
                    masking_type=MaskingType.chunked if L.chunk_size > 0 else MaskingType.causal,
                    masking_args={"size": L.chunk_size} if L.chunk_size > 0 else {},
                    positional_embedding_type=PositionalEmbeddingType.none, qk_unit_rms=L.qk_unit_rms,
                    qk_norm_eps=s.norm_eps, sink=L.sink), ec)
            else:
                mod = heuristics.instantiate_recurrent_mixer(DSRecurrentMixerConfig(
                    max_tokens=mt, kind=L.kind, model_dim=s.model_dim, n_heads=L.n_heads, n_heads_kv=L.n_heads_kv,
                    key_dim=L.key_dim, value_dim=L.value_dim, conv_taps=L.conv_taps, norm_groups=L.norm_groups,
                    eps=s.norm_eps, max_sequences=sm.max_ragged_sequence_count, input_dtype=dt, output_dtype=dt), ec)
            self.mixers.append(mod)
        n_cache = 0
        self._state_cfg = StatePoolConfig()
        shapes = []
        for r, (li, _) in enumerate(self._runs):
            L = s.layers[li]
            if L.kind == "attention":
                self._cache_of_run[r] = n_cache
                shapes.append((L.n_heads_kv, L.key_dim, L.value_dim))
                n_cache += 1
            else:
                (conv_shape, conv_dt), (mat_shape, mat_dt) = self.mixers[li].state_shapes()
                self._state_of_run[r] = (self._state_cfg.add(conv_shape, conv_dt), self._state_cfg.add(mat_shape, mat_dt))
        self._cache_shapes = tuple(shapes)

    # ------------------------------------------------------------------------------------------ properties
    @property
    def num_layers(self): return len(self.spec.layers)
    @property
    def model_dim(self): return self.spec.model_dim
    @property
    def vocab_size(self): return self.spec.vocab_size
    @property
    def activation_dtype(self): return DtypeEnum(self.spec.dtype)
    @property
    def max_sequence_length(self): return self.spec.max_seq_len

    # ------------------------------------------------------------------------------------------ memory planning
    def kv_cache_config(self, block_size: int) -> KVCacheConfig:
        """One (keys, values) pair per EXECUTION of an attention layer: a repeated layer keeps a cache per pass."""
        return KVCacheConfig(block_size=block_size, cache_shape=(len(self._cache_shapes), 1, 1),
                             cache_dtype=self.spec.dtype, layer_shapes=self._cache_shapes)

    def state_pool_config(self) -> StatePoolConfig:
        """Carried convolution inputs and matrix state per execution of a recurrent layer."""
        return self._state_cfg

    def get_kv_requirements(self, sequence, max_new_tokens: int, max_new_blocks: int):
        bs = self.state_manager.kv_block_size
        total = sequence.seen_tokens + max_new_tokens
        need = ceil_div(total, bs) - sequence.cur_allocated_blocks
        if need > max_new_blocks:
            fit = (sequence.cur_allocated_blocks + max_new_blocks) * bs - sequence.seen_tokens
            return max(0, fit), max_new_blocks
        return max_new_tokens, max(0, need)

    def get_remaining_block_capacity(self, sequence) -> int:
        return sequence.cur_allocated_blocks * self.state_manager.kv_block_size - sequence.seen_tokens

    def maybe_allocate_kv(self, sequence, n_new_tokens: int) -> None:
        _, need = self.get_kv_requirements(sequence, n_new_tokens, self.state_manager.free_blocks)
        if need > 0:
            sequence.extend_kv_cache(self.state_manager.allocate_blocks(need))

    def maybe_free_kv(self, sequence) -> None:
        """Chunk-local layers could return the pages before the current chunk; every page is kept."""

    # ------------------------------------------------------------------------------------------ forward
    def _feed_forward(self, L: HybridLayerSpec, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        h = self.linear(x, lw.w_gate_up)
        if h.is_cuda and h.dtype == torch.bfloat16 and L.ff_dim % 8 == 0:
            h = F.gated_act(h, L.ff_activation)
        else:
            h = M.gated_act_rows(h, L.ff_activation)
        return self.linear(h, lw.w_down)

    def _mixer(self, r: int, li: int, lw: LayerWeights, x: torch.Tensor, batch) -> torch.Tensor:
        L, mod, sm = self.spec.layers[li], self.mixers[li], self.state_manager
        proj = self.linear(x, lw.w_in)
        if L.kind == "attention":
            ctx = mod(proj, sm.get_cache(self._cache_of_run[r]), batch, None, lw.b_in, lw.sink)
        else:
            ci, si = self._state_of_run[r]
            ctx = mod(proj, lw, (sm.get_state(ci), sm.get_state(si)), batch)
        return self.linear(ctx, lw.wo)

    @torch.no_grad()
    def forward(self, batch) -> torch.Tensor:
        W, s = self.weights, self.spec
        resid = self.embed(batch, W["embed"])
        first = resid.clone() if any(again for _, again in self._runs) else None
        y = post = None                     # output of the last sublayer and its post-norm weight, not yet added
        for r, (li, again) in enumerate(self._runs):
            lw, L = W["layers"][li], s.layers[li]
            _, x = self.norm(resid, y, lw.norm1, None, post, first if again else None)
            y, post = self._mixer(r, li, lw, x, batch), lw.norm1b
            if L.ff_dim > 0:
                _, x = self.norm(resid, y, lw.norm2, None, post, None)
                y, post = self._feed_forward(L, lw, x), lw.norm2b
        rows = batch.last_token_index().long()
        if rows.numel() == 0:               # a step that only advances caches and states
            return torch.empty(0, s.vocab_size, dtype=torch.float32, device=resid.device)
        resid = resid.index_select(0, rows)
        _, x = self.norm(resid, None if y is None else y.index_select(0, rows), W["final_norm_w"], None, post, None)
        return self.linear(x, W["unembed"])[:, : s.vocab_size].float()
