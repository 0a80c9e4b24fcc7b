"""Kekopel: a decoder-only stack of post-scaled layers (``hybrid_model.py``, block form ``"post_scaled"``).  ``config.json``
lists every layer with its token mixer -- ``latent_attention`` (queries and keys / values through normalised latents, a
rotated key part shared by all heads, sliding window, sink logit) or ``mlstm`` (matrix-memory LSTM) -- the mixer's sizes
and its feed-forward: dense (squared ReLU, biases), a mixture of gated experts (sigmoid scores, the score scales the
expert's input) or none.  Every sublayer reads the stream through a short causal filter with a skip path, its output is
normalised with one gain and scaled per channel, and every layer hands on a learned mixture of all results so far.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1|norm2`` (one number each),
``l<i>.ls1|ls2``, ``l<i>.canon1|canon2`` (``[width, taps]``), ``l<i>.dwa`` (``i + 2`` mixture weights), ``l<i>.mix.*``
(latent attention: ``dq``, ``dq.norm``, ``uq``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``sink``, ``o``; mlstm: ``q``, ``k``,
``v``, ``g``, ``i``, ``i.b``, ``f``, ``f.b``, ``norm``, ``o``) and ``l<i>.mlp.*`` (dense: ``up``, ``up.b``, ``down``,
``down.b``; experts: ``router``, ``e<j>.gate|up|down``).  Linear weights are ``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..fomalix.policy import _cfg_dict
from ..hybrid_model import DSHybridModel, HybridLayerSpec, HybridSpec, pad_rows
from ..inference_policy_base import InferenceV2Policy
from ..inference_transformer_base import LayerWeights


class KekopelPolicy(InferenceV2Policy):

    def spec(self, model_config) -> HybridSpec:
        cfg = _cfg_dict(model_config)
        layers = []
        for L in cfg["layers"]:
            m, kind = L["mixer"], L["type"]
            mlp = L.get("mlp")
            ff: Dict[str, Any] = {}
            if mlp is not None:
                if mlp["kind"] == "dense":
                    ff = dict(ff_dim=int(mlp["ff"]), ff_kind="biased", ff_activation="relu_sq")
                elif mlp["kind"] == "moe":
                    ff = dict(ff_dim=int(mlp["expert"]["ff"]), ff_kind="moe", ff_activation="silu",
                              n_experts=int(mlp["router"]["experts"]), top_k=int(mlp["router"]["top"]),
                              moe_score="sigmoid", moe_weight_input=True)
                else:
                    raise ValueError(f"Unsupported feed-forward kind {mlp['kind']!r}")
            if kind == "latent_attention":
                mask, rot = m.get("mask") or {}, m.get("rot") or {}
                layers.append(HybridLayerSpec(
                    kind="latent_attention", n_heads=int(m["heads"]), n_heads_kv=1, key_dim=int(m["dim"]),
                    value_dim=int(m["vdim"]), attn_scale=float(m["scale"]), window=int(mask.get("size", 0)), sink=True,
                    q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), rot_dim=int(m["rot_dim"]),
                    rot_dims=int(rot.get("dims", m["rot_dim"])), rot_base=float(rot.get("base", 10000.0)), **ff))
            elif kind == "mlstm":
                layers.append(HybridLayerSpec(kind="mlstm", n_heads=int(m["heads"]), n_heads_kv=int(m["heads"]),
                                              key_dim=int(m["dim"]), value_dim=int(m["vdim"]),
                                              gate_cap=float(m["gate_cap"]), **ff))
            else:
                raise ValueError(f"Unknown mixer type {kind!r}")
        dt = getattr(model_config, "torch_dtype", None)
        return HybridSpec(vocab_size=int(cfg["vocab"]), model_dim=int(cfg["width"]), layers=layers,
                          norm_eps=float(cfg["norm"]["eps"]), sinusoid_base=None, block_form="post_scaled",
                          input_conv_taps=int(cfg["canon"]["taps"]), depth_mix=True,
                          dtype=dt if dt in (torch.bfloat16, torch.float32) else torch.bfloat16)

    # ------------------------------------------------------------------------------------------ weights
    def load_weights(self) -> Dict:
        if self._weights is not None:
            return self._weights
        spec = self.resolved_spec()
        dev, dt = self._device(), spec.dtype
        raw = {name: t.detach() for name, t in self._checkpoint_engine.parameters()}
        used = set()

        def get(name, dtype=dt):
            used.add(name)
            return raw[name].to(dev, dtype).contiguous()

        def cat(names, dtype=dt):
            return torch.cat([get(n, dtype) for n in names], dim=0)

        f32 = torch.float32
        weights: Dict[str, Any] = {"embed": get("embed"), "final_norm_w": get("final.norm", f32).reshape(1),
                                   "unembed": pad_rows(get("head")), "layers": []}
        for i, L in enumerate(spec.layers):
            p, lw = f"l{i}.", LayerWeights()
            lw["norm1"], lw["ls1"], lw["conv1"] = get(p + "norm1", f32).reshape(1), get(p + "ls1", f32), get(p + "canon1")
            lw["depth_mix"] = get(p + "dwa", f32)
            if lw["depth_mix"].numel() != i + 2:
                raise ValueError(f"{p}dwa has {lw['depth_mix'].numel()} weights, layer {i} mixes {i + 2} streams")
            m = p + "mix."
            if L.kind == "latent_attention":
                H, d, r, dv = L.n_heads, L.key_dim, L.kv_rank, L.value_dim
                lw["w_in"] = pad_rows(cat([m + "dq", m + "dkv"]))
                lw["q_norm"], lw["kv_norm"] = get(m + "dq.norm"), get(m + "dkv.norm")
                lw["w_uq"] = get(m + "uq")
                lw["w_uk"] = get(m + "uk").view(H, d, r).contiguous()
                lw["w_uv_t"] = get(m + "uv").view(H, dv, r).transpose(1, 2).contiguous()
                lw["sink"] = get(m + "sink", f32)
            else:
                lw["w_in"] = pad_rows(cat([m + "q", m + "k", m + "v", m + "g", m + "i", m + "f"]))
                lw["gate_bias_i"], lw["gate_bias_f"] = get(m + "i.b", f32), get(m + "f.b", f32)
                lw["norm"] = get(m + "norm")
            lw["wo"] = get(m + "o")
            if L.ff_dim > 0:
                lw["norm2"], lw["ls2"] = get(p + "norm2", f32).reshape(1), get(p + "ls2", f32)
                lw["conv2"] = get(p + "canon2")
                f = p + "mlp."
                if L.ff_kind == "moe":
                    lw["moe_gate"] = get(f + "router", f32)
                    lw["moe_w1"] = torch.stack([cat([f"{f}e{e}.gate", f"{f}e{e}.up"]) for e in range(L.n_experts)])
                    lw["moe_w2"] = torch.stack([get(f"{f}e{e}.down") for e in range(L.n_experts)]).contiguous()
                else:
                    lw["w_up"], lw["b_up"] = get(f + "up"), get(f + "up.b")
                    lw["w_down"], lw["b_down"] = get(f + "down"), get(f + "down.b")
            weights["layers"].append(lw)
        self.container_map.set_unmapped_params([n for n in raw if n not in used])
        self._weights = weights
        return weights

    def build_model(self, engine_config, mp_group=None, state_manager=None) -> DSHybridModel:
        self._engine_config = engine_config
        if mp_group is not None:
            self._mp_group = mp_group
        spec = self.resolved_spec()
        model = DSHybridModel(spec, self.load_weights(), engine_config, state_manager, self._mp_group)
        model.model_config = self._model_config
        return model
