"""Fomalix: a decoder-only stack whose ``config.json`` lists every layer with its token mixer (``attention``, ``delta``,
``mamba2``), the mixer's sizes and an optional dense feed-forward, plus a span of layers (``loop``) that is executed
several times.  Scaled token embedding + sinusoidal positions, RMS norms before and after every sublayer, no rotation.

Checkpoint names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.*`` (attention: ``q|k|v`` with ``.b`` biases, ``sink``, ``o``; delta: ``q|k|v`` with ``.conv`` filters, ``b``,
``a``, ``A_log``, ``dt_bias``, ``g``, ``norm``, ``o``; mamba2: ``in``, ``conv``, ``conv.b``, ``dt_bias``, ``A_log``, ``D``,
``norm``, ``o``) and ``l<i>.mlp.gate|up|down``.  Linear weights are ``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..hybrid_model import DSHybridModel, HybridLayerSpec, HybridSpec, pad_rows
from ..inference_policy_base import InferenceV2Policy
from ..inference_transformer_base import LayerWeights


def _cfg_dict(model_config: Any) -> Dict:
    if isinstance(model_config, dict):
        return model_config
    raw = getattr(model_config, "raw", None)
    if isinstance(raw, dict):
        return raw
    return model_config.to_dict()


class FomalixPolicy(InferenceV2Policy):

    def spec(self, model_config) -> HybridSpec:
        cfg = _cfg_dict(model_config)
        layers = []
        for L in cfg["layers"]:
            m, kind = L["mixer"], L["type"]
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"Unsupported feed-forward kind {mlp.get('kind')!r}")
            ff = int(mlp["ff"]) if mlp is not None else 0
            if kind == "attention":
                mask = m.get("mask") or {}
                layers.append(HybridLayerSpec(
                    kind="attention", n_heads=m["heads"], n_heads_kv=m["kv_heads"], key_dim=m["dim"],
                    value_dim=m["vdim"], attn_scale=float(m["scale"]), chunk_size=int(mask.get("size", 0)),
                    qk_unit_rms=True, sink=True, qkv_bias=True, ff_dim=ff))
            elif kind == "delta":
                layers.append(HybridLayerSpec(kind="delta", n_heads=m["heads"], n_heads_kv=m["kv_heads"],
                                              key_dim=m["dim"], value_dim=m["vdim"], conv_taps=int(m["conv"]), ff_dim=ff))
            elif kind == "mamba2":
                layers.append(HybridLayerSpec(kind="ssd", n_heads=m["heads"], n_heads_kv=m["groups"],
                                              key_dim=m["state"], value_dim=m["vdim"], conv_taps=int(m["conv"]),
                                              norm_groups=int(m.get("norm_groups", 1)), ff_dim=ff))
            else:
                raise ValueError(f"Unknown mixer type {kind!r}")
        loop = cfg.get("loop") or {}
        dt = getattr(model_config, "torch_dtype", None)
        return HybridSpec(vocab_size=cfg["vocab"], model_dim=cfg["width"], layers=layers,
                          norm_eps=float(cfg["norm"]["eps"]), embed_scale=float(cfg["embedding"]["scale"]),
                          loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                          loop_times=int(loop.get("times", 1)),
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

        weights: Dict[str, Any] = {"embed": get("embed"), "final_norm_w": get("final.norm"),
                                   "unembed": pad_rows(get("head")), "layers": []}
        for i, L in enumerate(spec.layers):
            p, lw = f"l{i}.", LayerWeights()
            lw["norm1"], lw["norm1b"] = get(p + "norm1"), get(p + "norm1b")
            m = p + "mix."
            if L.kind == "attention":
                lw["w_in"] = pad_rows(cat([m + "q", m + "k", m + "v"]))
                lw["b_in"] = cat([m + "q.b", m + "k.b", m + "v.b"])
                lw["sink"] = get(m + "sink", torch.float32)
            elif L.kind == "delta":
                lw["w_in"] = pad_rows(cat([m + "q", m + "k", m + "v", m + "g", m + "b", m + "a"]))
                lw["conv_w"] = cat([m + "q.conv", m + "k.conv", m + "v.conv"])
                lw["A_log"], lw["dt_bias"] = get(m + "A_log", torch.float32), get(m + "dt_bias", torch.float32)
                lw["norm"] = get(m + "norm")
            else:
                lw["w_in"] = pad_rows(get(m + "in"))
                lw["conv_w"], lw["conv_b"] = get(m + "conv"), get(m + "conv.b")
                lw["A_log"], lw["dt_bias"] = get(m + "A_log", torch.float32), get(m + "dt_bias", torch.float32)
                lw["D"], lw["norm"] = get(m + "D", torch.float32), get(m + "norm")
            lw["wo"] = get(m + "o")
            if L.ff_dim > 0:
                lw["norm2"], lw["norm2b"] = get(p + "norm2"), get(p + "norm2b")
                lw["w_gate_up"] = cat([p + "mlp.gate", p + "mlp.up"])
                lw["w_down"] = get(p + "mlp.down")
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
