"""Replay a recorded schedule of forwards through the ragged engine and write the logits it produces.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N  < steps.jsonl

Each input line is one engine step: ``{"step": n, "entries": [{"id": name, "tokens": [...], "want": [...]}], "end":
[names]}``.  All entries of a step form one ragged batch (``InferenceEngineV2.put``): prompt portions beside single
decode tokens, continuing from the KV pages and state slots earlier steps left.  ``want`` are the indices among an
entry's tokens whose logits are written, in entry order, to ``<out>/<step>.f32`` (little-endian float32
``[wanted, vocab]``); requests in ``end`` are flushed after the step.  ``done <step>`` is printed after every step.

The KV pool holds ``--max-tokens`` tokens in 64-token pages (each request rounded up to whole pages) and the state
manager tracks four requests, so pages and state slots are reused as requests end.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE = 64
MAX_LIVE = 4


def build_engine(model_dir: str, dtype_name: str, max_tokens: int):
    import torch
    from .config_v2 import RaggedInferenceEngineConfig
    from .engine_factory import build_hf_engine
    from .ragged.ragged_manager import DSStateManagerConfig
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype_name]
    pages = max(1, (max_tokens + PAGE - 1) // PAGE)
    sm = DSStateManagerConfig(max_tracked_sequences=MAX_LIVE, max_ragged_sequence_count=MAX_LIVE,
                              max_ragged_batch_size=max(pages * PAGE, MAX_LIVE), max_context=pages * PAGE,
                              num_kv_blocks=pages)
    cfg = RaggedInferenceEngineConfig(state_manager=sm, kv_block_size=PAGE)
    return build_hf_engine(model_dir, cfg, debug_level=40, dtype=dtype)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the KV pool holds")
    ap.add_argument("--device", default=None, help="default: the GPU; 'cpu' runs the PyTorch branch of every op")
    a = ap.parse_args(argv)
    import torch
    if a.device is None and not torch.cuda.is_available():
        print("no CUDA device: pass --device cpu to replay on the PyTorch branch", file=sys.stderr)
        return 4
    if a.device == "cpu":
        os.environ.setdefault("CUDA_VISIBLE_DEVICES", "")
    engine = build_engine(a.model, a.dtype, a.max_tokens)
    os.makedirs(a.out, exist_ok=True)
    uids, next_uid = {}, 0
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = step.get("entries", [])
        if entries:
            ids = []
            for e in entries:
                if e["id"] not in uids:
                    next_uid += 1
                    uids[e["id"]] = next_uid
                ids.append(uids[e["id"]])
            toks = [torch.tensor(e["tokens"], dtype=torch.int32) for e in entries]
            want = [list(e.get("want", [])) for e in entries]
            logits = engine.put(ids, toks, logit_positions=want)
            if logits.shape[0]:
                data = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4")
                tmp = os.path.join(a.out, f".{step['step']}.part")
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
            elif torch.cuda.is_available():
                torch.cuda.synchronize()
        for name in step.get("end", []):
            if name in uids:
                engine.flush(uids.pop(name))
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
