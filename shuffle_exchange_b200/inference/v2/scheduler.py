"""Continuous batching on top of :class:`InferenceEngineV2`: requests join and leave between forwards, prompts are cut
into portions that share a forward with other requests' single decode tokens (the reference leaves this loop to its
serving layer and only provides ``query`` / ``can_schedule`` / ``put`` / ``flush``, ``inference/v2/engine_v2.py:107-268``).

Every step: all requests that are decoding contribute one token; the remaining token budget goes to waiting prompts in
arrival order, as large a portion as budget and free KV blocks allow; a request that does not fit waits.  Finished
requests are flushed, which returns their KV blocks and state slot.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

import torch

from .sampling import SamplingParams, sample
from .scheduling_utils import SchedulingResult


@dataclass
class Request:
    uid: int
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_token_id: Optional[int] = None
    fed: int = 0                                  # prompt tokens already given to the engine
    output: List[int] = field(default_factory=list)
    done: bool = False
    _generator: Optional[torch.Generator] = None

    @property
    def decoding(self) -> bool:
        return self.fed >= len(self.prompt)


class RaggedScheduler:
    def __init__(self, engine, max_batch_tokens: Optional[int] = None, max_prompt_portion: Optional[int] = None) -> None:
        self.engine = engine
        sm = engine._config.state_manager
        self.max_batch_tokens = min(max_batch_tokens or sm.max_ragged_batch_size, sm.max_ragged_batch_size)
        self.max_prompt_portion = max_prompt_portion or self.max_batch_tokens
        self.max_batch_seqs = sm.max_ragged_sequence_count
        self.max_live = sm.max_tracked_sequences
        self._waiting: List[Request] = []
        self._live: Dict[int, Request] = {}
        self.finished: Dict[int, Request] = {}

    def add_request(self, uid: int, prompt: Iterable[int], max_new_tokens: int, sampling: SamplingParams = None,
                    eos_token_id: Optional[int] = None) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        r = Request(uid, prompt, max_new_tokens, sampling or SamplingParams(), eos_token_id)
        if r.sampling.seed is not None:
            r._generator = torch.Generator().manual_seed(r.sampling.seed)
        self._waiting.append(r)
        return r

    @property
    def pending(self) -> bool:
        return bool(self._waiting or self._live)

    def _plan(self):
        """[(request, tokens of this step)]: decode tokens first, then prompt portions while budget and blocks last."""
        plan, budget, blocks = [], self.max_batch_tokens, self.engine.free_blocks
        for r in self._live.values():
            if r.decoding and budget > 0 and len(plan) < self.max_batch_seqs:
                n, need = self.engine.query(r.uid, 1, blocks)
                if n == 1:
                    plan.append((r, [r.output[-1]]))
                    budget, blocks = budget - 1, blocks - need
        candidates = [r for r in self._live.values() if not r.decoding]
        admitted = 0
        while self._waiting and len(self._live) + admitted < self.max_live:
            candidates.append(self._waiting.pop(0))
            admitted += 1
        deferred = []
        for r in candidates:
            new = r.uid not in self._live
            n = 0
            if budget > 0 and len(plan) < self.max_batch_seqs:
                want = min(len(r.prompt) - r.fed, budget, self.max_prompt_portion)
                n, need = self._query_new(want, blocks) if new else self.engine.query(r.uid, want, blocks)
            if n <= 0:
                if new:
                    deferred.append(r)
                continue
            self._live[r.uid] = r
            plan.append((r, r.prompt[r.fed: r.fed + n]))
            budget, blocks = budget - n, blocks - need
        self._waiting[0:0] = deferred              # arrival order is kept
        return plan

    def _query_new(self, want: int, blocks: int):
        from .ragged.sequence_descriptor import PlaceholderSequenceDescriptor
        return self.engine.model().get_kv_requirements(PlaceholderSequenceDescriptor(), want, blocks)

    def step(self) -> Dict[int, int]:
        """One forward; returns {uid: token} for every request that produced a token in it."""
        plan = self._plan()
        if not plan:
            if self.pending:
                raise RuntimeError("nothing can be scheduled: the KV cache is too small for the waiting requests")
            return {}
        uids = [r.uid for r, _ in plan]
        toks = [torch.tensor(t, dtype=torch.int32) for _, t in plan]
        res = self.engine.can_schedule(uids, [len(t) for _, t in plan])
        if res != SchedulingResult.Success:
            raise RuntimeError(f"scheduler produced a batch the engine refuses: {res}")
        completes = [r.decoding or r.fed + len(t) >= len(r.prompt) for r, t in plan]
        rows = [[len(t) - 1] if c else [] for (r, t), c in zip(plan, completes)]
        logits = self.engine.put(uids, toks, do_checks=False, logit_positions=rows).cpu()
        out, k = {}, 0
        for (r, t), c in zip(plan, completes):
            if not r.decoding:
                r.fed += len(t)
            if not c:
                continue
            tok = int(sample(logits[k: k + 1], r.sampling, r._generator)[0])
            k += 1
            r.output.append(tok)
            out[r.uid] = tok
            if len(r.output) >= r.max_new_tokens or (r.eos_token_id is not None and tok == r.eos_token_id):
                r.done = True
                self.engine.flush(r.uid)
                self.finished[r.uid] = self._live.pop(r.uid)
        return out

    def run(self) -> Dict[int, List[int]]:
        while self.pending:
            self.step()
        return {uid: r.output for uid, r in self.finished.items()}


def generate(engine, prompts: List[List[int]], max_new_tokens: int, sampling: SamplingParams = None,
             eos_token_id: Optional[int] = None, max_batch_tokens: Optional[int] = None,
             max_prompt_portion: Optional[int] = None) -> List[List[int]]:
    """Generate continuations of token-id prompts through the scheduler; returns the new tokens per prompt."""
    sched = RaggedScheduler(engine, max_batch_tokens, max_prompt_portion)
    for i, p in enumerate(prompts):
        sched.add_request(i, p, max_new_tokens, sampling, eos_token_id)
    done = sched.run()
    return [done[i] for i in range(len(prompts))]
