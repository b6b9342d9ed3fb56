"""Scheduler and page pool of the stand-alone engine (vllm_neuron_b200/engine.py).

Inside vLLM the plugin's scheduler subclass and vLLM's KV-cache manager do this work; the stand-alone engine needs the same
two things without vLLM: pages handed out from a pool of fixed size and returned when a request ends, and a policy that
decides which tokens run in a step.  The policy functions are the ones the vLLM subclass uses (`admit_count`,
`stop_reason` in core/scheduler.py; reference: vllm_neuron/core/scheduler.py:69-166):
  * "exclusive" (dense decoders): a step is ONE whole-prompt prefill or a decode batch of every running request;
  * "mixed" (ragged-batch models): decodes and prompt portions share a step under a token budget, running requests first,
    then waiting ones while a line (state slot) and pages are free.
The output has the fields of vLLM's SchedulerOutput that the model runner reads.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from types import SimpleNamespace

from .scheduler import admit_count, stop_reason


class BlockPool:
    """Page ids 1 .. num_blocks - 1 (page 0 is the null page, never handed out).  Freed pages are reused first."""

    def __init__(self, num_blocks: int):
        self.num_blocks = num_blocks
        self._free = list(range(num_blocks - 1, 0, -1))  # pop() hands out 1, 2, ...

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> list[int]:
        if n > len(self._free):
            raise RuntimeError(f"KV pool exhausted: {n} pages wanted, {len(self._free)} free of {self.num_blocks - 1}")
        return [self._free.pop() for _ in range(n)]

    def free(self, ids) -> None:
        self._free.extend(reversed(list(ids)))


@dataclass
class EngineRequest:
    req_id: str
    tokens: list                      # every token known so far: the prompt, then what was generated (or forced)
    num_prompt: int
    max_new_tokens: int = 0
    sampling_params: object = None
    eos_token_id: int | None = None
    num_computed: int = 0
    block_ids: list = field(default_factory=list)
    admitted: bool = False            # the runner has seen it (it owns a row / state slot)
    finished: str | None = None

    @property
    def num_output(self) -> int:
        return len(self.tokens) - self.num_prompt


def make_output(new, cached, num_sched, finished):
    """new: [(EngineRequest, new block ids)], cached: [(EngineRequest, new block ids or None)]."""
    return SimpleNamespace(
        scheduled_new_reqs=[SimpleNamespace(req_id=r.req_id, prompt_token_ids=list(r.tokens), block_ids=(list(b),),
                                            num_computed_tokens=0, sampling_params=r.sampling_params, mm_features=[],
                                            lora_request=None) for r, b in new],
        scheduled_cached_reqs=SimpleNamespace(
            req_ids=[r.req_id for r, _ in cached], resumed_req_ids=set(),
            new_block_ids=[None if not b else (list(b),) for _, b in cached],
            num_computed_tokens=[r.num_computed for r, _ in cached], new_token_ids=[], num_output_tokens=[r.num_output for r, _ in cached]),
        num_scheduled_tokens=dict(num_sched), total_num_scheduled_tokens=sum(num_sched.values()),
        finished_req_ids=set(finished), scheduled_spec_decode_tokens={}, free_encoder_mm_hashes=[])


class EngineScheduler:
    def __init__(self, pool: BlockPool, *, block_size: int, max_num_seqs: int, max_model_len: int,
                 max_num_batched_tokens: int = 2048, policy: str = "mixed"):
        assert policy in ("mixed", "exclusive")
        self.pool, self.block_size, self.policy = pool, block_size, policy
        self.max_num_seqs, self.max_model_len, self.budget = max_num_seqs, max_model_len, max_num_batched_tokens
        self.waiting: deque[EngineRequest] = deque()
        self.running: list[EngineRequest] = []
        self._finished_ids: list[str] = []  # reported to the runner with the next step

    def add(self, req: EngineRequest) -> None:
        if len(req.tokens) + req.max_new_tokens > self.max_model_len:
            raise ValueError(f"request {req.req_id}: {len(req.tokens)} + {req.max_new_tokens} tokens exceed max_model_len "
                             f"{self.max_model_len}")
        self.waiting.append(req)

    def pages_for(self, req: EngineRequest, upto: int) -> list[int]:
        """Allocate the pages that holding tokens [0, upto) still needs; returns the new ids."""
        need = -(-upto // self.block_size) - len(req.block_ids)
        new = self.pool.allocate(need) if need > 0 else []
        req.block_ids += new
        return new

    def _can_hold(self, req: EngineRequest, upto: int) -> bool:
        return -(-upto // self.block_size) - len(req.block_ids) <= self.pool.num_free

    def finish(self, req: EngineRequest, reason: str = "stop") -> None:
        req.finished = reason
        if req in self.running:
            self.running.remove(req)
        self.pool.free(req.block_ids)
        req.block_ids = []
        if req.admitted:
            self._finished_ids.append(req.req_id)

    def take_finished(self) -> list[str]:
        out, self._finished_ids = self._finished_ids, []
        return out

    def schedule(self):
        new, cached, num = [], [], {}
        if self.policy == "exclusive":
            n = admit_count(len(self.running), len(self.waiting), self.max_num_seqs)
            if n and self._can_hold(self.waiting[0], len(self.waiting[0].tokens)):
                r = self.waiting.popleft()  # prefill step: the whole prompt of one request, nothing else
                new.append((r, self.pages_for(r, len(r.tokens))))
                num[r.req_id] = len(r.tokens)
                r.admitted = True
                self.running.append(r)
            else:
                for r in self.running:
                    cached.append((r, self.pages_for(r, r.num_computed + 1)))
                    num[r.req_id] = 1
            return make_output(new, cached, num, self.take_finished())
        left = self.budget
        for r in self.running:  # decodes (one token) and unfinished prompts (as much as the budget allows)
            n = min(len(r.tokens) - r.num_computed, left)
            if n <= 0 or not self._can_hold(r, r.num_computed + n):
                continue
            cached.append((r, self.pages_for(r, r.num_computed + n)))
            num[r.req_id] = n
            left -= n
        while self.waiting and left > 0 and admit_count(len(self.running), 1, self.max_num_seqs, max_prompt_batch=1 << 30):
            r = self.waiting[0]
            n = min(len(r.tokens), left)
            if not self._can_hold(r, n):
                break
            self.waiting.popleft()
            new.append((r, self.pages_for(r, n)))
            num[r.req_id] = n
            left -= n
            r.admitted = True
            self.running.append(r)
        return make_output(new, cached, num, self.take_finished())

    def update(self, sched, sampled: dict[str, list[int]]) -> list[EngineRequest]:
        """Advance the scheduled requests by what the step computed and sampled; returns those that finished."""
        done = []
        by_id = {r.req_id: r for r in self.running}
        for rid, n in sched.num_scheduled_tokens.items():
            r = by_id[rid]
            r.num_computed += n
            for tok in sampled.get(rid, ()):
                r.tokens.append(tok)
                why = stop_reason(num_tokens=len(r.tokens), num_output_tokens=r.num_output, max_tokens=r.max_new_tokens,
                                  max_model_len=self.max_model_len, min_tokens=0, last_token_id=tok,
                                  eos_token_id=r.eos_token_id, ignore_eos=r.eos_token_id is None)
                if why:
                    self.finish(r, why if isinstance(why, str) else why[0])
                    done.append(r)
                    break
        return done
