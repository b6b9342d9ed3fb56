"""Stand-alone engine: the model runner, a page pool and a scheduler without vLLM around them.

    engine = B200Engine.from_pretrained(model_dir, dtype="bfloat16", max_num_seqs=4, max_pool_tokens=4096)
    outputs = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)        # greedy unless sampling_params are given

    python -m vllm_neuron_b200.engine --model DIR --prompt 1,2,3 --prompt 4,5 --max-new-tokens 16

The model class comes from the registry (config.json's architecture); the step is `B200ModelRunner.execute_model`, the same
call the vLLM worker makes, fed with scheduler outputs built here (core/engine_scheduler.py).  The KV pool is sized in TOKENS
(`max_pool_tokens`, rounded up to pages, plus the null page) and is shared by the live requests; each request owns one of
`max_num_seqs` rows (block-table row = recurrent-state slot) for its lifetime, and both pages and rows return to their pools
when it ends.  `replay_step` teacher-forces given tokens through the same path and hands back logits at chosen positions
(vllm_neuron_b200/trace.py drives it).
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from types import SimpleNamespace

import torch

from .core.engine_scheduler import BlockPool, EngineRequest, EngineScheduler
from .registry import load_config, resolve

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class StepOutput:
    """The fields of vLLM's ModelRunnerOutput that the runner fills."""
    req_ids: list = field(default_factory=list)
    req_id_to_index: dict = field(default_factory=dict)
    sampled_token_ids: list = field(default_factory=list)
    logprobs: object = None
    prompt_logprobs_dict: dict = field(default_factory=dict)
    pooler_output: list = field(default_factory=list)


def _runner_config(*, max_num_seqs, max_model_len, block_size, num_blocks, max_num_batched_tokens):
    """The attributes of VllmConfig the runner reads."""
    return SimpleNamespace(
        model_config=SimpleNamespace(hf_config=None, max_model_len=max_model_len, seed=0, enforce_eager=True, dtype=torch.bfloat16),
        cache_config=SimpleNamespace(block_size=block_size, enable_prefix_caching=False, num_gpu_blocks_override=num_blocks),
        parallel_config=SimpleNamespace(tensor_parallel_size=1, world_size=1),
        scheduler_config=SimpleNamespace(max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                                         max_num_batched_tokens=max_num_batched_tokens),
        load_config=SimpleNamespace(load_format="auto"), additional_config={})


class B200Engine:
    def __init__(self, config, weights, *, entry=None, dtype="bfloat16", max_num_seqs: int = 4, max_pool_tokens: int = 4096,
                 block_size: int = 32, max_model_len: int | None = None, max_num_batched_tokens: int = 2048, device="cuda:0"):
        from .worker.b200_model_runner import B200ModelRunner

        if entry is None:
            _, entry = resolve(config.to_dict() if hasattr(config, "to_dict") else {"architectures": ["LlamaForCausalLM"]})
        dt = DTYPES[dtype]
        if dt not in entry.dtypes:
            raise ValueError(f"this model family is not served in {dtype}")
        self.device = torch.device(device)
        self.block_size = block_size
        pages = -(-max_pool_tokens // block_size)
        self.num_blocks = pages + 1  # + the null page
        self.max_model_len = max_model_len or pages * block_size
        self.max_num_seqs = max_num_seqs
        self.model = entry.build(config, weights, dtype=dt, num_blocks=self.num_blocks, max_num_seqs=max_num_seqs,
                                 max_model_len=self.max_model_len, block_size=block_size, device=self.device)
        mixed = bool(getattr(self.model, "mixed_batch", False))
        self.pool = BlockPool(self.num_blocks)
        self.scheduler = EngineScheduler(self.pool, block_size=block_size, max_num_seqs=max_num_seqs,
                                         max_model_len=self.max_model_len, max_num_batched_tokens=max_num_batched_tokens,
                                         policy="mixed" if mixed else "exclusive")
        cfg = _runner_config(max_num_seqs=max_num_seqs, max_model_len=self.max_model_len, block_size=block_size,
                             num_blocks=self.num_blocks, max_num_batched_tokens=max_num_batched_tokens)
        self.runner = B200ModelRunner(cfg, self.device, model=self.model)
        self.runner.use_cuda_graph = False
        self.runner.output_factory = (StepOutput(), StepOutput)
        self.runner.initialize_kv_cache(num_blocks=self.num_blocks)
        self.requests: dict[str, EngineRequest] = {}

    @classmethod
    def from_pretrained(cls, path: str, **kw) -> "B200Engine":
        _, entry, config = load_config(path)
        return cls(config, entry.open_weights(path, config), entry=entry, **kw)

    # ------------------------------------------------------------------ generation
    def add_request(self, req_id: str, prompt_token_ids, max_new_tokens: int = 16, sampling_params=None, eos_token_id=None):
        assert req_id not in self.requests and len(prompt_token_ids) > 0
        r = EngineRequest(req_id, [int(t) for t in prompt_token_ids], len(prompt_token_ids), max_new_tokens, sampling_params,
                          eos_token_id)
        self.requests[req_id] = r
        self.scheduler.add(r)
        return r

    def step(self) -> list[EngineRequest]:
        """One scheduler decision + one model step; returns the requests that finished in it."""
        sched = self.scheduler.schedule()
        out = self.runner.execute_model(sched)
        sampled = {rid: out.sampled_token_ids[i] for rid, i in out.req_id_to_index.items()}
        return self.scheduler.update(sched, sampled)

    def has_unfinished(self) -> bool:
        return bool(self.scheduler.waiting or self.scheduler.running)

    def generate(self, prompts, max_new_tokens: int = 16, sampling_params=None) -> list[list[int]]:
        reqs = [self.add_request(f"gen-{len(self.requests)}-{i}", p, max_new_tokens, sampling_params) for i, p in enumerate(prompts)]
        while self.has_unfinished():
            self.step()
        self._flush_finished()
        return [r.tokens[r.num_prompt:] for r in reqs]

    def _flush_finished(self):
        ids = self.scheduler.take_finished()
        if ids:
            from .core.engine_scheduler import make_output

            self.runner.execute_model(make_output([], [], {}, ids))

    # ------------------------------------------------------------------ teacher-forced replay
    def replay_step(self, entries, end=()) -> dict[str, torch.Tensor]:
        """entries: [(req_id, tokens, want)] -- each request's following tokens (an unknown id is a new request) and which
        of them to return logits for.  The whole list is one engine step.  `end`: ids to retire once the step has run; their
        pages and row go back to the pools.  Returns req_id -> fp32 logits [len(want), vocab] (host)."""
        from .core.engine_scheduler import make_output

        sch = self.scheduler
        new, cached, num = [], [], {}
        for rid, tokens, want in entries:
            tokens = [int(t) for t in tokens]
            if not tokens:
                continue
            r = self.requests.get(rid)
            if r is None:
                if len(sch.running) >= self.max_num_seqs:
                    raise RuntimeError(f"no free row for request {rid!r}: {self.max_num_seqs} are live")
                r = self.requests[rid] = EngineRequest(rid, tokens, len(tokens))
                r.admitted = True
                sch.running.append(r)
                new.append((r, sch.pages_for(r, len(tokens))))
            else:
                assert r.finished is None and r.num_computed == len(r.tokens), f"request {rid!r} cannot take forced tokens now"
                r.tokens += tokens
                r.num_prompt = len(r.tokens)
                self.runner.extend_prompt(rid, tokens)
                cached.append((r, sch.pages_for(r, len(r.tokens))))
            num[rid] = len(tokens)
            if want:
                self.runner.logit_taps[rid] = [int(p) for p in want]
        taps = {}
        if num:
            sched = make_output(new, cached, num, sch.take_finished())
            self.runner.execute_model(sched)
            for rid, n in num.items():
                self.requests[rid].num_computed += n
            taps = {rid: t.float().cpu() for rid, t in self.runner.tap_logits.items()}
            for r, _ in new + cached:  # the runner sampled a continuation for fully computed requests: forced runs drop it
                st = self.runner.requests[r.req_id]
                st.output_token_ids.clear()
        for rid in end:
            r = self.requests.pop(rid, None)
            if r is not None:
                sch.finish(r)
        return taps


def main(argv=None):
    ap = argparse.ArgumentParser(description="Greedy generation from token ids with the stand-alone B200 engine")
    ap.add_argument("--model", required=True, help="directory with config.json and *.safetensors")
    ap.add_argument("--prompt", action="append", required=True, help="comma-separated token ids (repeatable)")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-num-seqs", type=int, default=4)
    ap.add_argument("--max-pool-tokens", type=int, default=4096)
    a = ap.parse_args(argv)
    from . import build

    build.build()
    eng = B200Engine.from_pretrained(a.model, dtype=a.dtype, max_num_seqs=a.max_num_seqs, max_pool_tokens=a.max_pool_tokens)
    prompts = [[int(t) for t in p.split(",")] for p in a.prompt]
    for p, out in zip(prompts, eng.generate(prompts, a.max_new_tokens)):
        print(",".join(map(str, p)), "->", ",".join(map(str, out)))


if __name__ == "__main__":
    main()
