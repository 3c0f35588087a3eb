"""The generation loop above the step function.

Per batch: all prompts in one step, a token sampled for each sequence from the logits of its
prompt's last place, then one token per live sequence per step. `max_tokens` counts the token
sampled from the prompt's logits, so at least one token is always produced; a stop token is kept
in the output and counted, and ends its sequence; the last sampled token is not fed back
(model_f32.go:604-669). A prompt longer than the engine can hold keeps its tail
(model_f32.go:598-602). Sequences of a batch end independently; requests beyond what fits at once
run as further batches on the slots the earlier ones gave back.

The loop's decisions (who is live, who stops and why, how requests are split into batches) are
plain Python over token ids, so they can be tested with a scripted step function.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Sequence as Seq

import torch

from ..cache.needs import PAGE
from ..sampling.sampler import SamplingOptions


@dataclass
class GenerationResult:
    tokens: list[int]                 # sampled tokens, a final stop token included
    prompt_tokens: int
    finish_reason: str                # "stop" | "length" | "capacity" | "cancelled"
    prefill_ms: float = 0.0           # of the batch the request ran in
    decode_ms: float = 0.0

    @property
    def generated_tokens(self) -> int:
        return len(self.tokens)


def plan_batches(prompt_lens: Seq[int], max_tokens: int, max_seqs: int, page_capacity: int,
                 max_positions: int) -> list[list[int]]:
    """Split request indices, in order, into batches that fit `max_seqs` slots and `page_capacity`
    cache pages when every request runs to its longest (prompt + max_tokens - 1 tokens held)."""
    batches, cur, cur_pages = [], [], 0
    for i, n in enumerate(prompt_lens):
        held = min(max_positions, min(n, max_positions) + max_tokens - 1)
        pages = (max(held, 1) + PAGE - 1) // PAGE
        if pages > page_capacity:
            raise ValueError(f"request {i} needs {pages} cache pages ({held} tokens); the cache has {page_capacity}")
        if cur and (len(cur) >= max_seqs or cur_pages + pages > page_capacity):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += pages
    if cur:
        batches.append(cur)
    return batches


@dataclass
class _Live:
    request: int
    prompt: list[int]
    held: int                                     # tokens in the cache
    out: list[int] = field(default_factory=list)
    reason: str | None = None


class BatchState:
    """Who is live in a batch and what each has produced; no device code."""

    def __init__(self, requests: list[int], prompts: list[list[int]], max_tokens: int, stop_ids, max_positions: int):
        if max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        self.max_tokens, self.stop_ids, self.max_positions = max_tokens, frozenset(stop_ids or ()), max_positions
        self.seqs = []
        for r, p in zip(requests, prompts):
            if len(p) == 0:
                raise ValueError(f"request {r} has an empty prompt")
            self.seqs.append(_Live(r, list(p[-max_positions:]), 0))

    def live(self) -> list[int]:
        return [i for i, s in enumerate(self.seqs) if s.reason is None]

    def accept(self, idx: list[int], fed: list[int], sampled: list[int]) -> list[int]:
        """Sequences `idx` were fed `fed[i]` tokens and sampled `sampled[i]`; returns those that just ended."""
        ended = []
        for i, n, t in zip(idx, fed, sampled):
            s = self.seqs[i]
            s.held += n
            s.out.append(int(t))
            if int(t) in self.stop_ids:
                s.reason = "stop"
            elif len(s.out) >= self.max_tokens:
                s.reason = "length"
            elif s.held + 1 > self.max_positions:
                s.reason = "capacity"
            if s.reason:
                ended.append(i)
        return ended

    def ends_by_count(self, i: int, fed: int) -> bool:
        """Whether sequence i ends with its next accepted token whatever that token is."""
        s = self.seqs[i]
        return len(s.out) + 1 >= self.max_tokens or s.held + fed + 1 > self.max_positions

    def cancel(self) -> list[int]:
        ended = self.live()
        for i in ended:
            self.seqs[i].reason = "cancelled"
        return ended


class Generator:
    """Runs requests through an Engine (or anything with open()/step()) and a Sampler."""

    def __init__(self, engine, sampler):
        self.engine, self.sampler = engine, sampler

    def generate(self, prompts: list[list[int]], max_tokens: int = 100, options: SamplingOptions | None = None,
                 stop_ids=None, seed: int = 0, max_batch: int | None = None,
                 on_step: Callable[[int, dict[int, int]], bool | None] | None = None) -> list[GenerationResult]:
        from .step import StepEntry
        options = options or SamplingOptions()
        eng = self.engine
        stop = eng.layout.stop_ids if stop_ids is None else stop_ids
        max_seqs = min(eng.cache.n_slots, max_batch or eng.cache.n_slots)
        batches = plan_batches([len(p) for p in prompts], max_tokens, max_seqs, eng.cache.n_pages, eng.max_positions)
        results: list[GenerationResult | None] = [None] * len(prompts)
        # With an engine that keeps per-sequence state records on the device and a sampler that reads
        # them, a step's sampling takes nothing from the host: options and stop set go up once per call,
        # the sequences' seeds once per batch.
        on_device_state = hasattr(self.sampler, "sample_state") and hasattr(getattr(eng, "cache", None), "seq_state")
        if on_device_state:
            self.sampler.begin(options, stop)
        for batch in batches:
            state = BatchState(batch, [prompts[i] for i in batch], max_tokens, stop, eng.max_positions)
            seqs = {i: eng.open() for i in range(len(batch))}
            seeds = [seed + r for r in batch]               # one sampling stream per request
            if on_device_state:
                eng.cache.seed([seqs[i].slot for i in range(len(batch))], seeds)
            t_ev = [eng.new_event() for _ in range(3)]
            try:
                t_ev[0].record()
                live = state.live()
                if hasattr(eng, "prompt_step"):          # long batches of prompts go through in portions
                    logits, index = eng.prompt_step([StepEntry(seqs[i], state.seqs[i].prompt) for i in live])
                else:
                    logits = eng.step([StepEntry(seqs[i], state.seqs[i].prompt) for i in live])
                    index = eng.last_step if on_device_state else None
                fed = [len(state.seqs[i].prompt) for i in live]
                step_no = 0
                # When the engine replays its decode step, the next step is launched with the sampled ids
                # still on the device, before the host reads them: only a stop token can then end a
                # sequence one step "late", and its extra row is dropped.
                pipelined = bool(getattr(eng, "use_graphs", False)) and hasattr(eng, "decode_step_device") \
                    and not options.penalises
                while True:
                    recent = [state.seqs[i].prompt + state.seqs[i].out for i in live] if options.penalises else None
                    if on_device_state:
                        toks_dev = self.sampler.sample_state(logits, eng.cache, index, options, recent)
                    else:
                        toks_dev = self.sampler.sample(logits, options, [seeds[i] for i in live],
                                                       [len(state.seqs[i].out) for i in live], recent)
                    if step_no == 0:
                        t_ev[1].record()
                    ahead = None
                    # the ids start their way to the host before the next step is put on the stream
                    read = self.sampler.begin_read(toks_dev) if pipelined and hasattr(self.sampler, "begin_read") else toks_dev.tolist
                    if pipelined:
                        cont = [j for j, i in enumerate(live) if not state.ends_by_count(i, fed[j])]
                        if cont:
                            rows = toks_dev if len(cont) == len(live) else toks_dev[torch.as_tensor(cont, device=toks_dev.device)]
                            ahead = ([live[j] for j in cont], eng.decode_step_device([seqs[live[j]] for j in cont], rows),
                                     eng.last_step if on_device_state else None)
                    toks = read()
                    for i in state.accept(live, fed, toks):
                        seqs.pop(i).close()
                    if on_step is not None and on_step(step_no, {batch[i]: t for i, t in zip(live, toks)}):
                        for i in state.cancel():
                            seqs.pop(i).close()
                    live = state.live()
                    if not live:
                        break
                    if ahead is not None:
                        keep = [j for j, i in enumerate(ahead[0]) if state.seqs[i].reason is None]
                        if len(keep) == len(ahead[0]):
                            logits, index = ahead[1], ahead[2]
                        else:
                            rows = torch.as_tensor(keep, device=ahead[1].device)
                            logits, index = ahead[1][rows], (ahead[2].rows(rows) if on_device_state else None)
                    else:
                        logits = eng.step([StepEntry(seqs[i], [state.seqs[i].out[-1]]) for i in live])
                        index = eng.last_step if on_device_state else None
                    fed = [1] * len(live)
                    step_no += 1
                t_ev[2].record()
                t_ev[2].synchronize()
                if hasattr(eng, "check_errors"):
                    eng.check_errors()
                pre_ms, dec_ms = t_ev[0].elapsed_time(t_ev[1]), t_ev[1].elapsed_time(t_ev[2])
            finally:
                for s in seqs.values():
                    s.close()
            for s in state.seqs:
                results[s.request] = GenerationResult(s.out, len(s.prompt), s.reason or "cancelled", pre_ms, dec_ms)
        return results
