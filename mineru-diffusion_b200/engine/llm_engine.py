"""Step loop around scheduler and model runner.

The part of the reference's ``LLMEngine`` that drives the hot path
(``engines/nano_dvlm/nanovllm/engine/llm_engine.py:66-105``): schedule, run,
post-process, collect finished requests.  Tokenizer, processor and the CLI
stay with the reference; requests enter here as ``Sequence`` objects.
"""
from __future__ import annotations

from time import perf_counter

from .config import Config
from .scheduler import Scheduler
from .sequence import Sequence


class LLMEngine:

    def __init__(self, config: Config, model_runner):
        self.config = config
        self.model_runner = model_runner      # sets config.num_kvcache_blocks before the scheduler reads it
        self.scheduler = Scheduler(config)
        self.num_prefill_steps = 0
        self.num_decode_steps = 0

    def add_sequence(self, seq: Sequence):
        self.scheduler.add(seq)

    def step(self):
        seqs, is_prefill = self.scheduler.schedule()
        num_tokens = self.model_runner.call("run", seqs, is_prefill)
        self.scheduler.postprocess(seqs)
        outputs = [(seq.seq_id, seq.completion_token_ids, seq.step_map) for seq in seqs if seq.is_finished]
        if is_prefill:
            self.num_prefill_steps += 1
            num_tokens = sum(len(seq) for seq in seqs) + num_tokens
        else:
            self.num_decode_steps += 1
            num_tokens = -num_tokens
        return outputs, num_tokens

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    def generate(self, seqs: list[Sequence]):
        """Runs all requests to completion; returns ({seq_id: (token_ids,
        step_map)}, wall seconds)."""
        for seq in seqs:
            self.add_sequence(seq)
        done: dict[int, tuple[list[int], list[int]]] = {}
        start = perf_counter()
        while not self.is_finished():
            outputs, _ = self.step()
            for seq_id, token_ids, step_map in outputs:
                done[seq_id] = (token_ids, step_map)
        return done, perf_counter() - start
