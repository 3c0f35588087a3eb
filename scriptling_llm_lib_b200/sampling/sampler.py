"""Choosing the next token of every sequence of a batch from its logits, on the device.

Strategies and option names are the reference's (model.go:701-851; `llm.generate` keywords,
model.go:868-946): "greedy", "temperature", "top_k", "top_p", with `temperature`, `top_k`, `top_p`,
`repeat_penalty`, `repeat_last_n`. Greedy ignores temperature and penalty (model_f32.go:610-615);
a temperature of 0 means greedy. The reference draws from one clock-seeded generator
(sampling.go:14-18); here each sequence has its own seed and a draw counter, kept in its
fixed-size state record on the device (cache.seq_state) and advanced by the sampling kernel, so a
sequence's tokens do not depend on its batch mates and a sampled decode step takes nothing from
the host. `sample` (parameters packed on the host for every call) remains for callers without
sequences: kernel tests and measurements.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np
import torch

from ..csrc.bindings import SamplingKernels

STRATEGIES = ("greedy", "temperature", "top_k", "top_p")


@dataclass(frozen=True)
class SamplingOptions:
    strategy: str = "greedy"
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.9
    repeat_penalty: float = 0.0      # 0 or 1 disables; applied on the sampling strategies only
    repeat_last_n: int = 64

    def __post_init__(self):
        if self.strategy not in STRATEGIES:
            raise ValueError(f"unknown sampling strategy {self.strategy!r}; supported: {', '.join(STRATEGIES)}")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")

    @property
    def is_greedy(self) -> bool:
        return self.strategy == "greedy" or self.temperature == 0.0

    @property
    def penalises(self) -> bool:
        return (not self.is_greedy) and self.repeat_penalty > 0.0 and self.repeat_penalty != 1.0


def pack_params(options: SamplingOptions, seeds: list[int], draws: list[int]) -> np.ndarray:
    """Rows of 8 int32 words for the sampling kernel: strategy, temperature, top_k, top_p, seed
    (low, high), draw index (low, high)."""
    n = len(seeds)
    out = np.zeros((n, SamplingKernels.PARAM_WORDS), dtype=np.int32)
    strat = 0 if options.is_greedy else SamplingKernels.STRATEGIES[options.strategy]
    f2i = lambda f: struct.unpack("<i", struct.pack("<f", f))[0]
    u2i = lambda u: struct.unpack("<i", struct.pack("<I", u & 0xFFFFFFFF))[0]
    out[:, 0], out[:, 1], out[:, 2], out[:, 3] = strat, f2i(options.temperature), options.top_k, f2i(options.top_p)
    for i, (s, d) in enumerate(zip(seeds, draws)):
        out[i, 4], out[i, 5], out[i, 6], out[i, 7] = u2i(s), u2i(s >> 32), u2i(d), u2i(d >> 32)
    return out


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self.kernels = SamplingKernels()
        self._greedy_params = torch.zeros((0, SamplingKernels.PARAM_WORDS), dtype=torch.int32, device=self.device)
        self._host = torch.zeros((64, SamplingKernels.PARAM_WORDS), dtype=torch.int32).pin_memory()
        self._copied = torch.cuda.Event()

    def _params(self, options, seeds, draws) -> torch.Tensor:
        n = len(seeds)
        if options.is_greedy:                       # strategy word 0 in every row; nothing else is read
            if self._greedy_params.shape[0] < n:
                self._greedy_params = torch.zeros((max(64, 2 * n), SamplingKernels.PARAM_WORDS), dtype=torch.int32,
                                                  device=self.device)
            return self._greedy_params[:n]
        if self._host.shape[0] < n:
            self._host = torch.zeros((2 * n, SamplingKernels.PARAM_WORDS), dtype=torch.int32).pin_memory()
        self._copied.synchronize()                  # the last copy out of the pinned rows is done
        self._host[:n] = torch.from_numpy(pack_params(options, seeds, draws))
        dev = self._host[:n].to(self.device, non_blocking=True)
        self._copied.record()
        return dev

    def begin(self, options: SamplingOptions, stop_ids=()) -> None:
        """Put the options and the stop set of a generation call on the device (once per call, and
        only when they differ from the last call's); `sample_state` then takes nothing from the host."""
        key = (options.strategy if not options.is_greedy else "greedy", options.temperature, options.top_k, options.top_p,
               tuple(sorted(set(int(t) for t in stop_ids or ()))))
        if getattr(self, "_begun", None) == key:
            return
        words = pack_params(options, [0], [0])[0, :4].copy()
        self._options_dev = torch.from_numpy(words).to(self.device)
        self._stop_dev = torch.tensor(key[4], dtype=torch.int32, device=self.device) if key[4] else None
        self._begun = key

    def sample_state(self, logits: torch.Tensor, cache, index, options: SamplingOptions,
                     recent: list[list[int]] | None = None) -> torch.Tensor:
        """logits float32 [n, V] -> int32 token ids [n] on the device, every row's sampling key and draw
        counter taken from its sequence's state record on the device (`cache.seq_state` at
        `index.slots`), which the kernel advances (tokens held, generated count, last token, counter,
        finished flag on a stop token). Call `begin` first."""
        n = logits.shape[0]
        if options.penalises and recent is not None:
            logits = self._penalised(logits, options, recent)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        self.kernels.sample_rows_state(logits, self._options_dev, cache.seq_state, index.slots, index.pos_after,
                                       self._stop_dev, out)
        return out

    def _penalised(self, logits, options, recent):
        n = logits.shape[0]
        last_n = max(1, options.repeat_last_n)
        win = np.full((n, last_n), -1, dtype=np.int32)
        counts = np.zeros(n, dtype=np.int32)
        for i, r in enumerate(recent):
            tail = r[-last_n:]
            win[i, :len(tail)] = tail
            counts[i] = len(tail)
        logits = logits.clone()
        self.kernels.repeat_penalty(
            logits, torch.from_numpy(win).to(self.device), torch.from_numpy(counts).to(self.device),
            torch.full((n,), float(options.repeat_penalty), dtype=torch.float32, device=self.device), last_n)
        return logits

    def begin_read(self, tokens: torch.Tensor):
        """Start copying sampled ids to the host; returns a function that waits for that copy alone and
        gives the ids as a list. Called before later work is put on the stream, it lets the host read a
        step's tokens while the next step is already running (a plain read would wait for all of it).
        The copy runs on a stream of its own behind an event: a copy between two kernels of the
        compute stream costs that stream about 0.1 ms (measured), this one nothing."""
        n = tokens.shape[0]
        if getattr(self, "_host_ids", None) is None or self._host_ids.shape[0] < n:
            self._host_ids = torch.empty(max(64, n), dtype=torch.int32).pin_memory()
            self._read_stream = torch.cuda.Stream(device=self.device)
            self._sampled, self._ids_read = torch.cuda.Event(), torch.cuda.Event()
        host = self._host_ids[:n]
        self._sampled.record()
        self._read_stream.wait_event(self._sampled)
        with torch.cuda.stream(self._read_stream):
            host.copy_(tokens, non_blocking=True)
            self._ids_read.record()
        tokens.record_stream(self._read_stream)

        def result():
            self._ids_read.synchronize()
            return host.tolist()
        return result

    def sample(self, logits: torch.Tensor, options: SamplingOptions, seeds: list[int], draws: list[int],
               recent: list[list[int]] | None = None) -> torch.Tensor:
        """logits float32 [n, V] on the device -> int32 token ids [n] on the device.
        `recent`: each sequence's prompt and generated tokens so far (for the repeat penalty)."""
        n = logits.shape[0]
        if options.penalises and recent is not None:
            logits = self._penalised(logits, options, recent)
        params = self._params(options, seeds, draws)
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        self.kernels.sample_rows(logits, params, out)
        return out
