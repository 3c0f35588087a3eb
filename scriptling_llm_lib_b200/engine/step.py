"""The engine and its one step function.

The reference's step is Forward(tokenIDs, startPos): one sequence, its new tokens, logits of the
last position (model_f32.go:377-380). Here a step takes a batch of sequences with the next tokens
of each (a whole prompt, or one token), runs exactly those tokens as one packed batch against
the cache that earlier steps left, and returns float32 logits at the places asked for. A
sequence's rows see only that sequence's keys, so neither its batch mates nor padding change its
numbers.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..cache import PAGE, SequenceCache, pages_for
from ..config.registry import architecture_for, load_config
from ..csrc.bindings import CastKernels, KernelSet
from ..weights.loader import load_weights, stored_to_kept
from .graphs import DecodeGraphs
from .layout import ModelLayout
from .model import DecoderModel

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _draw_one(ts, spec, index, device):
    from ..weights.random_init import draw_device
    if device.type != "cuda":
        raise StepError(f"the engine runs on a CUDA device, not on {device}")
    with torch.cuda.device(device):
        return draw_device(ts, spec.seed, index, spec.dtype, device)


class StepError(ValueError):
    """A step that cannot run; raised before anything is launched or changed."""


class Sequence:
    """A live request: a cache slot and the number of tokens it holds."""

    def __init__(self, engine: "Engine", slot: int):
        self.engine, self.slot, self.closed = engine, slot, False

    @property
    def length(self) -> int:
        return self.engine.cache.length[self.slot]

    def close(self) -> None:
        if not self.closed:
            self.engine.cache.close(self.slot)
            self.closed = True


@dataclass
class StepEntry:
    sequence: Sequence
    tokens: list[int]
    want: list[int] | None = None      # places among `tokens` whose logits are wanted; None: the last


@dataclass
class StepIndex:
    """Device views of the last step's sequences, in entry order: their cache slots and the tokens each
    holds after the step. The sampler finds every row's state record through them without a copy."""
    slots: torch.Tensor
    pos_after: torch.Tensor

    def rows(self, keep: torch.Tensor) -> "StepIndex":
        return StepIndex(self.slots[keep].contiguous(), self.pos_after[keep].contiguous())


class StepContext:
    """What the parts see of a step: the kernels, the packed batch's index arrays, the cache."""

    def __init__(self, engine: "Engine"):
        self.engine = engine
        self.kernels = engine.kernels
        self.dtype = engine.dtype
        self.cache = engine.cache
        self.err_flag = engine.err_flag
        self.n_tokens = self.n_seqs = self.max_new = 0
        self.token_ids = self.tok_pos = self.tok_seq = self.seq_start = self.seq_pos0 = self.slots = None
        self.seq_pos_after = None
        self.block_tables: list[torch.Tensor] = []

    @property
    def kernels_f32(self):
        return self.engine.kernels_f32

    @property
    def casts(self):
        return self.engine.casts

    def decode_splits(self, n_heads: int, n_kv_heads: int, head_dim: int) -> int:
        """Over how many blocks a decode step splits each sequence's keys."""
        return self.kernels.decode.attention_splits(self.n_seqs, n_heads, n_kv_heads, head_dim, self.max_pages,
                                                    self.engine.sm_count)

    def unit_kv(self, unit: int):
        g = self.cache.group_of_unit[unit]
        k, v = self.cache.groups[g].unit_storage(unit)
        return k, v, self.block_tables[g]

    def unit_state(self, unit: int):
        """State tensor [n_slots, ...] of the unit; index it with `self.slots`."""
        return self.cache.state[unit]


class Engine:
    """One model on one GPU: weights, cache and the step function."""

    def __init__(self, layout: ModelLayout, tensors: dict, dtype, max_tokens: int, max_seqs: int | None = None,
                 device="cuda:0", use_graphs: bool = True):
        self.dtype = DTYPES[dtype]
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise StepError(f"the engine runs on a CUDA device, not on {self.device}")
        self.layout = layout
        self.kernels = KernelSet(self.dtype)
        self._kernels_f32 = self.kernels if self.dtype == torch.float32 else None
        self._casts = None
        self.model = DecoderModel(layout)
        self.model.bind(tensors, self.dtype, self.device)
        # decode steps are replayed as CUDA graphs when every mixer and feed-forward allows it
        self.use_graphs = use_graphs and self.model.graph_safe()
        self.decode_graphs = DecodeGraphs(self)
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._tickets = None
        self.last_step: StepIndex | None = None
        self.cache = None
        self.resize_cache(max_tokens, max_seqs)

    def resize_cache(self, max_tokens: int, max_seqs: int | None = None) -> None:
        """(Re)build the cache for `max_tokens` tokens held at once (each sequence's count rounded up
        to whole pages) and `max_seqs` live sequences. Only while no sequence is open."""
        if self.cache is not None and self.cache.slots.n_held:
            raise StepError("the cache cannot be resized while sequences are open")
        self.cache = None
        self.decode_graphs.clear()
        n_pages = max(1, pages_for(max_tokens))
        n_slots = max_seqs if max_seqs is not None else min(n_pages, 1024)
        self.cache = SequenceCache(self.model.cache_needs(), self.model.state_needs(), n_slots, n_pages, self.dtype,
                                   self.device)
        self.max_positions = min(self.layout.max_positions, n_pages * PAGE)
        self.model.prepare(self.max_positions, self.device)
        padded = 1
        while padded < n_slots:
            padded <<= 1
        self.tickets(padded * max([g.need.kv_heads for g in self.cache.groups] or [1]))

    def bytes_per_page(self) -> int:
        """Device bytes one page of PAGE tokens costs over all cache units."""
        width = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(units) * need.kv_heads * PAGE * need.head_dim * width
                   for need, units in ((g.need, g.units) for g in self.cache.groups))

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir, dtype="bfloat16", max_tokens: int = 4096, max_seqs: int | None = None,
                    device="cuda:0", use_graphs: bool = True) -> "Engine":
        """`model_dir`: a folder with config.json and model.safetensors, or a model that exists only as
        a configuration and a seed, `random:<config.json>[:seed[:bfloat16|float32]]`: its weights are
        drawn on the device and equal those of the folder that random-weights mode writes for the
        same configuration, seed and storage precision."""
        from .. import models  # noqa: F401  (registers the architectures)
        from ..weights.random_init import is_random_spec, parse_random_spec
        dev = torch.device(device)
        if is_random_spec(model_dir):
            import json
            spec = parse_random_spec(model_dir)
            with open(spec.config_path) as f:
                raw = json.load(f)
            archs = raw.get("architectures") or [None]
            arch = architecture_for(archs[0])
            cfg = arch.config_class.from_dict(raw, spec.config_path)
            layout = arch.layout(cfg)
            specs = DecoderModel(layout).tensor_specs()
            tensors = {}
            for i, ts in enumerate(specs):          # one at a time: the stored form of a tensor is dropped once widened
                t = _draw_one(ts, spec, i, dev)
                tensors[ts.name] = stored_to_kept(t, DTYPES[dtype]).contiguous()
        else:
            arch, cfg = load_config(model_dir)
            layout = arch.layout(cfg)
            specs = DecoderModel(layout).tensor_specs()
            tensors = load_weights(model_dir, specs, dev, DTYPES[dtype], ignore=layout.ignorable_tensors)
        eng = cls(layout, tensors, dtype, max_tokens, max_seqs, device, use_graphs)
        eng.config = cfg
        return eng

    @property
    def kernels_f32(self):
        if self._kernels_f32 is None:
            self._kernels_f32 = KernelSet(torch.float32)
        return self._kernels_f32

    @property
    def casts(self):
        if self._casts is None:
            self._casts = CastKernels()
        return self._casts

    # ------------------------------------------------------------------ sequences
    def open(self) -> Sequence:
        return Sequence(self, self.cache.open())

    def tickets(self, n: int) -> torch.Tensor:
        """Zeroed int32 counters that kernels of one stream draw tickets from and leave zero (which
        of several blocks finishes last). One buffer for the engine: its kernels run one after another.
        It is sized when the cache is (slots padded to a power of two x the most key/value heads of any
        cache unit), because captured decode steps hold its address: should a caller ever need more,
        the captured steps are dropped before the buffer is replaced, and are captured again on use."""
        if self._tickets is None or self._tickets.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise StepError(f"a part asked for {n} ticket counters while a decode step was being captured; the "
                                f"engine holds {0 if self._tickets is None else self._tickets.numel()} (ask for more "
                                "in the part's prepare())")
            self.decode_graphs.clear()
            self._tickets = torch.zeros(max(4096, 2 * n), dtype=torch.int32, device=self.device)
        return self._tickets

    def new_event(self):
        return torch.cuda.Event(enable_timing=True)

    # ------------------------------------------------------------------ the step
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Run the given tokens of every entry; returns float32 logits [wanted places, vocab] in the
        order of the entries and of each entry's `want`."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        V = self.layout.vocab_size
        seen, growth, want_rows = set(), [], []
        lens, pos0 = [], []
        row = 0
        for e in entries:
            s = e.sequence
            if s.closed or s.engine is not self:
                raise StepError("a step entry names a sequence that is closed or belongs to another engine")
            if s.slot in seen:
                raise StepError(f"the sequence in slot {s.slot} appears twice in one step")
            seen.add(s.slot)
            n = len(e.tokens)
            if n == 0:
                raise StepError("a step entry brings no tokens")
            if s.length + n > self.max_positions:
                raise StepError(f"sequence would reach {s.length + n} tokens; the engine holds at most "
                                f"{self.max_positions} per sequence")
            want = [n - 1] if e.want is None else list(e.want)
            for w in want:
                if not 0 <= w < n:
                    raise StepError(f"wanted place {w} is outside the entry's {n} tokens")
                want_rows.append(row + w)
            lens.append(n)
            pos0.append(s.length)
            growth.append((s.slot, n))
            row += n
        ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=row)
        if ids.min() < 0 or ids.max() >= V:
            bad = int(ids[(ids < 0) | (ids >= V)][0])
            raise StepError(f"token id {bad} is outside the vocabulary (0..{V - 1})")
        self.cache.reserve(growth)                      # CacheFull leaves everything as it was

        B, T = len(entries), row
        if self.use_graphs and T == B:
            slots = [e.sequence.slot for e in entries]
            tables = [self.cache.block_table(g, slots) for g in range(len(self.cache.groups))]
            logits = self.decode_graphs.run(ids, pos0, slots, tables)
            self.last_step = self.decode_graphs.last_index
            # the captured step's own buffer is overwritten by the next replay: the caller gets a copy
            if want_rows != list(range(B)):
                logits = logits[torch.as_tensor(want_rows, dtype=torch.long, device=self.device)] if want_rows else None
            else:
                logits = logits.clone()
        else:
            ctx = self._context(entries, ids, lens, pos0, want_rows)
            self.last_step = StepIndex(ctx.slots, ctx.seq_pos_after)
            logits = self._forward(ctx, want=bool(want_rows))
            if T > B:                                   # a prompt step is long enough to afford the read
                self.check_errors()
        self.cache.advance(growth)
        return logits if logits is not None else torch.empty((0, V), dtype=torch.float32, device=self.device)

    PROMPT_TOKENS_PER_STEP = 16384     # a prompt step's activations grow with its rows: longer batches go in portions

    def prompt_step(self, entries: list[StepEntry], max_tokens_per_step: int | None = None):
        """Whole prompts (or any token runs) of several sequences, in as many steps as it takes to keep
        each step at `max_tokens_per_step` rows or fewer: a sequence's run is cut into portions, each
        landing on what the portions before left in the cache. Returns the float32 logits of every
        entry's last token, [entries, vocab], and the StepIndex of those rows (for the sampler). The
        numbers are those of one big step, beyond rounding: a row sees its own sequence's keys only."""
        budget = max_tokens_per_step or self.PROMPT_TOKENS_PER_STEP
        if budget < 1:
            raise StepError("a step needs room for at least one token")
        if sum(len(e.tokens) for e in entries) <= budget:
            logits = self.step([StepEntry(e.sequence, e.tokens) for e in entries])
            return logits, self.last_step
        rows: list[torch.Tensor | None] = [None] * len(entries)
        done = [0] * len(entries)
        nxt = 0
        while nxt < len(entries):
            step, room, finishing = [], budget, []
            i = nxt
            while i < len(entries) and room > 0:
                toks = entries[i].tokens
                take = min(room, len(toks) - done[i])
                last = done[i] + take == len(toks)
                step.append(StepEntry(entries[i].sequence, toks[done[i]:done[i] + take], [take - 1] if last else []))
                done[i] += take
                room -= take
                if last:
                    finishing.append(i)
                    i += 1
                else:
                    break
            out = self.step(step)
            for j, k in enumerate(finishing):
                rows[k] = out[j:j + 1]
            nxt = i
        slots = torch.tensor([e.sequence.slot for e in entries], dtype=torch.int32)
        held = torch.tensor([e.sequence.length for e in entries], dtype=torch.int32)
        both = torch.stack([slots, held]).pin_memory().to(self.device, non_blocking=True)
        self.last_step = StepIndex(both[0], both[1])
        return torch.cat(rows), self.last_step

    def activation_reserve_bytes(self) -> int:
        """A generous bound on what a prompt step of PROMPT_TOKENS_PER_STEP rows allocates beside
        weights and cache (residual, products' outputs), plus the logits of the captured decode steps:
        what the cache must leave free."""
        width = 64 * self.layout.hidden_size                        # bytes a row, all buffers of a layer alive at once
        return self.PROMPT_TOKENS_PER_STEP * width + 4 * self.layout.vocab_size * 4 * 1024

    def check_errors(self) -> None:
        """Raises if a kernel of an earlier step reported an error (a wait on the device that ran out
        of time, a token id out of range). Reading the flag waits for the stream, so replayed decode
        steps do not do it themselves: the generation loop asks once per batch, trace replay after
        every step, and every prompt step asks for itself."""
        if int(self.err_flag) != 0:
            self.err_flag.zero_()
            raise StepError("a kernel reported an error during a step (a wait on the device ran out of time, or a "
                            "token id was out of range)")

    def decode_step_device(self, sequences: list[Sequence], ids: torch.Tensor) -> torch.Tensor:
        """One token for each of `sequences`, the ids taken from an int32 device tensor (what the
        sampler just wrote), logits of every row back. Lets a caller launch the next step before it
        has read the last step's tokens. Only for engines that replay their decode step. The logits
        are the captured step's own buffer: they hold until the next decode step is launched (sample
        from them first, as the generation loop does, or copy them)."""
        if not self.use_graphs:
            raise StepError("this engine does not replay its decode step; feed token ids from the host")
        if ids.dtype != torch.int32 or ids.device != self.device or ids.shape[0] != len(sequences):
            raise StepError("ids must be an int32 tensor on the engine's device, one per sequence")
        seen = set()
        for s in sequences:
            if s.closed or s.engine is not self or s.slot in seen:
                raise StepError("a sequence is closed, foreign, or named twice")
            seen.add(s.slot)
            if s.length + 1 > self.max_positions:
                raise StepError(f"sequence would reach {s.length + 1} tokens; the engine holds at most {self.max_positions}")
        growth = [(s.slot, 1) for s in sequences]
        self.cache.reserve(growth)
        slots = [s.slot for s in sequences]
        tables = [self.cache.block_table(g, slots) for g in range(len(self.cache.groups))]
        logits = self.decode_graphs.run(ids.contiguous(), [s.length for s in sequences], slots, tables)
        self.last_step = self.decode_graphs.last_index
        self.cache.advance(growth)
        return logits

    def _forward(self, ctx: StepContext, want: bool):
        """The model on the rows of `ctx`: embedding, the scheduled blocks, and for the wanted rows the
        final norm and the output head."""
        residual = self.model.embedding.forward(ctx.token_ids, ctx)
        delta = None
        schedule, blocks, rows = self.layout.schedule, self.model.blocks, residual.shape[0]
        for i, e in enumerate(schedule):
            block = blocks[e.layer]
            nxt = blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            if getattr(block, "folds_entry", False) and nxt is not None and getattr(nxt, "folds_entry", False):
                # the layer behind this one says what its first norm would let this layer's last sublayer prepare
                delta = block.forward(residual, delta, ctx, e.cache_unit, e.writes_cache,
                                      next_fold=lambda before, nxt=nxt: nxt.entry_fold(ctx, rows, residual, before))
            else:
                delta = block.forward(residual, delta, ctx, e.cache_unit, e.writes_cache)
        if not want:
            return None
        normed = self.model.final_norm.forward(residual, delta, ctx, rows=ctx.want_rows)
        return self.model.head.forward(normed, ctx)

    def _context(self, entries, ids, lens, pos0, want_rows) -> StepContext:
        B, T = len(lens), int(ids.shape[0])
        lens_a = np.asarray(lens, dtype=np.int32)
        pos0_a = np.asarray(pos0, dtype=np.int32)
        seq_start = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(lens_a, out=seq_start[1:])
        tok_seq = np.repeat(np.arange(B, dtype=np.int32), lens_a)
        tok_pos = (np.arange(T, dtype=np.int32) - seq_start[tok_seq] + pos0_a[tok_seq]).astype(np.int32)
        slots = [e.sequence.slot for e in entries]
        tables = [self.cache.block_table(g, slots) for g in range(len(self.cache.groups))]
        pieces = [ids.astype(np.int32), tok_pos, tok_seq, seq_start, pos0_a, np.asarray(slots, dtype=np.int32),
                  np.asarray(want_rows, dtype=np.int32), pos0_a + lens_a] + [t.reshape(-1) for t in tables]
        sizes = [p.shape[0] for p in pieces]
        host = torch.from_numpy(np.concatenate(pieces)).pin_memory()
        dev = host.to(self.device, non_blocking=True)
        views, off = [], 0
        for n in sizes:
            views.append(dev[off:off + n])
            off += n
        ctx = StepContext(self)
        ctx.n_tokens, ctx.n_seqs, ctx.max_new = T, B, int(lens_a.max())
        ctx.token_ids, ctx.tok_pos, ctx.tok_seq, ctx.seq_start, ctx.seq_pos0, ctx.slots, ctx.want_rows, ctx.seq_pos_after = views[:8]
        ctx.block_tables = [v.view(B, t.shape[1]) for v, t in zip(views[8:], tables)]
        ctx.is_decode = bool((lens_a == 1).all())
        ctx.max_pages = int(-(-(int((pos0_a + lens_a).max())) // PAGE))
        ctx._host_keepalive = host
        return ctx
