"""CUDA graphs of the decode step.

A decode step launches a few hundred small kernels whose sizes depend only on the batch size, so
it is captured once per (padded batch size, block-table width) and replayed: the step's index
arrays live in one static device buffer that is refreshed from pinned host memory before each
replay. Rows added to fill the batch up to its padded size read and write a spare cache page and a
spare state slot of their own, so they change nothing a real row sees.
"""
from __future__ import annotations

import gc

import numpy as np
import torch

from ..cache.needs import PAGE


def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


class DecodeGraph:
    def __init__(self, engine, batch: int, width: int):
        from .step import StepContext
        self.engine, self.batch, self.width = engine, batch, width
        n_groups = len(engine.cache.groups)
        B = batch
        # layout of the index buffer (int32): ids, pos, seq, seq_start, pos0, slots, want_rows, pos after, block tables
        self.sizes = [B, B, B, B + 1, B, B, B, B] + [B * width] * n_groups
        total = sum(self.sizes)
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=engine.device)
        self.copied = torch.cuda.Event()
        views, off = [], 0
        for n in self.sizes:
            views.append(self.dev[off:off + n])
            off += n
        ctx = StepContext(engine)
        ctx.n_tokens = ctx.n_seqs = B
        ctx.max_new = 1
        ctx.token_ids, ctx.tok_pos, ctx.tok_seq, ctx.seq_start, ctx.seq_pos0, ctx.slots, ctx.want_rows, ctx.seq_pos_after = views[:8]
        ctx.block_tables = [v.view(B, width) for v in views[8:]]
        ctx.is_decode = True
        ctx.max_pages = width
        self.ctx = ctx
        self._fill_host([], [], [], [])
        self.dev.copy_(self.host)
        # warm-up outside capture (lazy attribute calls, allocator growth), then capture
        side = torch.cuda.Stream(device=engine.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            engine._forward(ctx, want=True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..csrc import bindings
        before = bindings.LAUNCHES[0]
        self.graph = torch.cuda.CUDAGraph()
        # No garbage collection while the capture is under way: the graphs of an engine that is no longer
        # in use (they hang in reference cycles) would be destroyed whenever the collector happens to
        # run, and destroying a graph is not permitted while any stream captures; it invalidates the capture.
        # What is garbage now is collected before.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=engine.decode_graphs.pool):
                self.logits = engine._forward(ctx, want=True)
        finally:
            if collecting:
                gc.enable()
        self.kernels_per_replay = bindings.LAUNCHES[0] - before

    def _fill_host(self, ids, pos0, slots, tables):
        B, W, eng = self.batch, self.width, self.engine
        n = len(ids)
        h = self.host.numpy()
        off = 0
        h[off:off + B] = 0
        h[off:off + n] = ids
        off += B
        h[off:off + B] = 0
        h[off:off + n] = pos0
        off += B
        h[off:off + B] = np.arange(B)
        off += B
        h[off:off + B + 1] = np.arange(B + 1)
        off += B + 1
        h[off:off + B] = 0
        h[off:off + n] = pos0
        off += B
        h[off:off + B] = eng.cache.n_slots            # the spare state slot
        h[off:off + n] = slots
        off += B
        h[off:off + B] = np.arange(B)
        off += B
        h[off:off + B] = 1
        h[off:off + n] = np.asarray(pos0, dtype=np.int64) + 1 if n else 0
        off += B
        for g in range(len(eng.cache.groups)):
            tab = h[off:off + B * W].reshape(B, W)
            tab[:] = eng.cache.n_pages               # the spare page
            if n:
                t = tables[g]
                tab[:n, :t.shape[1]] = np.where(t >= 0, t, eng.cache.n_pages)
            off += B * W

    def run(self, ids, pos0, slots, tables) -> torch.Tensor:
        """`ids`: token ids on the host (a sequence of ints), or an int32 device tensor (the sampler's
        output fed straight back, so that the host need not have seen the tokens yet)."""
        self.copied.synchronize()
        on_device = isinstance(ids, torch.Tensor)
        n = ids.shape[0] if on_device else len(ids)
        self._fill_host([0] * n if on_device else ids, pos0, slots, tables)
        if on_device:
            B = self.batch
            self.dev[B:].copy_(self.host[B:], non_blocking=True)        # everything but the ids
            self.dev[:n].copy_(ids)
            if n < B:
                self.dev[n:B].zero_()
        else:
            self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        self.graph.replay()
        from ..csrc import bindings
        bindings.LAUNCHES[0] += self.kernels_per_replay
        return self.logits[:n]

    def index(self, n: int):
        from .step import StepIndex
        return StepIndex(self.ctx.slots[:n], self.ctx.seq_pos_after[:n])

    @property
    def h2d_bytes(self) -> int:
        """Bytes copied to the device before each replay when the token ids are there already."""
        return 4 * (self.host.numel() - self.batch)


class DecodeGraphs:
    """The graphs of one engine, captured on first use. They share one memory pool (their replays
    never overlap: one stream, one step after another), so a graph's buffers, its logits included,
    hold a step's values only until the next replay of any of them. At most MAX_GRAPHS are kept;
    the one replayed longest ago goes first."""
    MAX_GRAPHS = 48

    def __init__(self, engine):
        self.engine = engine
        self.graphs: dict[tuple[int, int], DecodeGraph] = {}
        self.pool = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None
        self.last_index = None
        self.last_graph: DecodeGraph | None = None

    def clear(self):
        self.graphs.clear()

    def run(self, ids, pos0, slots, tables) -> torch.Tensor:
        need = max(1, max(t.shape[1] for t in tables)) if tables else 1
        cap = -(-self.engine.max_positions // PAGE)
        width = min(max(8, _next_pow2(need)), max(cap, need))
        batch = _next_pow2(ids.shape[0] if isinstance(ids, torch.Tensor) else len(ids))
        key = (batch, width)
        g = self.graphs.pop(key, None)
        if g is None:
            while len(self.graphs) >= self.MAX_GRAPHS:
                self.graphs.pop(next(iter(self.graphs)))          # the dict is kept in order of last use
            g = DecodeGraph(self.engine, batch, width)
        self.graphs[key] = g
        out = g.run(ids, pos0, slots, tables)
        self.last_graph, self.last_index = g, g.index(out.shape[0])
        return out
