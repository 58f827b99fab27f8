"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

A `Row` is one request's share of a step: any number >= 1 of new tokens at positions
`start, start + 1, ...`, everything before `start` being in the cache already, and `want`, the
places among these tokens whose logits are asked for. A step may mix whole prompts, portions
of prompts cut anywhere and single decoded tokens; all rows run as one flat batch of T tokens
with no padding, the keys and values of every token are written to the request's pages, and
the function returns float32 logits [number of wanted places, vocab] in the order of the rows
and of `want` (atomserve/runner.py:42-56, 87-180 is the reference's form of this contract).

The runner reads requests and never changes them: reserving pages before a step and
advancing counters after it belong to the caller (the scheduler, or the trace replayer).

Everything the kernels need to know about the batch is packed into one int32 buffer on the
host and copied to the device once per step (atomserve/runner.py:215-241). Steps made only of
single tokens are replayed from CUDA graphs, captured per (requests, table width) bucket.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field

import numpy as np
import torch

from atomserve_b200.cache.manager import CacheManager, RequestCache
from atomserve_b200.ops.library import launches, note_replay
from atomserve_b200.ops.status import status_for
from atomserve_b200.parts.base import CacheView, StepContext
from atomserve_b200.parts.model import DecoderModel


@dataclass
class Row:
    tokens: list[int]
    start: int
    cache: RequestCache
    want: list[int] = field(default_factory=list)  # indices into `tokens`


def slot_of(block_table: list[int], position: int, block_size: int) -> int:
    """Cache slot of `position`: page * block_size + offset (atomserve/runner.py:37-39)."""
    return block_table[position // block_size] * block_size + position % block_size


def _round_up(n: int, to: int) -> int:
    return -(-n // to) * to


class _Packed:
    """Lays several int32 arrays out in one buffer; the same names and sizes give the same
    offsets, so a captured graph finds its inputs where it left them."""

    def __init__(self):
        self.parts: list[tuple[str, int, int]] = []
        self.size = 0

    def add(self, name: str, length: int) -> None:
        self.parts.append((name, self.size, length))
        self.size += _round_up(max(length, 1), 4)  # 16-byte aligned parts

    def views(self, buffer: torch.Tensor) -> dict[str, torch.Tensor]:
        return {name: buffer[off : off + n] for name, off, n in self.parts}


GRAPH_BATCHES = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def batch_bucket(requests: int) -> int | None:
    """The number of requests a decode graph is captured for: the batch rounded up to a few
    sizes and padded with dummy requests; None beyond the largest."""
    for b in GRAPH_BATCHES:
        if b >= requests:
            return b
    return None


def width_bucket(pages: int) -> int:
    """Block-table width of a decode graph: the pages of the longest request, to a power of two."""
    width = 16
    while width < pages:
        width *= 2
    return width


def context_bucket(max_context: int) -> int:
    """The longest context rounded up by less than 256 keys or at most a quarter. The attention kernels size their
    key partitions for the rounded value, so a coarser bucket would leave partitions empty."""
    step = 256 if max_context <= 2048 else (512 if max_context <= 8192 else 1024)
    return -(-max_context // step) * step


class GraphCache:
    """Captured decode graphs by shape key, at most `limit` of them: the one unused longest is
    dropped when a new one comes, and with it the memory only it held. All graphs write their
    logits into one buffer that the runner owns, so a graph keeps nothing of its own but its
    kernels' arguments."""

    def __init__(self, limit: int = 48):
        self.limit = limit
        self._entries: OrderedDict[tuple, tuple] = OrderedDict()

    def __len__(self) -> int:
        return len(self._entries)

    def get(self, key: tuple):
        entry = self._entries.get(key)
        if entry is not None:
            self._entries.move_to_end(key)
        return entry

    def put(self, key: tuple, entry: tuple) -> None:
        self._entries[key] = entry
        self._entries.move_to_end(key)
        while len(self._entries) > self.limit:
            self._entries.popitem(last=False)

    def clear(self) -> None:
        self._entries.clear()


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, cuda_graphs: bool = True):
        self.model, self.cache = model, cache
        self.device = model.device
        self.block_size = cache.block_size
        # how kernels report that they could not finish (none on the CPU stand-ins of the tests)
        self.device_status = status_for(self.device) if self.device.type == "cuda" else None
        self.views: list[CacheView | None] = [cache.entry_view(i) for i in range(len(model.schedule))]
        # Graphs replay the same kernels on new inputs; a part that updates state of its own in
        # place would be run again by capture and warm-up, so such models step eagerly.
        self.use_graphs = cuda_graphs and self.device.type == "cuda" and not cache.entry_state
        self._copy_done: torch.cuda.Event | None = None
        self._graphs = GraphCache()
        self._graph_pool = None
        self._graph_logits: torch.Tensor | None = None  # [largest batch bucket met, vocab]: every graph's output
        # request uid -> (generation, per group a numpy copy of its block table, extended as it grows)
        self._tables: dict[int, tuple[int, list[np.ndarray]]] = {}
        # decode steps: per group a host matrix [state slot, page] of the live requests' block tables,
        # kept up to date row by row, so that a step's tables are one gather instead of a loop of copies
        self._matrix: list[np.ndarray] = [np.zeros((0, 0), dtype=np.int32) for _ in cache.groups]
        self._row_owner: list[dict[int, tuple[int, int, int]]] = [{} for _ in cache.groups]  # slot -> (uid, generation, pages held)
        self._host: torch.Tensor | None = None
        self._dev: torch.Tensor | None = None
        self.last_upload_bytes = 0  # size of the last step's packed host-to-device copy

    # ---- building the batch ---------------------------------------------------------------------

    def validate(self, rows: list[Row]) -> None:
        bs = self.block_size
        vocab = self.model.spec.vocab_size
        groups = self.cache.groups
        for r in rows:
            tokens = r.tokens
            n = len(tokens)
            if n < 1:
                raise ValueError("a row must bring at least one token")
            lowest, highest = (tokens[0], tokens[0]) if n == 1 else (min(tokens), max(tokens))
            if lowest < 0 or highest >= vocab:
                raise ValueError(f"a token id lies outside [0, {vocab})")
            if r.start < 0:
                raise ValueError(f"a row starts at position {r.start}")
            for w in r.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted places {r.want} lie outside the row's {n} tokens")
            if len(r.cache.block_tables) != len(groups):
                raise ValueError("the row's request has block tables for another set of cache groups")
            for g, table in zip(groups, r.cache.block_tables):
                if (r.start + n) > len(table) * bs:
                    raise ValueError(f"block table holds {len(table) * bs} slots, the row needs {r.start + n}")
                if g.window is not None:  # only windows release pages before a request ends
                    first = self.cache.first_needed_block(g, r.start)
                    if any(b < 0 for b in table[first : -(-(r.start + n) // bs)]):
                        raise ValueError("a page the row still reads has been released")

    def _table_array(self, rc: RequestCache, g: int) -> np.ndarray:
        """The request's block table of group g as int32, kept between steps and extended by the
        pages added since (entries a window released keep their old page id: never read)."""
        entry = self._tables.get(rc.uid)
        if entry is None or entry[0] != rc.generation:  # new, or freed and started again
            if len(self._tables) > 4096:
                self._tables.clear()
            entry = self._tables[rc.uid] = (rc.generation, [np.zeros(0, dtype=np.int32) for _ in rc.block_tables])
        cached = entry[1]
        table, have = rc.block_tables[g], cached[g]
        if len(table) > len(have):
            have = np.concatenate([have, np.asarray(table[len(have) :], dtype=np.int32)])
        cached[g] = have
        return have

    def _table_matrix(self, g: int, rows: list[Row], slot_ids: list[int], width: int) -> np.ndarray:
        """Group g's matrix with the rows of these requests (each in its state slot) brought up to
        date: a row is zeroed when its slot passes to another request or the request starts again,
        and takes the pages added since (entries a window released keep their old id: never read)."""
        m = self._matrix[g]
        need_rows, need_cols = max(slot_ids) + 1, width
        if m.shape[0] < need_rows or m.shape[1] < need_cols:
            grown = np.zeros((max(need_rows, m.shape[0]), max(2 * need_cols, m.shape[1])), dtype=np.int32)
            grown[: m.shape[0], : m.shape[1]] = m
            m = self._matrix[g] = grown
            for slot, (uid, generation, held) in list(self._row_owner[g].items()):
                self._row_owner[g][slot] = (uid, generation, min(held, m.shape[1]))
        owners = self._row_owner[g]
        cap = m.shape[1]
        for r, slot in zip(rows, slot_ids):
            rc = r.cache
            table = rc.block_tables[g]
            owner = owners.get(slot)
            if owner is None or owner[0] != rc.uid or owner[1] != rc.generation:
                m[slot, :] = 0
                held = 0
            else:
                held = owner[2]
                if held >= len(table):
                    continue
            upto = min(len(table), cap)
            m[slot, held:upto] = table[held:upto]
            owners[slot] = (rc.uid, rc.generation, upto)
        return m

    def _layout(self, T: int, R: int, W: list[int], B: int) -> _Packed:
        lay = _Packed()
        lay.add("token_ids", T)
        lay.add("positions", T)
        lay.add("req_q_start", R + 1)
        lay.add("req_pos_start", R)
        lay.add("state_slots", R)
        lay.add("logits_rows", B)
        for g, w in enumerate(W):
            lay.add(f"slots{g}", T)
            lay.add(f"tables{g}", R * w)
        return lay

    def _buffers(self, size: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self._host is None or self._host.shape[0] < size:
            cap = max(size, 1 << 16)
            pin = self.device.type == "cuda"
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=pin)
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._graphs.clear()  # captured graphs point into the old buffer
        return self._host, self._dev

    def prepare(self, rows: list[Row], pad_requests: int | None = None, pad_width: int | None = None):
        """Pack the rows; returns (ctx, per-group (slots, tables), layout key).

        `pad_requests` (decode-only steps) appends dummy single-token requests up to that count:
        token 0 at position 0, nothing stored (slot -1), an all-zero block table, and a wanted
        row each, so that a few captured graph shapes serve every batch size. Their logits are
        computed and dropped by the caller."""
        self.validate(rows)
        bs = self.block_size
        real = len(rows)
        pad = max(0, (pad_requests or 0) - real)
        R = real + pad
        T = sum(len(r.tokens) for r in rows) + pad
        widths = []
        for g in range(len(self.cache.groups)):
            w = max(-(-(r.start + len(r.tokens)) // bs) for r in rows)
            widths.append(pad_width if pad_width is not None else w)
        B = sum(len(r.want) for r in rows) + pad
        lay = self._layout(T, R, widths, B)
        host, dev = self._buffers(lay.size)
        if self._copy_done is not None:
            self._copy_done.synchronize()  # the last step's upload has left the host buffer
        hv = lay.views(host)
        tok, pos = hv["token_ids"].numpy(), hv["positions"].numpy()
        qs, ps, ss, lr = (hv[k].numpy() for k in ("req_q_start", "req_pos_start", "state_slots", "logits_rows"))
        flat = b = 0
        max_context = 0
        single = T == R  # every row brings one token (a decode step): no per-token loops
        if single:
            starts = [r.start for r in rows]
            tok[:real] = [r.tokens[0] for r in rows]
            pos[:real] = starts
            ps[:real] = starts
            qs[:real] = range(real)
            ss[:real] = [r.cache.state_slot for r in rows]
            for i, r in enumerate(rows):
                if r.want:
                    lr[b] = i
                    b += 1
            flat = real
            max_context = max(starts) + 1
        for i, r in enumerate(() if single else rows):
            n = len(r.tokens)
            tok[flat : flat + n] = r.tokens
            pos[flat : flat + n] = range(r.start, r.start + n)
            qs[i], ps[i], ss[i] = flat, r.start, r.cache.state_slot
            for w in r.want:
                lr[b] = flat + w
                b += 1
            flat += n
            max_context = max(max_context, r.start + n)
        for i in range(real, R):  # padding requests
            tok[flat], pos[flat], qs[i], ps[i], ss[i], lr[b] = 0, 0, flat, 0, 0, flat
            flat += 1
            b += 1
        qs[R] = flat
        slot_ids = [r.cache.state_slot for r in rows] if single else []
        gather = single and real > 0 and min(slot_ids) >= 0  # every request sits in a state slot of its own
        for g, width in enumerate(widths):
            slots, tables = hv[f"slots{g}"].numpy(), hv[f"tables{g}"].numpy().reshape(R, width)
            flat = 0
            if gather:
                m = self._table_matrix(g, rows, slot_ids, width)
                at, first = np.asarray(slot_ids), np.asarray(starts)
                tables[:real] = m[at, :width]
                slots[:real] = m[at, first // bs].astype(np.int64) * bs + first % bs
                flat = real
            for i, r in enumerate(() if gather else rows):
                table = self._table_array(r.cache, g)
                n = len(r.tokens)
                used = min(len(table), width)
                tables[i, :used] = table[:used]
                tables[i, used:] = 0
                if n == 1:
                    slots[flat] = int(table[r.start // bs]) * bs + r.start % bs
                else:
                    p = np.arange(r.start, r.start + n)
                    slots[flat : flat + n] = table[p // bs].astype(np.int64) * bs + p % bs
                flat += n
            if pad:
                tables[real:] = 0
                slots[flat : flat + pad] = -1
        dev[: lay.size].copy_(host[: lay.size], non_blocking=True)
        self.last_upload_bytes = lay.size * 4
        if self.device.type == "cuda":
            self._copy_done = torch.cuda.Event()
            self._copy_done.record()
        dv = lay.views(dev)
        ctx = StepContext(
            num_tokens=T, num_requests=R, token_ids=dv["token_ids"], positions=dv["positions"],
            req_q_start=dv["req_q_start"], req_pos_start=dv["req_pos_start"],
            state_slots=dv["state_slots"], logits_rows=dv["logits_rows"], max_context=max_context,
            host_q_lens=[len(r.tokens) for r in rows] + [1] * pad, host_pos_start=[r.start for r in rows] + [0] * pad,
            host_state_slots=[r.cache.state_slot for r in rows] + [0] * pad,
        )  # fmt: skip
        groups = [(dv[f"slots{g}"], dv[f"tables{g}"].view(R, w)) for g, w in enumerate(widths)]
        return ctx, groups, (T, R, tuple(widths), B)

    def _bind(self, groups) -> None:
        for i, view in enumerate(self.views):
            if view is not None and i in self.cache.entry_group:
                g, _ = self.cache.entry_group[i]
                view.slots, view.block_tables = groups[g]

    # ---- running --------------------------------------------------------------------------------

    @torch.inference_mode()
    def step(self, rows: list[Row], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run one step; float32 logits [sum(len(row.want)), vocab]. `device_tokens` (int32, one
        per row, on the device) stands in for the rows' token ids where the host does not know
        them yet: a step of single tokens launched before its predecessor's sampled ids were read;
        the rows then carry placeholders."""
        if not rows:
            return torch.empty(0, self.model.spec.vocab_size, device=self.device, dtype=torch.float32)
        if device_tokens is not None and (device_tokens.shape[0] != len(rows) or any(len(r.tokens) != 1 for r in rows)):
            raise ValueError("tokens from the device are one per row of a step of single tokens")
        if self.use_graphs and all(len(r.tokens) == 1 for r in rows):
            return self._step_graph(rows, device_tokens)
        ctx, groups, _ = self.prepare(rows)
        if device_tokens is not None:
            ctx.token_ids[: len(rows)].copy_(device_tokens)
        self._bind(groups)
        return self.model.forward(ctx, self.views)

    def _step_graph(self, rows: list[Row], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Decode-only step through a captured graph. The graph is keyed by everything that
        fixes kernel shapes and buffer offsets: requests (rounded up to a bucket and padded with
        dummy requests when every row wants its logits, as in generation), table width (rounded
        up to a power of two), wanted rows, and the bucket of the longest context (which sets
        the key partitions). At most GraphCache.limit graphs are kept, and they share one pool of
        memory and one logits buffer, [the batch bucket of the engine's sequence limit, vocab] float32: 39 MB at 64 requests
        of a 151,936-token vocabulary, 156 MB at 256. The returned logits are a view of that
        buffer: read them before the next step."""
        bs = self.block_size
        pad_w = width_bucket(max(-(-(r.start + 1) // bs) for r in rows))
        wanted = sum(len(r.want) for r in rows)
        pad_r = batch_bucket(len(rows)) if wanted == len(rows) else None
        ctx, groups, key = self.prepare(rows, pad_requests=pad_r, pad_width=pad_w)
        if device_tokens is not None:  # behind the upload, before anything reads the ids
            ctx.token_ids[: len(rows)].copy_(device_tokens)
        ctx.max_context = context_bucket(ctx.max_context)
        key = (*key, ctx.max_context)
        self._bind(groups)
        out_rows = key[3]
        if self._graph_logits is None or self._graph_logits.shape[0] < out_rows:
            # once, for the largest batch the state slots allow (a batch that grows step by step
            # would otherwise replace the buffer, and with it every graph, at each new bucket)
            largest = batch_bucket(min(self.cache.state.num_slots, GRAPH_BATCHES[-1])) or GRAPH_BATCHES[-1]
            self._graphs.clear()  # they write into the buffer that is being replaced
            self._graph_logits = torch.empty(max(out_rows, largest), self.model.spec.vocab_size, device=self.device, dtype=torch.float32)
        logits = self._graph_logits[:out_rows]
        entry = self._graphs.get(key)
        if entry is None:
            # warm up outside capture (lazy library initialisation must not be captured)
            self.model.forward(ctx, self.views, logits)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                # one memory pool for all graphs: only one of them runs at a time
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = launches()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                self.model.forward(ctx, self.views, logits)
            entry = (graph, launches() - before)
            self._graphs.put(key, entry)
        graph, recorded = entry
        graph.replay()
        note_replay(recorded)  # the replay ran what the capture recorded
        return logits[:wanted]


def rows_for(seqs, num_new_tokens: list[int]) -> list[Row]:
    """The usual rows of a scheduled step: each sequence's next uncomputed tokens, with logits
    wanted at the last one only if that reaches the end of its known tokens
    (atomserve/runner.py:59-68)."""
    rows = []
    for seq, n in zip(seqs, num_new_tokens, strict=True):
        start, tokens = seq.num_computed_tokens, seq.token_ids
        known = len(tokens)
        if n < 1 or start + n > known:
            raise ValueError(f"cannot run tokens {start}:{start + n} of {known}")
        rows.append(Row(tokens[start : start + n], start, seq.cache, [n - 1] if start + n == known else []))
    return rows
