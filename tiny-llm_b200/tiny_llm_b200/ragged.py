"""Ragged batches: one model step over several requests, each bringing any number of new tokens.

A continuous-batching step is a flat list of tokens: a portion of one request's prompt beside single decoded tokens of
others.  ``RaggedEntry`` names one request's share, ``RaggedPlan`` is what the kernels need, built on the host from the
requests' page lists and moved to the device as ONE pinned block:

    ids [T] | tok_pos [T] | tok_seq [T] | want_rows [W] | block_table [S, max_pages] | tiles [n, 3] per tile size | seq_info [S, 4]

``tok_pos`` is the position of a token in its sequence, ``tok_seq`` its row in this step's block table, ``tiles`` the
attention kernels' work lists (runs of at most ``tile`` consecutive tokens of one sequence; one list per tile size
the model's layers ask for, ``tiles_for(size)``), ``seq_info`` one row per sequence for kernels that walk a sequence's new
tokens in order (first flat token, token count, position of the first token, the request's recurrent-state slot or -1).
Building the plan also
does the step's cache bookkeeping: every request's page list grows by its new tokens (pages come from the pool's free
list first), before anything is launched.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch


@dataclass
class RaggedEntry:
    tokens: Sequence[int]
    cache: list                       # the request's per-layer caches (model.create_kv_cache())
    want: Sequence[int] | None = None  # places among `tokens` whose logits are wanted; None = the last one


class RaggedPlan:
    @staticmethod
    def block_ints(tokens: int, wanted: int, seqs: int, max_pages: int, tiles: int) -> int:
        """Number of int32 in a plan's device block (``tiles`` summed over the tile sizes)."""
        return 3 * tokens + wanted + seqs * max_pages + 3 * tiles + 4 * seqs

    def __init__(self, entries: Sequence[RaggedEntry], device, tile, max_pages: int | None = None, into: torch.Tensor | None = None):
        """``max_pages`` fixes the block table's width (at least what the longest request needs) and ``into`` names a
        preallocated int32 device block to upload into: a captured graph reads the same addresses every step."""
        sizes = sorted({int(tile)} if isinstance(tile, int) else {int(t) for t in tile})
        owners = []
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError("a ragged entry needs at least one token")
            owner = getattr(e.cache[0], "owner", e.cache[0])
            if any(owner is o for o in owners):
                raise ValueError("a request may appear once per step")
            owners.append(owner)
        starts = [o.offset for o in owners]
        done = []
        try:
            for o, e in zip(owners, entries):
                o.append_slots(len(e.tokens))
                done.append((o, len(e.tokens)))
        except Exception:
            for o, n in done:  # all-or-nothing: give the pages of this step back
                o.rewind(n)
            raise
        T = sum(len(e.tokens) for e in entries)
        S = len(entries)
        needed = max(o.num_pages for o in owners)
        if max_pages is not None and max_pages < needed:
            for o, n in done:
                o.rewind(n)
            raise ValueError(f"block table of {max_pages} pages, {needed} needed")
        max_pages = needed if max_pages is None else max_pages
        wants = [list(e.want) if e.want is not None else [len(e.tokens) - 1] for e in entries]
        W = sum(len(w) for w in wants)
        n_tiles = {size: sum(-(-len(e.tokens) // size) for e in entries) for size in sizes}
        total = self.block_ints(T, W, S, max_pages, sum(n_tiles.values()))
        host = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=torch.cuda.is_available() and torch.device(device).type == "cuda")
        buf = host.numpy()
        ids, pos, seq = buf[0:T], buf[T : 2 * T], buf[2 * T : 3 * T]
        want = buf[3 * T : 3 * T + W]
        table = buf[3 * T + W : 3 * T + W + S * max_pages].reshape(S, max_pages)
        table[:] = -1
        tile_at, at = {}, 3 * T + W + S * max_pages
        for size in sizes:
            tile_at[size] = (at, n_tiles[size])
            at += 3 * n_tiles[size]
        info = buf[at : at + 4 * S].reshape(S, 4)
        tile_rows = {size: [] for size in sizes}
        t = w = 0
        for s, (e, o, start) in enumerate(zip(entries, owners, starts)):
            n = len(e.tokens)
            ids[t : t + n] = np.asarray(e.tokens, dtype=np.int64)
            pos[t : t + n] = np.arange(start, start + n, dtype=np.int64)
            seq[t : t + n] = s
            for place in wants[s]:
                if not 0 <= place < n:
                    raise ValueError(f"wanted place {place} is outside the entry's {n} tokens")
                want[w] = t + place
                w += 1
            for size in sizes:
                tile_rows[size] += [(t + first, min(size, n - first), s) for first in range(0, n, size)]
            table[s, : o.num_pages] = o.page_ids
            info[s] = (t, n, start, getattr(o, "state_slot", -1))
            t += n
        for size in sizes:
            start, n = tile_at[size]
            buf[start : start + 3 * n] = np.asarray(tile_rows[size], dtype=np.int32).reshape(-1)
        self.num_tokens, self.num_seqs, self.num_want, self.max_pages = T, S, W, max_pages
        self.h2d_bytes = total * 4
        if into is None:
            dev = host.to(device, non_blocking=True)
        else:
            if into.numel() != total or into.dtype != torch.int32:
                raise ValueError("the device block does not fit this plan")
            dev = into
            dev.copy_(host[:total], non_blocking=True)
        self.total_ints = total
        self._host = host  # keep the pinned block alive until the copy has run
        self.ids, self.tok_pos, self.tok_seq = dev[0:T], dev[T : 2 * T], dev[2 * T : 3 * T]
        self.want_rows = dev[3 * T : 3 * T + W]
        self.block_table = dev[3 * T + W : 3 * T + W + S * max_pages].view(S, max_pages)
        self._tiles = {size: dev[start : start + 3 * n].view(n, 3) for size, (start, n) in tile_at.items()}
        self.seq_info = dev[at : at + 4 * S].view(S, 4)
        self.tiles = self._tiles[sizes[0]]
        self.max_context = max(o.offset for o in owners)  # the longest sequence after this step's append
        self.want_counts = [len(x) for x in wants]
        self.starts = starts
        self.max_tokens = max(len(e.tokens) for e in entries)  # the longest entry of the step
        self.owners = owners
        for o in owners:  # from here on the step runs: what it consumes cannot be taken back from a recurrent state
            if hasattr(o, "ran_offset"):
                o.ran_offset = o.offset

    def rope_tables(self, dims: int, base: float, factor: float = 1.0):
        """(cos, sin) fp32 ``[T, dims // 2]`` of this step's token positions, made once per step and rotation."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        key = (int(dims), float(base), float(factor))
        tables = self.__dict__.setdefault("_rope_tables", {})
        if key not in tables:
            tables[key] = blocks.rope_table(self.tok_pos, dims=key[0], base=key[1], factor=key[2])
        return tables[key]

    def tiles_for(self, size: int) -> torch.Tensor:
        """The work list cut into runs of at most ``size`` tokens (one of the sizes the plan was built for)."""
        return self._tiles[size]
