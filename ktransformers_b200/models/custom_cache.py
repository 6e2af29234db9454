"""StaticCache — the paged latent KV cache of absorbed MLA (archive/ktransformers/models/custom_cache.py:26-200).

Same contract as the reference's DeepSeek branch: per layer one buffer `[max_pages, page_size, 1, kv_lora_rank + rope]`
(page_size 64), a static identity page table per batch row, `update(ckv, k_pe, layer_idx, {"cache_position": ...})`
writes the new rows at `(pos // page, pos % page)` and returns `(buffer, page_table)`.  The write is one
`ktb200_mla_kv_write` launch (csrc/mla.cu) instead of two advanced-indexing copies; buffers never move, so the cache
is CUDA-graph safe."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from .. import native


class StaticCache:
    def __init__(self, config, max_batch_size: int, max_cache_len: int, device, dtype=torch.bfloat16, page_size: int = 64):
        assert dtype == torch.bfloat16, "the latent cache is bf16"
        self.config = config
        self._max_batch_size, self._max_cache_len = max_batch_size, max_cache_len
        self.page_size = page_size
        self.max_pages = (max_cache_len + page_size - 1) // page_size
        self.kv_lora_rank, self.qk_rope_head_dim = config.kv_lora_rank, config.qk_rope_head_dim
        self.device = torch.device(device)
        latent = (self.max_pages * max_batch_size, page_size, 1, self.kv_lora_rank + self.qk_rope_head_dim)
        self.key_cache = [torch.zeros(latent, dtype=dtype, device=device) for _ in range(config.num_hidden_layers)]
        self.value_cache = [None] * config.num_hidden_layers
        table = torch.arange(self.max_pages * max_batch_size, dtype=torch.int32, device=device).reshape(max_batch_size, self.max_pages)
        self.page_table_list = [table] * config.num_hidden_layers
        self.past_tokens = [0] * config.num_hidden_layers
        self.is_MLA = self.is_page = True

    @property
    def max_batch_size(self):
        return self._max_batch_size

    @property
    def max_cache_len(self):
        return self._max_cache_len

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.past_tokens[layer_idx]

    def get_usable_length(self, kv_seq_len: int, layer_idx: int = 0) -> int:
        return self.past_tokens[layer_idx]

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """key_states = compressed_kv [bsz, q_len, 1, 512], value_states = k_pe [bsz, q_len, 1, 64] (the reference's argument
        order, custom_cache.py:147-193); batch row b writes into its own page range."""
        cache_position = cache_kwargs.get("cache_position")
        k_out = self.key_cache[layer_idx]
        bsz, q_len = key_states.shape[0], key_states.shape[1]
        pos = cache_position.to(torch.int32).reshape(1, -1).expand(bsz, q_len)
        page_idx = (pos // self.page_size + torch.arange(bsz, device=pos.device, dtype=torch.int32).reshape(bsz, 1) * self.max_pages).reshape(-1).contiguous()
        page_off = (pos % self.page_size).reshape(-1).contiguous()
        ckv = key_states.reshape(-1, self.kv_lora_rank).contiguous()
        kpe = value_states.reshape(-1, self.qk_rope_head_dim).contiguous()
        native.check(native.lib().ktb200_mla_kv_write(k_out.data_ptr(), self.page_size, ckv.data_ptr(), kpe.data_ptr(), page_idx.data_ptr(),
                                                      page_off.data_ptr(), ckv.shape[0], torch.cuda.current_stream(k_out.device).cuda_stream))
        if not torch.cuda.is_current_stream_capturing():
            self.past_tokens[layer_idx] += q_len
        return k_out, self.page_table_list[layer_idx]

    def reset(self):
        for t in self.key_cache:
            t.zero_()
        self.past_tokens = [0] * len(self.past_tokens)


class ForwardBatch:
    """One step's ragged batch, flattened token-major: what the scheduler hands to a model's step function.

    `tokens`, `pos`, `slot` [T]; for layers that keep a previous-token row: `prev_idx` (row of the previous token inside this
    step or -1), `rd_row` / `wr_row` (state rows to read when the previous token came in an earlier step / to write for the
    last token of a sequence's portion; -1: none).  `seqs` [4, >= n_seqs]: the same per sequence portion, for layers whose
    state is a recurrence over the portion's tokens, and `seq_of` [T]: the portion a token belongs to (column of `seqs`), for
    layers that look further back than one token.  `want` [W]: rows whose logits the caller asked for."""

    N_META = 10      # index rows per token: pos, slot, prev_idx, rd_row, wr_row, the four rows of `seqs`, seq_of

    __slots__ = ("tokens", "pos", "slot", "prev_idx", "rd_row", "wr_row", "want", "n_tokens", "max_kv", "seqs", "n_seqs", "seq_of")

    def __init__(self, meta: torch.Tensor, tokens: torch.Tensor, want: torch.Tensor, max_kv: int, n_seqs: int = 0):
        self.pos, self.slot, self.prev_idx, self.rd_row, self.wr_row = meta[0], meta[1], meta[2], meta[3], meta[4]
        self.tokens, self.want, self.n_tokens, self.max_kv = tokens, want, int(tokens.shape[0]), max_kv
        # per sequence portion, for layers that carry a recurrent state: rows (first token's row, token count, state row to
        # read or -1, state row to write) in the first n_seqs columns
        self.seqs, self.n_seqs = (meta[5:9] if meta.shape[0] >= 9 else None), n_seqs
        self.seq_of = meta[9] if meta.shape[0] >= 10 else None


class PagedStateCache:
    """Pages of per-token cache rows plus fixed-size per-sequence state rows, for models whose layers keep a (windowed) latent
    cache and a previous-token row.

    * One pool of `num_pages` pages of `page_size` tokens; layer l's buffer is `[num_pages, page_size, row_widths[l]]` and all
      layers share the page ids, so a sequence has ONE page table row (`page_table[slot]`, device int32), used as a ring:
      logical page p sits in column `p % max_pages_per_seq`.
    * A sequence occupies a slot from `open()` to `close()`; `extend(slot, n)` reserves pages for the next n tokens and returns
      the first position; pages that fall wholly behind `window` (the largest look-back of any layer), or before the start of
      the current chunk when every layer's mask is chunked, are given back while the sequence is still running, and pages and slots are reused without being cleared: readers never look outside
      `[pos - window + 1, pos]`, and position 0 reads no state.
    * State rows are double-buffered per slot (`state[l]` is `[2 * max_slots, width]` fp32): a step reads row `2*slot + parity`
      and writes row `2*slot + 1 - parity`, then `commit()` flips the parity of the slots it touched, so no kernel launch
      reads a row it also writes.

    The reference's StaticCache (archive/ktransformers/models/custom_cache.py:26-200) keeps a static identity page table per
    batch row; this manager adds allocation, release and the recurrent rows."""

    def __init__(self, row_widths, state_width, max_tokens: int, max_slots: int, device, dtype=torch.bfloat16, page_size: int = 64,
                 window: Optional[int] = None, chunks=None):
        """`row_widths[l]`: cache values per token of cache layer l (0: the layer caches no rows); `state_width`: fp32 state
        values per sequence, one number for all layers or one per layer (0: none).  A model whose layers run several times
        with separate caches counts every run as a cache layer.  `window`: the largest sliding look-back of any caching layer
        (None: unbounded); `chunks`: the chunk lengths of the caching layers when EVERY one of them reads only keys of the
        query's own chunk (position p sees p - p mod C onwards) — then the pages before the earliest chunk start are given back."""
        self.device, self.dtype, self.page_size, self.window = torch.device(device), dtype, int(page_size), window
        self.chunks = sorted({int(c) for c in chunks}) if chunks else None
        self.max_slots = int(max_slots)
        # every live sequence may hold one partly filled page at each end of its range
        self.num_pages = (int(max_tokens) + page_size - 1) // page_size + 2 * self.max_slots
        self.max_pages_per_seq = (int(max_tokens) + page_size - 1) // page_size + 2
        self.key_cache = [torch.zeros((self.num_pages, page_size, int(w)), dtype=dtype, device=device) for w in row_widths]
        state_widths = [int(state_width)] * len(row_widths) if isinstance(state_width, int) else [int(w) for w in state_width]
        if len(state_widths) != len(row_widths):
            raise ValueError("one state width per cache layer")
        self.state = [torch.zeros((2 * self.max_slots, w), dtype=torch.float32, device=device) for w in state_widths]
        self.page_table = torch.zeros((self.max_slots, self.max_pages_per_seq), dtype=torch.int32, device=device)
        self._table_host = torch.zeros((self.max_slots, self.max_pages_per_seq), dtype=torch.int32)
        self._free_pages = list(range(self.num_pages - 1, -1, -1))
        self._free_slots = list(range(self.max_slots - 1, -1, -1))
        self._slot_of: Dict[Any, int] = {}
        self._len = [0] * self.max_slots            # tokens written so far
        self._first_page = [0] * self.max_slots     # logical pages below this index were given back
        self._parity = [0] * self.max_slots
        self._touched: set = set()
        self._dirty = False

    # -- sequences ---------------------------------------------------------------------------------
    def open(self, seq_id) -> int:
        if seq_id in self._slot_of:
            return self._slot_of[seq_id]
        if not self._free_slots:
            raise MemoryError("PagedStateCache: no free sequence slot")
        s = self._free_slots.pop()
        self._slot_of[seq_id] = s
        self._len[s], self._first_page[s], self._parity[s] = 0, 0, 0
        return s

    def close(self, seq_id) -> None:
        s = self._slot_of.pop(seq_id)
        n_pages = (self._len[s] + self.page_size - 1) // self.page_size
        for lp in range(self._first_page[s], n_pages):
            self._free_pages.append(int(self._table_host[s, lp % self.max_pages_per_seq]))
        self._len[s] = 0
        self._free_slots.append(s)

    def slot(self, seq_id) -> int:
        return self._slot_of[seq_id]

    def length(self, seq_id) -> int:
        return self._len[self._slot_of[seq_id]]

    def free_tokens(self) -> int:
        return len(self._free_pages) * self.page_size

    # -- pages -------------------------------------------------------------------------------------
    def extend(self, slot: int, n: int) -> int:
        """Reserve pages for positions [len, len + n); returns len."""
        start = self._len[slot]
        have = (start + self.page_size - 1) // self.page_size
        need = (start + n + self.page_size - 1) // self.page_size
        if need - self._first_page[slot] > self.max_pages_per_seq:      # the table row is a ring over the live pages
            raise MemoryError("PagedStateCache: sequence holds more pages than its page table row")
        if need - have > len(self._free_pages):
            raise MemoryError("PagedStateCache: out of pages")
        for lp in range(have, need):
            self._table_host[slot, lp % self.max_pages_per_seq] = self._free_pages.pop()
            self._dirty = True
        self._len[slot] = start + n
        self._touched.add(slot)
        return start

    def release_behind(self, slot: int) -> None:
        """Give back the pages that no later token of this sequence can look at."""
        if self.window is None and self.chunks is None:
            return
        nxt, first = self._len[slot], 0              # the next token's position, and the first key it (and so any later token) may read
        if self.window is not None:
            first = max(first, nxt - (self.window - 1))
        if self.chunks is not None:
            first = max(first, min(nxt - nxt % c for c in self.chunks))
        keep_from = first // self.page_size
        for lp in range(self._first_page[slot], keep_from):
            self._free_pages.append(int(self._table_host[slot, lp % self.max_pages_per_seq]))
        self._first_page[slot] = max(self._first_page[slot], keep_from)

    def sync_table(self) -> torch.Tensor:
        if self._dirty:
            self.page_table.copy_(self._table_host, non_blocking=False)
            self._dirty = False
        return self.page_table

    # -- state rows --------------------------------------------------------------------------------
    def state_rows(self, slot: int, start: int):
        """(row to read or -1 when the portion starts the sequence, row to write)"""
        p = self._parity[slot]
        return (2 * slot + p if start > 0 else -1), 2 * slot + 1 - p

    def commit(self) -> None:
        for s in self._touched:
            self._parity[s] ^= 1
            self.release_behind(s)
        self._touched.clear()

    def capacity_per_sequence(self) -> int:
        return self.max_pages_per_seq * self.page_size

    def build_batch(self, entries, want_all: bool = False, static=None) -> ForwardBatch:
        """entries: [(seq_id, tokens, want)] — reserve pages, lay out the per-token index rows, one host-to-device copy.
        `static` = (meta [ForwardBatch.N_META, T] int32, tokens [T] int64) device buffers of a captured step: the rows are copied into them and
        the batch is built on them, asking for every row (the caller picks the wanted ones from the captured output)."""
        rows, toks, want, base, max_kv = [[] for _ in range(ForwardBatch.N_META)], [], [], 0, 0
        for seq_id, tokens, w in entries:
            s = self.open(seq_id)
            n = len(tokens)
            start = self.extend(s, n)
            rd, wr = self.state_rows(s, start)
            rows[9] += [len(rows[5])] * n
            for r, v in zip(rows[5:9], (base, n, rd, wr)):
                r.append(v)
            rows[0] += range(start, start + n)
            rows[1] += [s] * n
            rows[2] += [-1] + list(range(base, base + n - 1))
            rows[3] += [rd] + [-1] * (n - 1)
            rows[4] += [-1] * (n - 1) + [wr]
            toks += tokens
            want += [base + i for i in (range(n) if want_all else w)]
            base += n
            max_kv = max(max_kv, start + n)
        n_seqs = len(rows[5])
        for r in rows[5:9]:
            r += [0] * (base - n_seqs)
        self.sync_table()
        if static is not None:
            static[0].copy_(torch.tensor(rows, dtype=torch.int32))
            static[1].copy_(torch.tensor(toks, dtype=torch.int64))
            b = ForwardBatch(static[0], static[1], torch.tensor(want, dtype=torch.int64).to(self.device, non_blocking=True), self.capacity_per_sequence(), n_seqs)
            return b
        meta = torch.tensor(rows, dtype=torch.int32).to(self.device, non_blocking=True)
        return ForwardBatch(meta, torch.tensor(toks, dtype=torch.int64).to(self.device, non_blocking=True),
                            torch.tensor(want, dtype=torch.int64).to(self.device, non_blocking=True), max_kv, n_seqs)
