"""Host-side page bookkeeping of the KV cache (pure Python, no torch, no device).

The contract is the reference allocator's (src/moba_opt/cache_layout.py:12-148):
  * a fixed number of sequence slots, each with `table_width` logical pages that map to arbitrary
    physical pages (-1 = unmapped);
  * a LIFO pool: pages are taken from the END of `free_pages`, which starts as (N-1, ..., 1, 0), so
    page 0 is handed out first and released pages are reused most-recent-first;
  * planning is side-effect free; `commit` publishes a plan only if it was made against the current
    version (`RuntimeError("stale ...")` otherwise);
  * every contract or capacity violation is a `ValueError` and leaves the state untouched.
"""
import numbers
from dataclasses import dataclass


def positive_int(value, name):
    """Returns int(value) for an integral, non-bool value > 0, else raises ValueError."""
    if isinstance(value, numbers.Integral) and not isinstance(value, bool) and value > 0:
        return int(value)
    raise ValueError(f"{name} must be a positive integer")


def _ceil_div(a, b):
    return (a + b - 1) // b


@dataclass(frozen=True)
class AppendPlan:
    """A fully computed next state plus where every appended token goes."""
    version: int
    tables: tuple
    lengths: tuple
    free_pages: tuple
    token_sequences: tuple    # sequence id of every appended token, in input order
    token_positions: tuple    # its position inside that sequence
    completed_chunks: tuple   # (sequence id, chunk index) for every chunk this append completes
    page_edits: tuple = ()    # (sequence id, logical page, physical page) for every page this append maps


@dataclass(frozen=True)
class StepPlan:
    """One new token for every leased sequence."""
    version: int
    positions: tuple          # position the new token of each leased sequence will take
    updates: tuple            # (sequence id, logical page, physical page) where a token opens a page


class PageAllocator:
    """Transactional allocator: `plan_append` computes, `commit` publishes, `reset` releases."""

    def __init__(self, batch_size, max_seq_len, page_size, num_pages, chunk_size):
        self.batch_size = positive_int(batch_size, "batch_size")
        self.max_seq_len = positive_int(max_seq_len, "max_seq_len")
        self.page_size = positive_int(page_size, "page_size")
        self.num_pages = positive_int(num_pages, "num_pages")
        self.chunk_size = positive_int(chunk_size, "chunk_size")
        if self.max_seq_len >= 1 << 30 or self.num_pages * self.page_size >= 1 << 31:
            raise ValueError("cache exceeds int32 indexing capacity")
        self.table_width = _ceil_div(self.max_seq_len, self.page_size)
        unmapped = (-1,) * self.table_width
        self.tables = (unmapped,) * self.batch_size
        self.lengths = (0,) * self.batch_size
        self.free_pages = tuple(range(self.num_pages - 1, -1, -1))
        self.version = 0

    # -- validation --------------------------------------------------------------------------
    def validate_ids(self, ids, *, unique=False):
        out = []
        for sid in ids:
            if not isinstance(sid, numbers.Integral) or isinstance(sid, bool):
                raise ValueError("sequence IDs must be integers")
            sid = int(sid)
            if sid < 0 or sid >= self.batch_size:
                raise ValueError("sequence ID outside cache batch slots")
            out.append(sid)
        if len(out) == 0 or (unique and len(set(out)) < len(out)):
            raise ValueError("nonempty unique sequence IDs required for append/reset")
        return tuple(out)

    def _pages_needed(self, ids, counts):
        total = 0
        for sid, n in zip(ids, counts):
            after = self.lengths[sid] + n
            if after > self.max_seq_len:
                raise ValueError("append exceeds max_seq_len")
            total += _ceil_div(after, self.page_size) - _ceil_div(self.lengths[sid], self.page_size)
        return total

    # -- planning / publishing ---------------------------------------------------------------
    def plan_append(self, sequence_ids, counts, tokens=True):
        """`tokens=False` leaves out the per-token (sequence, position) lists, which a whole-prompt append does not need."""
        ids = self.validate_ids(sequence_ids, unique=True)
        if len(ids) != len(counts):
            raise ValueError("one token count per sequence required")
        counts = tuple(positive_int(n, "append count") for n in counts)
        if self._pages_needed(ids, counts) > len(self.free_pages):
            raise ValueError("KV page pool exhausted; cache was not modified")
        pool = list(self.free_pages)
        rows = {}                                   # only the rows that receive a page are rebuilt
        lengths = list(self.lengths)
        where_seq, where_pos, closed, edits = [], [], [], []
        page, chunk = self.page_size, self.chunk_size
        for sid, n in zip(ids, counts):
            first, last = lengths[sid], lengths[sid] + n
            lo, hi = _ceil_div(first, page), _ceil_div(last, page)
            if hi > lo:
                fresh = [pool.pop() for _ in range(hi - lo)]
                old = self.tables[sid]
                rows[sid] = old[:lo] + tuple(fresh) + old[hi:]
                edits.extend((sid, lo + i, physical) for i, physical in enumerate(fresh))
            if tokens:
                where_seq.extend(sid for _ in range(n))
                where_pos.extend(range(first, last))
            closed.extend((sid, c) for c in range(first // chunk, last // chunk))
            lengths[sid] = last
        tables = tuple(rows.get(s, row) for s, row in enumerate(self.tables)) if rows else self.tables
        return AppendPlan(self.version, tables, tuple(lengths), tuple(pool), tuple(where_seq), tuple(where_pos),
                          tuple(closed), tuple(edits))

    def commit(self, plan):
        if plan.version != self.version:
            raise RuntimeError("stale append plan")
        self.tables, self.lengths, self.free_pages = plan.tables, plan.lengths, plan.free_pages
        self.version += 1

    def reset(self, sequence_ids):
        """Releases every page of the given sequences (in table order, onto the end of the pool)."""
        ids = self.validate_ids(sequence_ids, unique=True)
        pool = list(self.free_pages)
        tables, lengths = list(self.tables), list(self.lengths)
        for sid in ids:
            pool.extend(p for p in tables[sid] if p >= 0)
            tables[sid] = (-1,) * self.table_width
            lengths[sid] = 0
        self.tables, self.lengths, self.free_pages = tuple(tables), tuple(lengths), tuple(pool)
        self.version += 1

    def clone(self):
        twin = object.__new__(PageAllocator)
        twin.__dict__.update(self.__dict__)
        return twin


class IncrementalLayout:
    """Exclusive lease over a fixed set of sequences for token-by-token decode: per step only the
    leased sequences are touched; `publish` writes the state back into the allocator."""

    def __init__(self, layout, sequence_ids):
        self.ids = layout.validate_ids(sequence_ids, unique=True)
        self.tables = [list(row) for row in layout.tables]
        self.lengths = list(layout.lengths)
        self.free = list(layout.free_pages)
        self.version = layout.version
        self.page_size = layout.page_size
        self.max_seq_len = layout.max_seq_len

    def plan(self):
        positions = tuple(self.lengths[sid] for sid in self.ids)
        if max(positions) >= self.max_seq_len:
            raise ValueError("append exceeds max_seq_len")
        openers = [(sid, pos // self.page_size) for sid, pos in zip(self.ids, positions) if pos % self.page_size == 0]
        if len(openers) > len(self.free):
            raise ValueError("KV page pool exhausted; cache was not modified")
        # the i-th opener receives the i-th page from the end of the pool, exactly what pop() yields
        updates = tuple((sid, logical, self.free[-(i + 1)]) for i, (sid, logical) in enumerate(openers))
        return StepPlan(self.version, positions, updates)

    def commit(self, plan):
        if plan.version != self.version:
            raise RuntimeError("stale decode step plan")
        for sid, logical, physical in plan.updates:
            taken = self.free.pop()
            if taken != physical:
                raise RuntimeError("stale decode step plan")
            self.tables[sid][logical] = physical
        for sid in self.ids:
            self.lengths[sid] += 1
        self.version += 1

    def publish(self, layout):
        layout.tables = tuple(tuple(row) for row in self.tables)
        layout.lengths = tuple(self.lengths)
        layout.free_pages = tuple(self.free)
        layout.version = self.version
