"""Host-side model of how the balanced persistent kernel shares the work out (test support).

The kernel (csrc/paged_decode_balanced.cuh, ``Chunking``), its plan kernel and its merge kernel
all derive the partition from ``seq_lens`` alone; this module restates that arithmetic in Python
so that the partition can be inspected (which warp group streams which page pairs, where the
pieces of a cut sequence land in the workspace) and its invariants tested without a GPU.

Cost is counted in half page pairs: sequence ``b`` owns the cost range that starts at
``2 * pairs_before(b) + piece_cost * b``; its first ``piece_cost`` units stand for taking the
sequence up, then come two units per page pair.  The cost axis is cut into ``groups``
contiguous chunks whose lengths differ by at most one unit, and a page pair belongs to the
chunk that holds its first unit.
"""

from __future__ import annotations

from dataclasses import dataclass

PAGE = 16
WARPS_PER_SM = 8
PIECE_COST = 2
MIN_CHUNK_COST = 8


def pairs_of(seq_len: int, kv_start: int = 0) -> int:
    pages = -(-seq_len // PAGE) - kv_start // PAGE if seq_len > kv_start else 0
    return (pages + 1) // 2


@dataclass(frozen=True)
class Piece:
    sequence: int
    group: int        # warp group (chunk) that streams it
    first_pair: int   # pair range inside the sequence
    last_pair: int
    slot: int | None  # workspace slot 2 * group + which, None when the sequence is whole


class ChunkPlan:
    def __init__(self, seq_lens, num_kv_heads: int, sm_count: int = 148, *, kv_start: int = 0,
                 piece_cost: int = PIECE_COST, warps_per_sm: int = WARPS_PER_SM):
        self.pairs = [pairs_of(int(n), kv_start) for n in seq_lens]
        self.batch = len(self.pairs)
        self.piece_cost = piece_cost
        self.prefix = [0]
        for n in self.pairs:
            self.prefix.append(self.prefix[-1] + n)
        total = 2 * self.prefix[-1] + piece_cost * self.batch
        max_groups = max(sm_count * warps_per_sm // num_kv_heads, 1)
        self.groups = max(min(max_groups, total // MIN_CHUNK_COST), 1)
        self.base, self.rem = divmod(total, self.groups)
        self.total_cost = total

    # ---- the device functions, one to one
    def start_of(self, chunk: int) -> int:
        return chunk * self.base + min(chunk, self.rem)

    def chunk_of(self, unit: int) -> int:
        wide = self.rem * (self.base + 1)
        return unit // (self.base + 1) if unit < wide else self.rem + (unit - wide) // max(self.base, 1)

    def first_unit(self, sequence: int) -> int:
        return 2 * self.prefix[sequence] + self.piece_cost * (sequence + 1)

    # ---- derived views
    def pair_range(self, chunk: int) -> tuple[int, int]:
        """Pairs (indices into the flattened list of all sequences' pairs) of one chunk."""
        def before(cost: int) -> int:
            if cost >= self.total_cost:
                return self.prefix[-1]
            b = max(i for i in range(self.batch) if 2 * self.prefix[i] + self.piece_cost * i <= cost)
            off = cost - self.first_unit(b)
            return self.prefix[b] + min(max((off + 1) // 2, 0), self.pairs[b])
        if chunk >= self.groups:
            return self.prefix[-1], self.prefix[-1]
        return before(self.start_of(chunk)), before(self.start_of(chunk + 1))

    def pieces_of(self, sequence: int) -> list[Piece]:
        """What the merge kernel derives for one sequence: its pieces and their slots."""
        n = self.pairs[sequence]
        if n == 0:
            return []
        s0 = self.first_unit(sequence)
        first, last = self.chunk_of(s0), self.chunk_of(s0 + 2 * (n - 1))
        out = []
        for c in range(first, last + 1):
            lo, hi = self.pair_range(c)
            a = max(lo, self.prefix[sequence]) - self.prefix[sequence]
            e = min(hi, self.prefix[sequence + 1]) - self.prefix[sequence]
            which = 1 if s0 > self.start_of(c) else 0
            out.append(Piece(sequence, c, a, e - 1, None if first == last else 2 * c + which))
        return out
