"""Tensor-parallel shard plan for the packed-ternary decoder: which slice of which matrix a rank holds.

The reference keeps every projection whole (poly/bitnet_gpu.go:56-115 uploads Q/K/V/O and gate/up/down as
single buffers).  The split below is the one its integer arithmetic allows without changing a result bit:

* Q, K, V, gate, up: a contiguous slice of the ROWS (whole heads, whole intermediate units).  Each rank
  quantizes the same replicated input row, so nothing is exchanged.
* O, down: the matching slice of the COLUMNS.  Their input (attention output, gate product) exists only in
  slices, and the always-on inner RMSNorm and the absmax quantization run over the whole vector, so ranks
  exchange a float64 sum of squares, a float32 absmax and finally the int32 partial accumulators.

Packed rows are sequences of uint32 words with 16 two-bit codes each (poly/bitnet_cpu.go:17-30), so a column
slice must start on a multiple of 16 columns.  Every slice keeps the scale of the whole matrix.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def row_words(cols: int) -> int:
    return (cols + 15) // 16


def slice_rows(words: np.ndarray, rows: int, cols: int, r0: int, r1: int) -> np.ndarray:
    """Words of rows [r0, r1) of a packed [rows, cols] matrix."""
    if not (0 <= r0 <= r1 <= rows):
        raise ValueError("row slice [%d, %d) outside 0..%d" % (r0, r1, rows))
    w = np.asarray(words, dtype=np.uint32).reshape(rows, row_words(cols))
    return np.ascontiguousarray(w[r0:r1])


def slice_cols(words: np.ndarray, rows: int, cols: int, c0: int, c1: int) -> np.ndarray:
    """Words of columns [c0, c1) of a packed [rows, cols] matrix; c0 must be a multiple of 16 and so must
    c1 unless it is the last column."""
    if not (0 <= c0 <= c1 <= cols):
        raise ValueError("column slice [%d, %d) outside 0..%d" % (c0, c1, cols))
    if c0 % 16 or (c1 % 16 and c1 != cols):
        raise ValueError("column slice [%d, %d) does not fall on 16-column word boundaries" % (c0, c1))
    w = np.asarray(words, dtype=np.uint32).reshape(rows, row_words(cols))
    return np.ascontiguousarray(w[:, c0 // 16:row_words(c1)])


@dataclass(frozen=True)
class ShardPlan:
    """Slice bounds of one rank for a decoder with the given unsharded dimensions."""
    world: int
    rank: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    inter: int
    vocab: int

    def __post_init__(self):
        w = self.world
        if w < 1 or not (0 <= self.rank < w):
            raise ValueError("rank %d of %d" % (self.rank, w))
        if self.heads % w or self.kv_heads % w or self.inter % w:
            raise ValueError("heads %d, kv heads %d and intermediate %d must be multiples of the group size %d"
                             % (self.heads, self.kv_heads, self.inter, w))
        if w > 1 and ((self.heads // w * self.head_dim) % 16 or (self.inter // w) % 16):
            raise ValueError("per-rank widths %d and %d must be multiples of 16 columns"
                             % (self.heads // w * self.head_dim, self.inter // w))

    @property
    def q_rows(self):
        n = self.heads // self.world * self.head_dim
        return self.rank * n, (self.rank + 1) * n

    @property
    def kv_rows(self):
        n = self.kv_heads // self.world * self.head_dim
        return self.rank * n, (self.rank + 1) * n

    @property
    def inter_rows(self):
        n = self.inter // self.world
        return self.rank * n, (self.rank + 1) * n

    @property
    def vocab_rows(self):
        """Rows of the tied LM head this rank computes (the whole head when vocab does not divide)."""
        if self.world > 1 and self.vocab % self.world == 0:
            n = self.vocab // self.world
            return self.rank * n, (self.rank + 1) * n
        return 0, self.vocab

    def shard_block(self, words7, attn_inner=None, ffn_inner=None):
        """words7 = packed q, k, v, o, gate, up, down of one block (unsharded).  Returns the seven slices as
        (words, rows, cols) triples in the same order, and the slices of the two inner-norm vectors."""
        H, qd, kvd, I = self.hidden, self.heads * self.head_dim, self.kv_heads * self.head_dim, self.inter
        q0, q1 = self.q_rows
        k0, k1 = self.kv_rows
        i0, i1 = self.inter_rows
        out = [
            (slice_rows(words7[0], qd, H, q0, q1), q1 - q0, H),
            (slice_rows(words7[1], kvd, H, k0, k1), k1 - k0, H),
            (slice_rows(words7[2], kvd, H, k0, k1), k1 - k0, H),
            (slice_cols(words7[3], H, qd, q0, q1), H, q1 - q0),
            (slice_rows(words7[4], I, H, i0, i1), i1 - i0, H),
            (slice_rows(words7[5], I, H, i0, i1), i1 - i0, H),
            (slice_cols(words7[6], H, I, i0, i1), H, i1 - i0),
        ]

        def cut(v, a, b):
            # an inner-norm vector may be shorter than the row it scales: entries beyond it count as 1
            if v is None:
                return None
            v = np.asarray(v, dtype=np.float32)
            return np.ascontiguousarray(v[a:b]) if a < v.size else None

        return out, cut(attn_inner, q0, q1), cut(ffn_inner, i0, i1)
