"""CPU restatement of the reference's cached decode attention.  TEST INFRASTRUCTURE ONLY: imported by
tests/, the smoke check and the benchmark's CPU-baseline leg; the product never calls it.

Follows, in f32 numpy:
  * Rope::new / Rope::rotate       reference rope.rs:71-97, 170-225 (rotate-half: channel j pairs with j + head_dim/2)
  * KvCache                        reference attention.rs:19-78
  * MultiHeadAttention::forward_cached without its four Linear layers
                                   reference attention.rs:344-398 (head_scores :1100-1130, accumulate_head_output
                                   :1133-1160, scale = 1/sqrt(head_dim) :294-296, softmax activations.rs:56-70)
  * the attention of forward_train for one sequence (causal, full sequence), which the reference's own tests
    use as the ground truth of the cached path (attention.rs:1318-1362).

Pinned by the known answers and properties of the reference's tests: rope.rs:232-298 (identity at
position 0, the hand-computed rotation, inverse, norm, relative distance) and attention.rs:1318-1362
(cached decode and prefill-then-decode reproduce the full-sequence forward to 1e-5); see
tests/test_kv_attention_oracle.py.  The reference itself cannot be run here (no Rust toolchain).
"""
from __future__ import annotations

import numpy as np

F = np.float32


def rope_tables(head_dim: int, max_seq_len: int, base: float):
    """(cos, sin), each [max_seq_len, head_dim / 2] (rope.rs:77-90)."""
    if head_dim == 0 or head_dim % 2 != 0:
        raise ValueError("rope head_dim must be even and non-zero, got %d" % head_dim)
    half = head_dim // 2
    channel = np.arange(half, dtype=F)
    frequency = np.power(F(base), (F(-2.0) * channel / F(head_dim)).astype(F)).astype(F)
    angle = (np.arange(max_seq_len, dtype=F)[:, None] * frequency[None, :]).astype(F)
    return np.cos(angle).astype(F), np.sin(angle).astype(F)


def rope_apply(tensor: np.ndarray, heads: int, position_offset: int, cos: np.ndarray, sin: np.ndarray,
               direction: float = 1.0) -> np.ndarray:
    """Rope::apply (direction -1: apply_inverse): rows are tokens at positions offset, offset + 1, ..."""
    rows, cols = tensor.shape
    half = cos.shape[1]
    head_dim = 2 * half
    if cols != heads * head_dim:
        raise ValueError("rope expected %d columns for %d heads, got %d" % (heads * head_dim, heads, cols))
    if position_offset + rows > cos.shape[0]:
        raise ValueError("SequenceTooLong: length %d, max_seq_len %d" % (position_offset + rows, cos.shape[0]))
    x = tensor.astype(F).reshape(rows, heads, 2, half)
    c = cos[position_offset:position_offset + rows][:, None, :]
    s = (F(direction) * sin[position_offset:position_offset + rows])[:, None, :]
    low, high = x[:, :, 0, :], x[:, :, 1, :]
    out = np.empty_like(x)
    out[:, :, 0, :] = low * c - high * s
    out[:, :, 1, :] = high * c + low * s
    return out.reshape(rows, cols)


def softmax(values: np.ndarray) -> np.ndarray:
    """activations.rs:56-70 on a 1-d slice."""
    e = np.exp((values - values.max()).astype(F)).astype(F)
    total = e.sum(dtype=F)
    return e / total if total > 0 else e


def attend(queries: np.ndarray, keys: np.ndarray, values: np.ndarray, num_heads: int, kv_heads: int, head_dim: int,
           position_offset: int) -> np.ndarray:
    """head_scores + accumulate_head_output for every head: row i of `queries` sits at position
    position_offset + i and sees keys 0 ..= position_offset + i.  Returns the merged heads."""
    group = num_heads // kv_heads
    scale = F(1.0) / np.sqrt(F(head_dim))
    merged = np.zeros((queries.shape[0], num_heads * head_dim), F)
    for head in range(num_heads):
        qb, kb = head * head_dim, (head // group) * head_dim
        for i in range(queries.shape[0]):
            visible = position_offset + i + 1
            scores = (keys[:visible, kb:kb + head_dim] @ queries[i, qb:qb + head_dim]).astype(F) * scale
            merged[i, qb:qb + head_dim] = softmax(scores) @ values[:visible, kb:kb + head_dim]
    return merged


class KvCacheOracle:
    """One sequence: KvCache + the attention arithmetic of forward_cached."""

    def __init__(self, num_heads: int, kv_heads: int, head_dim: int, max_seq_len: int, rope_base: float = 10000.0,
                 rope: bool = True):
        if num_heads == 0 or kv_heads == 0 or kv_heads > num_heads or num_heads % kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.num_heads, self.kv_heads, self.head_dim, self.rope = num_heads, kv_heads, head_dim, rope
        self.cos, self.sin = rope_tables(head_dim, max_seq_len, rope_base)
        self.keys = np.zeros((0, kv_heads * head_dim), F)
        self.values = np.zeros((0, kv_heads * head_dim), F)

    def __len__(self) -> int:
        return self.keys.shape[0]

    def clear(self) -> None:
        self.keys, self.values = self.keys[:0], self.values[:0]

    def forward_cached(self, q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
        """q, k, v: the projections of the new rows (before rotation); returns the merged heads."""
        offset = len(self)
        q, k, v = q.astype(F), k.astype(F), v.astype(F)
        if self.rope:
            q = rope_apply(q, self.num_heads, offset, self.cos, self.sin)
            k = rope_apply(k, self.kv_heads, offset, self.cos, self.sin)
        self.keys = np.concatenate([self.keys, k])
        self.values = np.concatenate([self.values, v])
        return attend(q, self.keys, self.values, self.num_heads, self.kv_heads, self.head_dim, offset)


def full_sequence(q: np.ndarray, k: np.ndarray, v: np.ndarray, num_heads: int, kv_heads: int, head_dim: int,
                  max_seq_len: int, rope_base: float = 10000.0, rope: bool = True) -> np.ndarray:
    """The causal attention of forward_train for one sequence, written as one masked matrix product per
    head (an independent formulation: the cached path must reproduce it, attention.rs:1318-1340)."""
    rows = q.shape[0]
    q, k, v = q.astype(F), k.astype(F), v.astype(F)
    if rope:
        cos, sin = rope_tables(head_dim, max_seq_len, rope_base)
        q = rope_apply(q, num_heads, 0, cos, sin)
        k = rope_apply(k, kv_heads, 0, cos, sin)
    group = num_heads // kv_heads
    scale = F(1.0) / np.sqrt(F(head_dim))
    mask = np.tril(np.ones((rows, rows), bool))
    out = np.zeros((rows, num_heads * head_dim), F)
    for head in range(num_heads):
        qb, kb = head * head_dim, (head // group) * head_dim
        s = (q[:, qb:qb + head_dim] @ k[:, kb:kb + head_dim].T).astype(F) * scale
        s = np.where(mask, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        p = (e / e.sum(axis=1, keepdims=True)).astype(F)
        out[:, qb:qb + head_dim] = p @ v[:, kb:kb + head_dim]
    return out
