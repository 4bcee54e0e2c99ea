"""Host-side mirror of the reference's ``KvCache`` + ``MultiHeadAttention::forward_cached``
(attention.rs:19-78, 344-398) over the C ABI of include/kv_attention_b200.h, for many sequences.

The projections (query, key, value, output) stay with the caller; this object owns the caches and the
attention arithmetic between them.  There is no host implementation behind it.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np

from . import _lib
from .moe import CudaError, InvalidConfig, InvalidInput, NetworkError, _stream

_ERRORS = {_lib.INVALID_CONFIG: InvalidConfig, _lib.INVALID_INPUT: InvalidInput, _lib.UNSUPPORTED: InvalidConfig}


class KvCache:
    """``sequences`` caches of ``capacity`` positions (KvCache::with_capacity, attention.rs:39-48) and the
    RoPE tables for ``max_seq_len`` positions (Rope::new, rope.rs:71-97)."""

    def __init__(self, sequences: int, num_heads: int, kv_heads: int, head_dim: int, capacity: int,
                 max_seq_len: Optional[int] = None, rope_base: float = 10000.0, rope: bool = True,
                 precision: str = "bf16", device: int = 0):
        if precision not in ("f32", "bf16"):
            raise InvalidConfig("precision is 'f32' or 'bf16'")
        self.sequences, self.num_heads, self.kv_heads, self.head_dim = sequences, num_heads, kv_heads, head_dim
        self.capacity = capacity
        self.precision = precision
        self._h = C.c_void_p()
        cfg = _lib.KvCacheConfigC(sequences=sequences, num_heads=num_heads, kv_heads=kv_heads, head_dim=head_dim,
                                  capacity=capacity, max_seq_len=max_seq_len if max_seq_len is not None else capacity,
                                  rope_base=rope_base, rope=1 if rope else 0,
                                  precision=_lib.PRECISION_BF16 if precision == "bf16" else _lib.PRECISION_F32,
                                  device=device)
        rc = _lib.lib().kv_cache_create(C.byref(cfg), C.byref(self._h))
        if rc != _lib.OK:
            text = _lib.lib().kv_cache_last_error(self._h).decode(errors="replace") if self._h else "kv_cache_create failed"
            if self._h:
                _lib.lib().kv_cache_destroy(self._h)
                self._h = C.c_void_p()
            raise _ERRORS.get(rc, CudaError)(text)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            _lib.lib().kv_cache_destroy(h)
            self._h = C.c_void_p()

    def _check(self, rc: int) -> None:
        if rc != _lib.OK:
            text = _lib.lib().kv_cache_last_error(self._h).decode(errors="replace")
            raise _ERRORS.get(rc, CudaError)(text)

    # -- KvCache ------------------------------------------------------------------------------------
    def lengths(self, stream=None) -> List[int]:
        """``KvCache::len`` of every sequence."""
        out = (C.c_int32 * self.sequences)()
        self._check(_lib.lib().kv_cache_lengths(self._h, out, _stream(stream)))
        return list(out)

    def clear(self, sequence: int = -1, stream=None) -> None:
        self._check(_lib.lib().kv_cache_clear(self._h, sequence, _stream(stream)))

    def truncate(self, length: int, sequence: int = -1, stream=None) -> None:
        self._check(_lib.lib().kv_cache_truncate(self._h, sequence, length, _stream(stream)))

    def keys_values(self, sequence: int, stream=None):
        """Cached (post-RoPE) keys and values of one sequence as f32 [len, kv_heads * head_dim]."""
        n = self.lengths(stream)[sequence]
        W = self.kv_heads * self.head_dim
        k = np.empty((n, W), np.float32)
        v = np.empty((n, W), np.float32)
        fp = C.POINTER(C.c_float)
        self._check(_lib.lib().kv_cache_read(self._h, sequence, k.ctypes.data_as(fp), v.ctypes.data_as(fp), _stream(stream)))
        return k, v

    # -- forward_cached -----------------------------------------------------------------------------
    def forward_cached(self, q, k, v, rows_per_sequence: int = 1, first_sequence: int = 0,
                       n_sequences: Optional[int] = None, out=None, stream=None):
        """Device tensors q [rows, num_heads * head_dim] (scratch: may be rotated in place), k and v
        [rows, kv_heads * head_dim], rows = n_sequences * rows_per_sequence; returns the merged heads."""
        import torch
        n_seq = self.sequences - first_sequence if n_sequences is None else n_sequences
        rows = n_seq * rows_per_sequence
        dt = torch.bfloat16 if self.precision == "bf16" else torch.float32
        want = ((rows, self.num_heads * self.head_dim), (rows, self.kv_heads * self.head_dim), (rows, self.kv_heads * self.head_dim))
        for t, shape, name in zip((q, k, v), want, "qkv"):
            if not (t.is_cuda and t.is_contiguous() and t.dtype == dt and tuple(t.shape) == shape):
                raise InvalidInput("%s must be a contiguous %s device tensor of shape %s" % (name, dt, shape))
        if out is None:
            out = torch.empty_like(q)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        self._check(_lib.lib().kv_attention_forward_cached(self._h, first_sequence, n_seq, C.c_void_p(q.data_ptr()),
                                                          C.c_void_p(k.data_ptr()), C.c_void_p(v.data_ptr()),
                                                          rows_per_sequence, C.c_void_p(out.data_ptr()), _stream(stream)))
        return out


__all__ = ["KvCache", "NetworkError"]
