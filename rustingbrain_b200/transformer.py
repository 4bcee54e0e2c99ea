"""Host-side mirror of the reference's ``TransformerLm`` builder and training entry points over the C ABI of
include/transformer_b200.h (reference transformer.rs:236-450 builder, :676 forward_batch, :1394 train_step_batch,
:1519 accumulate_step, :1576 step, :1604 zero_grad; ``TotalLoss`` causal_lm_loss.rs:30-49; ``TokenBatch``
batch.rs:22-222).

Same names, argument meaning and error classes as the reference.  Weights are injected by the caller
(``set_param``): the reference's builder seed drives rand's StdRng, whose stream is not reproduced, so ``seed``
here fills the model from numpy's Philox with the reference's distributions (He-uniform projections,
param.rs:240-246; U(-0.02, 0.02) embedding, embedding.rs:26-33; unit norm weights).  There is no host
implementation behind this object: without the CUDA library every call raises.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field, replace
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from .moe import CudaError, InvalidConfig, InvalidInput, NetworkError, Timeout, DEFAULT_AUX_LOSS_WEIGHT, \
    DEFAULT_ROUTER_Z_LOSS_WEIGHT

_ERRORS = {_lib.INVALID_CONFIG: InvalidConfig, _lib.INVALID_INPUT: InvalidInput, _lib.TIMEOUT: Timeout,
           _lib.UNSUPPORTED: InvalidConfig}

(EMBEDDING, FINAL_NORM, HEAD, ATTENTION_NORM, WQ, WK, WV, WO, FFN_NORM, FFN_GATE, FFN_UP, FFN_DOWN, MOE_ROUTER, MOE_GATE,
 MOE_UP, MOE_DOWN, MOE_SHARED_GATE, MOE_SHARED_UP, MOE_SHARED_DOWN) = range(19)


@dataclass(frozen=True)
class Adam:
    """``Optimizer::adam(learning_rate)`` (optimizers.rs:65-73)."""
    learning_rate: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8
    weight_decay: float = 0.0


@dataclass(frozen=True)
class Sgd:
    """``Optimizer::sgd(learning_rate)`` (optimizers.rs:61-63)."""
    learning_rate: float = 1e-2


@dataclass(frozen=True)
class Lion:
    """``Optimizer::lion(learning_rate)`` / ``lion_with_weight_decay`` (optimizers.rs:86-104)."""
    learning_rate: float = 3e-5
    beta1: float = 0.9
    beta2: float = 0.99
    weight_decay: float = 0.0


@dataclass(frozen=True)
class TotalLoss:
    """causal_lm_loss.rs:30-49."""
    lm_loss: float
    auxiliary_loss: float

    def total(self) -> float:
        return self.lm_loss + self.auxiliary_loss

    def perplexity(self) -> float:
        return float(np.exp(self.lm_loss))


@dataclass(frozen=True)
class TransformerConfig:
    """transformer.rs:28-58 with the defaults of :99-125 (the 55M-total / 36M-active model)."""
    vocab_size: int = 32000
    d_model: int = 512
    n_layers: int = 8
    n_heads: int = 8
    n_kv_heads: int = 2
    head_dim: int = 64
    d_ff: int = 1408
    moe_d_ff: int = 352
    num_experts: int = 8
    experts_per_token: int = 2
    moe_layers: Tuple[int, ...] = tuple(range(2, 8))
    shared_expert: bool = True
    max_seq_len: int = 2048
    rope_base: float = 10000.0
    rmsnorm_eps: float = 1e-6
    tie_embeddings: bool = True
    causal: bool = True
    aux_loss_weight: float = DEFAULT_AUX_LOSS_WEIGHT
    router_z_loss_weight: float = DEFAULT_ROUTER_Z_LOSS_WEIGHT

    def is_moe_layer(self, layer: int) -> bool:
        return layer in self.moe_layers

    def _c(self, max_batch_rows: int, device: int) -> "_lib.LmConfigC":
        mask = 0
        for layer in self.moe_layers:
            if layer >= 64:
                raise InvalidConfig("moe_layers names layer %d, but at most 64 layers are supported" % layer)
            mask |= 1 << layer
        return _lib.LmConfigC(self.vocab_size, self.d_model, self.n_layers, self.n_heads, self.n_kv_heads, self.head_dim,
                              self.d_ff, self.moe_d_ff, self.num_experts, self.experts_per_token, int(self.shared_expert),
                              mask, self.max_seq_len, self.rope_base, self.rmsnorm_eps, int(self.tie_embeddings),
                              self.aux_loss_weight, self.router_z_loss_weight, max_batch_rows, device)

    def validate(self) -> None:
        """TransformerConfig::validate (transformer.rs:132-172) plus the shape rules of the device products."""
        if not self.causal:
            raise InvalidConfig("the device path trains causal models only")
        msg = C.create_string_buffer(256)
        if _lib.lib().lm_config_validate(C.byref(self._c(2, 0)), msg, 256) != _lib.OK:
            raise InvalidConfig(msg.value.decode())

    def parameter_counts(self) -> Tuple[int, int]:
        """(total, active), transformer.rs:195-235."""
        total, active = C.c_int64(), C.c_int64()
        _lib.lib().lm_parameter_counts(C.byref(self._c(2, 0)), C.byref(total), C.byref(active))
        return total.value, active.value


class TokenBatch:
    """Sequences right-padded to the longest (batch.rs:35-75); optional per-token loss mask (:127-146)."""

    def __init__(self, sequences: Sequence[Sequence[int]], loss_mask: Optional[Sequence[bool]] = None):
        if len(sequences) == 0:
            raise InvalidConfig("EmptyDataset")
        self.lengths = np.asarray([len(s) for s in sequences], np.int32)
        if int(self.lengths.min()) < 2:
            raise InvalidConfig("a causal language-modelling loss needs at least two tokens per sequence, got %d"
                                % int(self.lengths.min()))
        self.batch, self.seq_len = len(sequences), int(self.lengths.max())
        self.ids = np.zeros(self.batch * self.seq_len, np.uint32)
        for i, s in enumerate(sequences):
            self.ids[i * self.seq_len:i * self.seq_len + len(s)] = np.asarray(s, np.uint32)
        self.loss_mask = None
        if loss_mask is not None:
            if len(loss_mask) != len(self.ids):
                raise InvalidConfig("a loss mask covers %d token positions, not %d" % (len(loss_mask), len(self.ids)))
            self.loss_mask = np.ascontiguousarray(loss_mask, dtype=np.uint8)

    @property
    def rows(self) -> int:
        return len(self.ids)

    def is_padded(self) -> bool:
        return bool((self.lengths != self.seq_len).any())


class TransformerBuilder:
    """transformer.rs:271-450: one setter per configuration field, then ``build()``."""

    def __init__(self):
        self._config = TransformerConfig()
        self._optimizer = Adam(3e-4)
        self._seed: Optional[int] = None
        self._mixed_precision = True
        self._max_batch_rows = 8192
        self._device = 0

    def _set(self, **kw) -> "TransformerBuilder":
        self._config = replace(self._config, **kw)
        return self

    def config(self, config: TransformerConfig): self._config = config; return self
    def vocab_size(self, n: int): return self._set(vocab_size=n)
    def d_model(self, n: int): return self._set(d_model=n)
    def n_layers(self, n: int): return self._set(n_layers=n)
    def heads(self, n_heads: int, n_kv_heads: int, head_dim: int): return self._set(n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim)
    def d_ff(self, n: int): return self._set(d_ff=n)
    def moe_d_ff(self, n: int): return self._set(moe_d_ff=n)
    def experts(self, num_experts: int, experts_per_token: int): return self._set(num_experts=num_experts, experts_per_token=experts_per_token)
    def moe_layers(self, layers: Iterable[int]): return self._set(moe_layers=tuple(layers))
    def shared_expert(self, on: bool): return self._set(shared_expert=on)
    def max_seq_len(self, n: int): return self._set(max_seq_len=n)
    def rope_base(self, base: float): return self._set(rope_base=base)
    def rmsnorm_eps(self, eps: float): return self._set(rmsnorm_eps=eps)
    def bidirectional(self, on: bool): return self._set(causal=not on)
    def tie_embeddings(self, on: bool): return self._set(tie_embeddings=on)
    def aux_loss_weight(self, w: float): return self._set(aux_loss_weight=w)
    def router_z_loss_weight(self, w: float): return self._set(router_z_loss_weight=w)
    def optimizer(self, optimizer): self._optimizer = optimizer; return self
    def seed(self, seed: int): self._seed = seed; return self

    def mixed_precision(self, on: bool):
        """The device path computes in bf16 over f32 master weights; ``False`` is refused at ``build``."""
        self._mixed_precision = on
        return self

    def max_batch_rows(self, rows: int):
        """Not in the reference: the largest ``batch * seq_len`` a step will see (sizes the device workspace)."""
        self._max_batch_rows = rows
        return self

    def device(self, index: int): self._device = index; return self

    def parameter_counts(self) -> Tuple[int, int]:
        return self._config.parameter_counts()

    def build(self) -> "TransformerLm":
        return TransformerLm(self)


class TransformerLm:
    """``TransformerLm`` resident on one B200 (the state the reference reaches with ``to_cuda``)."""

    @staticmethod
    def builder() -> TransformerBuilder:
        return TransformerBuilder()

    def __init__(self, builder: TransformerBuilder):
        cfg = builder._config
        cfg.validate()
        if not builder._mixed_precision:
            raise InvalidConfig("the device path runs bf16 products over f32 master weights (mixed_precision)")
        self.config, self.optimizer = cfg, builder._optimizer
        self._h = C.c_void_p()
        rc = _lib.lib().lm_create(C.byref(cfg._c(builder._max_batch_rows, builder._device)), C.byref(self._h))
        if rc != _lib.OK:
            text = _lib.lib().lm_last_error(self._h).decode(errors="replace") if self._h else "lm_create failed"
            if self._h:
                _lib.lib().lm_destroy(self._h)
                self._h = C.c_void_p()
            raise _ERRORS.get(rc, CudaError)(text)
        if builder._seed is not None:
            self._init_from_seed(builder._seed)

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().lm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc: int) -> None:
        if rc != _lib.OK:
            raise _ERRORS.get(rc, CudaError)("status %d: %s" % (rc, _lib.lib().lm_last_error(self._h).decode(errors="replace")))

    # -- parameters ---------------------------------------------------------------------------------
    def param_shape(self, which: int) -> Tuple[int, int]:
        c = self.config
        HD, KD = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        return {EMBEDDING: (c.vocab_size, c.d_model), HEAD: (c.vocab_size, c.d_model), FINAL_NORM: (1, c.d_model),
                ATTENTION_NORM: (1, c.d_model), FFN_NORM: (1, c.d_model), WQ: (HD, c.d_model), WK: (KD, c.d_model),
                WV: (KD, c.d_model), WO: (c.d_model, HD), FFN_GATE: (c.d_ff, c.d_model), FFN_UP: (c.d_ff, c.d_model),
                FFN_DOWN: (c.d_model, c.d_ff), MOE_ROUTER: (c.num_experts, c.d_model), MOE_GATE: (c.moe_d_ff, c.d_model),
                MOE_UP: (c.moe_d_ff, c.d_model), MOE_DOWN: (c.d_model, c.moe_d_ff), MOE_SHARED_GATE: (c.moe_d_ff, c.d_model),
                MOE_SHARED_UP: (c.moe_d_ff, c.d_model), MOE_SHARED_DOWN: (c.d_model, c.moe_d_ff)}[which]

    def set_param(self, which: int, value, layer: int = 0, expert: int = 0) -> None:
        rows, cols = self.param_shape(which)
        a = np.ascontiguousarray(value, dtype=np.float32).reshape(rows, cols)
        self._ck(_lib.lib().lm_set_param(self._h, layer, which, expert, a.ctypes.data_as(C.c_void_p), rows, cols))

    def _read(self, fn, which: int, layer: int, expert: int) -> np.ndarray:
        rows, cols = self.param_shape(which)
        out = np.empty((rows, cols), np.float32)
        self._ck(fn(self._h, layer, which, expert, out.ctypes.data_as(C.c_void_p), rows, cols))
        return out[0] if rows == 1 else out

    def get_param(self, which: int, layer: int = 0, expert: int = 0) -> np.ndarray:
        return self._read(_lib.lib().lm_get_param, which, layer, expert)

    def get_grad(self, which: int, layer: int = 0, expert: int = 0) -> np.ndarray:
        return self._read(_lib.lib().lm_get_grad, which, layer, expert)

    def load_weights(self, w: dict) -> None:
        """A dict shaped like ``oracle.transformer.seeded_model_weights``: embedding, final_norm, (lm_head,) blocks[...]."""
        c = self.config
        self.set_param(EMBEDDING, w["embedding"])
        self.set_param(FINAL_NORM, w["final_norm"])
        if not c.tie_embeddings:
            self.set_param(HEAD, w["lm_head"])
        for layer, b in enumerate(w["blocks"]):
            for which, key in ((ATTENTION_NORM, "attention_norm"), (WQ, "wq"), (WK, "wk"), (WV, "wv"), (WO, "wo"), (FFN_NORM, "ffn_norm")):
                self.set_param(which, b[key], layer)
            if c.is_moe_layer(layer):
                m = b["moe"]
                self.set_param(MOE_ROUTER, m["router"], layer)
                for e in range(c.num_experts):
                    self.set_param(MOE_GATE, m["gate"][e], layer, e)
                    self.set_param(MOE_UP, m["up"][e], layer, e)
                    self.set_param(MOE_DOWN, m["down"][e], layer, e)
                if c.shared_expert:
                    for i, s in enumerate(m["shared"]):
                        self.set_param(MOE_SHARED_GATE + i, s, layer)
            else:
                self.set_param(FFN_GATE, b["gate"], layer)
                self.set_param(FFN_UP, b["up"], layer)
                self.set_param(FFN_DOWN, b["down"], layer)

    def _init_from_seed(self, seed: int) -> None:
        c, g = self.config, np.random.Generator(np.random.Philox(seed))
        he = lambda rows, cols: g.uniform(-np.sqrt(2.0 / cols), np.sqrt(2.0 / cols), (rows, cols)).astype(np.float32)
        ones = np.ones(c.d_model, np.float32)
        w = dict(embedding=g.uniform(-0.02, 0.02, (c.vocab_size, c.d_model)).astype(np.float32), final_norm=ones, blocks=[])
        if not c.tie_embeddings:
            w["lm_head"] = he(c.vocab_size, c.d_model)
        for layer in range(c.n_layers):
            b = dict(attention_norm=ones, ffn_norm=ones, wq=he(*self.param_shape(WQ)), wk=he(*self.param_shape(WK)),
                     wv=he(*self.param_shape(WV)), wo=he(*self.param_shape(WO)))
            if c.is_moe_layer(layer):
                E = c.num_experts
                b["moe"] = dict(router=he(E, c.d_model), gate=[he(c.moe_d_ff, c.d_model) for _ in range(E)],
                                up=[he(c.moe_d_ff, c.d_model) for _ in range(E)], down=[he(c.d_model, c.moe_d_ff) for _ in range(E)],
                                shared=(he(c.moe_d_ff, c.d_model), he(c.moe_d_ff, c.d_model), he(c.d_model, c.moe_d_ff)) if c.shared_expert else None)
            else:
                b.update(gate=he(c.d_ff, c.d_model), up=he(c.d_ff, c.d_model), down=he(c.d_model, c.d_ff))
            w["blocks"].append(b)
        self.load_weights(w)

    # -- passes ---------------------------------------------------------------------------------------
    @staticmethod
    def _batch(sequences_or_batch) -> TokenBatch:
        return sequences_or_batch if isinstance(sequences_or_batch, TokenBatch) else TokenBatch(sequences_or_batch)

    def _args(self, b: TokenBatch):
        return (b.ids.ctypes.data_as(C.c_void_p), b.lengths.ctypes.data_as(C.c_void_p) if b.is_padded() else None)

    def forward_batch(self, batch, return_router_logits: bool = False):
        """Logits [batch * seq_len, vocab] (f32, host); optionally the router logits of every MoE layer."""
        b = self._batch(batch)
        logits = np.empty((b.rows, self.config.vocab_size), np.float32)
        n_moe = len(self.config.moe_layers)
        router = np.empty((n_moe, b.rows, self.config.num_experts), np.float32) if return_router_logits and n_moe else None
        ids, lengths = self._args(b)
        self._ck(_lib.lib().lm_forward_logits(self._h, ids, lengths, b.batch, b.seq_len, logits.ctypes.data_as(C.c_void_p),
                                              router.ctypes.data_as(C.c_void_p) if router is not None else None))
        return (logits, router) if return_router_logits else logits

    forward_train = forward_batch

    def accumulate_step(self, batch) -> TotalLoss:
        b = self._batch(batch)
        lm, aux = C.c_float(), C.c_float()
        ids, lengths = self._args(b)
        mask = b.loss_mask.ctypes.data_as(C.c_void_p) if b.loss_mask is not None else None
        self._ck(_lib.lib().lm_accumulate_step(self._h, ids, lengths, mask, b.batch, b.seq_len, C.byref(lm), C.byref(aux)))
        return TotalLoss(lm.value, aux.value)

    def zero_grad(self) -> None:
        self._ck(_lib.lib().lm_zero_grad(self._h))

    def step(self, scale: float = 1.0) -> None:
        """``TransformerLm::step`` (transformer.rs:1576-1606) with whichever optimizer the model holds."""
        o = self.optimizer
        if isinstance(o, Sgd):
            self._ck(_lib.lib().lm_step_sgd(self._h, o.learning_rate, scale))
        elif isinstance(o, Lion):
            self._ck(_lib.lib().lm_step_lion(self._h, o.learning_rate, o.beta1, o.beta2, o.weight_decay, scale))
        else:
            self._ck(_lib.lib().lm_step_adam(self._h, o.learning_rate, o.beta1, o.beta2, o.epsilon, o.weight_decay, scale))

    def train_step_batch(self, batch) -> TotalLoss:
        o = self.optimizer
        if not isinstance(o, Adam):
            self.zero_grad()
            out = self.accumulate_step(batch)
            self.step(1.0)
            return out
        b = self._batch(batch)
        lm, aux = C.c_float(), C.c_float()
        ids, lengths = self._args(b)
        mask = b.loss_mask.ctypes.data_as(C.c_void_p) if b.loss_mask is not None else None
        self._ck(_lib.lib().lm_train_step(self._h, ids, lengths, mask, b.batch, b.seq_len, o.learning_rate, o.beta1, o.beta2,
                                          o.epsilon, o.weight_decay, C.byref(lm), C.byref(aux)))
        return TotalLoss(lm.value, aux.value)

    train_step = train_step_batch

    # -- KV-cached decode ---------------------------------------------------------------------------
    def new_kv_caches(self, sequences: int = 1, capacity: Optional[int] = None) -> "KvCaches":
        """One cache per layer (transformer.rs:649-660), for ``sequences`` sequences that decode together."""
        return KvCaches(self, sequences, capacity if capacity is not None else self.config.max_seq_len)

    def forward_cached(self, ids, caches: "KvCaches", first_sequence: int = 0) -> np.ndarray:
        """``ids``: one list of new token ids per sequence (equal lengths: the prompts for a prefill, one id each
        for a decode step), or a flat list for a single sequence.  Returns logits [sequences * rows, vocab]."""
        if len(ids) and not hasattr(ids[0], "__len__"):
            ids = [ids]
        per = len(ids[0])
        if per == 0 or any(len(s) != per for s in ids):
            raise InvalidInput("forward_cached takes the same number of new ids for every sequence")
        flat = np.ascontiguousarray(np.asarray(ids, np.uint32).reshape(-1))
        logits = np.empty((len(flat), self.config.vocab_size), np.float32)
        self._ck(_lib.lib().lm_forward_cached(self._h, caches._h, flat.ctypes.data_as(C.c_void_p), first_sequence, len(ids), per,
                                              logits.ctypes.data_as(C.c_void_p)))
        return logits

    def optimizer_step(self) -> int:
        return int(_lib.lib().lm_optimizer_step(self._h))

    def set_optimizer_step(self, step: int) -> None:
        self._ck(_lib.lib().lm_set_optimizer_step(self._h, step))

    def parameter_counts(self) -> Tuple[int, int]:
        return self.config.parameter_counts()

    def last_step_ms(self) -> List[float]:
        ms = (C.c_float * 4)()
        self._ck(_lib.lib().lm_last_step_ms(self._h, ms))
        return list(ms)

    def synchronize(self) -> None:
        self._ck(_lib.lib().lm_synchronize(self._h))


class KvCaches:
    """``Vec<KvCache>`` of the reference, batched over sequences; owned by the caller, tied to one model."""

    def __init__(self, model: TransformerLm, sequences: int, capacity: int):
        self._model, self.sequences, self.capacity = model, sequences, capacity
        self._h = C.c_void_p()
        model._ck(_lib.lib().lm_decoder_create(model._h, sequences, capacity, C.byref(self._h)))

    def clear(self, sequence: int = -1) -> None:
        self._model._ck(_lib.lib().lm_decoder_clear(self._model._h, self._h, sequence))

    def __del__(self):
        if getattr(self, "_h", None):
            _lib.lib().lm_decoder_destroy(self._h)
            self._h = C.c_void_p()


__all__ = ["KvCaches", "Adam", "Sgd", "Lion", "TotalLoss", "TransformerConfig", "TransformerBuilder", "TransformerLm", "TokenBatch", "NetworkError"]
