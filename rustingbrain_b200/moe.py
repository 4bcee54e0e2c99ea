"""Host-side mirror of the reference crate's MoE interface over the C ABI.

Names, argument meaning and error behaviour follow ``src/moe.rs`` of
``rusting_brain`` 2.0.2: ``MoeConfig`` (moe.rs:26-87), ``MoeLayer`` (:207-640) with
``forward`` / ``forward_train`` / ``backward``, and ``MoeCache`` (:131-188) with
``aux_loss`` / ``z_loss`` / ``auxiliary_loss`` / ``load_fractions``.  Every call
runs on the GPU through ``libmoe_b200.so``; nothing here computes the layer on the
host.

Activations may be numpy arrays (host memory: the library copies them in and out,
f32) or torch CUDA tensors (device memory: passed by pointer, f32 for an f32 layer,
bf16 for a bf16 layer).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, replace

import numpy as np

from . import _lib
from ._lib import (PRECISION_BF16, PRECISION_F32, PRECISION_Q8, W_DOWN, W_GATE, W_ROUTER, W_SHARED_DOWN,
                   W_SHARED_GATE, W_SHARED_UP, W_UP)

DEFAULT_AUX_LOSS_WEIGHT = 0.01          # moe.rs:20
DEFAULT_ROUTER_Z_LOSS_WEIGHT = 1e-3     # moe.rs:23
UNROUTED = -1                           # moe.rs:191 (usize::MAX there)

_PRECISIONS = {"f32": PRECISION_F32, "bf16": PRECISION_BF16, "q8": PRECISION_Q8}


class NetworkError(RuntimeError):
    """Base of the errors this path raises (the reference's ``NetworkError`` enum, network.rs:19-83)."""


class InvalidConfig(NetworkError):
    pass


class InvalidInput(NetworkError):
    pass


class CudaError(NetworkError):
    pass


class Timeout(NetworkError):
    """A bounded wait gave up: a device-side barrier wait, or a host-side wait behind a collective."""


_ERRORS = {_lib.INVALID_CONFIG: InvalidConfig, _lib.INVALID_INPUT: InvalidInput, _lib.TIMEOUT: Timeout}


@dataclass(frozen=True)
class MoeConfig:
    """``MoeConfig`` (moe.rs:26-66)."""
    num_experts: int
    experts_per_token: int
    d_ff: int
    shared_expert: bool = False
    aux_loss_weight: float = DEFAULT_AUX_LOSS_WEIGHT
    router_z_loss_weight: float = DEFAULT_ROUTER_Z_LOSS_WEIGHT

    def with_shared_expert(self, shared_expert: bool) -> "MoeConfig":
        return replace(self, shared_expert=shared_expert)

    def with_aux_loss_weight(self, weight: float) -> "MoeConfig":
        return replace(self, aux_loss_weight=weight)

    def with_router_z_loss_weight(self, weight: float) -> "MoeConfig":
        return replace(self, router_z_loss_weight=weight)

    def validate(self) -> None:
        """``MoeConfig::validate`` (moe.rs:68-86)."""
        if self.num_experts <= 0:
            raise InvalidConfig("a MoE layer needs at least one expert")
        if self.experts_per_token <= 0 or self.experts_per_token > self.num_experts:
            raise InvalidConfig("experts_per_token must be between 1 and num_experts (%d), got %d" %
                                (self.num_experts, self.experts_per_token))
        if self.d_ff <= 0:
            raise InvalidConfig("expert d_ff must be non-zero")


class MoeCache:
    """What ``forward_train`` returns beside the output (moe.rs:131-188).

    The tensors the backward pass needs stay on the device inside the layer handle;
    this object carries the losses and the routing table.  It is valid until the
    next forward call on the same layer.
    """

    def __init__(self, layer: "MoeLayer", tokens: int, generation: int):
        self._layer = layer
        self._generation = generation
        self.tokens = tokens
        self._losses = None
        self._routing = None

    def _check(self):
        if self._generation != self._layer._generation:
            raise InvalidInput("this MoeCache belongs to an earlier forward pass")

    def _get_losses(self):
        if self._losses is None:
            self._check()
            self._losses = self._layer._losses()
        return self._losses

    def aux_loss(self) -> float:
        """Load-balancing loss, already multiplied by ``aux_loss_weight`` (moe.rs:159-162)."""
        return self._get_losses()[0]

    def z_loss(self) -> float:
        """Router z-loss, already multiplied by its weight (moe.rs:164-168)."""
        return self._get_losses()[1]

    def auxiliary_loss(self) -> float:
        a, z = self._get_losses()
        return a + z

    def routing(self):
        """(expert_of [T,k], gates [T,k], counts [E], token_of [R], slot_of [R])."""
        if self._routing is None:
            self._check()
            self._routing = self._layer._routing(self.tokens)
        return self._routing

    def load_fractions(self):
        """Fraction of routed slots that went to each expert (moe.rs:175-182)."""
        counts = self.routing()[2].astype(np.float32)
        return counts / np.float32(max(int(counts.sum()), 1))


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


class MoeLayer:
    """``MoeLayer`` (moe.rs:207-640) resident on one GPU.

    ``MoeLayer::new`` draws He-uniform weights from the caller's ``StdRng``; that
    stream is not reproduced here, so weights start at zero and are uploaded with
    :meth:`set_weights` / :meth:`set_weight` in the reference's ``[out, in]`` layout.
    """

    def __init__(self, d_model: int, config: MoeConfig, *, precision: str = "bf16", max_tokens: int = 4096,
                 device: int = 0, training: bool = True, ep_rank: int = 0, ep_size: int = 1,
                 ep_capacity_factor: float = 0.0):
        config.validate()
        if precision not in _PRECISIONS:
            raise InvalidConfig("precision must be one of %s" % sorted(_PRECISIONS))
        self.config = config
        self._d = int(d_model)
        self.precision = precision
        self.max_tokens = int(max_tokens)
        self.device = int(device)
        self.training = bool(training)
        self._h = C.c_void_p()
        self._generation = 0
        self._keep = None
        c = _lib.MoeConfigC(self._d, config.num_experts, config.experts_per_token, config.d_ff,
                            int(config.shared_expert), config.aux_loss_weight, config.router_z_loss_weight,
                            _PRECISIONS[precision], self.max_tokens, self.device, int(self.training), ep_rank, ep_size,
                            ep_capacity_factor)
        self._cfg = c
        L = _lib.lib()
        msg = C.create_string_buffer(256)
        if L.moe_config_validate(C.byref(c), msg, 256) != _lib.OK:
            raise InvalidConfig(msg.value.decode())
        rc = L.moe_create(C.byref(c), C.byref(self._h))
        if rc != _lib.OK:
            text = L.moe_last_error(self._h).decode() if self._h else "no usable sm_100 device"
            if self._h:
                L.moe_destroy(self._h)
                self._h = C.c_void_p()
            raise _ERRORS.get(rc, CudaError)("moe_create failed (%d): %s" % (rc, text))

    # -- life cycle -------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc: int):
        if rc != _lib.OK:
            text = _lib.lib().moe_last_error(self._h).decode()
            raise _ERRORS.get(rc, CudaError)("status %d: %s" % (rc, text))

    @staticmethod
    def workspace_bytes(d_model, config: MoeConfig, precision="bf16", max_tokens=4096, training=True) -> int:
        c = _lib.MoeConfigC(d_model, config.num_experts, config.experts_per_token, config.d_ff,
                            int(config.shared_expert), config.aux_loss_weight, config.router_z_loss_weight,
                            _PRECISIONS[precision], max_tokens, 0, int(training), 0, 1, 0.0)
        return int(_lib.lib().moe_workspace_bytes(C.byref(c)))

    def d_model(self) -> int:
        return self._d

    # -- parameters -------------------------------------------------------
    def _shape(self, which):
        E, d, F = self.config.num_experts, self._d, self.config.d_ff
        if which == W_ROUTER:
            return (E, d)
        return (d, F) if which in (W_DOWN, W_SHARED_DOWN) else (F, d)

    def set_weight(self, which: int, expert: int, w):
        """Uploads one projection, f32 ``[out, in]`` (numpy array or torch tensor on any device)."""
        rows, cols = self._shape(which)
        if _is_torch(w):
            import torch
            w = w.detach().to(torch.float32).contiguous()
            if tuple(w.shape) != (rows, cols):
                raise InvalidInput("weight shape %s, expected %s" % (tuple(w.shape), (rows, cols)))
            ptr = w.data_ptr()
        else:
            w = np.ascontiguousarray(w, dtype=np.float32)
            if w.shape != (rows, cols):
                raise InvalidInput("weight shape %s, expected %s" % (w.shape, (rows, cols)))
            ptr = w.ctypes.data
        self._ck(_lib.lib().moe_set_weight_f32(self._h, which, expert, ptr, rows, cols))

    def set_weight_q8(self, which: int, expert: int, q, scales):
        """Uploads one int8 projection: values ``[out, in]`` and one f32 scale per output row
        (``Quantized``, quantized.rs:17-24).  Only for ``precision="q8"`` layers."""
        rows, cols = self._shape(which)
        q = np.ascontiguousarray(q, dtype=np.int8)
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        if q.shape != (rows, cols) or scales.shape != (rows,):
            raise InvalidInput("int8 weight shape %s / %s, expected %s" % (q.shape, scales.shape, (rows, cols)))
        self._ck(_lib.lib().moe_set_weight_q8(self._h, which, expert, q.ctypes.data, scales.ctypes.data, rows, cols))

    def load_snapshot(self, path, block: int):
        """Fills the layer from MoE block ``block`` of a weight file written by the reference's
        ``save_bin`` (transformer.rs:1809-1860), f32 or int8, whatever this layer's precision."""
        self._ck(_lib.lib().moe_load_snapshot_layer(self._h, str(path).encode(), int(block)))

    def load_optimizer_state(self, path, info, block: int) -> int:
        """Restores the Adam moments of MoE block ``block`` from a ``save_optimizer_state`` file
        (transformer.rs:1675-1696); ``info`` is `snapshot.snapshot_info` of the matching weight file.
        Returns the file's step counter."""
        step = C.c_int64(0)
        self._ck(_lib.lib().moe_load_optimizer_layer(self._h, str(path).encode(), C.byref(info._c), int(block),
                                                     C.byref(step)))
        return int(step.value)

    # ---- low-rank adapters on the expert projections (TransformerLm::add_lora / merge_lora) ----
    def lora_attach(self, rank: int, alpha: float = None):
        """Attaches `W + (alpha / rank) * up * down` adapters to every expert projection (not the router)
        and freezes the base weights (param.rs:635-714, moe.rs:502-514).  ``alpha`` defaults to ``rank``."""
        self._ck(_lib.lib().moe_lora_attach(self._h, int(rank), float(rank if alpha is None else alpha)))
        self._lora_rank = int(rank)

    def _lora_shapes(self, which):
        rows, cols = self._shape(which)
        r = getattr(self, "_lora_rank", 0)
        return (r, cols), (rows, r)

    def lora_set(self, which: int, expert: int, down, up):
        ds, us = self._lora_shapes(which)
        down = np.ascontiguousarray(down, dtype=np.float32)
        up = np.ascontiguousarray(up, dtype=np.float32)
        if down.shape != ds or up.shape != us:
            raise InvalidInput("adapter shapes %s / %s, expected %s / %s" % (down.shape, up.shape, ds, us))
        self._ck(_lib.lib().moe_lora_set(self._h, which, expert, down.ctypes.data, up.ctypes.data))

    def _lora_read(self, fn, which, expert):
        ds, us = self._lora_shapes(which)
        down, up = np.empty(ds, np.float32), np.empty(us, np.float32)
        self._ck(fn(self._h, which, expert, down.ctypes.data, up.ctypes.data))
        return down, up

    def lora_get(self, which: int, expert: int = 0):
        """(down [rank, in], up [out, rank])."""
        return self._lora_read(_lib.lib().moe_lora_get, which, expert)

    def lora_get_grad(self, which: int, expert: int = 0):
        """Gradients of (down, up) from the accumulated weight gradient (Lora::backward, param.rs:690-709)."""
        return self._lora_read(_lib.lib().moe_lora_get_grad, which, expert)

    def load_lora(self, path, info, block: int):
        """Fills the attached adapters from block ``block`` of a ``save_lora`` file
        (transformer.rs:1109-1202); ``info`` is `snapshot.snapshot_info` of the matching weight file."""
        self._ck(_lib.lib().moe_load_lora_layer(self._h, str(path).encode(), C.byref(info._c), int(block)))

    def lora_merge(self):
        """Adds the adapters into the weights and removes them (merge_lora)."""
        self._ck(_lib.lib().moe_lora_merge(self._h))
        self._lora_rank = 0

    def set_weights(self, router, gate, up, down, shared=None):
        """router [E,d]; gate/up [E,F,d]; down [E,d,F]; shared = (gate, up, down) of one expert."""
        self.set_weight(W_ROUTER, 0, router)
        for e in range(self.config.num_experts):
            self.set_weight(W_GATE, e, gate[e])
            self.set_weight(W_UP, e, up[e])
            self.set_weight(W_DOWN, e, down[e])
        if shared is not None:
            for which, w in zip((W_SHARED_GATE, W_SHARED_UP, W_SHARED_DOWN), shared):
                self.set_weight(which, 0, w)

    def _read(self, fn, which, expert):
        rows, cols = self._shape(which)
        out = np.empty((rows, cols), np.float32)
        self._ck(fn(self._h, which, expert, out.ctypes.data, rows, cols))
        return out

    def get_weight(self, which: int, expert: int = 0):
        return self._read(_lib.lib().moe_get_weight_f32, which, expert)

    def get_grad(self, which: int, expert: int = 0):
        """Plain dL/dW accumulated since the last :meth:`zero_grad` / optimizer step."""
        return self._read(_lib.lib().moe_get_grad_f32, which, expert)

    def get_moments(self, which: int, expert: int = 0):
        rows, cols = self._shape(which)
        m = np.empty((rows, cols), np.float32)
        v = np.empty((rows, cols), np.float32)
        self._ck(_lib.lib().moe_get_moments_f32(self._h, which, expert, m.ctypes.data, v.ctypes.data, rows, cols))
        return m, v

    def zero_grad(self):
        self._ck(_lib.lib().moe_zero_grad(self._h, None))

    def step_adam(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, scale=1.0, stream=None):
        """``Param::step`` with ``Optimizer::Adam`` over the whole layer (param.rs:562-589)."""
        self._ck(_lib.lib().moe_step_adam(self._h, lr, beta1, beta2, eps, weight_decay, step, scale, _stream(stream)))

    def step_sgd(self, lr=1e-2, scale=1.0, stream=None):
        """``Param::step`` with ``Optimizer::Sgd`` (param.rs:557-561)."""
        self._ck(_lib.lib().moe_step_sgd(self._h, lr, scale, _stream(stream)))

    def step_lion(self, lr=1e-4, beta1=0.9, beta2=0.99, weight_decay=0.0, scale=1.0, stream=None):
        """``Param::step`` with ``Optimizer::Lion`` (param.rs:590-613); betas default as ``Optimizer::lion``."""
        self._ck(_lib.lib().moe_step_lion(self._h, lr, beta1, beta2, weight_decay, scale, _stream(stream)))

    # -- forward / backward ----------------------------------------------
    def forward(self, x, valid=None, out=None, stream=None):
        """``MoeLayer::forward`` (moe.rs:237): the output only, nothing kept for a backward pass."""
        return self._forward(x, valid, out, stream, save=False, logits=None)[0]

    def forward_train(self, x, valid=None, out=None, stream=None, logits=None):
        """``MoeLayer::forward_train`` (moe.rs:243-341): ``(output, MoeCache)``.

        ``valid`` is the padding mask of ``Layout`` (batch.rs:225-269): rows with 0 are
        routed nowhere and left out of the auxiliary statistics.  ``logits`` (device
        f32 ``[T, E]``) replaces the router projection; the parity tests use it.
        """
        return self._forward(x, valid, out, stream, save=self.training, logits=logits)

    def _forward(self, x, valid, out, stream, save, logits):
        L = _lib.lib()
        self._generation += 1
        if _is_torch(x):
            import torch
            want = torch.float32 if self.precision == "f32" else torch.bfloat16
            if x.dim() != 2 or not x.is_cuda or x.dtype != want or not x.is_contiguous():
                raise InvalidInput("expected a contiguous CUDA %s tensor [tokens, d_model]" % want)
            T, cols = x.shape
            y = out if out is not None else torch.empty((T, self._d), dtype=want, device=x.device)
            v = None
            if valid is not None:
                v = torch.as_tensor(valid).to(device=x.device, dtype=torch.uint8).contiguous()
                if v.numel() != T:
                    raise InvalidConfig("padding mask covers %d rows, not %d" % (v.numel(), T))  # batch.rs:262-266
            st = _stream(stream if stream is not None else torch.cuda.current_stream(x.device).cuda_stream)
            vp = v.data_ptr() if v is not None else None
            if logits is not None:
                rc = L.moe_forward_from_logits(self._h, x.data_ptr(), logits.data_ptr(), T, cols, vp, y.data_ptr(), 0,
                                               int(save), st)
            else:
                rc = L.moe_forward(self._h, x.data_ptr(), T, cols, vp, y.data_ptr(), 0, int(save), st)
            self._ck(rc)
            self._keep = (x, v, logits)   # the backward pass reads x again
            return y, MoeCache(self, T, self._generation)
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim != 2:
            raise InvalidInput("expected [tokens, d_model]")
        T, cols = x.shape
        v = None
        if valid is not None:
            v = np.ascontiguousarray(valid, dtype=np.uint8)
            if v.size != T:
                raise InvalidConfig("padding mask covers %d rows, not %d" % (v.size, T))
        y = out if out is not None else np.empty((T, self._d), np.float32)
        fp, bp = C.POINTER(C.c_float), C.POINTER(C.c_uint8)
        self._ck(L.moe_forward_host(self._h, x.ctypes.data_as(fp), T, cols, v.ctypes.data_as(bp) if v is not None else None,
                                    y.ctypes.data_as(fp), int(save)))
        return y, MoeCache(self, T, self._generation)

    def backward(self, cache: MoeCache, grad_output, out=None, stream=None):
        """``MoeLayer::backward`` (moe.rs:348-489): accumulates weight gradients, returns dL/dinput."""
        cache._check()
        L = _lib.lib()
        if _is_torch(grad_output):
            import torch
            g = grad_output.contiguous()
            gx = out if out is not None else torch.empty_like(g)
            st = _stream(stream if stream is not None else torch.cuda.current_stream(g.device).cuda_stream)
            self._ck(L.moe_backward(self._h, g.data_ptr(), gx.data_ptr(), 0, st))
            return gx
        g = np.ascontiguousarray(grad_output, dtype=np.float32)
        gx = out if out is not None else np.empty_like(g)
        fp = C.POINTER(C.c_float)
        self._ck(L.moe_backward_host(self._h, g.ctypes.data_as(fp), gx.ctypes.data_as(fp)))
        return gx

    # -- cache read-back --------------------------------------------------
    def _losses(self):
        a, z = C.c_float(), C.c_float()
        self._ck(_lib.lib().moe_get_losses(self._h, C.byref(a), C.byref(z)))
        return a.value, z.value

    def _routing(self, T):
        k, E = self.config.experts_per_token, self.config.num_experts
        expert_of = np.empty((T, k), np.int32)
        gates = np.empty((T, k), np.float32)
        counts = np.empty(E, np.int32)
        token_of = np.empty(T * k, np.int32)
        slot_of = np.empty(T * k, np.int32)
        n = C.c_int32()
        ip, fp = C.POINTER(C.c_int32), C.POINTER(C.c_float)
        self._ck(_lib.lib().moe_get_routing(self._h, expert_of.ctypes.data_as(ip), gates.ctypes.data_as(fp),
                                            counts.ctypes.data_as(ip), token_of.ctypes.data_as(ip),
                                            slot_of.ctypes.data_as(ip), C.byref(n)))
        return expert_of, gates, counts, token_of[:n.value].copy(), slot_of[:n.value].copy()

    def router_cache(self, T):
        """(logits, probabilities, log-sum-exp) of the last forward, as numpy arrays."""
        E = self.config.num_experts
        logits = np.empty((T, E), np.float32)
        probs = np.empty((T, E), np.float32)
        lse = np.empty(T, np.float32)
        fp = C.POINTER(C.c_float)
        self._ck(_lib.lib().moe_get_router_cache(self._h, logits.ctypes.data_as(fp), probs.ctypes.data_as(fp),
                                                 lse.ctypes.data_as(fp)))
        return logits, probs, lse

    PROFILE_STAGES = ("router", "permute", "gemm_gate_up", "gemm_down", "combine", "grad_gather", "dgrad_down",
                      "wgrad_down", "dgrad_gate_up", "wgrad_gate_up", "router_bwd", "unpermute", "router_wgrad",
                      "shared_fwd", "shared_bwd", "adam")

    def profile(self, enable: bool):
        """Brackets every stage with CUDA events on the launching stream (measurement aid)."""
        self._ck(_lib.lib().moe_debug_profile(self._h, int(enable)))

    def profile_read(self):
        """{stage: (milliseconds, launches)} accumulated since the last read; synchronises."""
        n = len(self.PROFILE_STAGES)
        ms = (C.c_float * n)()
        cnt = (C.c_int32 * n)()
        self._ck(_lib.lib().moe_debug_profile_read(self._h, ms, cnt))
        return {name: (float(ms[i]), int(cnt[i])) for i, name in enumerate(self.PROFILE_STAGES)}

    def clear_error(self):
        """Lifts the sticky error state after a failed call (the reference's poisoned context has no such
        call: it is rebuilt; here the workspace is kept)."""
        self._ck(_lib.lib().moe_clear_error(self._h))

    def synchronize(self):
        self._ck(_lib.lib().moe_synchronize(self._h))

    def num_parameters(self) -> int:
        """moe.rs:528-536."""
        c = self.config
        per = 3 * c.d_ff * self._d
        return c.num_experts * self._d + c.num_experts * per + (per if c.shared_expert else 0)

    def active_parameters(self) -> int:
        """moe.rs:540-545."""
        c = self.config
        per = 3 * c.d_ff * self._d
        return c.num_experts * self._d + c.experts_per_token * per + (per if c.shared_expert else 0)


def _stream(s):
    if s is None:
        return None
    return C.c_void_p(int(s))
