"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

ctypes front end of ``libmoe_oracle.so`` (built from ``moe_oracle.cpp`` by the
Makefile beside it): a CPU restatement of the reference crate's
``MoeLayer`` (``src/moe.rs``), ``SwiGlu`` (``src/ffn.rs``), ``Quantized``
(``src/quantized.rs``) and Adam step (``src/param.rs:562-589``).

Only the tests, the smoke check and the CPU-baseline / reference legs of the
benchmark import this package.  The CUDA library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmoe_oracle.so")

ROUTER, GATE, UP, DOWN, SHARED_GATE, SHARED_UP, SHARED_DOWN = range(7)


def build(force: bool = False) -> str:
    """Compiles the restatement with the Makefile in this directory."""
    src = os.path.join(_HERE, "moe_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libmoe_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        fp, ip, bp, vp = C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_uint8), C.c_void_p
        L.orc_create.restype = vp
        L.orc_create.argtypes = [C.c_int] * 5 + [C.c_float] * 2
        L.orc_destroy.argtypes = [vp]
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_max_threads.restype = C.c_int
        L.orc_set_weight.argtypes = [vp, C.c_int, C.c_int, fp, C.c_int, C.c_int]
        L.orc_get_weight.argtypes = [vp, C.c_int, C.c_int, fp]
        L.orc_get_grad.argtypes = [vp, C.c_int, C.c_int, fp]
        L.orc_get_moments.argtypes = [vp, C.c_int, C.c_int, fp, fp]
        L.orc_set_weight_q8.argtypes = [vp, C.c_int, C.c_int, C.POINTER(C.c_int8), fp, C.c_int, C.c_int]
        L.orc_quantize.argtypes = [vp, C.c_int]
        L.orc_quantize_rows.argtypes = [fp, C.c_int, C.c_int, C.POINTER(C.c_int8), fp]
        L.orc_q8_matmul.argtypes = [fp, C.c_int, C.POINTER(C.c_int8), fp, C.c_int, C.c_int, fp]
        L.orc_softmax_rows.argtypes = [fp, C.c_int, C.c_int, fp, fp]
        L.orc_route.argtypes = [fp, C.c_int, C.c_int, C.c_int, bp, ip, fp]
        L.orc_silu.restype = C.c_float
        L.orc_silu.argtypes = [C.c_float]
        L.orc_silu_derivative.restype = C.c_float
        L.orc_silu_derivative.argtypes = [C.c_float]
        L.orc_forward.restype = C.c_int
        L.orc_forward.argtypes = [vp, fp, C.c_int, C.c_int, bp, C.c_int, fp, fp]
        L.orc_get_losses.argtypes = [vp, fp, fp]
        L.orc_get_routing.restype = C.c_int
        L.orc_get_routing.argtypes = [vp, ip, fp, ip, ip, ip]
        L.orc_get_router.argtypes = [vp, fp, fp, fp]
        L.orc_get_expert_rows.argtypes = [vp, fp, fp]
        L.orc_zero_grad.argtypes = [vp]
        L.orc_backward.restype = C.c_int
        L.orc_backward.argtypes = [vp, fp, fp]
        L.orc_adam_step.argtypes = [vp] + [C.c_float] * 5 + [C.c_int, C.c_float]
        L.orc_sgd_step.argtypes = [vp, C.c_float, C.c_float]
        L.orc_sgd_apply.argtypes = [vp, vp, C.c_longlong, C.c_float, C.c_float]
        L.orc_lion_apply.argtypes = [vp, vp, vp, C.c_longlong] + [C.c_float] * 5
        L.orc_lion_step.argtypes = [vp] + [C.c_float] * 5
        _lib = L
    return _lib


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return a.ctypes.data_as(C.POINTER(C.c_int))


def _b(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint8))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def softmax_rows(logits):
    """``moe.rs:643-656``: (probabilities, log-sum-exp) of each row."""
    logits = _f32(logits)
    T, E = logits.shape
    probs = np.empty((T, E), np.float32)
    lse = np.empty(T, np.float32)
    lib().orc_softmax_rows(_f(logits), T, E, _f(probs), _f(lse))
    return probs, lse


def route(probs, top_k, valid=None):
    """``MoeLayer::route`` (``moe.rs:553-593``): (expert_of [T,k] with -1 for padding, gates [T,k])."""
    probs = _f32(probs)
    T, E = probs.shape
    expert_of = np.empty((T, top_k), np.int32)
    gates = np.empty((T, top_k), np.float32)
    v = None if valid is None else np.ascontiguousarray(valid, dtype=np.uint8)
    lib().orc_route(_f(probs), T, E, top_k, None if v is None else _b(v), _i(expert_of), _f(gates))
    return expert_of, gates


def quantize_rows(w):
    """``Quantized::from_matrix`` (``quantized.rs:29-51``): (int8 values, f32 scale per row)."""
    w = _f32(w)
    q = np.empty(w.shape, np.int8)
    s = np.empty(w.shape[0], np.float32)
    lib().orc_quantize_rows(_f(w), w.shape[0], w.shape[1], q.ctypes.data_as(C.POINTER(C.c_int8)), _f(s))
    return q, s


def q8_matmul(x, q, scales):
    """``Quantized::matmul_rhs_transposed`` (``quantized.rs:55-99``)."""
    x = _f32(x)
    q = np.ascontiguousarray(q, dtype=np.int8)
    scales = _f32(scales)
    y = np.empty((x.shape[0], q.shape[0]), np.float32)
    lib().orc_q8_matmul(_f(x), x.shape[0], q.ctypes.data_as(C.POINTER(C.c_int8)), _f(scales), q.shape[0],
                        q.shape[1], _f(y))
    return y


def silu(x: float) -> float:
    return lib().orc_silu(float(x))


def silu_derivative(x: float) -> float:
    return lib().orc_silu_derivative(float(x))


def sgd_apply(value, grad, lr, scale=1.0):
    """Param::step, Sgd arm (param.rs:557-561), in place on two f32 arrays; the gradient is cleared."""
    assert value.dtype == np.float32 and grad.dtype == np.float32 and value.flags.c_contiguous and grad.flags.c_contiguous
    lib().orc_sgd_apply(value.ctypes.data, grad.ctypes.data, value.size, lr, scale)


def lion_apply(value, grad, moment, lr, beta1=0.9, beta2=0.99, wd=0.0, scale=1.0):
    """Param::step, Lion arm (param.rs:590-613), in place on three f32 arrays; the gradient is cleared."""
    for a in (value, grad, moment):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().orc_lion_apply(value.ctypes.data, grad.ctypes.data, moment.ctypes.data, value.size, lr, beta1, beta2, wd, scale)


class OracleMoe:
    """The reference's ``MoeLayer`` on the CPU.  Weights are ``[out, in]`` row-major f32."""

    def __init__(self, d_model, num_experts, top_k, d_ff, shared=False, aux_w=0.01, z_w=1e-3):
        self.d, self.E, self.k, self.F, self.shared = d_model, num_experts, top_k, d_ff, bool(shared)
        self.h = lib().orc_create(d_model, num_experts, top_k, d_ff, int(shared), aux_w, z_w)
        if not self.h:
            raise ValueError("invalid MoE config")  # MoeConfig::validate, moe.rs:68-86
        self.T = 0

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_destroy(self.h)
            self.h = None

    def _shape(self, which):
        if which == ROUTER:
            return (self.E, self.d)
        return (self.d, self.F) if which in (DOWN, SHARED_DOWN) else (self.F, self.d)

    def set_weight(self, which, expert, w):
        w = _f32(w)
        if lib().orc_set_weight(self.h, which, expert, _f(w), w.shape[0], w.shape[1]):
            raise ValueError("bad weight shape or index")

    def set_weight_q8(self, which, expert, q, scales):
        q = np.ascontiguousarray(q, dtype=np.int8)
        scales = _f32(scales)
        if lib().orc_set_weight_q8(self.h, which, expert, q.ctypes.data_as(C.POINTER(C.c_int8)), _f(scales),
                                   q.shape[0], q.shape[1]):
            raise ValueError("bad weight shape or index")

    def set_weights(self, router, gate, up, down, shared=None):
        """router [E,d]; gate/up [E,F,d]; down [E,d,F]; shared = (gate [F,d], up [F,d], down [d,F])."""
        self.set_weight(ROUTER, 0, router)
        for e in range(self.E):
            self.set_weight(GATE, e, gate[e])
            self.set_weight(UP, e, up[e])
            self.set_weight(DOWN, e, down[e])
        if shared is not None:
            for which, w in zip((SHARED_GATE, SHARED_UP, SHARED_DOWN), shared):
                self.set_weight(which, 0, w)

    def quantize(self, include_router=True):
        lib().orc_quantize(self.h, int(include_router))

    def get_weight(self, which, expert=0):
        out = np.empty(self._shape(which), np.float32)
        lib().orc_get_weight(self.h, which, expert, _f(out))
        return out

    def get_grad(self, which, expert=0):
        out = np.empty(self._shape(which), np.float32)
        lib().orc_get_grad(self.h, which, expert, _f(out))
        return out

    def get_moments(self, which, expert=0):
        m = np.empty(self._shape(which), np.float32)
        v = np.empty(self._shape(which), np.float32)
        lib().orc_get_moments(self.h, which, expert, _f(m), _f(v))
        return m, v

    def forward(self, x, valid=None, logits=None):
        """``forward_train``; returns y [T,d].  ``logits`` overrides the router product."""
        x = _f32(x)
        T, cols = x.shape
        v = None if valid is None else np.ascontiguousarray(valid, dtype=np.uint8)
        lg = None if logits is None else _f32(logits)
        y = np.empty((T, self.d), np.float32)
        rc = lib().orc_forward(self.h, _f(x), T, cols, None if v is None else _b(v), 0 if v is None else len(v),
                               None if lg is None else _f(lg), _f(y))
        if rc:
            raise ValueError("InvalidInput: expected %d columns, got %d (or a mask of the wrong length)" %
                             (self.d, cols))
        self.T = T
        return y

    def losses(self):
        a, z = C.c_float(), C.c_float()
        lib().orc_get_losses(self.h, C.byref(a), C.byref(z))
        return a.value, z.value

    def routing(self):
        """expert_of [T,k], gates [T,k], counts [E], token_of [R], slot_of [R] (stable, expert-major)."""
        expert_of = np.empty((self.T, self.k), np.int32)
        gates = np.empty((self.T, self.k), np.float32)
        counts = np.empty(self.E, np.int32)
        token_of = np.empty(self.T * self.k, np.int32)
        slot_of = np.empty(self.T * self.k, np.int32)
        n = lib().orc_get_routing(self.h, _i(expert_of), _f(gates), _i(counts), _i(token_of), _i(slot_of))
        return expert_of, gates, counts, token_of[:n].copy(), slot_of[:n].copy()

    def router_cache(self):
        logits = np.empty((self.T, self.E), np.float32)
        probs = np.empty((self.T, self.E), np.float32)
        lse = np.empty(self.T, np.float32)
        lib().orc_get_router(self.h, _f(logits), _f(probs), _f(lse))
        return logits, probs, lse

    def expert_rows(self):
        """hidden [R,F] and pre-gate expert outputs [R,d] in permuted order."""
        R = int(self.routing()[2].sum())
        hidden = np.empty((R, self.F), np.float32)
        outputs = np.empty((R, self.d), np.float32)
        lib().orc_get_expert_rows(self.h, _f(hidden), _f(outputs))
        return hidden, outputs

    def zero_grad(self):
        lib().orc_zero_grad(self.h)

    def backward(self, grad_out):
        grad_out = _f32(grad_out)
        grad_in = np.empty((self.T, self.d), np.float32)
        lib().orc_backward(self.h, _f(grad_out), _f(grad_in))
        return grad_in

    def adam_step(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1, scale=1.0):
        lib().orc_adam_step(self.h, lr, beta1, beta2, eps, wd, step, scale)

    def sgd_step(self, lr=1e-2, scale=1.0):
        lib().orc_sgd_step(self.h, lr, scale)

    def lion_step(self, lr=1e-4, beta1=0.9, beta2=0.99, wd=0.0, scale=1.0):
        lib().orc_lion_step(self.h, lr, beta1, beta2, wd, scale)
