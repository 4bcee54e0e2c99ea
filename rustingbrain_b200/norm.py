"""Host-side mirror of the reference's ``RmsNorm`` (norm.rs:22-129) over the C ABI of
include/rmsnorm_b200.h.  Device tensors in, device tensors out; no host implementation behind it."""
from __future__ import annotations

import ctypes as C

from . import _lib
from .moe import CudaError, InvalidConfig, InvalidInput, _stream

_ERRORS = {_lib.INVALID_CONFIG: InvalidConfig, _lib.INVALID_INPUT: InvalidInput, _lib.UNSUPPORTED: InvalidConfig}


class RmsNorm:
    """``RmsNorm::new(d_model, eps)``: weight of ones (f32, on the device), its gradient, `forward`, `backward`."""

    def __init__(self, d_model: int, eps: float = 1e-6, device: int = 0):
        import torch
        self.d_model, self.eps = d_model, float(eps)
        self.weight = torch.ones(d_model, dtype=torch.float32, device="cuda:%d" % device)
        self.grad = torch.zeros_like(self.weight)
        self.frozen = False
        self._scratch = None

    def _check(self, rc, msg):
        if rc != _lib.OK:
            raise _ERRORS.get(rc, CudaError)(msg.value.decode(errors="replace"))

    @staticmethod
    def _precision(t):
        import torch
        if t.dtype == torch.float32:
            return _lib.PRECISION_F32
        if t.dtype == torch.bfloat16:
            return _lib.PRECISION_BF16
        raise InvalidInput("activations are f32 or bf16 device tensors")

    def forward(self, x, out=None, stream=None):
        import torch
        if not (x.is_cuda and x.is_contiguous() and x.dim() == 2 and x.shape[1] == self.d_model):
            raise InvalidInput("expected a contiguous device tensor [tokens, %d]" % self.d_model)
        y = torch.empty_like(x) if out is None else out
        msg = C.create_string_buffer(256)
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        self._check(_lib.lib().rmsnorm_forward(C.c_void_p(x.data_ptr()), C.c_void_p(self.weight.data_ptr()),
                                               C.c_void_p(y.data_ptr()), x.shape[0], self.d_model, self.eps,
                                               self._precision(x), _stream(st), msg, len(msg)), msg)
        return y

    def backward(self, x, grad_y, stream=None):
        """Accumulates the weight gradient into ``self.grad`` (unless frozen) and returns dL/dx."""
        import torch
        if x.shape != grad_y.shape or x.dtype != grad_y.dtype or not (grad_y.is_cuda and grad_y.is_contiguous()):
            raise InvalidInput("grad_y must match x")
        need = int(_lib.lib().rmsnorm_scratch_bytes(x.shape[0], self.d_model))
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
        gx = torch.empty_like(x)
        msg = C.create_string_buffer(256)
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        gw = None if self.frozen else C.c_void_p(self.grad.data_ptr())
        self._check(_lib.lib().rmsnorm_backward(C.c_void_p(x.data_ptr()), C.c_void_p(self.weight.data_ptr()),
                                                C.c_void_p(grad_y.data_ptr()), C.c_void_p(gx.data_ptr()), gw,
                                                C.c_void_p(self._scratch.data_ptr()), x.shape[0], self.d_model, self.eps,
                                                self._precision(x), _stream(st), msg, len(msg)), msg)
        return gx


__all__ = ["RmsNorm"]
