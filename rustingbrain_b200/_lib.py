"""ctypes binding of libmoe_b200.so (the C ABI declared in include/moe_b200.h).

The library is the product: if it is missing or cannot be loaded this module
raises, it never substitutes a host implementation.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmoe_b200.so")

OK, INVALID_CONFIG, INVALID_INPUT, CUDA_ERROR, OUT_OF_MEMORY, UNSUPPORTED, TIMEOUT, COMM_ERROR, POISONED = range(9)
PRECISION_F32, PRECISION_BF16, PRECISION_Q8 = 0, 1, 2
W_ROUTER, W_GATE, W_UP, W_DOWN, W_SHARED_GATE, W_SHARED_UP, W_SHARED_DOWN = range(7)


class MoeConfigC(C.Structure):
    _fields_ = [
        ("d_model", C.c_int32), ("num_experts", C.c_int32), ("experts_per_token", C.c_int32), ("d_ff", C.c_int32),
        ("shared_expert", C.c_int32), ("aux_loss_weight", C.c_float), ("router_z_loss_weight", C.c_float),
        ("precision", C.c_int32), ("max_tokens", C.c_int32), ("device", C.c_int32), ("training", C.c_int32),
        ("ep_rank", C.c_int32), ("ep_size", C.c_int32), ("ep_capacity_factor", C.c_float),
    ]


class SnapshotInfoC(C.Structure):
    """moe_snapshot_info_t of include/moe_b200.h."""
    _fields_ = [(n, C.c_int64) for n in (
        "vocab_size", "d_model", "n_layers", "n_heads", "n_kv_heads", "head_dim", "d_ff", "moe_d_ff",
        "num_experts", "experts_per_token", "max_seq_len")] + [
        ("shared_expert", C.c_int32), ("tie_embeddings", C.c_int32), ("causal", C.c_int32),
        ("aux_loss_weight", C.c_float), ("router_z_loss_weight", C.c_float), ("rope_base", C.c_float),
        ("rmsnorm_eps", C.c_float), ("precision", C.c_int32), ("n_moe_layers", C.c_int32),
        ("moe_layers", C.c_int32 * 256), ("optimizer_step", C.c_int64), ("parameter_count", C.c_int64),
        ("dense_ffn_params", C.c_int32), ("lora_rank", C.c_int32), ("lora_alpha", C.c_float),
    ]


class KvCacheConfigC(C.Structure):
    """kv_cache_config_t of include/kv_attention_b200.h."""
    _fields_ = [("sequences", C.c_int32), ("num_heads", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("capacity", C.c_int32), ("max_seq_len", C.c_int32), ("rope_base", C.c_float), ("rope", C.c_int32),
                ("precision", C.c_int32), ("device", C.c_int32)]


class LmConfigC(C.Structure):
    """lm_config_t of include/transformer_b200.h."""
    _fields_ = [("vocab_size", C.c_int32), ("d_model", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("d_ff", C.c_int32), ("moe_d_ff", C.c_int32),
                ("num_experts", C.c_int32), ("experts_per_token", C.c_int32), ("shared_expert", C.c_int32),
                ("moe_layer_mask", C.c_uint64), ("max_seq_len", C.c_int32), ("rope_base", C.c_float),
                ("rmsnorm_eps", C.c_float), ("tie_embeddings", C.c_int32), ("aux_loss_weight", C.c_float),
                ("router_z_loss_weight", C.c_float), ("max_batch_rows", C.c_int32), ("device", C.c_int32)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libmoe_b200.so is not built (run `python -m rustingbrain_b200.build`); there is no host fallback")
    # The library needs libnccl.so.2.  When PyTorch is going to be used in the same process its bundled
    # (newer) NCCL has to be the copy that gets loaded: loading this library first would bind the
    # system's older libnccl, and `import torch` would then fail on symbols that copy lacks.
    try:
        import torch  # noqa: F401
    except ImportError:
        pass
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, i32, f32 = C.c_void_p, C.c_int32, C.c_float
    fp, ip, bp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_uint8)
    cfgp = C.POINTER(MoeConfigC)
    sig = {
        "moe_config_validate": (i32, [cfgp, C.c_char_p, i32]),
        "moe_workspace_bytes": (C.c_int64, [cfgp]),
        "moe_create": (i32, [cfgp, C.POINTER(vp)]),
        "moe_destroy": (None, [vp]),
        "moe_last_error": (C.c_char_p, [vp]),
        "moe_clear_error": (i32, [vp]),
        "moe_set_weight_f32": (i32, [vp, i32, i32, vp, i32, i32]),
        "moe_get_weight_f32": (i32, [vp, i32, i32, vp, i32, i32]),
        "moe_get_grad_f32": (i32, [vp, i32, i32, vp, i32, i32]),
        "moe_get_moments_f32": (i32, [vp, i32, i32, vp, vp, i32, i32]),
        "moe_set_moments_f32": (i32, [vp, i32, i32, vp, vp, i32, i32]),
        "moe_set_weight_q8": (i32, [vp, i32, i32, vp, vp, i32, i32]),
        "moe_forward": (i32, [vp, vp, i32, i32, vp, vp, i32, i32, vp]),
        "moe_forward_from_logits": (i32, [vp, vp, vp, i32, i32, vp, vp, i32, i32, vp]),
        "moe_backward": (i32, [vp, vp, vp, i32, vp]),
        "moe_zero_grad": (i32, [vp, vp]),
        "moe_step_adam": (i32, [vp, f32, f32, f32, f32, f32, i32, f32, vp]),
        "moe_step_sgd": (i32, [vp, f32, f32, vp]),
        "moe_step_lion": (i32, [vp, f32, f32, f32, f32, f32, vp]),
        "moe_forward_host": (i32, [vp, fp, i32, i32, bp, fp, i32]),
        "moe_backward_host": (i32, [vp, fp, fp]),
        "moe_get_losses": (i32, [vp, fp, fp]),
        "moe_get_routing": (i32, [vp, ip, fp, ip, ip, ip, ip]),
        "moe_get_router_cache": (i32, [vp, fp, fp, fp]),
        "moe_synchronize": (i32, [vp]),
        "moe_snapshot_info": (i32, [C.c_char_p, C.POINTER(SnapshotInfoC), C.c_char_p, i32]),
        "moe_load_snapshot_layer": (i32, [vp, C.c_char_p, i32]),
        "moe_load_optimizer_layer": (i32, [vp, C.c_char_p, C.POINTER(SnapshotInfoC), i32, C.POINTER(C.c_int64)]),
        "moe_lora_attach": (i32, [vp, i32, f32]),
        "moe_lora_set": (i32, [vp, i32, i32, vp, vp]),
        "moe_lora_get": (i32, [vp, i32, i32, vp, vp]),
        "moe_lora_get_grad": (i32, [vp, i32, i32, vp, vp]),
        "moe_lora_merge": (i32, [vp]),
        "moe_load_lora_layer": (i32, [vp, C.c_char_p, C.POINTER(SnapshotInfoC), i32]),
        "moe_route_noalloc": (i32, [vp, vp, i32, i32, i32, f32, f32, vp, vp, vp, vp, vp, vp, vp, C.c_char_p, i32]),
        "moe_ep_unique_id": (i32, [vp, i32]),
        "moe_ep_init": (i32, [vp, vp, i32]),
        "moe_ep_set_deadline_ms": (i32, [vp, C.c_int64]),
        "moe_debug_deadline_wait": (i32, [i32, i32, ip]),
        "moe_ep_export_buffers": (i32, [vp, vp, i32]),
        "moe_ep_import_buffers": (i32, [vp, i32, vp, i32]),
        "moe_ep_plan": (i32, [ip, i32, i32, i32, ip, ip, ip, ip, ip]),
        "lm_config_validate": (i32, [C.POINTER(LmConfigC), C.c_char_p, i32]),
        "lm_parameter_counts": (i32, [C.POINTER(LmConfigC), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
        "lm_create": (i32, [C.POINTER(LmConfigC), C.POINTER(vp)]),
        "lm_destroy": (None, [vp]),
        "lm_last_error": (C.c_char_p, [vp]),
        "lm_set_param": (i32, [vp, i32, i32, i32, vp, i32, i32]),
        "lm_get_param": (i32, [vp, i32, i32, i32, vp, i32, i32]),
        "lm_get_grad": (i32, [vp, i32, i32, i32, vp, i32, i32]),
        "lm_forward_logits": (i32, [vp, vp, vp, i32, i32, vp, vp]),
        "lm_accumulate_step": (i32, [vp, vp, vp, vp, i32, i32, fp, fp]),
        "lm_zero_grad": (i32, [vp]),
        "lm_step_adam": (i32, [vp, f32, f32, f32, f32, f32, f32]),
        "lm_step_sgd": (i32, [vp, f32, f32]),
        "lm_step_lion": (i32, [vp, f32, f32, f32, f32, f32]),
        "lm_train_step": (i32, [vp, vp, vp, vp, i32, i32, f32, f32, f32, f32, f32, fp, fp]),
        "lm_optimizer_step": (C.c_int64, [vp]),
        "lm_set_optimizer_step": (i32, [vp, C.c_int64]),
        "lm_decoder_create": (i32, [vp, i32, i32, C.POINTER(vp)]),
        "lm_decoder_destroy": (None, [vp]),
        "lm_decoder_clear": (i32, [vp, vp, i32]),
        "lm_forward_cached": (i32, [vp, vp, vp, i32, i32, i32, vp]),
        "lm_last_step_ms": (i32, [vp, fp]),
        "lm_synchronize": (i32, [vp]),
        "kv_cache_create": (i32, [C.POINTER(KvCacheConfigC), C.POINTER(vp)]),
        "kv_cache_destroy": (None, [vp]),
        "kv_cache_last_error": (C.c_char_p, [vp]),
        "kv_cache_clear": (i32, [vp, i32, vp]),
        "kv_cache_truncate": (i32, [vp, i32, i32, vp]),
        "kv_cache_lengths": (i32, [vp, ip, vp]),
        "kv_attention_forward_cached": (i32, [vp, i32, i32, vp, vp, vp, i32, vp, vp]),
        "kv_cache_read": (i32, [vp, i32, fp, fp, vp]),
        "rmsnorm_forward": (i32, [vp, vp, vp, i32, i32, f32, i32, vp, C.c_char_p, i32]),
        "rmsnorm_scratch_bytes": (C.c_int64, [i32, i32]),
        "rmsnorm_backward": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, f32, i32, vp, C.c_char_p, i32]),
        "moe_debug_tc_gemm": (i32, [i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp]),
        "moe_debug_launch_count": (C.c_int64, []),
        "moe_debug_set_tc_pair": (i32, [i32]),
        "moe_debug_starve_next_gemm": (i32, [C.c_int64]),
        "moe_debug_profile": (i32, [vp, i32]),
        "moe_debug_profile_read": (i32, [vp, fp, ip]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def exported_symbols():
    """Names the headers under include/ declare; used by the load test."""
    import re
    inc = os.path.join(_HERE, "..", "include")
    names = []
    for h in sorted(os.listdir(inc)):
        if h.endswith(".h"):
            text = open(os.path.join(inc, h)).read()
            names += re.findall(r"\b((?:moe|kv|rmsnorm|lm)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(n for n in names if n not in ("moe_status", "moe_precision", "moe_weight", "lm_param", "lm_config", "lm_model", "lm_decoder")))
