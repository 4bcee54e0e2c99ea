"""The C-ABI library loads and exports everything include/*.h declares (no GPU needed)."""
import ctypes as C

import pytest

from rustingbrain_b200 import _lib, MoeConfig, InvalidConfig


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = _lib.exported_symbols()
    assert "moe_forward" in names and "moe_backward" in names and "moe_create" in names
    for name in names:
        assert hasattr(L, name), "libmoe_b200.so does not export " + name


def _cfg(**kw):
    base = dict(d_model=64, num_experts=4, experts_per_token=2, d_ff=32, shared_expert=0, aux_loss_weight=0.01,
                router_z_loss_weight=1e-3, precision=_lib.PRECISION_F32, max_tokens=16, device=0, training=1,
                ep_rank=0, ep_size=1, ep_capacity_factor=0.0)
    base.update(kw)
    return _lib.MoeConfigC(**base)


def test_config_validation_follows_the_reference():  # moe.rs:68-86, 705-710
    L = _lib.lib()
    msg = C.create_string_buffer(256)
    assert L.moe_config_validate(C.byref(_cfg()), msg, 256) == _lib.OK
    for bad in (dict(experts_per_token=0), dict(experts_per_token=5), dict(num_experts=0), dict(d_ff=0)):
        assert L.moe_config_validate(C.byref(_cfg(**bad)), msg, 256) == _lib.INVALID_CONFIG
        assert msg.value
    # shape rule of the tensor-core path is reported, not silently worked around
    assert L.moe_config_validate(C.byref(_cfg(precision=_lib.PRECISION_BF16, d_model=40)), msg, 256) == _lib.INVALID_CONFIG
    assert L.moe_workspace_bytes(C.byref(_cfg())) > 0
    for k, e in ((0, 4), (5, 4), (1, 0)):
        with pytest.raises(InvalidConfig):
            MoeConfig(e, k, 6).validate()


def test_builder_style_config_helpers():  # moe.rs:42-66
    c = MoeConfig(8, 2, 1408).with_shared_expert(True).with_aux_loss_weight(0.0).with_router_z_loss_weight(0.5)
    assert c.shared_expert and c.aux_loss_weight == 0.0 and c.router_z_loss_weight == 0.5
    assert MoeConfig(8, 2, 1408).aux_loss_weight == 0.01 and MoeConfig(8, 2, 1408).router_z_loss_weight == 1e-3


def test_create_fails_closed_without_a_device():  # lib.rs:72-76: never a silent CPU fallback
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    rc = _lib.lib().moe_create(C.byref(_cfg()), C.byref(h))
    assert rc != _lib.OK


def test_rmsnorm_and_kv_cache_arguments_are_checked_before_any_device_work():
    L = _lib.lib()
    msg = C.create_string_buffer(128)
    assert L.rmsnorm_scratch_bytes(70, 64) == 3 * 64 * 4          # three tiles of 32 rows (norm.rs:14)
    assert L.rmsnorm_scratch_bytes(0, 64) == 0
    assert L.rmsnorm_forward(None, None, None, 4, 64, 1e-6, _lib.PRECISION_F32, None, msg, 128) == _lib.INVALID_INPUT
    assert b"null" in msg.value
    buf = (C.c_float * 64)()
    p = C.cast(buf, C.c_void_p)
    assert L.rmsnorm_forward(p, p, p, 1, 12, 1e-6, _lib.PRECISION_F32, None, msg, 128) == _lib.UNSUPPORTED
    assert L.rmsnorm_forward(p, p, p, 1, 16, 1e-6, 7, None, msg, 128) == _lib.INVALID_CONFIG
    for bad in (dict(num_heads=3, kv_heads=2), dict(kv_heads=8), dict(head_dim=7), dict(sequences=0),
                dict(capacity=64, max_seq_len=32), dict(precision=_lib.PRECISION_Q8)):      # attention.rs:173-186, rope.rs:72-76
        kw = dict(sequences=2, num_heads=4, kv_heads=2, head_dim=8, capacity=16, max_seq_len=16, rope_base=10000.0, rope=1,
                  precision=_lib.PRECISION_F32, device=0)
        kw.update(bad)
        h = C.c_void_p()
        assert L.kv_cache_create(C.byref(_lib.KvCacheConfigC(**kw)), C.byref(h)) == _lib.INVALID_CONFIG, bad
        assert L.kv_cache_last_error(h)
        L.kv_cache_destroy(h)
    h = C.c_void_p()
    kw = dict(sequences=2, num_heads=4, kv_heads=2, head_dim=6, capacity=16, max_seq_len=16, rope_base=10000.0, rope=1,
              precision=_lib.PRECISION_F32, device=0)
    assert L.kv_cache_create(C.byref(_lib.KvCacheConfigC(**kw)), C.byref(h)) == _lib.UNSUPPORTED   # even, but no kernel
    L.kv_cache_destroy(h)


def test_language_model_configuration_is_checked_without_a_device():  # transformer.rs:132-172, 195-235
    from rustingbrain_b200.transformer import TransformerConfig, TransformerLm, TokenBatch
    assert TransformerConfig().parameter_counts() == (55_181_824, 35_717_632)      # the README's 55.2M / 35.7M
    dense = TransformerConfig(moe_layers=())
    assert dense.parameter_counts()[0] == dense.parameter_counts()[1]
    TransformerConfig().validate()
    for bad, text in ((dict(moe_layers=(9,)), "moe_layers names layer 9"), (dict(n_heads=6, n_kv_heads=4), "multiple of n_kv_heads"),
                      (dict(head_dim=7), "head_dim must be even"), (dict(experts_per_token=9), "experts_per_token"),
                      (dict(d_model=100), "multiples of 32"), (dict(vocab_size=0), "vocab_size must be non-zero")):
        with pytest.raises(InvalidConfig, match=text):
            TransformerConfig(**bad).validate()
    with pytest.raises(InvalidConfig):
        TokenBatch([[1]])
    b = TokenBatch([[1, 2, 3, 4], [5, 6]])
    assert b.is_padded() and b.seq_len == 4 and list(b.ids) == [1, 2, 3, 4, 5, 6, 0, 0] and list(b.lengths) == [4, 2]
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(Exception):                      # fails closed: there is no host model behind the builder
            TransformerLm.builder().build()
