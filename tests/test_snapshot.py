"""Readers of the reference's binary snapshots (RBWTS001 weights, RBOPT001 Adam moments).

The reference's own test of the format (`a_binary_snapshot_round_trips_and_is_far_smaller_than_json`,
transformer.rs:2800-2846) checks three properties: an f32 file is lossless, an int8 file restores
every weight within one quantization step of its row, and the file sizes follow from the layout.
The same properties are checked here on files written by `rustingbrain_b200.snapshot.write_snapshot`
(a restatement of save_bin), read back by the library's C reader.
"""
import json
import os
import struct

import numpy as np
import pytest

import oracle
from rustingbrain_b200 import InvalidSnapshot, snapshot_info, write_optimizer_state, write_snapshot
from rustingbrain_b200.snapshot import parameter_names, quantize_rows


def tiny_config(**over):
    cfg = dict(vocab_size=48, d_model=64, n_layers=3, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=96, moe_d_ff=64,
               num_experts=4, experts_per_token=2, moe_layers=[1, 2], shared_expert=True, max_seq_len=16,
               rope_base=10000.0, rmsnorm_eps=1e-6, tie_embeddings=True, causal=True, aux_loss_weight=0.01,
               router_z_loss_weight=0.001)
    cfg.update(over)
    return cfg


def tensors_for(cfg, seed=3, dense=3):
    g = np.random.Generator(np.random.Philox(seed))
    names = parameter_names(cfg, dense)
    return names, [(g.standard_normal(shape) * 0.1).astype(np.float32) for _, shape in names]


@pytest.mark.parametrize("precision", ["F32", "Q8"])
def test_header_is_parsed_and_sizes_follow_the_layout(tmp_path, precision):
    cfg = tiny_config()
    names, ts = tensors_for(cfg)
    path = tmp_path / "model.rbw"
    write_snapshot(path, cfg, ts, precision, optimizer_step=41)
    info = snapshot_info(path)
    assert info.precision == precision
    assert info.parameter_count == len(names) and info.dense_ffn_params == 3
    assert info.moe_layers == [1, 2] and info.optimizer_step == 41
    for key in ("vocab_size", "d_model", "n_layers", "moe_d_ff", "num_experts", "experts_per_token", "shared_expert",
                "tie_embeddings"):
        assert info.config[key] == cfg[key], key
    assert info.config["aux_loss_weight"] == pytest.approx(0.01)
    header = len(json.dumps({"config": {**cfg, "lora": None}, "optimizer": {"Adam": {"learning_rate": 1e-3, "beta1": 0.9,
                             "beta2": 0.999, "epsilon": 1e-8, "weight_decay": 0.0}}, "optimizer_step": 41,
                             "precision": precision}, separators=(",", ":")))
    body = sum(16 + (r * c * 4 if precision == "F32" else r * (4 + c)) for _, (r, c) in names)
    assert os.path.getsize(path) == 8 + 8 + header + 8 + body


def test_dense_feed_forward_kind_follows_from_the_parameter_count(tmp_path):
    cfg = tiny_config()
    _, ts = tensors_for(cfg, dense=2)                 # GELU blocks: up, down (ffn.rs:216-220)
    write_snapshot(tmp_path / "gelu.rbw", cfg, ts)
    assert snapshot_info(tmp_path / "gelu.rbw").dense_ffn_params == 2
    cfg = tiny_config(moe_layers=[0, 1, 2], tie_embeddings=False)
    names, ts = tensors_for(cfg)
    write_snapshot(tmp_path / "all_moe.rbw", cfg, ts)
    info = snapshot_info(tmp_path / "all_moe.rbw")
    assert info.dense_ffn_params == 0 and info.parameter_count == len(names)
    assert names[-1][0] == "lm_head"


def test_bad_files_are_refused(tmp_path):
    cfg = tiny_config()
    _, ts = tensors_for(cfg)
    (tmp_path / "junk").write_bytes(b"RBWTS000" + b"\0" * 64)
    with pytest.raises(InvalidSnapshot, match="not a RustingBrain weight file"):
        snapshot_info(tmp_path / "junk")
    with pytest.raises(InvalidSnapshot):
        snapshot_info(tmp_path / "missing.rbw")
    write_snapshot(tmp_path / "short.rbw", cfg, ts[:-2])          # two parameters fewer than the configuration builds
    with pytest.raises(InvalidSnapshot, match="parameters"):
        snapshot_info(tmp_path / "short.rbw")
    (tmp_path / "cut.rbw").write_bytes(b"RBWTS001" + struct.pack("<Q", 500) + b"{}")
    with pytest.raises(InvalidSnapshot, match="truncated"):
        snapshot_info(tmp_path / "cut.rbw")
    write_snapshot(tmp_path / "lora.rbw", {**cfg, "lora": {"rank": 4, "alpha": 4.0, "seed": 0}}, ts)
    with pytest.raises(InvalidSnapshot, match="parameters"):      # an adapted model writes three matrices per projection
        snapshot_info(tmp_path / "lora.rbw")
    write_snapshot(tmp_path / "layers.rbw", {**cfg, "moe_layers": [1, 7]}, ts)
    with pytest.raises(InvalidSnapshot, match="moe_layers"):
        snapshot_info(tmp_path / "layers.rbw")


def test_the_int8_grid_is_the_reference_one():
    g = np.random.Generator(np.random.Philox(5))
    w = (g.standard_normal((37, 53)) * 0.3).astype(np.float32)
    w[4] = 0.0                                        # an all-zero row keeps scale 0 (transformer.rs:514-518)
    w[5, :4] = [0.5, -0.5, 1.5, -1.5]                 # halves round away from zero
    w[5, 4:] = 0.0
    w[5, 10] = 127.0
    q, s = quantize_rows(w)
    q2, s2 = oracle.quantize_rows(w)                  # restatement of Quantized::from_matrix (quantized.rs:29-51)
    assert np.array_equal(s, s2) and np.array_equal(q, q2)
    assert s[4] == 0 and not q[4].any()
    assert list(q[5, :4]) == [1, -1, 2, -2]
    # the reference's own check: every restored weight within one step of its row's scale
    assert np.all(np.abs(q.astype(np.float32) * s[:, None] - w) <= s[:, None] + 1e-12)


# ---------------------------------------------------------------------------
# On the device: the library reads the files into layers
# ---------------------------------------------------------------------------
def _gpu_imports():
    torch = pytest.importorskip("torch")
    from rustingbrain_b200 import MoeConfig, MoeLayer
    return torch, MoeConfig, MoeLayer


def _block_tensors(names, ts, block):
    return {n.split("moe.", 1)[1]: t for (n, _), t in zip(names, ts) if n.startswith("blocks.%d.moe." % block)}


WHICH = {"gate": 1, "up": 2, "down": 3}


@pytest.mark.gpu
@pytest.mark.parametrize("file_precision", ["F32", "Q8"])
def test_f32_layer_restores_what_load_bin_restores(tmp_path, file_precision):
    torch, MoeConfig, MoeLayer = _gpu_imports()
    cfg = tiny_config()
    names, ts = tensors_for(cfg)
    path = tmp_path / "m.rbw"
    write_snapshot(path, cfg, ts, file_precision)
    layer = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="f32", max_tokens=32)
    layer.load_snapshot(path, 2)
    want = _block_tensors(names, ts, 2)

    def expect(t):
        if file_precision == "F32":
            return t                                   # lossless
        q, s = quantize_rows(t)
        return q.astype(np.float32) * s[:, None]       # byte as i8 as f32 * scale (transformer.rs:1917-1927)

    assert np.array_equal(layer.get_weight(0, 0), expect(want["router"]))
    for e in range(4):
        for part, which in WHICH.items():
            assert np.array_equal(layer.get_weight(which, e), expect(want["experts.%d.%s" % (e, part)])), (e, part)
    for part, which in WHICH.items():
        assert np.array_equal(layer.get_weight(which + 3, 0), expect(want["shared.%s" % part]))


@pytest.mark.gpu
@pytest.mark.parametrize("file_precision", ["F32", "Q8"])
def test_int8_layer_takes_the_rows_as_stored(tmp_path, file_precision):
    torch, MoeConfig, MoeLayer = _gpu_imports()
    cfg = tiny_config()
    names, ts = tensors_for(cfg)
    path = tmp_path / "m.rbw"
    write_snapshot(path, cfg, ts, file_precision)
    loaded = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="q8", max_tokens=32, training=False)
    loaded.load_snapshot(path, 1)
    by_hand = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="q8", max_tokens=32, training=False)
    want = _block_tensors(names, ts, 1)
    router = want["router"]
    if file_precision == "Q8":
        q, s = quantize_rows(router)
        router = q.astype(np.float32) * s[:, None]
    by_hand.set_weight(0, 0, router)
    for e in range(4):
        for part, which in WHICH.items():
            by_hand.set_weight_q8(which, e, *quantize_rows(want["experts.%d.%s" % (e, part)]))
    for part, which in WHICH.items():
        by_hand.set_weight_q8(which + 3, 0, *quantize_rows(want["shared.%s" % part]))
    g = np.random.Generator(np.random.Philox(11))
    x = torch.from_numpy(g.standard_normal((32, 64)).astype(np.float32)).cuda().bfloat16()
    a = loaded.forward(x).float().cpu().numpy()
    b = by_hand.forward(x).float().cpu().numpy()
    assert np.array_equal(a, b)
    assert np.abs(a).max() > 0


@pytest.mark.gpu
def test_wrong_block_and_wrong_shape_are_refused(tmp_path):
    torch, MoeConfig, MoeLayer = _gpu_imports()
    from rustingbrain_b200 import InvalidConfig, InvalidInput
    cfg = tiny_config()
    _, ts = tensors_for(cfg)
    path = tmp_path / "m.rbw"
    write_snapshot(path, cfg, ts)
    layer = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="f32", max_tokens=8)
    with pytest.raises(InvalidInput, match="not a MoE block"):
        layer.load_snapshot(path, 0)
    other = MoeLayer(64, MoeConfig(8, 2, 64, True), precision="f32", max_tokens=8)
    with pytest.raises(InvalidConfig, match="experts"):
        other.load_snapshot(path, 1)
    with open(path, "r+b") as f:                       # cut the file inside block 2
        f.truncate(os.path.getsize(path) - 4000)
    with pytest.raises(InvalidInput, match="truncated"):
        layer.load_snapshot(path, 2)


@pytest.mark.gpu
def test_adam_moments_are_restored(tmp_path):
    torch, MoeConfig, MoeLayer = _gpu_imports()
    cfg = tiny_config(shared_expert=False)
    names, ts = tensors_for(cfg)
    write_snapshot(tmp_path / "m.rbw", cfg, ts)
    g = np.random.Generator(np.random.Philox(13))
    moments = [((g.standard_normal(s) * 1e-3).astype(np.float32), (g.random(s) * 1e-6).astype(np.float32))
               for _, s in names]
    frozen = [i for i, (n, _) in enumerate(names) if n == "blocks.1.moe.experts.2.up"][0]
    moments[frozen] = None                             # a frozen parameter wrote the 0 x 0 placeholder
    write_optimizer_state(tmp_path / "m.opt", moments, step=123)
    info = snapshot_info(tmp_path / "m.rbw")
    layer = MoeLayer(64, MoeConfig(4, 2, 64, False), precision="f32", max_tokens=8)
    assert layer.load_optimizer_state(tmp_path / "m.opt", info, 1) == 123
    for i, (n, _) in enumerate(names):
        if not n.startswith("blocks.1.moe."):
            continue
        key = n.split("moe.", 1)[1]
        which, e = (0, 0) if key == "router" else (WHICH[key.split(".")[2]], int(key.split(".")[1]))
        m, v = layer.get_moments(which, e)
        if i == frozen:
            assert not m.any() and not v.any()
        else:
            assert np.array_equal(m, moments[i][0]) and np.array_equal(v, moments[i][1]), n
    (tmp_path / "bad.opt").write_bytes(b"RBOPT000" + b"\0" * 32)
    from rustingbrain_b200 import InvalidInput
    with pytest.raises(InvalidInput, match="optimizer state"):
        layer.load_optimizer_state(tmp_path / "bad.opt", info, 1)


@pytest.mark.gpu
def test_adapter_file_fills_the_attached_adapters(tmp_path):
    torch, MoeConfig, MoeLayer = _gpu_imports()
    from rustingbrain_b200 import InvalidInput
    from rustingbrain_b200.snapshot import adapter_names, write_lora
    cfg = tiny_config()
    _, ts = tensors_for(cfg)
    write_snapshot(tmp_path / "m.rbw", cfg, ts)
    info = snapshot_info(tmp_path / "m.rbw")
    rank, alpha = 4, 8.0
    names = adapter_names(cfg, rank)
    g = np.random.Generator(np.random.Philox(17))
    ad = [(g.standard_normal(s) * 0.1).astype(np.float32) for _, s in names]
    write_lora(tmp_path / "m.lora", rank, alpha, ad)
    layer = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="f32", max_tokens=8)
    with pytest.raises(InvalidInput, match="moe_lora_attach"):
        layer.load_lora(tmp_path / "m.lora", info, 2)           # load_lora wants the adapters to exist already
    layer.lora_attach(rank, alpha)
    layer.load_lora(tmp_path / "m.lora", info, 2)
    by_name = {n: t for (n, _), t in zip(names, ad)}
    for e in range(4):
        for part, which in WHICH.items():
            down, up = layer.lora_get(which, e)
            key = "blocks.2.moe.experts.%d.%s.lora." % (e, part)
            assert np.array_equal(down, by_name[key + "down"]) and np.array_equal(up, by_name[key + "up"]), key
    for part, which in WHICH.items():
        down, up = layer.lora_get(which + 3, 0)
        key = "blocks.2.moe.shared.%s.lora." % part
        assert np.array_equal(down, by_name[key + "down"]) and np.array_equal(up, by_name[key + "up"])
    other = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="f32", max_tokens=8)
    other.lora_attach(rank, 4.0)
    with pytest.raises(InvalidInput, match="alpha"):
        other.load_lora(tmp_path / "m.lora", info, 2)           # rank and alpha must be the file's
    write_lora(tmp_path / "short.lora", rank, alpha, ad[:-2])
    with pytest.raises(InvalidInput, match="parameters"):
        layer.load_lora(tmp_path / "short.lora", info, 2)


def test_adapted_model_files_are_understood(tmp_path):
    cfg = tiny_config(lora={"rank": 4, "alpha": 8.0, "seed": 0})
    names, ts = tensors_for(cfg)
    assert sum(1 for n, _ in names if n.endswith(".lora.down")) == 4 * 3 + 3 + 2 * (4 * 3 + 3)   # attention + ffn linears
    write_snapshot(tmp_path / "adapted.rbw", cfg, ts)
    info = snapshot_info(tmp_path / "adapted.rbw")
    assert info.lora_rank == 4 and info.lora_alpha == 8.0 and info.parameter_count == len(names)


@pytest.mark.gpu
@pytest.mark.parametrize("file_precision", ["F32", "Q8"])
def test_adapted_model_file_fills_weights_and_adapters(tmp_path, file_precision):
    torch, MoeConfig, MoeLayer = _gpu_imports()
    cfg = tiny_config(lora={"rank": 4, "alpha": 8.0, "seed": 0})
    names, ts = tensors_for(cfg)
    write_snapshot(tmp_path / "adapted.rbw", cfg, ts, file_precision)
    by_name = {n: t for (n, _), t in zip(names, ts)}

    def expect(t):
        if file_precision == "F32":
            return t
        q, s = quantize_rows(t)
        return q.astype(np.float32) * s[:, None]

    plain = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="f32", max_tokens=8)
    plain.load_snapshot(tmp_path / "adapted.rbw", 1)                 # no adapters attached: base weights only
    assert np.array_equal(plain.get_weight(3, 2), expect(by_name["blocks.1.moe.experts.2.down"]))
    adapted = MoeLayer(64, MoeConfig(4, 2, 64, True), precision="f32", max_tokens=8)
    adapted.lora_attach(4, 8.0)
    adapted.load_snapshot(tmp_path / "adapted.rbw", 2)
    assert np.array_equal(adapted.get_weight(0, 0), expect(by_name["blocks.2.moe.router"]))
    for e in range(4):
        for part, which in WHICH.items():
            key = "blocks.2.moe.experts.%d.%s" % (e, part)
            assert np.array_equal(adapted.get_weight(which, e), expect(by_name[key])), key
            down, up = adapted.lora_get(which, e)
            assert np.array_equal(down, expect(by_name[key + ".lora.down"])) and np.array_equal(up, expect(by_name[key + ".lora.up"]))
    down, up = adapted.lora_get(6, 0)
    assert np.array_equal(down, expect(by_name["blocks.2.moe.shared.down.lora.down"]))
    assert np.array_equal(up, expect(by_name["blocks.2.moe.shared.down.lora.up"]))
