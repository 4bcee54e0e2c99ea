"""The language model around the MoE layer on the device (include/transformer_b200.h) against the numpy / C++
checker (oracle/transformer.py): logits, losses, every parameter gradient, accumulation, padding, one Adam step.

bf16 products over f32 master weights: tolerance 2e-2 relative L2 per tensor (the bf16 bar of the layer tests).
The checker is fed the devices' own router logits, so both sides route identically and the comparison is
of the arithmetic, not of near-tie flips."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from helpers import rel_l2
from oracle import transformer as T
from oracle import ROUTER, GATE, UP, DOWN, SHARED_GATE
from rustingbrain_b200 import InvalidConfig, InvalidInput
from rustingbrain_b200 import transformer as D

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def _round_weights(w):
    out = dict(embedding=_bf16(w["embedding"]), final_norm=w["final_norm"], blocks=[])
    if "lm_head" in w:
        out["lm_head"] = _bf16(w["lm_head"])
    for b in w["blocks"]:
        nb = {}
        for k, v in b.items():
            if k == "moe":
                nb[k] = dict(router=v["router"], gate=_bf16(v["gate"]), up=_bf16(v["up"]), down=_bf16(v["down"]),
                             shared=tuple(_bf16(s) for s in v["shared"]) if v["shared"] is not None else None)
            elif k.endswith("norm"):
                nb[k] = v
            else:
                nb[k] = _bf16(v)
        out["blocks"].append(nb)
    return out


def _config(**over):
    c = T.default_config(vocab_size=101, d_model=128, n_layers=3, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=96, moe_d_ff=64,
                         num_experts=4, experts_per_token=2, moe_layers=(1, 2), max_seq_len=64)
    c.update(over)
    c["moe_layers"] = tuple(c["moe_layers"])
    return c


def _pair(c, seed=3, std=0.08, rows=256, optimizer=None):
    w = _round_weights(T.seeded_model_weights(c, seed, std=std))
    ora = T.OracleLm(c, w)
    dc = D.TransformerConfig(**{k: v for k, v in c.items()})
    dev = D.TransformerLm.builder().config(dc).max_batch_rows(rows).optimizer(optimizer or D.Adam(1e-2)).build()
    dev.load_weights(w)
    return dev, ora, w


def _sequences(c, lengths, seed=1):
    g = np.random.Generator(np.random.Philox(seed))
    return [list(g.integers(0, c["vocab_size"], n)) for n in lengths]


def _router_logits(c, router):
    return None if router is None else {layer: router[i] for i, layer in enumerate(c["moe_layers"])}


def _check_grads(c, dev, ora, tol=TOL):
    worst = {}
    def cmp(name, a, b):
        worst[name] = rel_l2(a, b)
    cmp("embedding", dev.get_grad(D.EMBEDDING), ora.grads["embedding"])
    cmp("final_norm", dev.get_grad(D.FINAL_NORM), ora.grads["final_norm"])
    if not c["tie_embeddings"]:
        cmp("lm_head", dev.get_grad(D.HEAD), ora.grads["lm_head"])
    for layer in range(c["n_layers"]):
        gb = ora.grads["blocks"][layer]
        for which, key in ((D.ATTENTION_NORM, "attention_norm"), (D.WQ, "wq"), (D.WK, "wk"), (D.WV, "wv"), (D.WO, "wo"), (D.FFN_NORM, "ffn_norm")):
            cmp("%d.%s" % (layer, key), dev.get_grad(which, layer), gb[key])
        if layer in c["moe_layers"]:
            m = ora.moe[layer]
            cmp("%d.router" % layer, dev.get_grad(D.MOE_ROUTER, layer), m.get_grad(ROUTER))
            for e in range(c["num_experts"]):
                for which, ow in ((D.MOE_GATE, GATE), (D.MOE_UP, UP), (D.MOE_DOWN, DOWN)):
                    go = m.get_grad(ow, e)
                    if np.abs(go).max() > 0:
                        cmp("%d.e%d.%d" % (layer, e, ow), dev.get_grad(which, layer, e), go)
            if c["shared_expert"]:
                cmp("%d.shared_gate" % layer, dev.get_grad(D.MOE_SHARED_GATE, layer), m.get_grad(SHARED_GATE))
        else:
            for which, key in ((D.FFN_GATE, "gate"), (D.FFN_UP, "up"), (D.FFN_DOWN, "down")):
                cmp("%d.%s" % (layer, key), dev.get_grad(which, layer), gb[key])
    bad = {k: v for k, v in worst.items() if not v <= tol}
    assert not bad, "gradients beyond %g: %s" % (tol, bad)
    return worst


@pytest.mark.parametrize("over,lengths", [
    (dict(), [32, 32]),                                          # two full sequences, GQA 4/2, head_dim 64
    (dict(), [40, 23, 31]),                                      # ragged: padding rows, masks into the MoE layers
    (dict(head_dim=32, n_heads=4, n_kv_heads=1), [24, 24]),      # one kv head for all, head_dim 32
    (dict(tie_embeddings=False, moe_layers=(0,), shared_expert=False, n_layers=2), [16, 16, 16]),
    (dict(moe_layers=()), [32, 17]),                             # dense only
    # sequences longer than one tile of the attention products: the tiles and K-stages above the diagonal are skipped
    (dict(max_seq_len=512, n_layers=2, moe_layers=(1,)), [384, 300]),          # 128 | S: tiles line up with the heads
    (dict(max_seq_len=512, n_layers=2, moe_layers=()), [320]),                 # tiles that cross from one head into the next
    (dict(max_seq_len=512, n_layers=2, moe_layers=(), n_kv_heads=4), [416, 100]),   # one query head per key/value head
])
def test_logits_loss_and_every_gradient_match_the_checker(over, lengths):
    c = _config(**over)
    dev, ora, _ = _pair(c, rows=max(256, len(lengths) * max(lengths)))
    seqs = _sequences(c, lengths)
    logits, router = dev.forward_batch(seqs, return_router_logits=True)
    batch = T.TokenBatch(seqs)
    lo = ora.forward(batch, _router_logits(c, router))
    valid = batch.valid
    assert rel_l2(logits[valid], lo[valid]) <= TOL
    dev.zero_grad()
    loss = dev.accumulate_step(seqs)
    ora.zero_grad()
    router2 = dev.forward_batch(seqs, return_router_logits=True)[1]
    lm_o, aux_o = ora.accumulate_step(batch, _router_logits(c, router2))
    assert abs(loss.lm_loss - lm_o) <= 2e-2 * abs(lm_o)
    assert abs(loss.auxiliary_loss - aux_o) <= 1e-3 * max(abs(aux_o), 1e-6) + 1e-7
    for layer in c["moe_layers"]:
        pass
    _check_grads(c, dev, ora)
    dev.close()


def test_accumulating_without_zeroing_keeps_adding():  # transformer.rs:2118-2136
    c = _config()
    dev, ora, _ = _pair(c)
    seqs = _sequences(c, [32, 32], seed=5)
    dev.zero_grad()
    dev.accumulate_step(seqs)
    g1 = {k: dev.get_grad(k, 1).copy() for k in (D.WQ, D.WO, D.MOE_ROUTER)}
    e1 = dev.get_grad(D.EMBEDDING).copy()
    dev.accumulate_step(seqs)
    for k, v in g1.items():
        assert rel_l2(dev.get_grad(k, 1), 2 * v) <= 1e-3
    assert rel_l2(dev.get_grad(D.EMBEDDING), 2 * e1) <= 1e-3
    dev.zero_grad()
    assert np.all(dev.get_grad(D.WQ, 1) == 0) and np.all(dev.get_grad(D.MOE_ROUTER, 1) == 0)
    dev.close()


def test_a_loss_mask_zeroes_the_masked_positions():  # transformer.rs:2068-2104, batch.rs:329-358
    c = _config(moe_layers=())
    dev, ora, _ = _pair(c)
    seqs = _sequences(c, [16, 16], seed=8)
    mask = np.zeros(32, bool)
    mask[20:28] = True                                   # only part of the second sequence is a target
    dev.zero_grad()
    loss = dev.accumulate_step(D.TokenBatch(seqs, loss_mask=mask))
    ora.zero_grad()
    lm_o, _ = ora.accumulate_step(T.TokenBatch(seqs, loss_mask=mask))
    assert abs(loss.lm_loss - lm_o) <= 2e-2 * abs(lm_o)
    _check_grads(c, dev, ora)
    with pytest.raises(InvalidConfig):
        dev.accumulate_step(D.TokenBatch(seqs, loss_mask=np.zeros(32, bool)))
    dev.close()


def test_train_steps_follow_the_checker_and_drive_the_loss_down():
    c = _config()
    dev, ora, _ = _pair(c, std=0.05)
    seqs = _sequences(c, [32, 32], seed=2)
    batch = T.TokenBatch(seqs)
    dl, ol = [], []
    for step in range(6):
        router = dev.forward_batch(seqs, return_router_logits=True)[1]
        t = dev.train_step_batch(seqs)
        dl.append(t.lm_loss)
        ol.append(ora.train_step(batch, _router_logits(c, router), lr=1e-2)[0])
    assert dev.optimizer_step() == 6
    assert dl[-1] < dl[0] - 0.05
    assert abs(dl[0] - ol[0]) <= 2e-2 * ol[0]
    assert abs(dl[-1] - ol[-1]) <= 0.1 * ol[-1]          # bf16 weights drift from the f32 checker over steps; the trend must agree
    # the weights moved as Adam moves them: first step of size ~lr on every touched weight
    w_after = dev.get_param(D.WO, 0)
    assert np.isfinite(w_after).all()
    dev.close()


@pytest.mark.parametrize("kind", ["sgd", "lion"])
def test_sgd_and_lion_train_steps_follow_the_checker(kind):  # gpu_transformer.rs:1855-1884; param.rs:557-561, 590-613
    c = _config()
    opt = D.Sgd(0.05) if kind == "sgd" else D.Lion(1e-2, weight_decay=0.1)
    dev, ora, w = _pair(c, std=0.05, optimizer=opt)
    seqs = _sequences(c, [32, 32], seed=4)
    batch = T.TokenBatch(seqs)
    router = dev.forward_batch(seqs, return_router_logits=True)[1]
    before = [a.copy() for a in (w["blocks"][0]["wo"], w["blocks"][0]["down"], w["blocks"][1]["moe"]["router"],
                                 w["blocks"][2]["moe"]["down"][1], w["embedding"])]   # the checker steps `w` in place
    dev.train_step_batch(seqs)
    if kind == "sgd":
        ora.train_step(batch, _router_logits(c, router), lr=0.05, kind="sgd")
    else:
        ora.train_step(batch, _router_logits(c, router), lr=1e-2, beta1=0.9, beta2=0.99, wd=0.1, kind="lion")
    assert dev.optimizer_step() == 1
    after = [(dev.get_param(D.WO, 0), ora.w["blocks"][0]["wo"]),
             (dev.get_param(D.FFN_DOWN, 0), ora.w["blocks"][0]["down"]),
             (dev.get_param(D.MOE_ROUTER, 1), ora.moe[1].get_weight(0)),
             (dev.get_param(D.MOE_DOWN, 2, expert=1), ora.moe[2].get_weight(3, 1)),
             (dev.get_param(D.EMBEDDING), ora.w["embedding"])]
    for (after_dev, after_ora), before in zip(after, before):
        if kind == "sgd":
            assert rel_l2(after_dev - before, after_ora - before) <= TOL
        else:
            # every touched weight moves by the learning rate; the sign can differ only where the bf16 and f32
            # gradients straddle zero
            assert np.mean(np.abs(after_dev - after_ora) > 5e-3) <= 0.03
            assert np.abs(after_dev - before).max() <= 1e-2 * (1 + 0.1 * np.abs(before).max()) + 1e-6
    assert np.all(dev.get_grad(D.WO, 0) == 0)
    dev.close()


def test_errors_follow_the_reference():
    c = _config()
    dev, _, _ = _pair(c)
    with pytest.raises(InvalidInput, match="TokenOutOfRange"):
        dev.forward_batch([[1, 2, 500]])
    with pytest.raises(InvalidInput, match="SequenceTooLong"):
        dev.forward_batch([list(range(65))])
    with pytest.raises(InvalidConfig):
        D.TokenBatch([[7]])
    with pytest.raises(InvalidInput):
        dev.set_param(D.HEAD, np.zeros((101, 128), np.float32))       # tied: there is no separate head
    with pytest.raises(InvalidInput):
        dev.set_param(D.FFN_GATE, np.zeros((96, 128), np.float32), layer=1)   # layer 1 is a MoE layer
    dev.close()
    with pytest.raises(InvalidConfig, match="moe_layers names layer 5"):
        D.TransformerLm.builder().config(D.TransformerConfig(n_layers=3, moe_layers=(5,))).build()
    with pytest.raises(InvalidConfig, match="multiple of n_kv_heads"):
        D.TransformerLm.builder().heads(6, 4, 64).build()
    assert D.TransformerLm.builder().parameter_counts() == (55_181_824, 35_717_632)


def test_a_prefill_then_cached_decode_reproduces_the_full_forward():  # attention.rs:1318-1362 at model level
    c = _config()
    dev, _, _ = _pair(c)
    seqs = _sequences(c, [24, 24, 24], seed=4)
    full = dev.forward_batch(seqs).reshape(3, 24, -1)
    caches = dev.new_kv_caches(sequences=3, capacity=32)
    got = np.empty_like(full)
    got[:, :16] = dev.forward_cached([s[:16] for s in seqs], caches).reshape(3, 16, -1)     # prefill
    for t in range(16, 24):                                                                 # one token per sequence
        got[:, t] = dev.forward_cached([[s[t]] for s in seqs], caches)
    assert rel_l2(got, full) <= TOL
    # a cleared slot restarts at position 0 while the others keep their state
    caches.clear(1)
    again = dev.forward_cached([seqs[1][:8]], caches, first_sequence=1).reshape(8, -1)
    assert rel_l2(again, full[1, :8]) <= TOL
    with pytest.raises(InvalidInput, match="SequenceTooLong"):
        dev.forward_cached([list(seqs[0][:10])], caches, first_sequence=0)                  # 24 + 10 > 32
    dev.close()
