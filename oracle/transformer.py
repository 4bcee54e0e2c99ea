"""CPU restatement of the reference's language model around the MoE layer.  TEST INFRASTRUCTURE ONLY:
imported by tests/, the smoke check and the benchmark's CPU-baseline leg; the product never calls it.

Follows, in f32 numpy (the MoE feed-forward itself is the C++ restatement, ``OracleMoe``):
  * TransformerConfig defaults / validate / parameter_counts   reference transformer.rs:99-130, 132-172, 195-235
  * TokenBatch (right padding, `predicts`, `predicted`)         reference batch.rs:35-75, 148-160, 204-222
  * Embedding forward / backward / unembed / unembed_backward   reference embedding.rs:49-75, 80-118, 121-152
  * Linear forward / backward (`y = x W^T`, bias free)          reference param.rs:762-825
  * RMSNorm                                                     oracle/norm.py (reference norm.rs:41-129)
  * MultiHeadAttention forward_train / backward                 reference attention.rs:305-341, 404-556
      (project_batched :947-978, head_scores_batched :980-1044 with the causal prefix softmax,
       accumulate_head_output_batched :1046-1098, scale = 1/sqrt(head_dim) :294-296, RoPE rope.rs:129-146)
  * SwiGlu forward_train / backward                             reference ffn.rs:56-120, silu :227-238
  * TransformerBlock forward_train / backward                   reference transformer_block.rs:205-270
  * TransformerLm forward_batch / backward / train_step_batch   reference transformer.rs:676-735, 1214-1246, 1394-1425
  * causal_lm_loss_batch / cross_entropy_rows                   reference causal_lm_loss.rs:66-150
  * Param::step (Sgd, Adam, Lion)                               reference param.rs:547-617

Pinned by the reference's own tests, restated in tests/test_transformer_oracle.py: causal_lm_loss.rs:152-186
(uniform logits give ln(vocab), the last position has no target, gradient against finite differences),
embedding.rs:175-218 (gather, accumulate into repeated rows only, unembed), attention.rs:1208-1255 (weights sum to
one over the visible prefix, the causal mask zeroes future keys, a later token cannot change an earlier
output) and :1364-1437 (input and query-weight gradients against finite differences), transformer.rs:2009-2066
(two accumulated half batches sum the half gradients).  Float results are pinned to this restatement plus those
finite differences; the reference itself cannot run here (no Rust toolchain).
"""
from __future__ import annotations

import numpy as np

from . import norm as rms
from .attention import rope_apply, rope_tables

F = np.float32


def default_config(**over):
    """TransformerConfig::default (transformer.rs:99-125)."""
    c = dict(vocab_size=32000, d_model=512, n_layers=8, n_heads=8, n_kv_heads=2, head_dim=64, d_ff=1408, moe_d_ff=352,
             num_experts=8, experts_per_token=2, moe_layers=tuple(range(2, 8)), shared_expert=True, max_seq_len=2048,
             rope_base=10000.0, rmsnorm_eps=1e-6, tie_embeddings=True, causal=True, aux_loss_weight=0.01,
             router_z_loss_weight=1e-3)
    c.update(over)
    c["moe_layers"] = tuple(c["moe_layers"])
    return c


def validate(c):
    """TransformerConfig::validate (transformer.rs:132-172); raises ValueError("InvalidConfig: ...")."""
    for name in ("vocab_size", "d_model", "n_layers", "n_heads", "n_kv_heads", "head_dim", "d_ff", "max_seq_len"):
        if c[name] == 0:
            raise ValueError("InvalidConfig: %s must be non-zero" % name)
    if c["n_heads"] % c["n_kv_heads"] != 0 or c["n_kv_heads"] > c["n_heads"]:
        raise ValueError("InvalidConfig: n_heads (%d) must be a multiple of n_kv_heads (%d)" % (c["n_heads"], c["n_kv_heads"]))
    if c["head_dim"] % 2 != 0:
        raise ValueError("InvalidConfig: head_dim must be even for rotary embeddings, got %d" % c["head_dim"])
    for layer in c["moe_layers"]:
        if layer >= c["n_layers"]:
            raise ValueError("InvalidConfig: moe_layers names layer %d, but the model has %d layers" % (layer, c["n_layers"]))
    if c["moe_layers"]:
        if c["num_experts"] == 0 or not (1 <= c["experts_per_token"] <= c["num_experts"]) or c["moe_d_ff"] == 0:
            raise ValueError("InvalidConfig: bad mixture-of-experts configuration")


def parameter_counts(c):
    """(total, active): TransformerConfig::parameter_counts (transformer.rs:195-235)."""
    d = c["d_model"]
    query = d * c["n_heads"] * c["head_dim"]
    key_value = 2 * d * c["n_kv_heads"] * c["head_dim"]
    attention, norms = 2 * query + key_value, 2 * d
    dense_ffn, expert = 3 * d * c["d_ff"], 3 * d * c["moe_d_ff"]
    shared = expert if c["shared_expert"] else 0
    router = c["num_experts"] * d
    moe_total = router + c["num_experts"] * expert + shared
    moe_active = router + c["experts_per_token"] * expert + shared
    total = c["vocab_size"] * d + d + (0 if c["tie_embeddings"] else c["vocab_size"] * d)
    active = total
    for layer in range(c["n_layers"]):
        total += attention + norms
        active += attention + norms
        if layer in c["moe_layers"]:
            total += moe_total
            active += moe_active
        else:
            total += dense_ffn
            active += dense_ffn
    return total, active


class TokenBatch:
    """batch.rs:22-222: sequences right-padded to the longest; `predicts(row)`: the row has a successor that is a
    real token of the same sequence (and, with a loss mask, one that is flagged)."""

    def __init__(self, sequences, loss_mask=None):
        if len(sequences) == 0:
            raise ValueError("EmptyDataset")
        self.lengths = [len(s) for s in sequences]
        if min(self.lengths) < 2:
            raise ValueError("InvalidConfig: a causal language-modelling loss needs at least two tokens per sequence")
        self.seq_len = max(self.lengths)
        self.batch = len(sequences)
        self.ids = np.zeros(self.batch * self.seq_len, np.uint32)
        self.valid = np.zeros(self.batch * self.seq_len, bool)
        for i, s in enumerate(sequences):
            self.ids[i * self.seq_len:i * self.seq_len + len(s)] = np.asarray(s, np.uint32)
            self.valid[i * self.seq_len:i * self.seq_len + len(s)] = True
        self.supervised = None
        if loss_mask is not None:
            if len(loss_mask) != len(self.ids):
                raise ValueError("InvalidConfig: a loss mask covers %d token positions, not %d" % (len(loss_mask), len(self.ids)))
            self.supervised = np.asarray(loss_mask, bool)
            if self.predicted() == 0:
                raise ValueError("InvalidConfig: a loss mask left no position to predict")

    @property
    def rows(self):
        return len(self.ids)

    def is_padded(self):
        return any(n != self.seq_len for n in self.lengths)

    def predicts(self, row):
        if row % self.seq_len + 1 >= self.lengths[row // self.seq_len]:
            return False
        return True if self.supervised is None else bool(self.supervised[row + 1])

    def predicted(self):
        return sum(1 for r in range(self.rows) if self.predicts(r))

    def layout_valid(self):
        """Layout::valid: None unless the batch is padded (batch.rs:212-217)."""
        return self.valid.astype(np.uint8) if self.is_padded() else None


def linear_forward(x, w):
    return (x.astype(F) @ w.astype(F).T).astype(F)


def silu(x):
    return (x / (F(1.0) + np.exp(-x))).astype(F)                 # ffn.rs:231-233


def silu_derivative(x):
    s = (F(1.0) / (F(1.0) + np.exp(-x))).astype(F)
    return (s * (F(1.0) + x * (F(1.0) - s))).astype(F)           # ffn.rs:235-238


def softmax_prefix(scores, seq_len, causal=True):
    """head_scores_batched's normalisation: row r sees r % seq_len + 1 keys, the tail is exactly zero."""
    out = np.zeros_like(scores, dtype=F)
    for r in range(scores.shape[0]):
        visible = r % seq_len + 1 if causal else seq_len
        v = scores[r, :visible].astype(F)
        e = np.exp((v - v.max()).astype(F)).astype(F)
        t = e.sum(dtype=F)
        out[r, :visible] = e / t if t > 0 else e
    return out


def attention_forward(x, wq, wk, wv, wo, H, Hkv, hd, seq_len, cos, sin, causal=True, rope=True):
    """MultiHeadAttention::forward_train; returns (output, cache)."""
    q, k, v = linear_forward(x, wq), linear_forward(x, wk), linear_forward(x, wv)
    if rope:
        q = np.concatenate([rope_apply(q[s:s + seq_len], H, 0, cos, sin) for s in range(0, x.shape[0], seq_len)])
        k = np.concatenate([rope_apply(k[s:s + seq_len], Hkv, 0, cos, sin) for s in range(0, x.shape[0], seq_len)])
    group, scale = H // Hkv, F(1.0) / np.sqrt(F(hd))
    rows = x.shape[0]
    merged = np.zeros((rows, H * hd), F)
    probs = []
    for head in range(H):
        qb, kb = head * hd, (head // group) * hd
        scores = np.zeros((rows, seq_len), F)
        for s0 in range(0, rows, seq_len):
            scores[s0:s0 + seq_len] = (q[s0:s0 + seq_len, qb:qb + hd] @ k[s0:s0 + seq_len, kb:kb + hd].T).astype(F) * scale
        p = softmax_prefix(scores, seq_len, causal)
        for s0 in range(0, rows, seq_len):
            merged[s0:s0 + seq_len, qb:qb + hd] = p[s0:s0 + seq_len] @ v[s0:s0 + seq_len, kb:kb + hd]
        probs.append(p)
    out = linear_forward(merged, wo)
    return out, dict(x=x, q=q, k=k, v=v, probs=probs, merged=merged, seq_len=seq_len)


def attention_backward(cache, grad_out, wq, wk, wv, wo, H, Hkv, hd, cos, sin, rope=True):
    """MultiHeadAttention::backward; returns (grad_input, {wq, wk, wv, wo gradients})."""
    x, q, k, v, merged, seq_len = cache["x"], cache["q"], cache["k"], cache["v"], cache["merged"], cache["seq_len"]
    rows = x.shape[0]
    group, scale = H // Hkv, F(1.0) / np.sqrt(F(hd))
    g_wo = (grad_out.T @ merged).astype(F)
    g_merged = (grad_out @ wo).astype(F)
    gq, gk, gv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    for head in range(H):
        p = cache["probs"][head]
        qb, kb = head * hd, (head // group) * hd
        for s0 in range(0, rows, seq_len):
            sl = slice(s0, s0 + seq_len)
            gp = (g_merged[sl, qb:qb + hd] @ v[sl, kb:kb + hd].T).astype(F)
            gv[sl, kb:kb + hd] += (p[sl].T @ g_merged[sl, qb:qb + hd]).astype(F)
            dot = (p[sl] * gp).sum(axis=1, keepdims=True, dtype=F)
            gs = (p[sl] * (gp - dot) * scale).astype(F)
            gq[sl, qb:qb + hd] += (gs @ k[sl, kb:kb + hd]).astype(F)
            gk[sl, kb:kb + hd] += (gs.T @ q[sl, qb:qb + hd]).astype(F)
    if rope:
        gq = np.concatenate([rope_apply(gq[s:s + seq_len], H, 0, cos, sin, -1.0) for s in range(0, rows, seq_len)])
        gk = np.concatenate([rope_apply(gk[s:s + seq_len], Hkv, 0, cos, sin, -1.0) for s in range(0, rows, seq_len)])
    grads = dict(wq=(gq.T @ x).astype(F), wk=(gk.T @ x).astype(F), wv=(gv.T @ x).astype(F), wo=g_wo)
    g_in = (gq @ wq + gk @ wk + gv @ wv).astype(F)
    return g_in, grads


def swiglu_forward(x, wg, wu, wd):
    gate, up = linear_forward(x, wg), linear_forward(x, wu)
    hidden = (silu(gate) * up).astype(F)
    return linear_forward(hidden, wd), dict(x=x, gate=gate, up=up, hidden=hidden)


def swiglu_backward(cache, grad_out, wg, wu, wd):
    g_hidden = (grad_out @ wd).astype(F)
    g_wd = (grad_out.T @ cache["hidden"]).astype(F)
    g_gate = (g_hidden * cache["up"] * silu_derivative(cache["gate"])).astype(F)
    g_up = (g_hidden * silu(cache["gate"])).astype(F)
    g_in = (g_gate @ wg + g_up @ wu).astype(F)
    return g_in, dict(gate=(g_gate.T @ cache["x"]).astype(F), up=(g_up.T @ cache["x"]).astype(F), down=g_wd)


def causal_lm_loss(logits, batch: TokenBatch):
    """(loss, grad_logits, predicted): causal_lm_loss_batch (causal_lm_loss.rs:66-150)."""
    rows, vocab = logits.shape
    if rows != batch.rows:
        raise ValueError("InvalidTarget: expected %d rows, got %d" % (rows, batch.rows))
    predicted = batch.predicted()
    if predicted == 0:
        raise ValueError("InvalidConfig: a causal language-modelling loss needs at least two tokens")
    inv = F(1.0) / F(predicted)
    grad = np.zeros((rows, vocab), F)
    total = F(0.0)
    for r in range(rows):
        if not batch.predicts(r):
            continue
        target = int(batch.ids[r + 1])
        if target >= vocab:
            raise ValueError("TokenOutOfRange: id %d, vocab_size %d" % (target, vocab))
        v = logits[r].astype(F)
        e = np.exp((v - v.max()).astype(F)).astype(F)
        p = (e / e.sum(dtype=F)).astype(F)
        total = F(total + F(-np.log(max(p[target], np.finfo(F).tiny))))
        grad[r] = p * inv
        grad[r, target] -= inv
    return float(total / F(predicted)), grad, predicted


def seeded_model_weights(c, seed, std=0.02):
    """A full set of weights, N(0, std) (embedding U(-0.02, 0.02) like Embedding::new, embedding.rs:26-33); the
    builder-seed -> weights stream of the reference (rand's StdRng) is not reproduced, weights are injected."""
    g = np.random.Generator(np.random.Philox(seed))
    d, H, Hkv, hd = c["d_model"], c["n_heads"], c["n_kv_heads"], c["head_dim"]
    n = lambda *shape: (g.standard_normal(shape) * std).astype(F)
    w = dict(embedding=g.uniform(-0.02, 0.02, (c["vocab_size"], d)).astype(F), final_norm=np.ones(d, F), blocks=[])
    if not c["tie_embeddings"]:
        w["lm_head"] = n(c["vocab_size"], d)
    for layer in range(c["n_layers"]):
        b = dict(attention_norm=(1.0 + 0.1 * g.standard_normal(d)).astype(F), wq=n(H * hd, d), wk=n(Hkv * hd, d),
                 wv=n(Hkv * hd, d), wo=n(d, H * hd), ffn_norm=(1.0 + 0.1 * g.standard_normal(d)).astype(F))
        if layer in c["moe_layers"]:
            E, Fm = c["num_experts"], c["moe_d_ff"]
            b["moe"] = dict(router=n(E, d), gate=n(E, Fm, d), up=n(E, Fm, d), down=n(E, d, Fm),
                            shared=(n(Fm, d), n(Fm, d), n(d, Fm)) if c["shared_expert"] else None)
        else:
            b["gate"], b["up"], b["down"] = n(c["d_ff"], d), n(c["d_ff"], d), n(d, c["d_ff"])
        w["blocks"].append(b)
    w["final_norm"] = (1.0 + 0.1 * g.standard_normal(d)).astype(F)
    return w


class OracleLm:
    """TransformerLm on the host: forward_batch, backward, train_step_batch, with injected weights (stepped in place)."""

    def __init__(self, config, weights):
        from . import OracleMoe
        validate(config)
        self.c, self.w = config, weights
        self.cos, self.sin = rope_tables(config["head_dim"], config["max_seq_len"], config["rope_base"])
        self.moe = {}
        for layer in config["moe_layers"]:
            m = OracleMoe(config["d_model"], config["num_experts"], config["experts_per_token"], config["moe_d_ff"],
                          config["shared_expert"], config["aux_loss_weight"], config["router_z_loss_weight"])
            mw = weights["blocks"][layer]["moe"]
            m.set_weights(mw["router"], mw["gate"], mw["up"], mw["down"], mw["shared"])
            self.moe[layer] = m
        self.grads = None
        self.step_count = 0
        self.moments = {}

    # -- forward_batch (transformer.rs:676-735) ---------------------------------------------------
    def forward(self, batch: TokenBatch, moe_logits=None):
        """Returns logits [rows, vocab]; keeps the caches.  `moe_logits[layer]` overrides a router product."""
        c, w = self.c, self.w
        if batch.seq_len > c["max_seq_len"]:
            raise ValueError("SequenceTooLong: length %d, max_seq_len %d" % (batch.seq_len, c["max_seq_len"]))
        if int(batch.ids.max()) >= c["vocab_size"]:
            raise ValueError("TokenOutOfRange")
        hidden = w["embedding"][batch.ids.astype(np.int64)].astype(F)
        valid = batch.layout_valid()
        self.caches, self.aux = [], 0.0
        for layer, b in enumerate(w["blocks"]):
            normed = rms.forward(hidden, b["attention_norm"], c["rmsnorm_eps"])
            attended, ac = attention_forward(normed, b["wq"], b["wk"], b["wv"], b["wo"], c["n_heads"], c["n_kv_heads"],
                                             c["head_dim"], batch.seq_len, self.cos, self.sin, c["causal"])
            residual = (attended + hidden).astype(F)
            normed2 = rms.forward(residual, b["ffn_norm"], c["rmsnorm_eps"])
            if layer in self.moe:
                lg = None if moe_logits is None else moe_logits.get(layer)
                projected = self.moe[layer].forward(normed2, valid=valid, logits=lg)
                a, z = self.moe[layer].losses()
                self.aux += a + z
                fc = None
            else:
                projected, fc = swiglu_forward(normed2, b["gate"], b["up"], b["down"])
            out = (projected + residual).astype(F)
            self.caches.append(dict(input=hidden, attention=ac, residual=residual, normed2=normed2, ffn=fc))
            hidden = out
        self.final_input = hidden
        self.final_output = rms.forward(hidden, w["final_norm"], c["rmsnorm_eps"])
        head = w["embedding"] if c["tie_embeddings"] else w["lm_head"]
        self.batch = batch
        return linear_forward(self.final_output, head)

    # -- backward (transformer.rs:1214-1246) ------------------------------------------------------
    def backward(self, grad_logits):
        """Accumulates into self.grads (created zero by zero_grad)."""
        c, w, g = self.c, self.w, self.grads
        head_key = "embedding" if c["tie_embeddings"] else "lm_head"
        head = w[head_key]
        g[head_key] = (g[head_key] + grad_logits.T @ self.final_output).astype(F)
        gh = (grad_logits @ head).astype(F)
        gh, g["final_norm"] = rms.backward(self.final_input, w["final_norm"], gh, c["rmsnorm_eps"], g["final_norm"])
        for layer in reversed(range(c["n_layers"])):
            b, cache, gb = w["blocks"][layer], self.caches[layer], g["blocks"][layer]
            if layer in self.moe:
                g_proj = self.moe[layer].backward(gh)
            else:
                g_proj, fg = swiglu_backward(cache["ffn"], gh, b["gate"], b["up"], b["down"])
                for k in ("gate", "up", "down"):
                    gb[k] = (gb[k] + fg[k]).astype(F)
            g_res, gb["ffn_norm"] = rms.backward(cache["residual"], b["ffn_norm"], g_proj, c["rmsnorm_eps"], gb["ffn_norm"])
            g_res = (g_res + gh).astype(F)
            g_att, ag = attention_backward(cache["attention"], g_res, b["wq"], b["wk"], b["wv"], b["wo"], c["n_heads"],
                                           c["n_kv_heads"], c["head_dim"], self.cos, self.sin)
            for k in ("wq", "wk", "wv", "wo"):
                gb[k] = (gb[k] + ag[k]).astype(F)
            g_in, gb["attention_norm"] = rms.backward(cache["input"], b["attention_norm"], g_att, c["rmsnorm_eps"], gb["attention_norm"])
            gh = (g_in + g_res).astype(F)
        np.add.at(g["embedding"], self.batch.ids.astype(np.int64), gh)      # Embedding::backward, in row order

    def zero_grad(self):
        w = self.w
        self.grads = dict(embedding=np.zeros_like(w["embedding"]), final_norm=np.zeros_like(w["final_norm"]), blocks=[])
        if "lm_head" in w:
            self.grads["lm_head"] = np.zeros_like(w["lm_head"])
        for layer, b in enumerate(w["blocks"]):
            self.grads["blocks"].append({k: np.zeros_like(v) for k, v in b.items() if k != "moe"})
        for m in self.moe.values():
            m.zero_grad()

    def accumulate_step(self, batch, moe_logits=None):
        """(lm_loss, auxiliary_loss): forward, loss, backward into the existing gradients (transformer.rs:1519-1545)."""
        logits = self.forward(batch, moe_logits)
        loss, grad_logits, _ = causal_lm_loss(logits, batch)
        if self.grads is None:
            self.zero_grad()
        self.backward(grad_logits)
        return loss, self.aux

    def step(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, scale=1.0, kind="adam"):
        """TransformerLm::step over every parameter with Param::step's Sgd, Adam or Lion arm (param.rs:547-617);
        clears the gradients.  The step counter advances for every kind."""
        self.step_count += 1
        t = self.step_count

        def upd(key, wv, gv):
            gsc = (gv * F(scale)).astype(F)
            if kind == "sgd":
                wv -= (F(lr) * gv * F(scale)).astype(F)
                return
            m, v = self.moments.get(key, (np.zeros_like(wv), np.zeros_like(wv)))
            if kind == "lion":
                update = (F(beta1) * m + F(1 - beta1) * gsc).astype(F)
                m = (F(beta2) * m + F(1 - beta2) * gsc).astype(F)
                self.moments[key] = (m, v)
                wv -= (F(lr) * (np.sign(update).astype(F) + F(wd) * wv)).astype(F)
                return
            m = (F(beta1) * m + F(1 - beta1) * gsc).astype(F)
            v = (F(beta2) * v + F(1 - beta2) * gsc * gsc).astype(F)
            self.moments[key] = (m, v)
            wv -= F(lr) * F(wd) * wv
            mh = m / F(1 - beta1 ** t)
            vh = v / F(1 - beta2 ** t)
            wv -= (F(lr) * mh / (np.sqrt(vh) + F(eps))).astype(F)

        w, g = self.w, self.grads
        upd("embedding", w["embedding"], g["embedding"])
        upd("final_norm", w["final_norm"], g["final_norm"])
        if "lm_head" in w:
            upd("lm_head", w["lm_head"], g["lm_head"])
        for layer, b in enumerate(w["blocks"]):
            for k in b:
                if k != "moe":
                    upd((layer, k), b[k], g["blocks"][layer][k])
        for m in self.moe.values():
            if kind == "sgd":
                m.sgd_step(lr, scale)
            elif kind == "lion":
                m.lion_step(lr, beta1, beta2, wd, scale)
            else:
                m.adam_step(lr, beta1, beta2, eps, wd, t, scale)
        self.zero_grad()

    def train_step(self, batch, moe_logits=None, **adam):
        """train_step_batch (transformer.rs:1394-1425): zero_grad, forward, loss, backward, step."""
        self.zero_grad()
        out = self.accumulate_step(batch, moe_logits)
        self.step(**adam)
        return out
