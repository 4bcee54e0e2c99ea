"""The reference's binary snapshot files, seen from the MoE layer.

Reading is done by the library (`moe_snapshot_info`, `moe_load_snapshot_layer`,
`moe_load_optimizer_layer` in include/moe_b200.h); this module wraps those calls and adds the
two writers, which follow `TransformerLm::save_bin` (reference transformer.rs:1809-1860) and
`save_optimizer_state` (transformer.rs:1675-1696) byte for byte, so that a MoE layer trained or
quantized here can be handed back to the reference and so that tests can build files.

File order of the parameters is `TransformerLm::params_mut` (transformer.rs:1620-1630); see
`parameter_names`.
"""
from __future__ import annotations

import ctypes as C
import json
import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib

WEIGHTS_MAGIC = b"RBWTS001"
OPTIMIZER_MAGIC = b"RBOPT001"
LORA_MAGIC = b"RBLOR001"


class InvalidSnapshot(ValueError):
    """NetworkError::InvalidSnapshot of the reference."""


@dataclass
class SnapshotInfo:
    """Header of a weight file (BinHeader, transformer.rs:503-510) plus what the parameter count implies."""
    config: Dict[str, object]
    precision: str                 # "F32" or "Q8"
    optimizer_step: int
    parameter_count: int
    dense_ffn_params: int          # 3 SwiGLU, 2 GELU, 0 when every block is MoE
    moe_layers: List[int] = field(default_factory=list)
    lora_rank: int = 0             # config.lora.rank when the file holds adapters
    lora_alpha: float = 0.0
    _c: Optional[_lib.SnapshotInfoC] = None


def snapshot_info(path: str) -> SnapshotInfo:
    """Parses the header of a weight file with the library's reader (host only)."""
    c = _lib.SnapshotInfoC()
    msg = C.create_string_buffer(512)
    rc = _lib.lib().moe_snapshot_info(str(path).encode(), C.byref(c), msg, len(msg))
    if rc != _lib.OK:
        raise InvalidSnapshot(msg.value.decode(errors="replace"))
    names = ("vocab_size", "d_model", "n_layers", "n_heads", "n_kv_heads", "head_dim", "d_ff", "moe_d_ff",
             "num_experts", "experts_per_token", "max_seq_len")
    config: Dict[str, object] = {n: int(getattr(c, n)) for n in names}
    config.update(shared_expert=bool(c.shared_expert), tie_embeddings=bool(c.tie_embeddings), causal=bool(c.causal),
                  aux_loss_weight=float(c.aux_loss_weight), router_z_loss_weight=float(c.router_z_loss_weight),
                  rope_base=float(c.rope_base), rmsnorm_eps=float(c.rmsnorm_eps))
    layers = [int(c.moe_layers[i]) for i in range(c.n_moe_layers)]
    config["moe_layers"] = layers
    return SnapshotInfo(config=config, precision="Q8" if c.precision == _lib.PRECISION_Q8 else "F32",
                        optimizer_step=int(c.optimizer_step), parameter_count=int(c.parameter_count),
                        dense_ffn_params=int(c.dense_ffn_params), moe_layers=layers, lora_rank=int(c.lora_rank),
                        lora_alpha=float(c.lora_alpha), _c=c)


def parameter_names(config: Dict[str, object], dense_ffn_params: int = 3) -> List[Tuple[str, Tuple[int, int]]]:
    """(name, (rows, cols)) of every parameter in file order (params_mut, transformer.rs:1620-1630;
    block order transformer_block.rs:286-292; MoE order moe.rs:516-525; SwiGLU order ffn.rs:126-131).
    With ``config["lora"]`` set every adapted projection is followed by its adapter's down and up
    (Linear::params_mut, param.rs:859-865)."""
    base = _base_parameter_names(config, dense_ffn_params)
    lora = config.get("lora")
    if not lora:
        return base
    rank = int(lora["rank"])
    out: List[Tuple[str, Tuple[int, int]]] = []
    for name, (rows, cols) in base:
        out.append((name, (rows, cols)))
        if _adapted(name):
            out += [(name + ".lora.down", (rank, cols)), (name + ".lora.up", (rows, rank))]
    return out


def _adapted(name: str) -> bool:
    part = name.split(".")
    return len(part) > 2 and (part[2] in ("attention", "ffn") or (part[2] == "moe" and part[3] != "router"))


def _base_parameter_names(config: Dict[str, object], dense_ffn_params: int = 3) -> List[Tuple[str, Tuple[int, int]]]:
    d = int(config["d_model"]); V = int(config["vocab_size"]); F = int(config["d_ff"]); Fm = int(config["moe_d_ff"])
    H = int(config["n_heads"]); Hkv = int(config["n_kv_heads"]); hd = int(config["head_dim"]); E = int(config["num_experts"])
    moe = set(int(i) for i in config["moe_layers"])
    out: List[Tuple[str, Tuple[int, int]]] = [("embedding", (V, d))]
    for b in range(int(config["n_layers"])):
        p = "blocks.%d." % b
        out += [(p + "attention_norm", (1, d)), (p + "attention.query", (H * hd, d)), (p + "attention.key", (Hkv * hd, d)),
                (p + "attention.value", (Hkv * hd, d)), (p + "attention.output", (d, H * hd)),
                (p + "feed_forward_norm", (1, d))]
        if b in moe:
            out.append((p + "moe.router", (E, d)))
            for e in range(E):
                q = p + "moe.experts.%d." % e
                out += [(q + "gate", (Fm, d)), (q + "up", (Fm, d)), (q + "down", (d, Fm))]
            if config.get("shared_expert"):
                q = p + "moe.shared."
                out += [(q + "gate", (Fm, d)), (q + "up", (Fm, d)), (q + "down", (d, Fm))]
        elif dense_ffn_params == 2:
            out += [(p + "ffn.up", (F, d)), (p + "ffn.down", (d, F))]
        else:
            out += [(p + "ffn.gate", (F, d)), (p + "ffn.up", (F, d)), (p + "ffn.down", (d, F))]
    out.append(("final_norm", (1, d)))
    if not config.get("tie_embeddings"):
        out.append(("lm_head", (V, d)))
    return out


def quantize_rows(w: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """The reference's int8 grid (transformer.rs:514-519, 1843-1851): scale = max|row| / 127,
    round half away from zero, clamp to +-127; a zero row has scale 0 and all-zero bytes."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    scale = (np.abs(w).max(axis=1) if w.shape[1] else np.zeros(w.shape[0], np.float32)).astype(np.float32) / np.float32(127.0)
    safe = np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)
    r = (w / safe[:, None]).astype(np.float32)
    r = np.sign(r) * np.floor(np.abs(r) + np.float32(0.5))      # f32::round: halves away from zero
    q = np.clip(r, -127, 127).astype(np.int8)
    q[scale == 0] = 0
    return q, scale.astype(np.float32)


def write_snapshot(path: str, config: Dict[str, object], tensors: Iterable[np.ndarray], precision: str = "F32",
                   optimizer: Optional[Dict[str, object]] = None, optimizer_step: int = 0) -> None:
    """save_bin: `tensors` are the f32 parameters in file order (see `parameter_names`)."""
    if precision not in ("F32", "Q8"):
        raise ValueError("precision is 'F32' or 'Q8'")
    cfg = dict(config)
    cfg.setdefault("lora", None)
    if optimizer is None:
        optimizer = {"Adam": {"learning_rate": 1e-3, "beta1": 0.9, "beta2": 0.999, "epsilon": 1e-8, "weight_decay": 0.0}}
    header = json.dumps({"config": cfg, "optimizer": optimizer, "optimizer_step": int(optimizer_step),
                         "precision": precision}, separators=(",", ":")).encode()
    tensors = [np.ascontiguousarray(t, dtype=np.float32) for t in tensors]
    with open(path, "wb") as f:
        f.write(WEIGHTS_MAGIC)
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        f.write(struct.pack("<Q", len(tensors)))
        for t in tensors:
            if t.ndim != 2:
                raise ValueError("every parameter is a matrix")
            f.write(struct.pack("<QQ", t.shape[0], t.shape[1]))
            if precision == "F32":
                f.write(t.astype("<f4").tobytes())
            else:
                q, scale = quantize_rows(t)
                rec = np.empty((t.shape[0], 4 + t.shape[1]), np.uint8)
                rec[:, :4] = scale.astype("<f4").view(np.uint8).reshape(-1, 4)
                rec[:, 4:] = q.view(np.uint8)
                f.write(rec.tobytes())


def write_optimizer_state(path: str, moments: Sequence[Optional[Tuple[np.ndarray, np.ndarray]]], step: int) -> None:
    """save_optimizer_state: (first, second) per parameter in file order; None writes the 0 x 0
    placeholder of a frozen parameter (transformer.rs:1729-1735)."""
    with open(path, "wb") as f:
        f.write(OPTIMIZER_MAGIC)
        f.write(struct.pack("<QQ", len(moments), int(step)))
        for mv in moments:
            if mv is None:
                f.write(struct.pack("<QQ", 0, 0))
                continue
            m, v = (np.ascontiguousarray(a, dtype=np.float32) for a in mv)
            if m.shape != v.shape or m.ndim != 2:
                raise ValueError("the two moments of a parameter have its shape")
            f.write(struct.pack("<QQ", m.shape[0], m.shape[1]))
            f.write(m.astype("<f4").tobytes())
            f.write(v.astype("<f4").tobytes())


def adapter_names(config: Dict[str, object], rank: int, dense_ffn_params: int = 3) -> List[Tuple[str, Tuple[int, int]]]:
    """(name, (rows, cols)) of every adapter matrix in `save_lora` order: per block the four attention
    projections, then the feed-forward projections (MoE: every expert's and the shared expert's, never
    the router; transformer_block.rs:274-278, moe.rs:502-514), `down` [rank, in] before `up` [out, rank]
    (param.rs:711-713)."""
    out: List[Tuple[str, Tuple[int, int]]] = []
    for name, (rows, cols) in _base_parameter_names(config, dense_ffn_params):
        if _adapted(name):
            out += [(name + ".lora.down", (rank, cols)), (name + ".lora.up", (rows, rank))]
    return out


def write_lora(path: str, rank: int, alpha: float, tensors: Iterable[np.ndarray], seed: int = 0) -> None:
    """save_lora: the adapter matrices in `adapter_names` order."""
    header = json.dumps({"rank": int(rank), "alpha": float(alpha), "seed": int(seed)}, separators=(",", ":")).encode()
    tensors = [np.ascontiguousarray(t, dtype=np.float32) for t in tensors]
    with open(path, "wb") as f:
        f.write(LORA_MAGIC)
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        f.write(struct.pack("<Q", len(tensors)))
        for t in tensors:
            f.write(struct.pack("<QQ", t.shape[0], t.shape[1]))
            f.write(t.astype("<f4").tobytes())
