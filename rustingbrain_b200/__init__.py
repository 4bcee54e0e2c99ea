"""B200-native (sm_100a) mixture-of-experts feed-forward layer.

A from-scratch CUDA implementation of the hot path of the reference crate's
``src/moe.rs`` behind a C ABI (``include/moe_b200.h``).  This package is the
host-side mirror of the reference's ``MoeConfig`` / ``MoeLayer`` / ``MoeCache``
interface over that ABI.
"""
from .moe import (CudaError, InvalidConfig, InvalidInput, MoeCache, MoeConfig, MoeLayer, NetworkError, Timeout,
                  DEFAULT_AUX_LOSS_WEIGHT, DEFAULT_ROUTER_Z_LOSS_WEIGHT)

from .snapshot import InvalidSnapshot, SnapshotInfo, snapshot_info, write_optimizer_state, write_snapshot

__all__ = ["InvalidSnapshot", "SnapshotInfo", "snapshot_info", "write_snapshot", "write_optimizer_state",
           "MoeConfig", "MoeLayer", "MoeCache", "NetworkError", "InvalidConfig", "InvalidInput", "CudaError", "Timeout",
           "DEFAULT_AUX_LOSS_WEIGHT", "DEFAULT_ROUTER_Z_LOSS_WEIGHT"]
