"""Fused communication + compute kernels.

``AllGatherLinear`` runs ``y = x W^T`` for a weight whose rows are sharded over the ranks of a
symmetric region: a few CTAs of the GEMM kernel pull the peers' shards over NVLink into the local
gathered buffer while the remaining CTAs already multiply the chunks that have landed
(``fsb_gemm_bf16_allgather`` in ``csrc/gemm_bf16.cu``). The gathered weight stays valid after the
call, so the backward pass (dgrad) reuses it without a second gather.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import count_launch

_declared = False
BN = 256


def _ensure():
    global _declared
    if not _declared:
        c = ctypes
        vp, i32, i64, u32 = c.c_void_p, c.c_int, c.c_longlong, c.c_uint
        _lib.declare("fsb_gemm_bf16_allgather", [vp, vp, vp, vp, i32, i32, i32, i64, i64, i32, i32, i32, vp, i32,
                                                 i32, vp, u32, u32, vp, vp])
        _declared = True


class AllGatherLinear:
    """State of one row-sharded weight for the fused all-gather -> GEMM kernel.

    ``peer_shard_addrs[r]`` is the address (in this process) of rank r's ``[shard_rows, K]`` bf16
    shard; ``out_features`` may be smaller than ``world * shard_rows`` (padding in the last shard).
    """

    def __init__(self, peer_shard_addrs, out_features: int, in_features: int, shard_rows: int,
                 device: torch.device, n_stagers: int = 12, flag_row_addr: int = 0, max_polls: int = 20_000_000):
        _ensure()
        self.addrs = (ctypes.c_ulonglong * len(peer_shard_addrs))(*peer_shard_addrs)
        self.world = len(peer_shard_addrs)
        self.N, self.K, self.shard_rows = out_features, in_features, shard_rows
        if (shard_rows * in_features * 2) % 16384 != 0 or (BN * in_features * 2) % 16384 != 0:
            raise ValueError("shard and chunk sizes must be multiples of 16 KB for the bulk-copy ring")
        self.device = device
        self.gathered = torch.empty(out_features, in_features, dtype=torch.bfloat16, device=device)
        self.counters = torch.zeros(-(-out_features // BN), dtype=torch.int32, device=device)
        self.calls = 0
        self.n_stagers = n_stagers
        self.flag_row_addr = flag_row_addr
        self.max_polls = max_polls

    def __call__(self, x: torch.Tensor, epoch: int = 0, out_dtype=torch.bfloat16) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        assert x2.dtype == torch.bfloat16 and x2.shape[1] == self.K and x2.stride(1) == 1
        M = x2.shape[0]
        out = torch.empty(M, self.N, dtype=out_dtype, device=x.device)
        self.calls += 1
        status = _lib.status_word(x.device)
        rc = _lib.load().fsb_gemm_bf16_allgather(
            x2.data_ptr(), self.addrs, self.gathered.data_ptr(), out.data_ptr(), M, self.N, self.K,
            x2.stride(0), out.stride(0), int(out_dtype == torch.float32), self.world, self.shard_rows,
            self.counters.data_ptr(), self.calls, self.n_stagers,
            self.flag_row_addr if self.flag_row_addr else None, epoch & 0xFFFFFFFF, self.max_polls,
            status.data_ptr(), _lib.stream_ptr(x.device))
        _lib.check(rc, "fsb_gemm_bf16_allgather")
        count_launch()
        return out.view(*x.shape[:-1], self.N)

    def reset(self) -> None:
        """Forget the progress counters. The counters grow by one chunk's pieces per call and every call waits
        for ``pieces * call_index``; after a call that reported a timeout (``ops.check_status()`` raised) some
        chunks never reached their count, so every later call would time out as well. Call this (on every rank
        of the group, with the stream idle) before using the object again."""
        self.counters.zero_()
        self.calls = 0
