"""Tensor-parallel plumbing: exchange of the per-rank IPC handles over torch.distributed.

The data path never goes through torch: row-parallel products push their partial sums into the peers'
exchange buffers with plain NVLink stores inside the product kernel itself (csrc/tp_device.cuh); this module
only carries 64 opaque bytes per rank between the processes once, at set-up.
"""
from __future__ import annotations

import ctypes as C

HANDLE_BYTES = 64


def gather_handles(dist, mine: bytes):
    """All ranks' handles, in rank order (any backend: goes through all_gather_object)."""
    world = dist.get_world_size()
    out = [None] * world
    dist.all_gather_object(out, bytes(mine))
    if any(h is None or len(h) != HANDLE_BYTES for h in out):
        raise RuntimeError("handle exchange returned a malformed entry")
    return out


def attach(model, dist) -> None:
    """Export this rank's exchange buffer, gather everybody's handles, map the peers, then barrier so that no
    rank starts pushing before every buffer is mapped and cleared."""
    lib = model.lib
    buf = C.create_string_buffer(HANDLE_BYTES)
    lib.check(lib.swlm_tp_export(model.state, buf))
    handles = gather_handles(dist, buf.raw)
    blob = b"".join(handles)
    lib.check(lib.swlm_tp_attach(model.state, C.c_char_p(blob)))
    dist.barrier()


def status(model) -> int:
    """0, or SWLM_ERR_TIMEOUT (-5) when a bounded wait on another rank expired."""
    return int(model.lib.swlm_tp_status(model.state))


def shard_range(lib, shard_kind: int, n: int, k: int, rank: int, size: int):
    out = (C.c_int * 4)()
    lib.check(lib.swlm_shard_range(shard_kind, n, k, rank, size, out))
    return tuple(out)
