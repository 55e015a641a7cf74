"""The library's own communicator over the C ABI (phx_comm_*): sharded retrieval and sharded gather-sum as single
native calls, with no framework collective on the path.  One process per GPU: rank 0 calls `unique_id()`, the host
ships the bytes to the other processes by its own means (a pipe, a file, a key-value store), every rank constructs a
`Communicator` (collective).  Mirrors the bootstrap of the reference's row-sharded embedding
(phoenix/xrex/cuda/row_emb/src/row_emb_comm.cc:283-345)."""
from __future__ import annotations

import ctypes as C
from typing import List

from . import _lib
from ._lib import PhoenixError, lib

ID_BYTES = 128


def unique_id() -> bytes:
    buf = (C.c_uint8 * ID_BYTES)()
    st = lib.phx_comm_unique_id(buf)
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())
    return bytes(buf)


class Communicator:
    def __init__(self, id_bytes: bytes, rank: int, world: int, device: int):
        assert len(id_bytes) == ID_BYTES
        self.rank, self.world, self.device = rank, world, device
        self._h = C.c_void_p()
        st = lib.phx_comm_create((C.c_uint8 * ID_BYTES).from_buffer_copy(id_bytes), rank, world, device, C.byref(self._h))
        if st != 0:
            raise PhoenixError(st, lib.phx_global_error().decode())

    def _check(self, st: int):
        if st != 0:
            raise PhoenixError(st, lib.phx_comm_last_error(self._h).decode())

    def close(self):
        if self._h:
            lib.phx_comm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def nccl_version(self) -> int:
        v = C.c_int32()
        self._check(lib.phx_comm_info(self._h, None, None, C.byref(v)))
        return int(v.value)

    def barrier(self, stream: int = 0):
        self._check(lib.phx_comm_barrier(self._h, stream or None))

    def retrieve_topk(self, shard, users, B: int, k: int, scores, ids, stream: int = 0):
        """Top-k of the whole row-sharded corpus for the same queries on every rank (collective, returns when the
        result is ready): users f32 [B,dim], scores f32 [B,k], ids int64 [B,k] CUDA tensors."""
        self._check(lib.phx_retrieve_topk(self._h, shard._h, int(users.data_ptr()), B, k, int(scores.data_ptr()),
                                          int(ids.data_ptr()), stream or None))

    def gather_setup(self, engine, max_ids: int, recv_factor: float = 2.0):
        self._check(lib.phx_gather_sharded_setup(self._h, engine._h, max_ids, float(recv_factor)))

    def gather_sum(self, engine, family: int, ids, n: int, out, stream: int = 0):
        """Multi-hash gather-sum of this rank's ids over the row-sharded table (collective): ids int64 [n], out int16
        view of bf16 [n, emb_size]; asynchronous on `stream` after the one host wait inside."""
        self._check(lib.phx_gather_sum_sharded(self._h, engine._h, family, int(ids.data_ptr()), n, int(out.data_ptr()),
                                               stream or None))

    def gather_sum_multi(self, engine, families, counts, ids, out, stream: int = 0):
        """The same for several features in one exchange: ids holds the runs back to back, run i = counts[i] ids of hash
        family families[i] (0 user, 1 item, 2 author, 3 ip).  Lookups that spread over the table's regions load every
        owner alike."""
        m = len(families)
        fam = (C.c_int32 * m)(*[int(f) for f in families])
        cnt = (C.c_int64 * m)(*[int(c) for c in counts])
        self._check(lib.phx_gather_sum_sharded_multi(self._h, engine._h, m, fam, cnt, int(ids.data_ptr()), int(out.data_ptr()),
                                                     stream or None))

    def gather_phase_ms(self) -> List[float]:
        buf = (C.c_float * 7)()
        self._check(lib.phx_gather_sharded_phase_ms(self._h, buf))
        return [float(x) for x in buf]
