"""Corpus shards and exhaustive dot-product top-k (phoenix/xrex/models/recsys_two_tower_model.py:
2455-2516, 193-221; phoenix/xrex/cuda/top_k_by_key/__init__.py:56-94) over the C ABI."""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import numpy as np

from . import _lib
from ._lib import PhoenixError, lib


class CorpusShard:
    """Rows [row_offset, row_offset + rows) of the post corpus on one device."""

    def __init__(self, rows: int, dim: int, row_offset: int = 0, max_queries: int = 256, max_k: int = 1000,
                 device: int = 0):
        self.rows, self.dim, self.row_offset, self.device = rows, dim, row_offset, device
        self.max_queries, self.max_k = max_queries, max_k
        self._h = C.c_void_p()
        st = lib.phx_corpus_create(device, rows, dim, row_offset, max_queries, max_k, C.byref(self._h))
        if st != 0:
            raise PhoenixError(st, lib.phx_global_error().decode())

    def _check(self, st: int):
        if st != 0:
            raise PhoenixError(st, lib.phx_corpus_last_error(self._h).decode())

    def close(self):
        if self._h:
            lib.phx_corpus_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def upload(self, row0: int, rows_bf16_bits: np.ndarray):
        a = np.ascontiguousarray(rows_bf16_bits, dtype=np.uint16)
        self._check(lib.phx_corpus_upload(self._h, row0, a.shape[0], a.ctypes.data))

    def fill_synthetic(self, seed: int):
        self._check(lib.phx_corpus_fill_synthetic(self._h, seed))

    def upload_int8(self, row0: int, q8: np.ndarray, scales: np.ndarray):
        """The int8 form of rows [row0, row0 + n): q8 int8 [n, dim], scales f32 [n] (the reference's post_q8 /
        post_scales, recsys_two_tower_model.py:2518-2533)."""
        q = np.ascontiguousarray(q8, dtype=np.int8); sc = np.ascontiguousarray(scales, dtype=np.float32)
        assert q.shape == (sc.shape[0], self.dim)
        self._check(lib.phx_corpus_upload_int8(self._h, row0, q.shape[0], q.ctypes.data, sc.ctypes.data))

    def quantize_int8(self):
        """Derive the int8 form from the resident bf16 rows on the device (scale = max|row| / 127)."""
        self._check(lib.phx_corpus_quantize_int8(self._h))

    def set_int8(self, on: bool):
        """Score every later top-k with the int8 form (half the bytes per row)."""
        self._check(lib.phx_corpus_set_int8(self._h, int(bool(on))))

    def read_int8_device(self, row0: int, nrows: int, q8, scales):
        self._check(lib.phx_corpus_read_int8_device(self._h, row0, nrows, int(q8.data_ptr()), int(scales.data_ptr())))

    def topk_device(self, users, B: int, k: int, scores, ids):
        """users f32 [B,dim], scores f32 [B,k], ids int64 [B,k]: torch CUDA tensors; asynchronous."""
        self._check(lib.phx_corpus_topk_device(self._h, int(users.data_ptr()), B, k, int(scores.data_ptr()),
                                               int(ids.data_ptr())))

    def set_mask(self, eligible):
        """Restrict every later top-k on this shard to the rows whose entry of `eligible` (bool [rows], or None to lift
        the restriction) is true: the reference's per-post type / eligibility mask
        (recsys_two_tower_model.py:2486-2493)."""
        if eligible is None:
            self._check(lib.phx_corpus_set_mask(self._h, None))
            return
        bits = np.packbits(np.asarray(eligible, dtype=bool), bitorder="little")
        words = np.zeros((len(eligible) + 31) // 32 * 4, np.uint8)
        words[:bits.size] = bits
        self._check(lib.phx_corpus_set_mask(self._h, words.view(np.uint32).ctypes.data))

    def topk_window_device(self, users, B: int, k: int, row_begin: int, row_end: int, scores, ids):
        """Top-k over shard-local rows [row_begin, row_end) only: one retrieval dataset of the reference's post table
        (recsys_two_tower_model.py:2660-2686); ids are global rows as in `topk_device`."""
        self._check(lib.phx_corpus_topk_window_device(self._h, int(users.data_ptr()), B, k, row_begin, row_end,
                                                      int(scores.data_ptr()), int(ids.data_ptr())))

    def topk_keys_device(self, users, B: int, k: int, keys):
        """The shard's top-k as sorted 64-bit keys int64 [B,k] (score and row in one word): the form the lists are
        gathered in before a merge."""
        self._check(lib.phx_corpus_topk_keys_device(self._h, int(users.data_ptr()), B, k, int(keys.data_ptr())))

    def merge_keys_device(self, keys, P: int, B: int, k: int, out_scores, out_ids):
        self._check(lib.phx_topk_merge_keys_device(self._h, int(keys.data_ptr()), P, B, k, int(out_scores.data_ptr()),
                                                   int(out_ids.data_ptr())))

    def set_stream(self, stream):
        """Run the shard's later work on this CUDA stream (an integer handle, 0 = the default stream; None = the
        shard's own stream)."""
        self._check(lib.phx_corpus_set_stream(self._h, stream or None, 1 if stream is None else 0))

    def merge_device(self, scores, ids, P: int, B: int, k: int, out_scores, out_ids):
        self._check(lib.phx_topk_merge_device(self._h, int(scores.data_ptr()), int(ids.data_ptr()), P, B, k,
                                              int(out_scores.data_ptr()), int(out_ids.data_ptr())))

    def sync(self):
        self._check(lib.phx_corpus_sync(self._h))

    def finish(self) -> bool:
        """Wait for the shard's work; True when the last top-k had to be done again with exact thresholds (its output
        buffers then hold the exact answer)."""
        r = C.c_int32()
        self._check(lib.phx_corpus_finish(self._h, C.byref(r)))
        return bool(r.value)

    def set_exact(self, on: bool):
        self._check(lib.phx_corpus_set_exact(self._h, int(bool(on))))

    def exact_runs(self) -> int:
        n = C.c_int64()
        self._check(lib.phx_corpus_exact_runs(self._h, C.byref(n)))
        return int(n.value)

    def last_device_ms(self) -> float:
        ms = C.c_float()
        self._check(lib.phx_corpus_last_device_ms(self._h, C.byref(ms)))
        return float(ms.value)


def merge_topk_static(scores, ids, P: int, B: int, k: int, out_scores, out_ids, device: "int | None" = None,
                      stream: "int | None" = None):
    """Merge [P,B,k] per-shard lists into [B,k] without allocating device memory: the scratch is a
    fixed array inside the library (limit P*B*k <= 2,097,152).  For callers whose device memory is
    owned by someone else.  Torch CUDA tensors; asynchronous on `stream` (default: torch's current
    stream of the tensors' device, which is also the default for `device`)."""
    import torch
    if device is None:
        device = scores.device.index if scores.device.index is not None else torch.cuda.current_device()
    if stream is None:
        stream = torch.cuda.current_stream(device).cuda_stream
    st = lib.phx_topk_merge_static(device, int(scores.data_ptr()), int(ids.data_ptr()), P, B, k,
                                   int(out_scores.data_ptr()), int(out_ids.data_ptr()), stream or None)
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())


def merge_topk_static_status(device: int = 0, stream: "int | None" = None) -> int:
    """Wait for `stream` and return the status word of the allocation-free merge (0 = every entry was merged, bit 2 =
    an id did not fit 32 bits and was left out)."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream(device).cuda_stream
    v = C.c_int32()
    st = lib.phx_topk_merge_static_status(device, stream or None, C.byref(v))
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())
    return int(v.value)


class Retriever:
    """User tower -> per-shard top-k -> merge.  With torch.distributed initialised, each rank holds one
    shard and the per-shard lists are merged after an all-gather (the reference's shard-local top-k +
    all_gather + top_k merge, recsys_two_tower_model.py:215-220); otherwise the local shards are merged
    directly."""

    def __init__(self, shards: Sequence[CorpusShard]):
        self.shards = list(shards)

    def retrieve(self, users, k: int, check: bool = True):
        """Top-k rows of the whole corpus for users f32 [B, dim] (CUDA tensor) -> (scores f32 [B,k], rows int64 [B,k]).
        Everything is enqueued on torch's current stream - per-shard top-k as 64-bit keys, one all-gather of those
        keys, the merge - with no host synchronisation in between.  check=True (default) then waits for the shards and,
        if the sampled pivot missed on any shard of any rank, takes that shard's exact list and merges again: the
        answer is always the exhaustive top-k.  check=False returns at once; the caller owns the check
        (CorpusShard.finish) before it trusts the result."""
        import torch
        B = users.shape[0]
        dev = users.device
        P = len(self.shards)
        stream = torch.cuda.current_stream(dev).cuda_stream
        dist = torch.distributed
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        keys = torch.empty((P, B, k), dtype=torch.int64, device=dev)
        out_s = torch.empty((B, k), dtype=torch.float32, device=dev)
        out_i = torch.empty((B, k), dtype=torch.int64, device=dev)
        for sh in self.shards:
            sh.set_stream(stream)

        def gather_and_merge():
            all_keys, n = keys, P
            if multi:
                W = dist.get_world_size()
                all_keys = torch.empty((W * P, B, k), dtype=torch.int64, device=dev)
                dist.all_gather_into_tensor(all_keys, keys)
                n = W * P
            self.shards[0].merge_keys_device(all_keys, n, B, k, out_s, out_i)

        try:
            for p, sh in enumerate(self.shards):
                sh.topk_keys_device(users, B, k, keys[p])
            gather_and_merge()
            if check:
                redo = False
                for sh in self.shards:
                    redo = sh.finish() or redo          # an exact re-run rewrites keys[p] in place
                if multi:
                    flag = torch.tensor([1 if redo else 0], dtype=torch.int32, device=dev)
                    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                    redo = bool(flag.item())
                if redo:
                    gather_and_merge()
                    self.shards[0].sync()
        finally:
            for sh in self.shards:
                sh.set_stream(None)     # back to the shard's own stream: the caller's stream may not outlive this call
        return out_s, out_i

    def user_vector(self, tower, history):
        """The user tower's vector of one history (list of plugin.HistoryItem): f32 [1, D] CUDA tensor."""
        import torch
        cfg = tower.cfg
        S = cfg.history_len
        hist = [h for h in history if h.post_id != 0 and h.author_id != 0][-S:]
        hp = np.zeros((1, S), np.int64); ha = np.zeros((1, S), np.int64)
        act = np.zeros((1, S), np.int32); srf = np.zeros((1, S), np.int32)
        for j, h in enumerate(hist):
            hp[0, j], ha[0, j], act[0, j], srf[0, j] = h.post_id, h.author_id, h.action, h.surface
        dev = torch.device("cuda", tower.device)
        t = [torch.from_numpy(a).to(dev) for a in (hp, ha, act, srf)]
        users = torch.empty((1, cfg.emb_size), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        tower.user_tower_device(1, *t, users)
        tower.sync()
        return users

    def retrieve_for_history(self, tower, history, k: int):
        s, i = self.retrieve(self.user_vector(tower, history), k)
        s, i = s[0].cpu().numpy(), i[0].cpu().numpy()
        for sh in self.shards:
            sh.sync()      # surfaces a device-side error of the scan (bounded wait, survivor overflow) as PhoenixError
        return s, i
