"""Python face of the engine: owns a phx_engine handle and moves numpy / torch buffers through the
C ABI.  Mirrors the model runner's per-batch sequence (phoenix/xrex/inference/model_runner.py:4141-4222):
featurised ids in, log-probabilities / continuous predictions / weighted scores out."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np

from . import _lib
from ._lib import PhoenixError, lib
from .config import PhoenixConfig


@dataclass
class RankInputs:
    """One batch of requests (id 0 = padding, history front-filled): the buffers of the reference's
    RankingBatchPrep (xai-recsys-engine/src/python.rs:1394-1440) with raw ids instead of hashes."""
    hist_post_ids: np.ndarray      # int64 [B,S]
    hist_author_ids: np.ndarray    # int64 [B,S]
    hist_actions: np.ndarray       # int32 [B,S]
    hist_surfaces: np.ndarray      # int32 [B,S]
    cand_post_ids: np.ndarray      # int64 [B,C]
    cand_author_ids: np.ndarray    # int64 [B,C]

    @property
    def batch(self) -> int:
        return int(self.hist_post_ids.shape[0])


@dataclass
class RankOutputs:
    log_probs: np.ndarray    # f32 [B,C,V]
    continuous: np.ndarray   # f32 [B,C,NC]
    scores: Optional[np.ndarray]  # f64 [B,C] or None when no blend is set


def _ptr(a) -> int:
    if a is None:
        return 0
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return int(a.data_ptr())  # torch tensor


class PhoenixEngine:
    def __init__(self, cfg: PhoenixConfig, device: int = 0):
        self.cfg = cfg
        self.device = device
        self._h = C.c_void_p()
        self._ccfg = cfg.to_c()
        st = lib.phx_engine_create(C.byref(self._ccfg), device, C.byref(self._h))
        if st != 0:
            raise PhoenixError(st, lib.phx_global_error().decode())
        self._has_blend = False

    # -- plumbing ------------------------------------------------------------------------------
    def _check(self, st: int):
        if st != 0:
            raise PhoenixError(st, lib.phx_last_error(self._h).decode())

    def close(self):
        if self._h:
            lib.phx_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- parameters ----------------------------------------------------------------------------
    def load_weights(self, weights: Dict[str, np.ndarray]):
        for name, arr in weights.items():
            a = np.ascontiguousarray(arr, dtype=np.float32)
            rows, cols = (1, a.shape[0]) if a.ndim == 1 else a.shape
            self._check(lib.phx_load_param(self._h, name.encode(), a.ctypes.data, rows, cols))

    def table_upload(self, row0: int, rows_bf16_bits: np.ndarray):
        a = np.ascontiguousarray(rows_bf16_bits, dtype=np.uint16)
        self._check(lib.phx_table_upload(self._h, row0, a.shape[0], a.ctypes.data))

    def table_fill_synthetic(self, seed: int, amp: float):
        self._check(lib.phx_table_fill_synthetic(self._h, seed, amp))

    # -- row-sharded table: export this engine's shard / map the others ---------------------------
    def table_ipc_handle(self) -> bytes:
        buf = (C.c_uint8 * 64)()
        self._check(lib.phx_table_ipc_handle(self._h, buf))
        return bytes(buf)

    def table_attach_peer(self, rank: int, handle: bytes):
        buf = (C.c_uint8 * 64).from_buffer_copy(handle)
        self._check(lib.phx_table_attach_peer(self._h, rank, buf))

    def table_local_ptr(self) -> int:
        p = C.c_void_p()
        self._check(lib.phx_table_local_ptr(self._h, C.byref(p)))
        return int(p.value)

    def table_attach_peer_ptr(self, rank: int, ptr: int):
        self._check(lib.phx_table_attach_peer_ptr(self._h, rank, ptr))

    def set_blend(self, spec: _lib.BlendSpec):
        self._check(lib.phx_set_blend(self._h, C.byref(spec)))
        self._has_blend = True

    # -- ranking ---------------------------------------------------------------------------------
    def _batch_struct(self, B, hp, ha, act, srf, cp, ca) -> _lib.RankBatch:
        b = _lib.RankBatch()
        b.batch = B
        b.hist_post_ids, b.hist_author_ids, b.hist_actions, b.hist_surfaces = _ptr(hp), _ptr(ha), _ptr(act), _ptr(srf)
        b.cand_post_ids, b.cand_author_ids = _ptr(cp), _ptr(ca)
        return b

    def rank(self, inp: RankInputs, out: "RankOutputs | None" = None) -> RankOutputs:
        """Host buffers in, host buffers out (copies inside the call).  `out`: a RankOutputs of an earlier call with
        the same batch size to write into (a server reuses its result buffers; fresh 10 MB arrays cost a page fault
        per 4 KB on every call)."""
        cfg, B = self.cfg, inp.batch
        arrs = [np.ascontiguousarray(inp.hist_post_ids, np.int64), np.ascontiguousarray(inp.hist_author_ids, np.int64),
                np.ascontiguousarray(inp.hist_actions, np.int32), np.ascontiguousarray(inp.hist_surfaces, np.int32),
                np.ascontiguousarray(inp.cand_post_ids, np.int64), np.ascontiguousarray(inp.cand_author_ids, np.int64)]
        assert arrs[0].shape == (B, cfg.history_len) and arrs[4].shape == (B, cfg.num_candidates)
        if out is not None and out.log_probs.shape == (B, cfg.num_candidates, cfg.num_actions):
            lp, cont, sc = out.log_probs, out.continuous, out.scores
            if self._has_blend and sc is None:
                sc = np.empty((B, cfg.num_candidates), np.float64)
        else:
            lp = np.empty((B, cfg.num_candidates, cfg.num_actions), np.float32)
            cont = np.empty((B, cfg.num_candidates, cfg.num_continuous), np.float32)
            sc = np.empty((B, cfg.num_candidates), np.float64) if self._has_blend else None
        b = self._batch_struct(B, *arrs)
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward(self._h, C.byref(b), C.byref(o)))
        return RankOutputs(lp, cont, sc)

    def rank_hashed(self, hist_post_hashes, hist_author_hashes, hist_actions, hist_surfaces, cand_post_hashes,
                    cand_author_hashes) -> RankOutputs:
        """The forward from the reference batch-prep's own buffers (xai-recsys-engine/src/python.rs:1394-1440):
        int32 unified-table rows [B,S,H] / [B,C,H], already hashed on the host; host arrays in and out."""
        cfg = self.cfg
        arrs = [np.ascontiguousarray(a, np.int32) for a in (hist_post_hashes, hist_author_hashes, hist_actions,
                                                             hist_surfaces, cand_post_hashes, cand_author_hashes)]
        B = arrs[0].shape[0]
        assert arrs[0].shape == (B, cfg.history_len, cfg.num_hashes) and arrs[4].shape == (B, cfg.num_candidates, cfg.num_hashes)
        lp = np.empty((B, cfg.num_candidates, cfg.num_actions), np.float32)
        cont = np.empty((B, cfg.num_candidates, cfg.num_continuous), np.float32)
        sc = np.empty((B, cfg.num_candidates), np.float64) if self._has_blend else None
        b = self._batch_struct(B, *arrs)
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_hashed(self._h, C.byref(b), C.byref(o)))
        return RankOutputs(lp, cont, sc)

    def rank_hashed_device(self, B, hp, ha, act, srf, cp, ca, lp, cont, sc=None):
        """Same with device tensors (int32 rows), asynchronous on the engine's stream."""
        b = self._batch_struct(B, hp, ha, act, srf, cp, ca)
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_hashed_device(self._h, C.byref(b), C.byref(o)))

    _PREP_FIELDS = (("user_hashes", np.int32), ("user_ip_hashes", np.int32), ("history_post_hashes", np.int32),
                    ("history_auth_hashes", np.int32), ("history_product_surfaces", np.int32), ("history_actions", np.bool_),
                    ("history_continuous_actions", np.float32), ("candidate_post_hashes", np.int32),
                    ("candidate_auth_hashes", np.int32), ("candidate_product_surfaces", np.int32))

    def rank_prep(self, prep) -> RankOutputs:
        """The forward over the mandatory buffers of the reference's batch-prep, under its attribute names
        (RankingBatchPrep, xai-recsys-engine/src/python.rs:1394-1404): `prep` is any object with those attributes as
        host arrays - user_hashes i32 [B,Hu], user_ip_hashes i32 [B,Hip] (or None), history_post_hashes /
        history_auth_hashes i32 [B,S,H], history_product_surfaces i32 [B,S], history_actions bool [B,S,V],
        history_continuous_actions f32 [B,S,8], candidate_post_hashes / candidate_auth_hashes i32 [B,C,H],
        candidate_product_surfaces i32 [B,C].  Which of them are read follows the engine's configuration."""
        cfg = self.cfg
        b = _lib.RankBatchPrep()
        keep = []
        for name, dt in self._PREP_FIELDS:
            a = getattr(prep, name, None)
            if a is None:
                continue
            a = np.ascontiguousarray(a, dt)
            keep.append(a)
            setattr(b, name, a.ctypes.data)
        hp = np.asarray(prep.history_post_hashes)
        B = hp.shape[0]
        assert hp.shape == (B, cfg.history_len, cfg.num_hashes)
        assert np.asarray(prep.history_actions).shape == (B, cfg.history_len, cfg.num_action_types)
        assert np.asarray(prep.candidate_post_hashes).shape == (B, cfg.num_candidates, cfg.num_hashes)
        b.batch = B
        lp = np.empty((B, cfg.num_candidates, cfg.num_actions), np.float32)
        cont = np.empty((B, cfg.num_candidates, cfg.num_continuous), np.float32)
        sc = np.empty((B, cfg.num_candidates), np.float64) if self._has_blend else None
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_prep(self._h, C.byref(b), C.byref(o)))
        return RankOutputs(lp, cont, sc)

    def rank_prep_device(self, B: int, prep, lp, cont, sc=None):
        """Same with device tensors as the attributes of `prep` (history_actions as a uint8 / bool tensor), asynchronous on
        the engine's stream."""
        b = _lib.RankBatchPrep()
        b.batch = B
        for name, _ in self._PREP_FIELDS:
            a = getattr(prep, name, None)
            if a is not None:
                setattr(b, name, _ptr(a))
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_prep_device(self._h, C.byref(b), C.byref(o)))

    def rank_submit(self, inp: RankInputs, slot: int) -> None:
        """Start a host-buffer request in pipeline slot 0 or 1 and return at once (the inputs are copied before the
        call returns).  `rank_collect(slot)` delivers its results; with both slots in flight the host-side copies of
        one request overlap the forward of the other."""
        cfg, B = self.cfg, inp.batch
        arrs = [np.ascontiguousarray(inp.hist_post_ids, np.int64), np.ascontiguousarray(inp.hist_author_ids, np.int64),
                np.ascontiguousarray(inp.hist_actions, np.int32), np.ascontiguousarray(inp.hist_surfaces, np.int32),
                np.ascontiguousarray(inp.cand_post_ids, np.int64), np.ascontiguousarray(inp.cand_author_ids, np.int64)]
        assert arrs[0].shape == (B, cfg.history_len) and arrs[4].shape == (B, cfg.num_candidates)
        b = self._batch_struct(B, *arrs)
        self._check(lib.phx_rank_submit(self._h, C.byref(b), slot))
        self._slot_batch = getattr(self, "_slot_batch", {})
        self._slot_batch[slot] = B

    def rank_collect(self, slot: int, out: "RankOutputs | None" = None) -> RankOutputs:
        """Wait for the request submitted to `slot` and return its results (into `out` when given)."""
        cfg = self.cfg
        B = getattr(self, "_slot_batch", {}).get(slot)
        if B is None:
            raise PhoenixError(6, "rank_collect: nothing was submitted to this slot")
        if out is not None and out.log_probs.shape == (B, cfg.num_candidates, cfg.num_actions):
            lp, cont, sc = out.log_probs, out.continuous, out.scores
            if self._has_blend and sc is None:
                sc = np.empty((B, cfg.num_candidates), np.float64)
        else:
            lp = np.empty((B, cfg.num_candidates, cfg.num_actions), np.float32)
            cont = np.empty((B, cfg.num_candidates, cfg.num_continuous), np.float32)
            sc = np.empty((B, cfg.num_candidates), np.float64) if self._has_blend else None
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_collect(self._h, slot, C.byref(o)))
        del self._slot_batch[slot]
        return RankOutputs(lp, cont, sc)

    def rank_device(self, B, hp, ha, act, srf, cp, ca, lp, cont, sc=None):
        """Device tensors (torch) in and out; asynchronous on the engine's stream."""
        b = self._batch_struct(B, hp, ha, act, srf, cp, ca)
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_device(self._h, C.byref(b), C.byref(o)))

    def rank_packed_device(self, B, hp, ha, act, srf, cp, ca, hist_off, cand_off, hist_rows: int, cand_rows: int, lp, cont, sc=None):
        """rank_device over the valid rows only (pack_ragged engines): hist_off / cand_off are int32 CUDA tensors
        [B + 1] as `plan_ragged` makes them, hist_rows / cand_rows their last entries."""
        b = self._batch_struct(B, hp, ha, act, srf, cp, ca)
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_packed_device(self._h, C.byref(b), _ptr(hist_off), _ptr(cand_off), hist_rows,
                                                       cand_rows, C.byref(o)))

    def rank_rows_device(self, B, hp, ha, act, srf, cp, ca, rows, stream=None):
        """Unified-table rows of every token slot of the batch (int32 [B, S+C, 2*num_hashes]) -> `rows`; the first
        half of a forward whose rows are exchanged between ranks (parallel.ShardedRanker)."""
        b = self._batch_struct(B, hp, ha, act, srf, cp, ca)
        self._check(lib.phx_rank_rows_device(self._h, C.byref(b), _ptr(rows), stream))

    def rank_forward_rows_device(self, B, hp, ha, act, srf, cp, ca, landing_ptr, pos, lp, cont, sc=None):
        """The forward with slot j of token t taken from row pos[t * 2*num_hashes + j] of the landing buffer at device
        address `landing_ptr` instead of the table."""
        b = self._batch_struct(B, hp, ha, act, srf, cp, ca)
        o = _lib.RankOut(_ptr(lp), _ptr(cont), _ptr(sc))
        self._check(lib.phx_rank_forward_rows_device(self._h, C.byref(b), landing_ptr, _ptr(pos), C.byref(o)))

    def rank_prefetch_device(self, B, hp, ha, act, srf, cp, ca):
        """Build the tokens of the batch the next rank_device call will carry, on a side stream (overlaps the
        forward enqueued right after this call; matters when the table is row-sharded over GPUs)."""
        b = self._batch_struct(B, hp, ha, act, srf, cp, ca)
        self._check(lib.phx_rank_prefetch_device(self._h, C.byref(b)))

    def user_tower_device(self, B, hp, ha, act, srf, users):
        b = self._batch_struct(B, hp, ha, act, srf, None, None)
        self._check(lib.phx_user_tower_device(self._h, C.byref(b), _ptr(users)))

    def sync(self):
        self._check(lib.phx_sync(self._h))

    def set_wait_limit_us(self, microseconds: int):
        """Limit of every bounded device-side wait of this engine's kernels (0 = the 2 s default)."""
        self._check(lib.phx_set_wait_limit_us(self._h, int(microseconds)))

    def wait_selftest(self):
        """Let one device-side wait run out: raises PhoenixError(PHX_E_TIMEOUT) when the mechanism works."""
        self._check(lib.phx_wait_selftest(self._h))

    def last_device_ms(self) -> float:
        ms = C.c_float()
        self._check(lib.phx_last_device_ms(self._h, C.byref(ms)))
        return float(ms.value)

    def last_launch_count(self) -> int:
        n = C.c_int32()
        self._check(lib.phx_last_launch_count(self._h, C.byref(n)))
        return int(n.value)

    def mark(self, slot: int):
        self._check(lib.phx_mark(self._h, slot))

    def mark_wait(self, slot: int):
        self._check(lib.phx_mark_wait(self._h, slot))

    def elapsed_ms(self, a: int, b: int) -> float:
        ms = C.c_float()
        self._check(lib.phx_elapsed_ms(self._h, a, b, C.byref(ms)))
        return float(ms.value)

    KERNEL_CLASSES = ("tokens", "rmsnorm", "gemm", "qknorm_rope", "attention", "heads")

    def profile_enable(self, on: bool):
        self._check(lib.phx_profile_enable(self._h, int(on)))

    def profile_read(self):
        ms = (C.c_float * 6)()
        n = (C.c_int32 * 6)()
        self._check(lib.phx_profile_read(self._h, ms, n))
        return {k: (float(ms[i]), int(n[i])) for i, k in enumerate(self.KERNEL_CLASSES)}

    def debug_read(self, what: str, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype)
        self._check(lib.phx_debug_read(self._h, what.encode(), out.ctypes.data, out.nbytes))
        return out

    # -- stand-alone operators ---------------------------------------------------------------------
    def hash_ids_device(self, family: int, ids, n: int, out):
        self._check(lib.phx_hash_ids_device(self._h, family, _ptr(ids), n, _ptr(out)))

    def gather_sum_device(self, family: int, ids, n: int, out):
        self._check(lib.phx_gather_sum_device(self._h, family, _ptr(ids), n, _ptr(out)))


def dispatch_counts() -> Dict[str, int]:
    """Launch counts by kernel variant over the life of the process (phx_dispatch_counts)."""
    n = lib.phx_dispatch_counts(None, 0)
    buf = (C.c_int64 * n)()
    lib.phx_dispatch_counts(buf, n)
    return {lib.phx_dispatch_name(i).decode(): int(buf[i]) for i in range(n)}


def ranker_attention(q, k, v, seg, hist_len: int, sm_scale: float, cap: float = -1.0, cap_method: int = 0,
                     device: int = 0):
    """Candidate-isolated attention on torch bf16 tensors [B,T,H,dh]; returns (out, device_ms)."""
    import torch
    B, T, Hq, dh = q.shape
    out = torch.empty_like(q)
    ms = C.c_float()
    torch.cuda.synchronize()
    st = lib.phx_ranker_attention_device(device, _ptr(q), _ptr(k), _ptr(v), _ptr(seg), _ptr(out), B, T, Hq,
                                         k.shape[2], dh, hist_len, sm_scale, cap, cap_method, C.byref(ms))
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())
    return out, float(ms.value)


def gemm(a, wt, residual=None, epilogue: int = 0, impl: int = 0, device: int = 0):
    """epilogue(A[M,K] @ Wt[N,K]^T) on torch bf16 tensors; returns (C, device_ms)."""
    import torch
    M, K = a.shape
    N = wt.shape[0]
    c = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    ms = C.c_float()
    torch.cuda.synchronize()
    st = lib.phx_gemm_device(device, _ptr(a), _ptr(wt), _ptr(residual), _ptr(c), M, N, K, epilogue, impl, C.byref(ms))
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())
    return c, float(ms.value)


def plan_ragged(hist_post_ids: np.ndarray, cand_post_ids: np.ndarray):
    """Offsets of the packed rows of a batch (host arrays int64 [B,S] / [B,C], 0 = padding): exclusive prefix sums
    (hist_off, cand_off), int32 [B + 1] each, of every request's leading non-padding slots; at least one history row
    per request; all slots when a request has padding in front of a valid slot.  No GPU involved."""
    hp = np.ascontiguousarray(hist_post_ids, np.int64)
    cp = np.ascontiguousarray(cand_post_ids, np.int64)
    B, S = hp.shape
    ho = np.zeros(B + 1, np.int32); co = np.zeros(B + 1, np.int32)
    st = lib.phx_plan_ragged(hp.ctypes.data, cp.ctypes.data, B, S, cp.shape[1], ho.ctypes.data, co.ctypes.data)
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())
    return ho, co
