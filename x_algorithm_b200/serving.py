"""Request queue and admission control of the serving shell over the C ABI (phx_queue_*, phx_admission_*): the duties
of the reference's engine between its wire layer and the dispatch loop (xai-recsys-engine/src/request_queue.rs,
admission.rs)."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

from . import _lib
from ._lib import PhoenixError, lib

NEVER = (1 << 64) - 1


def now_us() -> int:
    return int(lib.phx_now_us())


class RequestQueue:
    """Bounded queue of request ids with staleness / deadline drops (request_queue.rs:29-155)."""

    def __init__(self, batch_size: int, channel_size: int, max_staleness_us: int = NEVER, batch_wait_us: int = 0):
        self.batch_size = batch_size
        self._h = C.c_void_p()
        st = lib.phx_queue_create(batch_size, channel_size, max_staleness_us, batch_wait_us, C.byref(self._h))
        if st != 0:
            raise PhoenixError(st, "phx_queue_create: bad argument")

    def close(self):
        if self._h:
            lib.phx_queue_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def push(self, request_id: int, enqueue_time_us: int, deadline_us: int = 0) -> bool:
        """False when the channel is full (the caller sheds the request)."""
        st = lib.phx_queue_push(self._h, request_id, enqueue_time_us, deadline_us)
        if st not in (0, 5):
            raise PhoenixError(st, "phx_queue_push")
        return st == 0

    def dequeue(self, now: Optional[int] = None) -> Tuple[List[int], List[int]]:
        """(request ids of the next batch in arrival order, ids dropped as stale since the last call)."""
        ids = (C.c_uint64 * self.batch_size)()
        dropped = (C.c_uint64 * 4096)()
        n, nd = C.c_int32(), C.c_int32()
        st = lib.phx_queue_dequeue(self._h, now_us() if now is None else now, ids, self.batch_size, C.byref(n), dropped, 4096,
                                   C.byref(nd))
        if st != 0:
            raise PhoenixError(st, "phx_queue_dequeue")
        return [int(ids[i]) for i in range(n.value)], [int(dropped[i]) for i in range(nd.value)]

    def waiting(self) -> int:
        w = C.c_int32()
        lib.phx_queue_stats(self._h, C.byref(w), None)
        return int(w.value)


class AdmissionController:
    """Deadline-aware admission (admission.rs:44-227)."""

    def __init__(self, enabled: bool = True, batch_size: int = 32, margin_us: int = 0, post_us: int = 0,
                 fallback_budget_us: int = 0, ewma_alpha: float = 0.2, pipeline_depth: int = 0, eta_model: str = "loop"):
        model = {"loop": 0, "python": 0, "pipeline": 1, "rust": 1}.get(eta_model.strip().lower())
        if model is None:
            raise ValueError(f"unknown admission eta model '{eta_model}' (want loop|python or pipeline|rust)")
        self.fallback_budget_us = fallback_budget_us or None
        cfg = _lib.AdmissionConfig(int(enabled), model, batch_size, margin_us, post_us, fallback_budget_us, pipeline_depth, ewma_alpha)
        self._h = C.c_void_p()
        st = lib.phx_admission_create(C.byref(cfg), C.byref(self._h))
        if st != 0:
            raise PhoenixError(st, "phx_admission_create: bad argument")

    def close(self):
        if self._h:
            lib.phx_admission_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_enabled(self, on: bool):
        lib.phx_admission_set_enabled(self._h, int(on))

    def reset_estimates(self):
        lib.phx_admission_reset(self._h)

    def record_service_time_us(self, sample_us: int):
        lib.phx_admission_record_service_us(self._h, sample_us)

    def record_sojourn_us(self, sample_us: int, admit_backlog: int):
        lib.phx_admission_record_sojourn_us(self._h, sample_us, admit_backlog)

    def predicted_eta_us(self, queue_depth: int, model: Optional[str] = None) -> Optional[int]:
        eta = C.c_uint64()
        m = -1 if model is None else {"loop": 0, "pipeline": 1}[model]
        return int(eta.value) if lib.phx_admission_predicted_eta_us(self._h, queue_depth, m, C.byref(eta)) else None

    def should_reject(self, remaining_us: Optional[int], queue_depth: int) -> bool:
        return bool(lib.phx_admission_should_reject(self._h, -1 if remaining_us is None else remaining_us, queue_depth))

    def service_time_us(self) -> int:
        s = C.c_uint64()
        lib.phx_admission_estimates(self._h, C.byref(s), None)
        return int(s.value)

    def pipeline_time_us(self) -> int:
        p = C.c_uint64()
        lib.phx_admission_estimates(self._h, None, C.byref(p))
        return int(p.value)
