"""Diversity rerank on the GPU (phx_dpp_rescore_device): greedy DPP selection and its sliding-window variant for a
batch of requests, the job of vm-ranker/dpp.rs behind the value model."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

from . import _lib
from ._lib import PhoenixError, lib


@dataclass
class DppConfig:
    """vm-ranker/dpp.rs:14-29."""
    top_k: int = 10
    theta: float = 0.5
    max_selected_rank: int = 50
    greedy_order: bool = False
    window_size: Optional[int] = None        # not None: sliding-window selection
    half_distance: float = 0.0
    sid_lambda: float = 0.0


def dpp_rescore(cfg: DppConfig, scores, embeddings_f16, norms, missing=None, l1=None, num_valid=None, ctx_embeddings_f16=None,
                ctx_norms=None, ctx_missing=None, ctx_l1=None, num_context_valid=None, has_seed: bool = False, stream: int = 0):
    """scores f64 [B,C], embeddings float16 [B,C,E], norms f64 [B,C] (torch CUDA tensors; the optional ones likewise:
    missing uint8, l1 int32, context arrays [B,Hc,...] with the seed first when has_seed).  Returns (index int32
    [B,top_k] of the candidate served at each position, -1 behind the last pick; score f64 [B,top_k]; count int32 [B])."""
    import torch
    B, Cn, E = embeddings_f16.shape
    dev = scores.device
    Hc = 0 if ctx_embeddings_f16 is None else ctx_embeddings_f16.shape[1]
    ccfg = _lib.DppConfig(cfg.top_k, cfg.max_selected_rank, int(cfg.greedy_order), int(cfg.window_size is not None), cfg.theta,
                          min(cfg.window_size if cfg.window_size is not None else 0, 2**31 - 1), 0, cfg.half_distance, cfg.sid_lambda)
    p = lambda t: None if t is None else int(t.data_ptr())
    cin = _lib.DppInputs(B, Cn, E, Hc, p(scores), p(embeddings_f16), p(norms), p(missing), p(l1), p(num_valid), p(ctx_embeddings_f16),
                         p(ctx_norms), p(ctx_missing), p(ctx_l1), p(num_context_valid), int(has_seed), 0)
    idx = torch.empty((B, cfg.top_k), dtype=torch.int32, device=dev)
    sc = torch.empty((B, cfg.top_k), dtype=torch.float64, device=dev)
    cnt = torch.empty((B,), dtype=torch.int32, device=dev)
    st = lib.phx_dpp_rescore_device(dev.index or 0, C.byref(ccfg), C.byref(cin), p(idx), p(sc), p(cnt), stream or None)
    if st != 0:
        raise PhoenixError(st, lib.phx_global_error().decode())
    return idx, sc, cnt
