"""Generate golden fixtures by EXECUTING reference functions (run once, in a container that has
the reference checkout; the resulting .npz files are committed and the GPU box never needs the
reference).

    python tests/golden/gen_golden.py /path/to/reference

The reference's model modules import jax/haiku, which are not installed, so whole modules cannot
be imported.  Instead the source text of individual pure functions is cut out of the reference
files with `ast` and executed unchanged:
  * `_hash_ids_batch` runs under numba exactly as in the reference (it only needs numpy+numba);
  * the jnp-only helpers (rope_angles, apply_rope, rotate_half, rms_normalize, _split_merged_qkv,
    attention_segment_ids, history_candidate_mask) and the reference's own plain candidate-isolation
    attention (`attention_reference` with `_apply_cap`, `tanh`, `_abs` of
    pallas/ranker_attention_fa3.py) run with a small NumPy stand-in for the `jnp` / `jax.lax` names
    they use.  The arithmetic library is therefore NumPy, not XLA; the
    control flow, constants and operation order are the reference's own.
Nothing from the reference is copied into this repository; only inputs and outputs are stored.
"""
from __future__ import annotations

import ast
import os
import sys
import types

import numpy as np


def cut(path: str, names):
    src = open(path).read()
    tree = ast.parse(src)
    out = {}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = [d for d in node.decorator_list if "njit" in ast.unparse(d)]
            out[node.name] = ast.unparse(node)
    missing = set(names) - set(out)
    assert not missing, f"{path}: missing {missing}"
    return out


class _Lax:
    @staticmethod
    def rsqrt(x):
        return (np.float32(1.0) / np.sqrt(x)).astype(np.float32)

    @staticmethod
    def logistic(x):
        x = np.asarray(x)
        return (1.0 / (1.0 + np.exp(-x))).astype(x.dtype)

    @staticmethod
    def broadcasted_iota(dtype, shape, dim):
        return np.broadcast_to(np.arange(shape[dim], dtype=dtype).reshape([-1 if i == dim else 1 for i in range(len(shape))]), shape)


def _jnp():
    m = types.SimpleNamespace()
    for k in ("arange", "asarray", "einsum", "tile", "split", "concatenate", "mean", "square", "where",
              "broadcast_to", "logical_or", "logical_not", "float32", "int32", "bfloat16", "ndarray", "any", "exp",
              "inf", "log2", "abs", "tanh"):
        if hasattr(np, k):
            setattr(m, k, getattr(np, k))
    return m


def main(ref: str, outdir: str):
    models = os.path.join(ref, "phoenix/xrex/models")
    rng = np.random.Generator(np.random.PCG64(1234))

    # ---- hashing: the reference function itself, under numba --------------------------------
    import numba

    ns = {"np": np, "numba": numba}
    exec(cut(os.path.join(models, "recsys_embedding.py"), ["_hash_ids_batch"])["_hash_ids_batch"], ns)
    fn = ns["_hash_ids_batch"]
    ids = np.concatenate([
        np.array([0, 1, 2, 42, -1, -5, 999_999_937, 1_780_416_091_123_456_789,
                  np.iinfo(np.int64).max, np.iinfo(np.int64).min, (1 << 40) - 1, 1 << 40], dtype=np.int64),
        rng.integers(1, 1 << 40, size=2000, dtype=np.int64),
        rng.integers(np.iinfo(np.int64).min, np.iinfo(np.int64).max, size=500, dtype=np.int64),
    ])
    fams = {  # (scales, biases, modulus) = HashKeys defaults; several bucket counts
        "user": ([196742702, 1852108266], [1935840681, 167407236], 2_859_568_897),
        "item": ([2161410491, 1754358832], [1935840681, 167407236], 2_361_375_383),
        "author": ([371965780, 328930218], [139686260, 37755056], 631_860_353),
        "ip": ([529_482_163, 1_327_604_891], [742_961_053, 318_205_477], 1_073_741_789),
        "item4": ([2161410491, 1754358832, 371965780, 328930218], [1935840681, 167407236, 139686260, 37755056], 2_361_375_383),
    }
    hash_out = {"ids": ids}
    for name, (sc, bi, mod) in fams.items():
        for buckets in (100_000, 1 << 17, 1 << 22, 1 << 24):
            res = fn(ids, np.array(sc, dtype=np.int64), np.array(bi, dtype=np.int64), mod, buckets)
            hash_out[f"{name}_{buckets}"] = res
            hash_out[f"{name}_{buckets}_params"] = np.array(sc + bi + [mod, buckets], dtype=np.int64)
    np.savez_compressed(os.path.join(outdir, "hash_golden.npz"), **hash_out)

    # ---- jnp-only helpers with a NumPy stand-in ----------------------------------------------
    jnp = _jnp()
    jax = types.SimpleNamespace(Array=np.ndarray, lax=_Lax, numpy=jnp)
    base = {"jnp": jnp, "jax": jax, "lax": _Lax, "np": np, "Optional": __import__("typing").Optional,
            "Callable": __import__("typing").Callable, "checkpoint_name": lambda x, n: x}
    ns = dict(base)
    for s in cut(os.path.join(models, "layers.py"), ["rope_angles", "apply_rope", "rotate_half", "_split_merged_qkv"]).values():
        exec("from __future__ import annotations\n" + s, ns)
    for s in cut(os.path.join(models, "normalization.py"), ["rms_normalize"]).values():
        exec("from __future__ import annotations\n" + s, ns)
    for s in cut(os.path.join(models, "recsys_model.py"), ["attention_segment_ids"]).values():
        exec("from __future__ import annotations\n" + s, ns)
    for s in cut(os.path.join(ref, "phoenix/xrex/pallas/ranker_attention_utils.py"), ["history_candidate_mask"]).values():
        exec("from __future__ import annotations\n" + s, ns)

    B, T, H, dh = 2, 12, 3, 16
    pos = np.concatenate([np.arange(8), np.full(4, 8)]).astype(np.float32)[None].repeat(B, 0)
    ang = ns["rope_angles"](dh, 10000, T, pos)
    xq = rng.standard_normal((B, T, H, dh), dtype=np.float32)
    roped = ns["apply_rope"](xq, np.cos(ang), np.sin(ang))
    xin = rng.standard_normal((B, T, 40), dtype=np.float32) * 3
    gain = (1 + 0.1 * rng.standard_normal(40, dtype=np.float32)).astype(np.float32)
    normed = ns["rms_normalize"](xin, gain, 1e-5)
    qkv = rng.standard_normal((B, T, 2, 4, dh), dtype=np.float32)  # Hkv=2, g=2
    q, k, v = ns["_split_merged_qkv"](qkv)
    pad = rng.random((3, 16)) > 0.3
    seg = ns["attention_segment_ids"](pad, 10, False)
    # mask: history [0,5), candidates [8,14) inside a 16x16 window
    hmask = ns["history_candidate_mask"](0, 16, 0, 16, 0, 5, 8, 14)
    np.savez_compressed(
        os.path.join(outdir, "elementwise_golden.npz"),
        rope_pos=pos, rope_angles=ang, rope_x=xq, rope_out=roped,
        rms_x=xin, rms_gain=gain, rms_out=normed,
        qkv=qkv, q=q, k=k, v=v, pad=pad, seg=seg, hmask=hmask,
    )

    # ---- the reference's plain candidate-isolation attention (pallas/ranker_attention_fa3.py:1185-1236) ----------
    import math
    ns_a = dict(base)
    ns_a.update(math=math, Tuple=__import__("typing").Tuple,
                ranker_attention_utils=types.SimpleNamespace(history_candidate_mask=ns["history_candidate_mask"]))
    for name, src in cut(os.path.join(ref, "phoenix/xrex/pallas/ranker_attention_fa3.py"),
                         ["tanh", "_abs", "_apply_cap", "attention_reference"]).items():
        exec("from __future__ import annotations\n" + src, ns_a)
    att = {}
    cases = [  # (name, B, T, Hq, Hkv, dh, bound, cap, cap_method)
        ("full", 2, 40, 4, 4, 32, (0, 32, 32, 40), -1.0, "tanh"),
        ("ragged", 2, 48, 4, 2, 32, (0, 19, 32, 43), -1.0, "tanh"),       # padded history tail and padded candidates, GQA
        ("offset", 1, 40, 2, 2, 64, (3, 30, 33, 40), 20.0, "soft_sign"),  # history not starting at 0, soft-sign cap
        ("tanhcap", 2, 24, 2, 1, 32, (0, 16, 16, 24), 15.0, "tanh"),
    ]
    for name, B_, T_, Hq_, Hkv_, dh_, bound, cap, method in cases:
        q_ = (rng.standard_normal((B_, T_, Hq_, dh_), dtype=np.float32) * 1.5).astype(np.float32)
        k_ = (rng.standard_normal((B_, T_, Hkv_, dh_), dtype=np.float32) * 1.5).astype(np.float32)
        v_ = rng.standard_normal((B_, T_, Hkv_, dh_), dtype=np.float32)
        sm = math.sqrt(128.0) / dh_
        o_ = ns_a["attention_reference"](q_, k_, v_, bound=bound, sm_scale=sm, cap=cap, cap_method=method)
        att.update({f"{name}_q": q_, f"{name}_k": k_, f"{name}_v": v_, f"{name}_out": np.asarray(o_, dtype=np.float32),
                    f"{name}_bound": np.array(bound, dtype=np.int32),
                    f"{name}_params": np.array([sm, cap, 1.0 if method == "tanh" else 0.0], dtype=np.float64)})
    np.savez_compressed(os.path.join(outdir, "attention_golden.npz"), **att)
    print("wrote", outdir)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/gen_golden.py <path to a checkout of xai-org/x-algorithm>")
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
