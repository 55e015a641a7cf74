"""Golden fixtures for the COMPOSED model, made by EXECUTING the reference's own class bodies.

    python tests/golden/gen_golden_model.py /path/to/reference      ->  tests/golden/model_golden.npz

The reference's modules import jax / haiku / chex, which are not installed, so whole modules cannot be
imported.  As in gen_golden.py the source text of single definitions is cut out of the reference files with
`ast` and executed unchanged, here whole classes:

  transformer.py     DecoderLayer, MHABlock, FFNLayer, DenseBlock, FeedForwardConfig   (how a layer is wired)
  layers.py          MultiHeadAttention, Linear, rope_angles, apply_rope, rotate_half, _split_merged_qkv
  linear_layer.py    LinearImpl, LinearConfig
  normalization.py   RMSNorm, rms_normalize, qk_norm, all_heads_qk_norm
  scaling.py         ScaleConfig                                                         (input / output / attention scales)
  utils/utils.py     ffn_size, gelu_fn, remat_less
  recsys_model.py    decode, decode_continuous, _apply_activation, _rescale_sigmoid_heads_for_inference
  recsys_two_tower_model.py   strided_dataset_top_k, and the pooling lines of user_representation
  pallas/ranker_attention_fa3.py   attention_reference (the reference's plain candidate-isolation attention)

What stands in for the libraries: `jnp` / `jax.lax` / `jax.nn` are NumPy functions (the arithmetic library is NumPy,
not XLA; control flow, constants, operation order and dtype casts are the reference's own); `hk.Module` is a plain
base class whose `get_parameter` hands back arrays supplied by this script, keyed by the module's name; sharding
helpers are identities; the attention class the layer dispatches to calls `attention_reference` with the arguments
the reference's own wrapper builds (recsys_attention.py:36-66).  Nothing of the reference is stored: inputs,
parameters and outputs only.
"""
from __future__ import annotations

import ast
import dataclasses
import math
import os
import sys
import types
import typing

import numpy as np


def cut(path: str, names, methods_of: str | None = None):
    """Source text of top-level functions / classes `names` of a file (decorators kept), or of the methods `names` of
    the class `methods_of` as plain functions."""
    tree = ast.parse(open(path).read())
    body = tree.body
    if methods_of:
        body = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == methods_of).body
    out = {}
    for node in body:
        if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in names:
            if methods_of or isinstance(node, ast.FunctionDef):
                node.decorator_list = []        # jit / remat wrappers of free functions; class decorators are kept
            out[node.name] = ast.unparse(node)
    missing = set(names) - set(out)
    assert not missing, f"{path}: missing {missing}"
    return [out[n] for n in names]


# ---- NumPy standing in for jax.numpy / jax.lax / jax.nn ---------------------------------------------------------------

class JArr(np.ndarray):
    """ndarray with the functional update `x.at[idx].set(v)`."""

    @property
    def at(self):
        arr = self

        class _At:
            def __getitem__(self, idx):
                class _Set:
                    def set(self, v):
                        out = np.array(arr).view(JArr)
                        out[idx] = v
                        return out
                return _Set()
        return _At()


def jarr(x):
    return np.asarray(x).view(JArr)


def _top_k(x, k):
    """jax.lax.top_k: largest first, equal values in index order."""
    x = np.asarray(x)
    idx = np.arange(x.shape[-1])
    order = np.stack([np.lexsort((idx, -row.astype(np.float64)))[:k] for row in x.reshape(-1, x.shape[-1])])
    order = order.reshape(*x.shape[:-1], k)
    return np.take_along_axis(x, order, axis=-1), order.astype(np.int32)


def _gelu(x, approximate=True):
    x = np.asarray(x)
    assert approximate
    c = np.float32(math.sqrt(2.0 / math.pi))
    return (np.float32(0.5) * x * (np.float32(1.0) + np.tanh(c * (x + np.float32(0.044715) * x * x * x)))).astype(x.dtype)


def _sigmoid(x):
    x = np.asarray(x)
    return (1.0 / (1.0 + np.exp(-x))).astype(x.dtype)


def _softplus(x):
    x = np.asarray(x)
    return np.logaddexp(x, 0).astype(x.dtype)


def make_jax():
    jnp = types.SimpleNamespace()
    for k in ("arange", "asarray", "array", "einsum", "tile", "split", "concatenate", "mean", "square", "where", "broadcast_to",
              "logical_or", "logical_not", "float32", "int32", "ndarray", "any", "exp", "inf", "log2", "abs", "tanh",
              "reshape", "dot", "ones", "zeros", "cos", "sin", "sqrt", "maximum", "minimum", "sum", "cumsum", "full",
              "take_along_axis", "isin", "bool_", "finfo", "power", "repeat", "expand_dims", "clip", "log1p"):
        setattr(jnp, k, getattr(np, k))
    jnp.bfloat16 = np.float32      # parameters are supplied bf16-representable; activations run in float32 here
    lax = types.SimpleNamespace(
        rsqrt=lambda x: (np.float32(1.0) / np.sqrt(x)).astype(np.float32),
        top_k=_top_k,
        dynamic_slice_in_dim=lambda x, start, size, axis=0: np.take(x, np.arange(int(start), int(start) + size), axis=axis),
        logistic=_sigmoid,
        broadcasted_iota=lambda dtype, shape, dim: np.broadcast_to(
            np.arange(shape[dim], dtype=dtype).reshape([-1 if i == dim else 1 for i in range(len(shape))]), shape),
    )

    class _Scope:
        def __init__(self, *a, **k): pass
        def __enter__(self): return self
        def __exit__(self, *a): return False

    jax = types.SimpleNamespace(
        Array=np.ndarray, numpy=jnp, lax=lax, named_scope=_Scope,
        nn=types.SimpleNamespace(gelu=_gelu, sigmoid=_sigmoid, softplus=_softplus),
        tree=types.SimpleNamespace(map=lambda f, t: tuple(f(x) for x in t)),
    )
    return jax, jnp, lax, _Scope


# ---- haiku stand-in: modules with names, parameters looked up by "<module name>/<parameter name>" -----------------------

class ParamStore:
    def __init__(self):
        self.params: dict[str, np.ndarray] = {}
        self.stack: list[str] = []
        self.asked: list[str] = []

    def get(self, name, shape, dtype=None, init=None, **kw):
        key = (self.stack[-1] + "/" if self.stack and self.stack[-1] else "") + name
        self.asked.append(key)
        p = self.params[key]
        assert tuple(p.shape) == tuple(shape), (key, p.shape, shape)
        return jarr(p.astype(np.float32))


def make_hk(store: ParamStore):
    class Module:
        def __init__(self, name=None):
            self.name = name

        def __init_subclass__(cls, **kw):
            super().__init_subclass__(**kw)
            call = cls.__dict__.get("__call__")
            if call is not None and not getattr(call, "_transparent", False):
                def wrapped(self, *a, _call=call, **k):
                    store.stack.append(getattr(self, "name", None) or "")
                    try:
                        return _call(self, *a, **k)
                    finally:
                        store.stack.pop()
                cls.__call__ = wrapped

    def transparent(f):
        f._transparent = True
        return f

    init = types.SimpleNamespace(VarianceScaling=lambda *a, **k: None, TruncatedNormal=lambda *a, **k: None, Initializer=object)
    return types.SimpleNamespace(Module=Module, transparent=transparent, initializers=init)


def main(ref: str, outdir: str):
    X = os.path.join(ref, "phoenix/xrex")
    rng = np.random.Generator(np.random.PCG64(4321))
    jax, jnp, lax, Scope = make_jax()
    store = ParamStore()
    hk = make_hk(store)
    ident = lambda x, *a, **k: x

    class ShardingContext:                       # sharding is an identity on one device
        mesh = None
        def logical_axis_to_physical(self, *a, **k): return None
        def sharding_specs(self, *a, **k): return None
        def logical_group_size(self, *a, **k): return 1

    base = dict(
        jax=jax, jnp=jnp, lax=lax, np=np, hk=hk, math=math, dataclass=dataclasses.dataclass, replace=dataclasses.replace,
        partial=__import__("functools").partial, Optional=typing.Optional, Callable=typing.Callable, Tuple=typing.Tuple,
        Union=typing.Union, Sequence=typing.Sequence, Type=typing.Type, TypeAlias=typing.TypeAlias,
        abc=__import__("collections").abc, configclass=dataclasses.dataclass, Config=object,
        chex=types.SimpleNamespace(dataclass=lambda **k: dataclasses.dataclass(kw_only=True)),
        P=lambda *a: tuple(a), NamedSharding=lambda *a, **k: None, NamedShape=lambda *a, **k: None,
        with_sharding_constraint_unless_manual=ident, shard_map_unless_manual=lambda f, **k: f,
        checkpoint_name=ident, checkpoint_as_bits=ident, set_xla_metadata=Scope, get_parameter=store.get,
        ShardingContext=ShardingContext, logger=types.SimpleNamespace(debug=lambda *a, **k: None),
        Fp8Gemms=types.SimpleNamespace(OFF=0), Fp8Dot=lambda *a, **k: np.dot,
        TypeVar=typing.TypeVar, Any=typing.Any, F=typing.TypeVar("F"),
    )
    ns = dict(base)

    def run(srcs):
        for s in srcs:
            exec("from __future__ import annotations\n" + s, ns)

    run(cut(os.path.join(X, "utils/utils.py"), ["ffn_size", "gelu_fn", "remat_less"]))
    run(cut(os.path.join(X, "models/scaling.py"), ["ScaleConfig"]))
    run(cut(os.path.join(X, "models/normalization.py"), ["rms_normalize", "RMSNorm", "qk_norm", "all_heads_qk_norm"]))
    run(cut(os.path.join(X, "models/linear_layer.py"), ["LinearConfig", "LinearImpl"]))
    run(cut(os.path.join(X, "models/layers.py"), ["rope_angles", "rotate_half", "apply_rope", "_split_merged_qkv", "Linear"]))
    run(cut(os.path.join(X, "utils/model.py"), ["MemoryModelOutput"]))
    ns["MultiHeadAttentionOutput"] = ns["MemoryModelOutput"]
    run(cut(os.path.join(X, "models/layers.py"), ["MultiHeadAttention"]))
    run(cut(os.path.join(X, "pallas/ranker_attention_utils.py"), ["history_candidate_mask"]))
    ns["ranker_attention_utils"] = types.SimpleNamespace(history_candidate_mask=ns["history_candidate_mask"])
    run(cut(os.path.join(X, "pallas/ranker_attention_fa3.py"), ["tanh", "_abs", "_apply_cap", "attention_reference"]))
    run(cut(os.path.join(X, "models/transformer.py"), ["FeedForwardConfig", "DecoderOutput", "FFNLayerOutput", "MHABlock",
                                                        "DenseBlock", "FFNLayer", "DecoderLayer"]))
    ns["DecoderInput"] = np.ndarray

    # The attention class a layer dispatches to: the argument list of the reference's own wrapper around its ranker
    # kernel (PallasRankerAttention.sharded_custom_op_with_extra_args, recsys_attention.py:36-66), with the reference's
    # plain attention in the kernel's place.
    class RankerAttention:
        def __init__(self, config, scale_config, sharding_context=None):
            self.config, self.scale_config = config, scale_config

        def __call__(self, q, k, v, segment_ids, segment_ids_k, temp, **kw):
            history_upper = self.config.num_user_prefix_tokens + self.config.history_seq_len
            bound = (0, history_upper, history_upper, q.shape[1])
            return ns["attention_reference"](q, k, v, bound=bound, sm_scale=self.scale_config.attn_output_scale(self.config.key_size),
                                             cap=self.config.attn_logit_cap, cap_method=self.config.attn_logit_cap_method), None

    MHA = ns["MultiHeadAttention"]
    MHA._get_attn_impl = lambda self, extra, *, mask, seqpack_layout: (RankerAttention, extra)
    MHA._fused_qk_norm_rope_supported = lambda self, qkv, pspec: False      # a kernel-dispatch question, not semantics

    @dataclasses.dataclass
    class AttnConfig:                            # the fields of RecsysAttentionConfig the executed code reads
        num_q_heads: int; num_kv_heads: int; key_size: int; history_seq_len: int
        num_user_prefix_tokens: int = 0
        qkv_merge: bool = True; qk_norm: bool = False; rotary: bool = True; rope_type: str = "1d"
        rope_base_exponent: int = 10000; with_bias: bool = False; attn_impl: str = "pallas_ranker_attn"
        attn_output_gate: bool = False; attn_sharding_namespace: str | None = None
        attn_logit_cap: float = -1.0; attn_logit_cap_method: str = "tanh"; causal: bool = False

    out = {}
    scale = ns["ScaleConfig"]()
    out["scales"] = np.array([scale.input_scale(128), scale.output_scale(128), scale.attn_output_scale(64),
                              scale.input_scale(512), scale.output_scale(512), scale.attn_output_scale(32)], np.float64)
    out["ffn_sizes"] = np.array([ns["ffn_size"](128, 4.0), ns["ffn_size"](100, 2.0), ns["ffn_size"](512, 4.0)], np.int64)

    def bf16(x):
        u = np.ascontiguousarray(x, np.float32).view(np.uint32)
        r = ((u >> 16) & 1) + np.uint32(0x7FFF)
        return ((u + r) & np.uint32(0xFFFF0000)).view(np.float32)

    # ---- two decoder layers, three model shapes ----------------------------------------------------------------------
    cases = [  # name, B, S, C, D, Hq, Hkv, dh, widening, qk_norm, primer, cap, cap_method
        ("plain", 2, 16, 8, 128, 2, 2, 64, 4.0, False, False, -1.0, "tanh"),
        ("gqa_qknorm", 2, 12, 6, 128, 4, 2, 32, 2.0, True, False, 20.0, "soft_sign"),
        ("primer", 1, 10, 5, 64, 1, 1, 64, 4.0, False, True, 15.0, "tanh"),
    ]
    for name, B, S, C, D, Hq, Hkv, dh, wf, qkn, primer, cap, method in cases:
        T, L = S + C, 2
        F = ns["ffn_size"](D, wf)
        acfg = AttnConfig(num_q_heads=Hq, num_kv_heads=Hkv, key_size=dh, history_seq_len=S, qk_norm=qkn,
                          attn_logit_cap=cap, attn_logit_cap_method=method)
        fcfg = ns["FeedForwardConfig"](widening_factor=wf)
        x = bf16(rng.standard_normal((B, T, D), dtype=np.float32) * np.float32(math.sqrt(D)) * np.float32(0.3))
        pos = np.minimum(np.arange(T), S).astype(np.float32)[None, :, None].repeat(B, 0).repeat(3, 2)   # [B,T,3]; column 0 is read
        seg = np.where(np.arange(T) < S, 1, -1).astype(np.int32)[None].repeat(B, 0)
        mask = np.ones((B, 1, T, T), bool)                                                               # shape-checked only
        h = jarr(x)
        for l in range(L):
            g = lambda n: bf16(np.float32(1.0) + rng.standard_normal(n, dtype=np.float32) * np.float32(0.05))
            m = lambda *s: bf16(rng.standard_normal(s, dtype=np.float32) * np.float32(0.05))
            P_ = {"pre_attn_norm/scale": g(D), "qkv/w": m(D, (Hq + 2 * Hkv) * dh), "out/w": m(Hq * dh, D),
                  "pre_ffn_norm/scale": g(D), "up_proj/w": m(D, F), "down_proj/w": m(F, D)}
            if qkn:
                P_.update({"q_norm/scale": g(Hq * dh), "k_norm/scale": g(Hkv * dh)})
            if primer:
                P_.update({"post_attn_norm/scale": g(D), "post_ffn_norm/scale": g(D)})
            store.params = P_
            store.asked = []
            layer = ns["DecoderLayer"](attn_config=acfg, ffn_config=fcfg, scale_config=scale, primer_norm=primer,
                                       sharding_context=ShardingContext(), name=f"decoder_layer_{l}")
            res = layer(h, mask, seg, positions=pos)
            assert sorted(set(store.asked)) == sorted(P_), (sorted(set(store.asked)), sorted(P_))
            h = jarr(res.output)
            for k_, v_ in P_.items():
                out[f"{name}_l{l}_{k_.replace('/', '.')}"] = v_
            out[f"{name}_l{l}_out"] = np.asarray(res.output, np.float32)
        out[f"{name}_x"] = x
        out[f"{name}_dims"] = np.array([B, S, C, D, Hq, Hkv, dh, F, int(qkn), int(primer), 1 if method == "tanh" else 0], np.int64)
        out[f"{name}_cap"] = np.array([wf, cap], np.float64)

    # ---- heads: final norm -> decode / decode_continuous -> inference rescale ----------------------------------------
    RM = os.path.join(X, "models/recsys_model.py")
    cls = "RecsysAggregatedModel"
    tree = ast.parse(open(RM).read())
    owner = next(n.name for n in tree.body if isinstance(n, ast.ClassDef)
                 and any(isinstance(m, ast.FunctionDef) and m.name == "decode_continuous" for m in n.body))
    run(cut(RM, ["decode", "decode_continuous", "_apply_activation"], methods_of=owner))
    run(cut(RM, ["_get_surface_mask", "_rescale_sigmoid_heads_for_inference"]))
    ns["PURCHASE_VALUE_ACTION_INDEX"] = -1
    B, C, D, V, NC = 2, 7, 128, 19, 3
    hcand = bf16(rng.standard_normal((B, C, D), dtype=np.float32))
    unemb = bf16(rng.standard_normal((D, V), dtype=np.float32) * np.float32(0.05))
    cunemb = bf16(rng.standard_normal((D, NC), dtype=np.float32) * np.float32(0.05))
    fgain = bf16(np.float32(1.0) + rng.standard_normal(D, dtype=np.float32) * np.float32(0.05))

    @dataclasses.dataclass
    class Norm:
        norm_scale: float

    @dataclasses.dataclass
    class LossCfg:                               # the fields of ContinuousActionLossConfig the executed code reads
        action_index: int; activation: str; loss_type: str = "mae"; loss_weight: float = 1.0
        output_cap: float = 0.0; product_surfaces: tuple = (); exclude_product_surfaces: tuple = ()
        norm_config: Norm = dataclasses.field(default_factory=lambda: Norm(30.0)); metric_name: str | None = None

    losses = [LossCfg(0, "sigmoid", norm_config=Norm(30.0)), LossCfg(1, "softplus", loss_type="tweedie"),
              LossCfg(2, "sigmoid", loss_type="binary")]
    self_ = types.SimpleNamespace(
        config=types.SimpleNamespace(continuous_action_losses=losses, purchase_value_enabled=False),
        _get_unembedding=lambda: unemb, _get_continuous_unembedding=lambda: cunemb)
    self_._apply_activation = lambda logits, act: ns["_apply_activation"](self_, logits, act)
    store.params = {"final_layer_norm/scale": fgain}
    normed = ns["RMSNorm"](axis=-1, eps=1e-5, name="final_layer_norm")(jarr(hcand))
    logits = ns["decode"](self_, normed)
    cont, _ = ns["decode_continuous"](self_, normed)
    cont_inf = ns["_rescale_sigmoid_heads_for_inference"](jarr(cont), losses, None)
    out.update(heads_x=hcand, heads_final_gain=fgain, heads_unembed=unemb, heads_cont_unembed=cunemb,
               heads_normed=np.asarray(normed, np.float32), heads_logits=np.asarray(logits, np.float32),
               heads_cont=np.asarray(cont, np.float32), heads_cont_inference=np.asarray(cont_inf, np.float32))

    # ---- user-tower pooling: the lines of user_representation between the transformer and the return --------------------
    TT = os.path.join(X, "models/recsys_two_tower_model.py")
    src = open(TT).read().splitlines()
    i0 = next(i for i, l in enumerate(src) if "user_mask_float = user_padding_mask.astype(jnp.float32)" in l)
    i1 = next(i for i, l in enumerate(src) if i > i0 and "user_representation = user_representation / user_norm" in l)
    block = [l for l in src[i0:i1 + 1]]
    ind = len(block[0]) - len(block[0].lstrip())
    # the block starts inside a branch and ends after it: flatten to one level (the inner `if` keeps its relative indent)
    low = min(len(l) - len(l.lstrip()) for l in block if l.strip())
    pool_src = "\n".join(l[(ind if len(l) - len(l.lstrip()) >= ind else low):] if l.strip() else l for l in block)
    const = next(l for l in src if l.startswith("EPS"))
    pool_ns = dict(jnp=jnp, self=types.SimpleNamespace(config=types.SimpleNamespace(user_query_heads=0)))
    exec(const, pool_ns)
    Bp, Sp, Dp = 3, 9, 32
    pool_x = rng.standard_normal((Bp, Sp, Dp), dtype=np.float32)
    pool_mask = np.ones((Bp, Sp), bool); pool_mask[1, 5:] = False; pool_mask[2, :] = False
    pool_ns.update(user_outputs=pool_x, user_padding_mask=pool_mask)
    exec(pool_src, pool_ns)
    out.update(pool_x=pool_x, pool_mask=pool_mask, pool_out=np.asarray(pool_ns["user_representation"], np.float32),
               pool_eps=np.array([pool_ns["EPS"]], np.float64))

    # ---- sharded top-k with dataset windows and merge (strided_dataset_top_k) -----------------------------------------------
    run(cut(TT, ["strided_dataset_top_k"]))
    fn = ns["strided_dataset_top_k"]
    num_shards, rows_local, Bq, k = 4, 50, 3, 6
    scores = bf16(rng.standard_normal((num_shards, Bq, rows_local), dtype=np.float32))
    scores[:, :, ::7] = scores[0, 0, 0]                      # ties across shards and rows
    ranges = np.array([[0, 120], [120, 200], [37, 58]], np.int32)          # global (strided) row ranges of three datasets
    caps = (120, 80, 24)                                                   # the last window holds fewer rows than its capacity
    rec: dict = {}

    def run_shard(shard, gathered):
        calls = {"n": 0}

        def all_gather(x, axis_name, axis=1, tiled=True):
            i = calls["n"]; calls["n"] += 1
            if gathered is None:
                rec.setdefault(i, {})[shard] = np.asarray(x)
                return np.concatenate([np.asarray(x)] * num_shards, axis=axis)
            return np.concatenate([gathered[i][s] for s in range(num_shards)], axis=axis)
        lax.axis_index = lambda name: shard
        lax.all_gather = all_gather
        return fn(scores[shard], ranges, caps, k, "shards", num_shards, _top_k)

    for s in range(num_shards):
        run_shard(s, None)
    res = [run_shard(s, rec) for s in range(num_shards)]
    for d in range(len(caps)):
        for s in range(1, num_shards):                       # every shard holds the same merged answer
            assert np.array_equal(res[s][d][0], res[0][d][0]) and np.array_equal(res[s][d][1], res[0][d][1])
        out[f"topk_rows_{d}"] = np.asarray(res[0][d][0], np.int64)
        out[f"topk_scores_{d}"] = np.asarray(res[0][d][1], np.float32)
    out.update(topk_scores=scores, topk_ranges=ranges, topk_caps=np.array(caps, np.int64), topk_k=np.array([k], np.int64))

    # ---- input stage over batch-prep buffers: block_user_reduce / block_history_reduce / block_candidate_reduce ---------
    RM = os.path.join(X, "models/recsys_model.py")
    # the column of the purchase-value action is an enum value of the reference's protobuf schema, which is not a Python
    # source; block_history_reduce only compares against it (that column gets no embedding), so any column works here
    ns["PURCHASE_VALUE_ACTION_INDEX"] = 7
    run(cut(RM, ["normalize_continuous_value", "project_continuous_value_to_embedding", "block_user_reduce",
                 "block_history_reduce", "block_candidate_reduce"]))
    prng = np.random.Generator(np.random.PCG64(97))
    Bq, Sq, Cq, Dq, Hq, Vq, HIDq = 3, 5, 4, 32, 2, 4, 64
    keys = types.SimpleNamespace(num_user_hashes=Hq, num_ip_hashes=Hq, num_item_hashes=Hq, num_author_hashes=Hq)
    emb = lambda *shape: bf16(prng.standard_normal(shape, dtype=np.float32) * np.float32(0.1))
    prep = dict(
        prep_user_rows=emb(Bq, Hq, Dq), prep_ip_rows=emb(Bq, Hq, Dq),
        prep_user_hashes=np.array([[5, 9], [0, 0], [3, 0]], np.int32),
        prep_hist_post_rows=emb(Bq, Sq * Hq, Dq), prep_hist_auth_rows=emb(Bq, Sq * Hq, Dq),
        prep_hist_surface_rows=emb(Bq, Sq, Dq),
        prep_hist_post_hashes=prng.integers(0, 3, size=(Bq, Sq, Hq)).astype(np.int32),
        prep_hist_cont=(prng.random((Bq, Sq, 8), dtype=np.float32) * np.float32(80.0) - np.float32(10.0)),
        prep_cand_post_rows=emb(Bq, Cq * Hq, Dq), prep_cand_auth_rows=emb(Bq, Cq * Hq, Dq),
        prep_cand_surface_rows=emb(Bq, Cq, Dq),
        prep_cand_post_hashes=prng.integers(0, 3, size=(Bq, Cq, Hq)).astype(np.int32),
        prep_proj_user=emb(Hq * Dq, Dq), prep_proj_hist=emb((2 * Hq + 2) * Dq, Dq), prep_proj_cand=emb((2 * Hq + 1) * Dq, Dq),
    )
    # history action rows the reference's way: the action sets through multi_hot_to_embeddings
    run(cut(RM, ["multi_hot_to_embeddings"], methods_of="RecsysAggregatedModel"))
    ns["DTYPE_BY_NAME"] = {"float32": np.float32}
    prep["prep_hist_actions"] = prng.random((Bq, Sq, Vq)) < 0.4
    prep["prep_hist_actions"][0, 1] = False                                  # an empty set: the row is zero
    prep["prep_action_vector"] = emb(1, Dq)
    store.stack = []
    store.params = {"history_actions_table": prep["prep_action_vector"]}
    mh_self = types.SimpleNamespace(config=types.SimpleNamespace(fprop_dtype="float32"))
    act_rows, _ = ns["multi_hot_to_embeddings"](mh_self, jarr(prep["prep_hist_actions"]), Vq, Dq, 1.0, "history_actions_table")
    prep["prep_hist_action_rows"] = np.asarray(act_rows, np.float32)
    norm = lambda scale, use_log: types.SimpleNamespace(norm_scale=scale, use_log=use_log)
    loss = lambda idx, wt, name, nc: types.SimpleNamespace(action_index=idx, loss_weight=wt, metric_name=name, norm_config=nc)
    # columns 0 (log) and 3 (linear) get an embedding; column 3 is listed twice (used once), column 5 has no weight,
    # and the purchase-value column is skipped
    losses_in = [loss(0, 1.0, "dwell", norm(30.0, True)), loss(3, 0.5, "watch", norm(60.0, False)),
                 loss(3, 1.0, "watch_again", norm(10.0, False)), loss(5, 0.0, "unused", norm(5.0, False)),
                 loss(7, 1.0, "purchase", norm(5.0, False))]
    store.stack = []
    store.params = {"proj_mat_1": prep["prep_proj_user"], "proj_mat_3": prep["prep_proj_hist"], "proj_mat_2": prep["prep_proj_cand"]}
    for nm in ("dwell", "watch"):
        prep[f"prep_{nm}_proj1"] = emb(1, HIDq) * np.float32(10.0)
        prep[f"prep_{nm}_proj2"] = emb(HIDq, Dq)
        store.params[f"{nm}_proj_proj1"], store.params[f"{nm}_proj_proj2"] = prep[f"prep_{nm}_proj1"], prep[f"prep_{nm}_proj2"]
    lrm = lambda n: 1.0
    u_tok, u_mask = ns["block_user_reduce"](jarr(prep["prep_user_hashes"]), jarr(prep["prep_user_rows"]), keys, lrm, 1.0,
                                            user_ip_embeddings=jarr(prep["prep_ip_rows"]), use_ip_address=True)
    u_tok_noip, _ = ns["block_user_reduce"](jarr(prep["prep_user_hashes"]), jarr(prep["prep_user_rows"]), keys, lrm, 1.0)
    h_tok, h_mask = ns["block_history_reduce"](
        jarr(prep["prep_hist_post_hashes"]), None, jarr(prep["prep_hist_post_rows"]), jarr(prep["prep_hist_auth_rows"]),
        jarr(prep["prep_hist_surface_rows"]), jarr(prep["prep_hist_action_rows"]), keys, lrm, 1.0, True,
        history_continuous_actions=jarr(prep["prep_hist_cont"]), fprop_dtype=np.float32, continuous_action_losses=losses_in,
        continuous_action_hidden_dim=HIDq)
    c_tok, c_mask = ns["block_candidate_reduce"](
        jarr(prep["prep_cand_post_hashes"]), None, jarr(prep["prep_cand_post_rows"]), jarr(prep["prep_cand_auth_rows"]),
        jarr(prep["prep_cand_surface_rows"]), keys, lrm, 1.0, use_product_surface=True, fprop_dtype=np.float32)
    vals = np.array([-3.0, 0.0, 0.5, 7.0, 29.0, 30.0, 31.0, 1e6], np.float32)
    prep.update(
        prep_user_tok=np.asarray(u_tok, np.float32), prep_user_tok_noip=np.asarray(u_tok_noip, np.float32),
        prep_user_mask=np.asarray(u_mask, bool), prep_hist_tok=np.asarray(h_tok, np.float32), prep_hist_mask=np.asarray(h_mask, bool),
        prep_cand_tok=np.asarray(c_tok, np.float32), prep_cand_mask=np.asarray(c_mask, bool), prep_norm_in=vals,
        prep_norm_log=np.asarray(ns["normalize_continuous_value"](jarr(vals), norm(30.0, True)), np.float32),
        prep_norm_lin=np.asarray(ns["normalize_continuous_value"](jarr(vals), norm(30.0, False)), np.float32))
    out.update(prep)

    np.savez_compressed(os.path.join(outdir, "model_golden.npz"), **out)
    print("wrote", os.path.join(outdir, "model_golden.npz"), len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/gen_golden_model.py <path to a checkout of xai-org/x-algorithm>")
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
