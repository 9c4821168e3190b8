"""TEST INFRASTRUCTURE -- numpy front end over the CPU checkers in this directory.

`libpluto_oracle.so` is this repository's C restatement of the reference arithmetic
(pluto_oracle.c); `_ref/libpluto_ref.so` is the reference project's own
AttentionLayerReference compiled from its sources (ref_shim.cc, Makefile), and
`_ref/libpluto_ref_specs.so` holds the scalar specifications the reference keeps in its GPU layer
tests (ref_specs_shim.cc; the `spec_*` functions below).  Only tests, the
smoke check and the benchmark's CPU-baseline leg import this package; the engine in
`pluto_b200` never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libpluto_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libpluto_ref.so")
_SPECS_SO = os.path.join(_HERE, "_ref", "libpluto_ref_specs.so")


def build(quiet: bool = True) -> None:
    """Compile the C restatement, and the reference's own layer when its tree is present."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        _lib = C.CDLL(_ORACLE_SO)
        _lib.oracle_gdn_decay.restype = C.c_float
        _lib.oracle_gdn_decay.argtypes = [C.c_float] * 3
        _lib.oracle_gdn_beta.restype = C.c_float
        _lib.oracle_gdn_beta.argtypes = [C.c_float, C.c_int]
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


def ref() -> C.CDLL:
    global _ref
    if _ref is None:
        _ref = C.CDLL(_REF_SO)
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------- the reference's own specifications
_specs = None


def have_ref_specs() -> bool:
    return os.path.exists(_SPECS_SO)


def ref_specs() -> C.CDLL:
    global _specs
    if _specs is None:
        _specs = C.CDLL(_SPECS_SO)
    return _specs


def _f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def _f64(x):
    return np.ascontiguousarray(x, dtype=np.float64)


def spec_attention_steps(query_heads, key_value_heads, head_dim, rotary_dim, capacity, epsilon, theta,
                         rnd, q_gate, key, value, q_norm, k_norm):
    """class AttentionReference (cached_attention_ops_test.cc:43-131) stepped over
    q_gate [steps, Hq, 2, D], key/value [steps, Hkv, D].  Returns (out [steps, Hq, D], list of
    per-step probability arrays [Hq, t+1])."""
    steps = q_gate.shape[0]
    out = np.empty((steps, query_heads, head_dim), np.float32)
    probs = np.empty((query_heads * steps * (steps + 1) // 2,), np.float32)
    ref_specs().ref_spec_attention_steps(
        query_heads, key_value_heads, head_dim, rotary_dim, capacity, C.c_float(epsilon), C.c_float(theta),
        int(rnd), steps, _p(_f32(q_gate)), _p(_f32(key)), _p(_f32(value)), _p(_f32(q_norm)),
        _p(_f32(k_norm)), _p(out), _p(probs))
    rows, offset = [], 0
    for t in range(steps):
        rows.append(probs[offset:offset + query_heads * (t + 1)].reshape(query_heads, t + 1))
        offset += query_heads * (t + 1)
    return out, rows


def spec_delta_steps(key_heads, value_heads, key_dim, value_dim, kernel, epsilon, rnd, qkv, z, a, b,
                     weights, a_log, dt_bias, norm):
    """class DeltaReference (cached_attention_ops_test.cc:133-220) stepped from a fresh state over
    qkv [steps, channels], z [steps, Hv*dv], a, b [steps, Hv].  Returns out [steps, Hv, dv]."""
    steps = qkv.shape[0]
    out = np.empty((steps, value_heads, value_dim), np.float32)
    ref_specs().ref_spec_delta_steps(
        key_heads, value_heads, key_dim, value_dim, kernel, C.c_float(epsilon), int(rnd), steps,
        _p(_f32(qkv)), _p(_f32(z)), _p(_f32(a)), _p(_f32(b)), _p(_f32(weights)), _p(_f32(a_log)),
        _p(_f32(dt_bias)), _p(_f32(norm)), _p(out))
    return out


def _example_sizes(length, kh, vh, kd, vd, kernel):
    channels = 2 * kh * kd + vh * vd
    return [length * channels, length * vh * vd, length * vh, length * vh, channels * kernel, vh, vh, vd]


def _pointer_array(arrays):
    return (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])


def spec_sequence_delta_example(length, kh, vh, kd, vd, rnd):
    """MakeExample of sequence_delta_net_test.cc:31-62 (kernel 3, epsilon 0.03): the eight tensors
    QKV, Z, A, B, convolution, A_log, dt_bias, norm (float64, flat) and the upstream gradient."""
    tensors = [np.empty((n,), np.float64) for n in _example_sizes(length, kh, vh, kd, vd, 3)]
    upstream = np.empty((length * vh * vd,), np.float32)
    ref_specs().ref_spec_sequence_delta_example(length, kh, vh, kd, vd, int(rnd), _pointer_array(tensors),
                                                _p(upstream))
    return tensors, upstream


def spec_sequence_delta_forward(length, kh, vh, kd, vd, kernel, epsilon, rnd, tensors):
    """Reference(...) of sequence_delta_net_test.cc:66-159: out [T, Hv, dv] float64."""
    tensors = [_f64(t) for t in tensors]
    out = np.empty((length, vh, vd), np.float64)
    ref_specs().ref_spec_sequence_delta_forward(length, kh, vh, kd, vd, kernel, C.c_float(epsilon), int(rnd),
                                                _pointer_array(tensors), _p(out))
    return out


def spec_sequence_delta_gradients(length, kh, vh, kd, vd, kernel, epsilon, rnd, tensors, upstream, step):
    """Numerical BPTT of sequence_delta_net_test.cc:299-373 with the specification's own Loss:
    central differences (frozen rounding offsets) in every coordinate of the eight tensors."""
    tensors = [_f64(t) for t in tensors]
    grads = [np.empty_like(t) for t in tensors]
    ref_specs().ref_spec_sequence_delta_gradients(length, kh, vh, kd, vd, kernel, C.c_float(epsilon), int(rnd),
                                                  _pointer_array(tensors), _p(_f32(upstream)),
                                                  C.c_double(step), _pointer_array(grads))
    return grads


def spec_qwen_sequence_forward(query_heads, key_value_heads, head_dim, rotary_dim, epsilon, theta, rnd, length,
                               qg, k, v, qw, kw):
    """Reference(...) of qwen_attention_test.cc:26-95: out [T, Hq, D] float64."""
    out = np.empty((length, query_heads, head_dim), np.float64)
    ref_specs().ref_spec_qwen_sequence_forward(
        query_heads, key_value_heads, head_dim, rotary_dim, C.c_float(epsilon), C.c_float(theta), int(rnd),
        length, _p(_f64(qg)), _p(_f64(k)), _p(_f64(v)), _p(_f64(qw)), _p(_f64(kw)), _p(out))
    return out


def spec_qwen_sequence_gradients(query_heads, key_value_heads, head_dim, rotary_dim, epsilon, theta, rnd,
                                 length, qg, k, v, qw, kw, upstream, step):
    """Central differences of qwen_attention_test.cc:230-301 with the specification's own
    Reference: gradients of sum(out * upstream) with respect to qg, k, v, qw, kw."""
    inputs = [_f64(x) for x in (qg, k, v, qw, kw)]
    grads = [np.empty_like(x) for x in inputs]
    ref_specs().ref_spec_qwen_sequence_gradients(
        query_heads, key_value_heads, head_dim, rotary_dim, C.c_float(epsilon), C.c_float(theta), int(rnd),
        length, *[_p(x) for x in inputs], _p(_f64(upstream)), C.c_double(step), _pointer_array(grads))
    return grads


# ---------------------------------------------------------------------------- bf16 helpers
def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even (reference_internal.h:109-115)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = b + 0x7FFF + ((b >> 16) & 1)
    return (b >> 16).astype(np.uint16)


def from_bf16_bits(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return from_bf16_bits(to_bf16_bits(x))


# ---------------------------------------------------------------------------- causal MHA
def attention_fwd(qkv, context, heads, embed, bf16, threads=1, want_probs=False, use_ref=False):
    """qkv: [rows, 3E] float32 (fp32 policy) or uint16 bf16 bits.  Returns dict(out, maxima,
    normalizers[, probs]).  use_ref=True runs the reference's own compiled layer (no stats)."""
    rows = qkv.shape[0]
    qkv = np.ascontiguousarray(qkv)
    assert qkv.dtype == (np.uint16 if bf16 else np.float32) and qkv.shape[1] == 3 * embed
    out = np.empty((rows, embed), dtype=qkv.dtype)
    if use_ref:
        code = ref().pluto_ref_attention(_p(qkv), None, rows, context, heads, embed, int(bf16),
                                         threads, _p(out), None)
        if code:
            raise ValueError(f"reference status code {code}")
        return {"out": out}
    batch = rows // context if context > 0 and rows % context == 0 else 0
    maxima = np.empty((batch * heads * context,), dtype=np.float32)
    normalizers = np.empty_like(maxima)
    probs = np.empty((batch, heads, context, context), np.float32) if want_probs else None
    code = lib().oracle_attention_fwd(_p(qkv), rows, context, heads, embed, int(bf16), threads,
                                      _p(out), _p(maxima), _p(normalizers), _p(probs))
    if code:
        raise ValueError(f"oracle status code {code}")
    res = {"out": out, "maxima": maxima, "normalizers": normalizers}
    if want_probs:
        res["probs"] = probs
    return res


def attention_fwd_bwd(qkv, d_out, context, heads, embed, bf16, threads=1, use_ref=False):
    """Forward then backward.  Returns (out, d_qkv fp32 [rows, 3E])."""
    rows = qkv.shape[0]
    qkv = np.ascontiguousarray(qkv)
    d_out = np.ascontiguousarray(d_out, dtype=np.float32)
    out = np.empty((rows, embed), dtype=qkv.dtype)
    d_qkv = np.empty((rows, 3 * embed), dtype=np.float32)
    if use_ref:
        code = ref().pluto_ref_attention(_p(qkv), _p(d_out), rows, context, heads, embed,
                                         int(bf16), threads, _p(out), _p(d_qkv))
        if code:
            raise ValueError(f"reference status code {code}")
        return out, d_qkv
    out = attention_fwd(qkv, context, heads, embed, bf16, threads)["out"]
    code = lib().oracle_attention_bwd(_p(qkv), _p(out), _p(d_out), rows, context, heads, embed,
                                      int(bf16), threads, _p(d_qkv))
    if code:
        raise ValueError(f"oracle status code {code}")
    return out, d_qkv


def attention_bwd(qkv, out, d_out, context, heads, embed, bf16, threads=1):
    rows = qkv.shape[0]
    d_qkv = np.empty((rows, 3 * embed), dtype=np.float32)
    qkv, out = np.ascontiguousarray(qkv), np.ascontiguousarray(out)
    d_out = np.ascontiguousarray(d_out, dtype=np.float32)
    code = lib().oracle_attention_bwd(_p(qkv), _p(out), _p(d_out), rows, context, heads, embed,
                                      int(bf16), threads, _p(d_qkv))
    if code:
        raise ValueError(f"oracle status code {code}")
    return d_qkv


# ---------------------------------------------------------------------------- Qwen GQA
def qk_prepare(q_gate, k, v, q_norm, k_norm, position, rotary, eps, theta, rnd, keys, values):
    """One token.  q_gate [Hq,2,D], k,v [Hkv,D] fp32; keys/values: fp32 cache [cap,Hkv,D] updated
    in place at `position`.  Returns queries [Hq,D]."""
    hq, _, d = q_gate.shape
    hkv = k.shape[0]
    queries = np.empty((hq, d), np.float32)
    f = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    q_gate, k, v, q_norm, k_norm = map(f, (q_gate, k, v, q_norm, k_norm))
    lib().oracle_qk_prepare(_p(q_gate), _p(k), _p(v), _p(q_norm), _p(k_norm), hq, hkv, d, rotary,
                            position, C.c_float(eps), C.c_float(theta), int(rnd), _p(queries),
                            _p(keys), _p(values))
    return queries


def gqa_decode(queries, q_gate, keys, values, length, rnd):
    """queries [Hq,D] fp32, q_gate [Hq,2,D] or None, keys/values [>=length,Hkv,D] fp32 or uint16."""
    hq, d = queries.shape
    hkv = keys.shape[1]
    out = np.empty((hq, d), np.float32)
    queries = np.ascontiguousarray(queries, dtype=np.float32)
    if q_gate is not None:
        q_gate = np.ascontiguousarray(q_gate, dtype=np.float32)
    assert keys.flags.c_contiguous and values.flags.c_contiguous
    lib().oracle_gqa_decode(_p(queries), _p(q_gate), _p(keys), _p(values),
                            int(keys.dtype == np.uint16), hq, hkv, d, length, int(rnd), _p(out))
    return out


def gqa_decode_batch(q, keys, values, lengths, rnd=True, threads=1):
    """q [B,Hq,D] (uint16 bf16 bits or fp32); keys/values: lists of [L_b(or more),Hkv,D] arrays."""
    b, hq, d = q.shape
    hkv = keys[0].shape[1]
    q = np.ascontiguousarray(q)
    out = np.empty_like(q)
    kp = (C.c_void_p * b)(*[k.ctypes.data for k in keys])
    vp = (C.c_void_p * b)(*[v.ctypes.data for v in values])
    lens = np.ascontiguousarray(lengths, dtype=np.int32)
    lib().oracle_gqa_decode_batch(_p(q), kp, vp, _p(lens), b, int(q.dtype == np.uint16),
                                  int(keys[0].dtype == np.uint16), hq, hkv, d, int(rnd), threads,
                                  _p(out))
    return out


def gqa_prefill_rows(q, k, v, rows, rnd=True, threads=1):
    """Rows `rows` (a list of token indices) of the ungated sequence forward: q [T,Hq,D], k,v
    [T,Hkv,D] -> [len(rows),Hq,D].  Row r of the sequence layer is the cached step at position r
    over keys [0, r] (the reference pins the two paths to each other,
    qwen_attention_test.cc:155-228), so each sampled row costs only its own prefix instead of
    the whole triangle."""
    rows = np.asarray(rows, dtype=np.int64)
    k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
    return gqa_decode_batch(np.ascontiguousarray(q[rows]), [k] * len(rows), [v] * len(rows),
                            (rows + 1).astype(np.int32), rnd=rnd, threads=threads)


def gqa_probabilities(queries, keys, length):
    hq, d = queries.shape
    hkv = keys.shape[1]
    probs = np.empty((hq, length), np.float32)
    queries = np.ascontiguousarray(queries, dtype=np.float32)
    lib().oracle_gqa_probabilities(_p(queries), _p(keys), int(keys.dtype == np.uint16), hq, hkv, d,
                                   length, _p(probs))
    return probs


def gqa_prefill(q, k, v, gate=None, rnd=True, threads=1, rows=None, q_token_stride=None,
                q_head_stride=None, want_core=False, want_lse=False, shape=None):
    """q [T,Hq,D], k,v [T,Hkv,D] (uint16 bf16 bits or fp32).  `rows=(begin,end)` limits the query
    rows computed (others left zero).  For a strided q view pass the base array plus strides and
    shape=(T,Hq,D)."""
    t, hq, d = shape if shape is not None else q.shape
    hkv = k.shape[1]
    bf16 = k.dtype == np.uint16
    out = np.zeros((t, hq, d), dtype=k.dtype)
    core = np.zeros((t, hq, d), np.float32) if want_core else None
    lse = np.zeros((hq, t), np.float32) if want_lse else None
    rb, re = rows if rows is not None else (0, t)
    qts = q_token_stride if q_token_stride is not None else hq * d
    qhs = q_head_stride if q_head_stride is not None else d
    lib().oracle_gqa_prefill(_p(q), _p(gate), _p(np.ascontiguousarray(k)),
                             _p(np.ascontiguousarray(v)), int(bf16), t, hq, hkv, d,
                             C.c_size_t(qts), C.c_size_t(qhs), int(rnd), threads, rb, re, _p(out),
                             _p(core), _p(lse))
    res = {"out": out}
    if want_core:
        res["core"] = core
    if want_lse:
        res["lse"] = lse
    return res


def gqa_sequence_bwd(qg, k, v, q_norm, k_norm, dy, rotary, eps, theta, rnd=True, dqw=None, dkw=None):
    """QwenAttentionLayer sequence forward + backward (qwen_attention.cc:124-239, 450-499) for one
    sequence.  fp32 arrays: qg [T,Hq,2,D], k,v [T,Hkv,D], norms [D], dy [T,Hq,D].  dqw / dkw are
    fp32 [D] arrays accumulated into (None = frozen norm).  Returns dqg, dk, dv and the forward
    output y."""
    qg = np.ascontiguousarray(qg, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    dy = np.ascontiguousarray(dy, np.float32)
    t, hq, _, d = qg.shape
    hkv = k.shape[1]
    dqg = np.zeros_like(qg)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    y = np.zeros((t, hq, d), np.float32)
    rc = lib().oracle_gqa_sequence_bwd(
        _p(qg), _p(k), _p(v), _p(np.ascontiguousarray(q_norm, np.float32)),
        _p(np.ascontiguousarray(k_norm, np.float32)), _p(dy), t, hq, hkv, d, int(rotary),
        C.c_float(eps), C.c_float(theta), int(rnd), _p(dqg), _p(dk), _p(dv), _p(dqw), _p(dkw), _p(y))
    if rc != 0:
        raise MemoryError("oracle_gqa_sequence_bwd scratch allocation failed")
    return {"dqg": dqg, "dk": dk, "dv": dv, "y": y}


# ---------------------------------------------------------------------------- gated delta-net
def gdn_decay(a, dt_bias, a_log):
    return np.array([lib().oracle_gdn_decay(float(x), float(y), float(z))
                     for x, y, z in zip(np.ravel(a), np.ravel(dt_bias), np.ravel(a_log))],
                    np.float32).reshape(np.shape(a))


def gdn_beta(b, rnd):
    return np.array([lib().oracle_gdn_beta(float(x), int(rnd)) for x in np.ravel(b)],
                    np.float32).reshape(np.shape(b))


def gdn_recurrence(q, k, v, g, beta, state, normalize_qk=True, q_scale=1.0, rnd=True, threads=1):
    """q,k [B,T,Hk,dk]; v [B,T,Hv,dv] (uint16 bf16 bits or fp32); g,beta fp32 [B,T,Hv];
    state fp32 [B,Hv,dk,dv] updated IN PLACE.  Returns out like v."""
    b, t, hk, dk = q.shape
    hv, dv = v.shape[2], v.shape[3]
    q, k, v = map(np.ascontiguousarray, (q, k, v))
    g = np.ascontiguousarray(g, dtype=np.float32)
    beta = np.ascontiguousarray(beta, dtype=np.float32)
    assert state.dtype == np.float32 and state.flags.c_contiguous
    out = np.empty_like(v)
    code = lib().oracle_gdn_recurrence(_p(q), _p(k), _p(v), _p(g), _p(beta),
                                       int(v.dtype == np.uint16), b, t, hk, hv, dk, dv,
                                       int(normalize_qk), C.c_float(q_scale), int(rnd), threads,
                                       _p(state), _p(out))
    if code:
        raise ValueError(f"oracle status code {code}")
    return out


def gdn_conv_step(x, weight, state, rnd):
    """x [channels] fp32, weight [channels,width], state [channels,width] updated in place."""
    ch, width = weight.shape
    out = np.empty((ch,), np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    lib().oracle_gdn_conv_step(_p(x), _p(weight), ch, width, int(rnd), _p(state), _p(out))
    return out


def gdn_output(core, z, norm_weight, eps, rnd, final_round=True):
    heads, dim = core.shape
    out = np.empty((heads, dim), np.float32)
    f = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    core, z, norm_weight = map(f, (core, z, norm_weight))
    lib().oracle_gdn_output(_p(core), _p(z), _p(norm_weight), heads, dim, C.c_float(eps), int(rnd),
                            int(final_round), _p(out))
    return out


def gdn_sequence_bwd(qkv, z, a, b, conv_w, a_log, dt_bias, norm, dy, kh, vh, kd, vd, eps, rnd=True,
                     d_conv=None, d_a_log=None, d_dt_bias=None, d_norm=None):
    """SequenceDeltaNetLayer forward + backward (sequence_delta_net.cc:31-339, 482-561) for one
    sequence; fp32 arrays qkv [T,channels], z [T,vh*vd], a,b [T,vh], conv_w [channels,kernel],
    dy [T,vh*vd].  The d_* arrays (fp32) are accumulated into when given.  Returns dqkv, dz, da,
    db and the forward output y (before its bf16 store)."""
    f = lambda x: np.ascontiguousarray(x, np.float32)
    qkv, z, a, b, conv_w, dy = f(qkv), f(z), f(a), f(b), f(conv_w), f(dy)
    t, channels = qkv.shape
    kernel = conv_w.shape[1]
    dqkv, dz = np.zeros_like(qkv), np.zeros_like(z)
    da, db = np.zeros_like(a), np.zeros_like(b)
    y = np.zeros_like(z)
    rc = lib().oracle_gdn_sequence_bwd(
        _p(qkv), _p(z), _p(a), _p(b), _p(conv_w), _p(f(a_log)), _p(f(dt_bias)), _p(f(norm)), _p(dy),
        t, kh, vh, kd, vd, kernel, C.c_float(eps), int(rnd), _p(dqkv), _p(dz), _p(da), _p(db),
        _p(d_conv), _p(d_a_log), _p(d_dt_bias), _p(d_norm), _p(y))
    if rc != 0:
        raise MemoryError("oracle_gdn_sequence_bwd scratch allocation failed")
    return {"dqkv": dqkv, "dz": dz, "da": da, "db": db, "y": y}


# ---------------------------------------------------------------------------- imported projections
def float_to_e4m3(x: np.ndarray) -> np.ndarray:
    """fp32 -> FP8 E4M3 bytes (round to nearest even, saturating), element by element."""
    L = lib()
    L.oracle_float_to_e4m3.restype = C.c_uint8
    L.oracle_float_to_e4m3.argtypes = [C.c_float]
    flat = np.asarray(x, np.float32).ravel()
    return np.array([L.oracle_float_to_e4m3(float(v)) for v in flat], np.uint8).reshape(np.shape(x))


def e4m3_to_float(b: np.ndarray) -> np.ndarray:
    L = lib()
    L.oracle_e4m3_to_float.restype = C.c_float
    L.oracle_e4m3_to_float.argtypes = [C.c_uint8]
    flat = np.asarray(b, np.uint8).ravel()
    return np.array([L.oracle_e4m3_to_float(int(v)) for v in flat], np.float32).reshape(np.shape(b))


def quantize_imported_input(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros_like(x)
    lib().oracle_quantize_imported_input(_p(x), x.size, _p(out))
    return out


def linear_imported(weights: np.ndarray, storage: str, x: np.ndarray, scales=None) -> np.ndarray:
    """FullyConnectedLayer::ImportedForward (fully_connected.cc:295-341) for one token: weights
    [rows, cols] as fp32 ("fp32"), bf16 bits uint16 ("bf16") or e4m3 bytes uint8 ("fp8", with fp32
    block scales [ceil(rows/128), ceil(cols/128)]); x fp32 values of the bf16 activation.
    Returns the bf16 output as fp32."""
    code = {"fp32": 0, "bf16": 1, "fp8": 2}[storage]
    rows, cols = weights.shape
    w = np.ascontiguousarray(weights)
    out = np.zeros(rows, np.uint16)
    sc = None if scales is None else np.ascontiguousarray(scales, np.float32)
    lib().oracle_linear_imported(_p(w), code, _p(sc), _p(np.ascontiguousarray(x, np.float32)), cols,
                                 rows, _p(out))
    return from_bf16_bits(out)


# ---------------------------------------------------------------------------- dense projections
def _mma_cast(a: np.ndarray, bf16: bool) -> np.ndarray:
    """Operand type of the reference's tile MMAs (fully_connected.cc:31-33): bf16 for bf16
    activations, fp16 for the fp32-activation policy."""
    a = np.asarray(a, np.float32)
    return round_bf16(a) if bf16 else a.astype(np.float16).astype(np.float32)


def dense_fwd(x, w, bias, bf16: bool) -> np.ndarray:
    """DenseForwardKernel (fully_connected.cc:97-132): cast(x) @ cast(w) + bias, accumulated in
    higher precision than the reference's fp32 tiles; output rounded to bf16 for bf16 layers."""
    y = _mma_cast(x, bf16).astype(np.float64) @ _mma_cast(w, bf16).astype(np.float64) + np.asarray(bias, np.float64)
    y = y.astype(np.float32)
    return round_bf16(y) if bf16 else y


def dense_bwd(x, w, dy, bf16: bool):
    """DenseInputGradientKernel, DenseWeightGradientKernel, DenseBiasGradientKernel (:134-232)."""
    xc, wc, gc = (_mma_cast(a, bf16).astype(np.float64) for a in (x, w, dy))
    return {"dx": (gc @ wc.T).astype(np.float32), "dw": (xc.T @ gc).astype(np.float32),
            "db": np.asarray(dy, np.float64).sum(0).astype(np.float32)}


def block_linear_fwd(w_bf16, x_bf16, output_float32: bool) -> np.ndarray:
    """LinearForward (block_training.cc:38-56): y[t][r] = sum_c x[t][c] w[r][c] over the bf16
    values in fp32 arithmetic (here in double: every product is exact, only the sum order differs)."""
    y = (np.asarray(x_bf16, np.float64) @ np.asarray(w_bf16, np.float64).T).astype(np.float32)
    return y if output_float32 else round_bf16(y)


def block_linear_bwd(w_bf16, x_bf16, dy):
    """LinearInputGradient / LinearWeightGradient (block_training.cc:58-98): fp32 dy against the
    bf16 weight and input values; dw is the increment the layer adds to its accumulator."""
    dy = np.asarray(dy, np.float64)
    return {"dx": (dy @ np.asarray(w_bf16, np.float64)).astype(np.float32),
            "dw": (dy.T @ np.asarray(x_bf16, np.float64)).astype(np.float32)}
