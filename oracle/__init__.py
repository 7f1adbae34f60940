"""ctypes front end of the CPU parity oracle (``liborc.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / reference legs of ``bench.py``.  The product package ``tang_b200`` never imports it.

Each wrapper takes and returns numpy arrays and forwards to the C function of the same name in
``tang_oracle.cpp`` / ``tang_oracle_models.cpp``, whose comments cite the reference file:line
they restate.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborc.so")

KIND_Q4_F32 = 0   # tang-infer Q4Block: f32 scale per 32 weights
KIND_Q4_F16 = 1   # same blocks, scale stored as IEEE half
KIND_Q8_F32 = 2   # tang-infer Q8Block
KIND_I8_ROW = 3   # int8 [rows, cols] with one f32 scale per row


def build(force: bool = False) -> str:
    """Compile liborc.so with the Makefile beside this file (no-op if it is up to date)."""
    if force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH)
        for f in ("tang_oracle.cpp", "tang_oracle_models.cpp", "Makefile")
    ):
        subprocess.run(["make", "-C", _HERE, "-s"] + (["-B"] if force else []), check=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


_sz = C.c_size_t
_p = C.c_void_p


def _declare(L: C.CDLL) -> None:
    L.orc_f16_to_f32.restype = C.c_float
    L.orc_f16_to_f32.argtypes = [C.c_uint16]
    L.orc_f32_to_bf16.restype = C.c_uint16
    L.orc_f32_to_bf16.argtypes = [C.c_float]
    L.orc_bf16_to_f32.restype = C.c_float
    L.orc_bf16_to_f32.argtypes = [C.c_uint16]
    L.orc_f32_to_f16.restype = C.c_uint16
    L.orc_f32_to_f16.argtypes = [C.c_float]
    L.orc_argmax_f64.restype = _sz
    L.orc_kth_largest_f64.restype = C.c_double
    L.orc_max_threads.restype = C.c_int
    for name in ("orc_argmax_f64",):
        getattr(L, name).argtypes = [_p, _sz]
    L.orc_kth_largest_f64.argtypes = [_p, _sz, _sz]


def _ptr(a: np.ndarray) -> C.c_void_p:
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return C.c_void_p(a.ctypes.data)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ----------------------------------------------------------------------------- conversions

def f16_bits_to_f32(bits) -> np.ndarray:
    bits = _c(bits, np.uint16)
    out = np.empty(bits.shape, np.float32)
    f = lib().orc_f16_to_f32
    flat_in, flat_out = bits.reshape(-1), out.reshape(-1)
    for i in range(flat_in.size):
        flat_out[i] = f(int(flat_in[i]))
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    """Vectorised restatement of orc_f32_to_bf16 (same add-0x7FFF+lsb rule) for large arrays."""
    u = _c(x, np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + (0x7FFF + lsb).astype(np.uint32)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits) -> np.ndarray:
    return (_c(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_bf16(x) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, np.float32)))


# ----------------------------------------------------------------------------- quantisation

def n_blocks(n: int) -> int:
    return (n + 31) // 32


def quantize_q8(data):
    data = _c(data, np.float32).reshape(-1)
    nb = n_blocks(data.size)
    scales = np.empty(nb, np.float32)
    values = np.empty(nb * 32, np.int8)
    lib().orc_quantize_q8(_ptr(data), _sz(data.size), _ptr(scales), _ptr(values))
    return scales, values


def quantize_q4(data):
    data = _c(data, np.float32).reshape(-1)
    nb = n_blocks(data.size)
    scales = np.empty(nb, np.float32)
    packed = np.empty(nb * 16, np.uint8)
    lib().orc_quantize_q4(_ptr(data), _sz(data.size), _ptr(scales), _ptr(packed))
    return scales, packed


def dequantize_q8(scales, values) -> np.ndarray:
    scales, values = _c(scales, np.float32), _c(values, np.int8)
    out = np.empty(scales.size * 32, np.float32)
    lib().orc_dequantize_q8(_ptr(scales), _ptr(values), _sz(scales.size), _ptr(out))
    return out


def dequantize_q4(scales, packed) -> np.ndarray:
    scales, packed = _c(scales, np.float32), _c(packed, np.uint8)
    out = np.empty(scales.size * 32, np.float32)
    lib().orc_dequantize_q4(_ptr(scales), _ptr(packed), _sz(scales.size), _ptr(out))
    return out


def unpack_q4(packed) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    out = np.empty(packed.size * 2, np.int8)
    lib().orc_unpack_q4(_ptr(packed), _sz(packed.size), _ptr(out))
    return out


def quantize_matrix_q8(data, rows: int, cols: int):
    data = _c(data, np.float32).reshape(-1)
    assert data.size == rows * cols
    bpr = n_blocks(cols)
    scales = np.empty((rows, bpr), np.float32)
    values = np.empty((rows, bpr * 32), np.int8)
    lib().orc_quantize_matrix_q8(_ptr(data), _sz(rows), _sz(cols), _ptr(scales), _ptr(values))
    return scales, values


def quantize_matrix_q4(data, rows: int, cols: int):
    data = _c(data, np.float32).reshape(-1)
    assert data.size == rows * cols
    bpr = n_blocks(cols)
    scales = np.empty((rows, bpr), np.float32)
    packed = np.empty((rows, bpr * 16), np.uint8)
    lib().orc_quantize_matrix_q4(_ptr(data), _sz(rows), _sz(cols), _ptr(scales), _ptr(packed))
    return scales, packed


_SCALE_DTYPE = {KIND_Q4_F32: np.float32, KIND_Q4_F16: np.uint16, KIND_Q8_F32: np.float32, KIND_I8_ROW: np.float32}
_PAYLOAD_DTYPE = {KIND_Q4_F32: np.uint8, KIND_Q4_F16: np.uint8, KIND_Q8_F32: np.int8, KIND_I8_ROW: np.int8}


def qmatmul(kind: int, scales, payload, rows: int, cols: int, x, threads: int = 0) -> np.ndarray:
    """y[m, rows] = x[m, cols] . W^T, one reference matvec per activation row, f64."""
    scales = _c(scales, _SCALE_DTYPE[kind])
    payload = _c(payload, _PAYLOAD_DTYPE[kind])
    x = _c(x, np.float64)
    x2 = x.reshape(-1, cols)
    y = np.empty((x2.shape[0], rows), np.float64)
    lib().orc_qmatmul(C.c_int(kind), _ptr(scales), _ptr(payload), _sz(rows), _sz(cols), _ptr(x2),
                      _sz(x2.shape[0]), _ptr(y), C.c_int(threads))
    return y.reshape(x.shape[:-1] + (rows,))


def q8_matvec(scales, values, rows, cols, x, threads: int = 1):
    return qmatmul(KIND_Q8_F32, scales, values, rows, cols, np.asarray(x, np.float64).reshape(cols), threads)


def q4_matvec(scales, packed, rows, cols, x, threads: int = 1):
    return qmatmul(KIND_Q4_F32, scales, packed, rows, cols, np.asarray(x, np.float64).reshape(cols), threads)


# ----------------------------------------------------------------------------- CpuDevice (f32)

def matmul_f32(a, b, m, k, n):
    a, b = _c(a, np.float32), _c(b, np.float32)
    c = np.empty(m * n, np.float32)
    lib().orc_matmul_f32(_ptr(a), _ptr(b), _ptr(c), _sz(m), _sz(k), _sz(n))
    return c


def matmul_b_transposed_f32(a, b, m, k, n):
    a, b = _c(a, np.float32), _c(b, np.float32)
    c = np.empty(m * n, np.float32)
    lib().orc_matmul_b_transposed_f32(_ptr(a), _ptr(b), _ptr(c), _sz(m), _sz(k), _sz(n))
    return c


def softmax_f32(x, n_rows, row_len):
    x = _c(x, np.float32)
    out = np.empty(n_rows * row_len, np.float32)
    lib().orc_softmax_f32(_ptr(x), _ptr(out), _sz(n_rows), _sz(row_len))
    return out


def rms_norm_f32(x, w, n_groups, dim, eps):
    x, w = _c(x, np.float32), _c(w, np.float32)
    out = np.empty(n_groups * dim, np.float32)
    lib().orc_rms_norm_f32(_ptr(x), _ptr(w), _ptr(out), _sz(n_groups), _sz(dim), C.c_float(eps))
    return out


def rms_norm_residual_f32(x, res, w, n_groups, dim, eps):
    x, res, w = _c(x, np.float32), _c(res, np.float32), _c(w, np.float32)
    out = np.empty(n_groups * dim, np.float32)
    s = np.empty(n_groups * dim, np.float32)
    lib().orc_rms_norm_residual_f32(_ptr(x), _ptr(res), _ptr(w), _ptr(out), _ptr(s), _sz(n_groups), _sz(dim),
                                    C.c_float(eps))
    return out, s


def embedding_f32(weight, ids, dim):
    weight, ids = _c(weight, np.float32), _c(ids, np.uint32)
    out = np.empty(ids.size * dim, np.float32)
    lib().orc_embedding_f32(_ptr(weight), _ptr(ids), _ptr(out), _sz(ids.size), _sz(dim))
    return out


def kv_attention_f32(q, k_cache, v_cache, cache_start, q_len, n_heads, n_kv_heads, head_dim):
    q, k_cache, v_cache = _c(q, np.float32), _c(k_cache, np.float32), _c(v_cache, np.float32)
    out = np.empty(q_len * n_heads * head_dim, np.float32)
    lib().orc_kv_attention_f32(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _sz(cache_start), _sz(q_len),
                               _sz(n_heads), _sz(n_kv_heads), _sz(head_dim))
    return out


def rope_tables_f32(head_dim, max_seq_len, base):
    half = head_dim // 2
    cos = np.empty(max_seq_len * half, np.float32)
    sin = np.empty(max_seq_len * half, np.float32)
    lib().orc_rope_tables_f32(_sz(head_dim), _sz(max_seq_len), C.c_double(base), _ptr(cos), _ptr(sin))
    return cos, sin


def rope_forward_f32(x, cos, sin, seq_len, n_heads, head_dim, start_pos):
    x, cos, sin = _c(x, np.float32), _c(cos, np.float32), _c(sin, np.float32)
    out = np.empty_like(x)
    lib().orc_rope_forward_f32(_ptr(x), _ptr(out), _ptr(cos), _ptr(sin), _sz(seq_len), _sz(n_heads), _sz(head_dim),
                               _sz(start_pos))
    return out


def swiglu_f32(gate, up):
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().orc_swiglu_f32(_ptr(gate), _ptr(up), _ptr(out), _sz(gate.size))
    return out


# ----------------------------------------------------------------------------- f64 model pieces

def rms_norm_f64(x, w, eps):
    x, w = _c(x, np.float64), _c(w, np.float64)
    out = np.empty_like(x)
    lib().orc_rms_norm_f64(_ptr(x), _ptr(w), _ptr(out), _sz(x.size), C.c_double(eps))
    return out


def rope_heads_f64(x, n_heads, head_dim, pos, base):
    x = _c(x, np.float64)
    out = np.empty_like(x)
    lib().orc_rope_heads_f64(_ptr(x), _ptr(out), _sz(n_heads), _sz(head_dim), _sz(pos), C.c_double(base))
    return out


def attention_decode_f64(q, k_cache, v_cache, total_seq, n_heads, n_kv_heads, head_dim, threads: int = 0):
    q, k_cache, v_cache = _c(q, np.float64), _c(k_cache, np.float64), _c(v_cache, np.float64)
    out = np.empty(n_heads * head_dim, np.float64)
    lib().orc_attention_decode_f64(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _sz(total_seq), _sz(n_heads),
                                   _sz(n_kv_heads), _sz(head_dim), C.c_int(threads))
    return out


def swiglu_f64(gate, up):
    gate, up = _c(gate, np.float64), _c(up, np.float64)
    out = np.empty_like(gate)
    lib().orc_swiglu_f64(_ptr(gate), _ptr(up), _ptr(out), _sz(gate.size))
    return out


# ----------------------------------------------------------------------------- selection

def argmax_f64(v) -> int:
    v = _c(v, np.float64)
    return int(lib().orc_argmax_f64(_ptr(v), _sz(v.size)))


def kth_largest_f64(v, k) -> float:
    v = _c(v, np.float64)
    return float(lib().orc_kth_largest_f64(_ptr(v), _sz(v.size), _sz(k)))


def topk_filter_f64(logits, k):
    logits = _c(logits, np.float64)
    out = np.empty_like(logits)
    lib().orc_topk_filter_f64(_ptr(logits), _sz(logits.size), _sz(k), _ptr(out))
    return out


def topk_indices_f64(v, k):
    v = _c(v, np.float64)
    out = np.empty(k, np.int32)
    lib().orc_topk_indices_f64(_ptr(v), _sz(v.size), _sz(k), _ptr(out))
    return out


class SamplerConfig(C.Structure):
    """``SamplingConfig`` (crates/tang-infer/src/sampling.rs:6-20) without the loop controls."""
    _fields_ = [("temperature", C.c_double), ("top_k", C.c_uint64), ("top_p", C.c_double), ("repetition_penalty", C.c_double)]


def lcg_next_f64(state: int):
    """One step of the sampler's LCG: returns (fraction in [0, 1), new state)."""
    st = C.c_uint64(state)
    lib().orc_lcg_next_f64.restype = C.c_double
    r = lib().orc_lcg_next_f64(C.byref(st))
    return float(r), int(st.value)


def sampler_sample(logits, cfg: "SamplerConfig", rng_state: int, past=()):
    """``Sampler::sample`` (sampling.rs:86-158): returns (token, new rng state)."""
    logits = _c(logits, np.float64)
    past = _c(np.asarray(past, np.int64), np.int64)
    st = C.c_uint64(rng_state)
    lib().orc_sampler_sample.restype = C.c_int64
    tok = lib().orc_sampler_sample(_ptr(logits), _sz(logits.size), _ptr(past), _sz(past.size), C.byref(cfg), C.byref(st))
    return int(tok), int(st.value)


# ----------------------------------------------------------------------------- layer compositions

class QWeight(C.Structure):
    _fields_ = [("kind", C.c_int32), ("_pad", C.c_int32), ("scales", C.c_void_p), ("payload", C.c_void_p),
                ("rows", C.c_uint64), ("cols", C.c_uint64)]


class LlamaLayer(C.Structure):
    _fields_ = [(n, QWeight) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down")] + [
        ("attn_norm_bf16", C.c_void_p), ("ffn_norm_bf16", C.c_void_p)]


class LlamaDims(C.Structure):
    _fields_ = [("d_model", C.c_uint64), ("n_heads", C.c_uint64), ("n_kv_heads", C.c_uint64),
                ("head_dim", C.c_uint64), ("ffn", C.c_uint64), ("rope_base", C.c_double), ("eps", C.c_double)]


class MlaDims(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("n_heads", "kv_lora", "nope", "rope_dim", "v_dim")]


def qweight(kind, scales, payload, rows, cols) -> QWeight:
    """The arrays must stay alive (and contiguous) for as long as the struct is used."""
    assert scales.flags["C_CONTIGUOUS"] and payload.flags["C_CONTIGUOUS"]
    assert scales.dtype == _SCALE_DTYPE[kind] and payload.dtype == _PAYLOAD_DTYPE[kind]
    return QWeight(kind, 0, scales.ctypes.data, payload.ctypes.data, rows, cols)


def llama_layer_f64(dims: LlamaDims, layer: LlamaLayer, hidden: np.ndarray, k_cache: np.ndarray,
                    v_cache: np.ndarray, pos: int, threads: int = 0, rope_pos: int | None = None) -> None:
    """One decode token through one block: appended at cache row `pos`, rotated for position `rope_pos` (= pos unless
    the cache has been trimmed)."""
    assert hidden.dtype == np.float64 and k_cache.dtype == np.uint16 and v_cache.dtype == np.uint16
    lib().orc_llama_layer_at_f64(C.byref(dims), C.byref(layer), _ptr(hidden), _ptr(k_cache), _ptr(v_cache),
                                 C.c_uint64(pos), C.c_uint64(pos if rope_pos is None else rope_pos), C.c_int(threads))


def kv_trim_to(rows: np.ndarray, seq_len: int, keep: int) -> int:
    """``KVCache::trim_to(keep)`` (crates/tang-infer/src/kv_cache.rs:138-149) on one layer's rows [>= seq_len, kv_dim] of
    16-bit elements, in place; returns the new seq_len."""
    assert rows.dtype == np.uint16 and rows.ndim == 2 and rows.flags.c_contiguous
    f = lib().orc_kv_trim_to
    f.restype = C.c_uint64
    return int(f(_ptr(rows), C.c_uint64(seq_len), C.c_uint64(rows.shape[1]), C.c_uint64(keep)))


def llama_head_f64(dims: LlamaDims, final_norm_bf16: np.ndarray, lm_head: QWeight, hidden: np.ndarray,
                   threads: int = 0) -> np.ndarray:
    logits = np.empty(int(lm_head.rows), np.float64)
    lib().orc_llama_head_f64(C.byref(dims), _ptr(final_norm_bf16), C.byref(lm_head), _ptr(hidden), _ptr(logits),
                             C.c_int(threads))
    return logits


def router_f64(h, wg, n_experts, top_k, renormalize=False):
    h, wg = _c(h, np.float64), _c(wg, np.float64)
    idx = np.empty(top_k, np.int32)
    w = np.empty(top_k, np.float64)
    logits = np.empty(n_experts, np.float64)
    lib().orc_router_f64(_ptr(h), _ptr(wg), _sz(n_experts), _sz(h.size), _sz(top_k), C.c_int(int(renormalize)),
                         _ptr(idx), _ptr(w), _ptr(logits))
    return idx, w, logits


def expert_ffn_f64(gate: QWeight, up: QWeight, down: QWeight, x, threads: int = 0) -> np.ndarray:
    x = _c(x, np.float64)
    out = np.empty(int(down.rows), np.float64)
    lib().orc_expert_ffn_f64(C.byref(gate), C.byref(up), C.byref(down), _ptr(x), _ptr(out), C.c_int(threads))
    return out


def mla_decode_f64(dims: MlaDims, q_nope, q_rope, cache_bf16, ctx, w_qk, w_qk_scale, w_uv, w_uv_scale,
                   absorbed=True, threads: int = 0) -> np.ndarray:
    q_nope, q_rope = _c(q_nope, np.float64), _c(q_rope, np.float64)
    cache_bf16 = _c(cache_bf16, np.uint16)
    w_qk, w_uv = _c(w_qk, np.int8), _c(w_uv, np.int8)
    w_qk_scale, w_uv_scale = _c(w_qk_scale, np.float32), _c(w_uv_scale, np.float32)
    out = np.empty(int(dims.n_heads * dims.v_dim), np.float64)
    lib().orc_mla_decode_f64(C.byref(dims), _ptr(q_nope), _ptr(q_rope), _ptr(cache_bf16), C.c_uint64(ctx), _ptr(w_qk),
                             _ptr(w_qk_scale), _ptr(w_uv), _ptr(w_uv_scale), C.c_int(int(absorbed)), _ptr(out),
                             C.c_int(threads))
    return out
