"""ctypes loader for libtangq.so.  There is no fallback: a missing library is an ImportError-like
failure the first time any operator is used."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtangq.so")

TQ_OK, TQ_EINVAL, TQ_ECUDA, TQ_ENCCL, TQ_ETIMEOUT, TQ_ENOMEM, TQ_EUNSUPPORTED = range(7)
F32, BF16, F16, I8, U8, I32, F64 = range(7)
Q4_F32, Q4_F16, Q8_F32, I8_ROW = range(4)

_STATUS = {0: "TQ_OK", 1: "TQ_EINVAL", 2: "TQ_ECUDA", 3: "TQ_ENCCL", 4: "TQ_ETIMEOUT", 5: "TQ_ENOMEM",
           6: "TQ_EUNSUPPORTED"}


class TangqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{_STATUS.get(status, status)}: {message}")
        self.status = status


_p, _sz, _i = C.c_void_p, C.c_size_t, C.c_int
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); must list every symbol include/tangq.h declares
PROTOTYPES = {
    "tq_version": (_i, []),
    "tq_ctx_create": (_i, [_i, _p, _pp]),
    "tq_ctx_destroy": (_i, [_p]),
    "tq_last_error": (C.c_char_p, [_p]),
    "tq_sync": (_i, [_p]),
    "tq_ctx_stream": (_p, [_p]),
    "tq_buf_alloc": (_i, [_p, _sz, _pp]),
    "tq_buf_free": (_i, [_p, _p]),
    "tq_upload": (_i, [_p, _p, _p, _sz]),
    "tq_download": (_i, [_p, _p, _p, _sz]),
    "tq_memset": (_i, [_p, _p, _i, _sz]),
    "tq_convert": (_i, [_p, _p, _i, _p, _i, _sz]),
    "tq_qweight_from_blocks": (_i, [_p, _i, _p, _sz, _sz, _pp]),
    "tq_qweight_from_arrays": (_i, [_p, _i, _p, _p, _sz, _sz, _pp]),
    "tq_quantize_matrix": (_i, [_p, _p, _i, _sz, _sz, _sz, _i, _pp]),
    "tq_qweight_from_device_arrays": (_i, [_p, _i, _p, _p, _sz, _sz, _pp]),
    "tq_qweight_free": (_i, [_p, _p]),
    "tq_qweight_shape": (_i, [_p, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_i)]),
    "tq_qweight_bytes": (_sz, [_p]),
    "tq_dequantize": (_i, [_p, _p, _p, _p]),
    "tq_qlinear": (_i, [_p, _p, _p, _i, _sz, _sz, _p, _i, _sz, _p]),
    "tq_q_matvec_host": (_i, [_p, _p, _p, _p, _i, _sz]),
    "tq_q_matvec_host_async": (_i, [_p, _p, _p, _p, _i, _sz]),
    "tq_qweight_interleave_gate_up": (_i, [_p, _p, _pp]),
    "tq_qweight_concat_rows": (_i, [_p, _pp, _sz, _pp]),
    "tq_rms_norm": (_i, [_p, _p, _i, _p, _p, _i, _sz, _sz, C.c_float, _p, _i, _p]),
    "tq_rope_tables": (_i, [_p, _sz, _sz, C.c_double, _p, _p]),
    "tq_rope_forward": (_i, [_p, _p, _i, _p, _p, _p, _sz, _sz, _sz, _sz, _p, _i]),
    "tq_swiglu": (_i, [_p, _p, _p, _i, _sz, _sz, _sz, _p, _i]),
    "tq_embedding": (_i, [_p, _p, _i, _p, _sz, _sz, _sz, _p, _i]),
    "tq_argmax_rows": (_i, [_p, _p, _sz, _sz, _sz, _p]),
    "tq_sample": (_i, [_p, _p, _sz, _sz, _sz, _p, _p, _p, _p, _sz, _p]),
    "tq_generate_advance": (_i, [_p, _p, _sz, _p, _p, _p, _sz, _p, _p]),
    "tq_kv_attention": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _p]),
    "tq_gqa_decode": (_i, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, _p, _i]),
    "tq_gqa_prefill": (_i, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, _p, _i]),
    "tq_gqa_decode_noalloc": (_i, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, _p, _i]),
    "tq_comm_unique_id": (_i, [_p]),
    "tq_comm_create": (_i, [_p, _p, _i, _i, _pp]),
    "tq_comm_destroy": (_i, [_p, _p]),
    "tq_comm_abort": (_i, [_p]),
    "tq_comm_rank": (_i, [_p]),
    "tq_comm_world": (_i, [_p]),
    "tq_comm_enable_peer": (_i, [_p, _p, _sz]),
    "tq_comm_peer_local": (_i, [_p, _i, _i, _pp, _sz, _pp]),
    "tq_comm_peer_bytes": (_sz, [_i, _sz]),
    "tq_comm_set_wait_limit": (_i, [_p, C.c_uint]),
    "tq_all_reduce_f32": (_i, [_p, _p, _p, _sz]),
    "tq_all_gather": (_i, [_p, _p, _p, _p, _sz]),
    "tq_all_to_all": (_i, [_p, _p, _p, _p, _sz]),
    "tq_llama_create": (_i, [_p, _p, _p, _pp]),
    "tq_llama_destroy": (_i, [_p]),
    "tq_llama_set_layer": (_i, [_p, _sz, _p, _p, _p, _p, _p, _p]),
    "tq_llama_set_head": (_i, [_p, _p, _p, _p]),
    "tq_llama_kv_cache": (_i, [_p, _sz, _pp, _pp, C.POINTER(_sz)]),
    "tq_llama_decode_at": (_i, [_p, _p, _p, _p, _sz, _sz, _p]),
    "tq_llama_kv_trim": (_i, [_p, _p, _sz, _sz]),
    "tq_llama_hidden": (_i, [_p, _pp]),
    "tq_llama_decode": (_i, [_p, _p, _p, _sz, _sz, _p]),
    "tq_llama_prefill": (_i, [_p, _p, _p, _sz, _sz, _p]),
    "tq_moe_router": (_i, [_p, _p, _p, _sz, _sz, _sz, _sz, _i, _p, _p, _p]),
    "tq_moe_create": (_i, [_p, _p, _p, _p, _p, _p, _p, _pp]),
    "tq_moe_destroy": (_i, [_p]),
    "tq_moe_ffn": (_i, [_p, _p, _sz, _p, _p, _p, _p]),
    "tq_moe_ffn_dispatch": (_i, [_p, _p, _sz, _p, _p, _p, _p]),
    "tq_mla_decode": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _sz, C.c_float, _p]),
    "tq_mla_absorb_q": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _p]),
    "tq_mla_unabsorb": (_i, [_p, _p, _p, _sz, _sz, _sz, _p, _i]),
    "tq_mla_create": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _pp]),
    "tq_mla_destroy": (_i, [_p]),
    "tq_mla_layer_decode": (_i, [_p, _p, _p, _p, _sz, _sz, _sz, _p, _p]),
    "tq_graph_begin": (_i, [_p]),
    "tq_graph_end": (_i, [_p, _pp]),
    "tq_graph_launch": (_i, [_p, _p]),
    "tq_graph_free": (_i, [_p, _p]),
    "tq_launch_count": (C.c_ulonglong, [_p]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library and binds every prototype.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TangqError(TQ_EUNSUPPORTED,
                             f"{LIB_PATH} is missing; build it with `python -m tang_b200._build` (needs nvcc). "
                             "There is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
