"""tang_b200 — sm_100a kernels for tang-infer's quantised decode path behind a C ABI.

``tang_b200.device`` mirrors the reference's host interfaces over ``libtangq.so``
(``include/tangq.h``).  The package needs that library; there is no CPU path.
"""
from ._lib import (BF16, F16, F32, F64, I8, I32, I8_ROW, Q4_F16, Q4_F32, Q8_F32, U8, TangqError, load)
from .device import Buffer, Graph, QBuffer, QuantComputeDevice, QuantizedQ4, QuantizedQ8, SamplerConfig
from .checkpoint import SafetensorsError, TensorView, quantize_linear, read_safetensors, write_safetensors
from .llama import Comm, LlamaConfig, LlamaLayerWeights, LlamaModel
from .mla import MlaConfig, MlaLayer, mla_decode
from .moe import MoeConfig, MoeLayer, moe_router

__all__ = ["read_safetensors", "write_safetensors", "quantize_linear", "TensorView", "SafetensorsError", "SamplerConfig", "mla_decode", "MlaLayer", "MlaConfig", "MoeLayer", "MoeConfig", "moe_router", "LlamaModel", "LlamaConfig", "LlamaLayerWeights", "Comm", "Graph", "QuantComputeDevice", "QuantizedQ4", "QuantizedQ8", "Buffer", "QBuffer", "TangqError", "load",
           "F32", "BF16", "F16", "I8", "U8", "I32", "F64", "Q4_F32", "Q4_F16", "Q8_F32", "I8_ROW"]
