"""B200-native weight-only quantised GEMM (W4A16 / W8A16): a drop-in for the
WeightOnlyQuantMatmul / WeightOnlyGroupwiseQuantMatmul path of TensorRT-LLM.

    ops        GPU entry points (functional form + plugin mirrors) over the C ABI
    quantize   host-side quantise / pack / layout ops with the reference's names
    torch_ops  registers both under torch.ops.trtllm.*
    mapping    tensor-parallel rank math (Mapping)
    tp         column / row-parallel linears, the peer-memory all-reduce helper
    checkpoint GPTQ / AutoAWQ tensors -> the library's tensors and layers
"""
from . import _lib, ops, quantize  # noqa: F401
from ._lib import (BIAS, FP8_ALPHA, INT8_WEIGHT, PRE_QUANT_SCALE, W4_REGIME_AUTO, W4_REGIME_GEMM,  # noqa: F401
                   W4_REGIME_GEMV, ZERO, W4Error)
from .ops import (WeightOnlyGroupwiseQuantMatmulPlugin, WeightOnlyQuantMatmulPlugin,  # noqa: F401
                  weight_only_groupwise_quant_matmul, weight_only_quant_matmul)

__version__ = "0.1.0"
