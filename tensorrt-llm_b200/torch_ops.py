"""Loads the C++ ``torch.ops.trtllm`` registrations of this library (csrc/trtllm_ops.cpp).

The five host-side ops keep the schemas of cpp/tensorrt_llm/thop/weightOnlyQuantOp.cpp:358-385 of
TensorRT-LLM. The two GEMM ops are new (that reference version ships no weight-only GEMM torch op);
they follow the conventions of its other GEMM ops (cpp/tensorrt_llm/thop/cutlassScaledMM.cpp:121-175):
CUDA tensors in, output allocated on the input's device, current stream. All seven are registered
from C++ with TORCH_LIBRARY_FRAGMENT / TORCH_LIBRARY_IMPL; this module only loads the shared object
(built in-tree by csrc/build_ops.sh) and raises if it is missing: there is no Python fallback.
"""
from __future__ import annotations

import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
OPS_LIB_PATH = os.path.join(_HERE, "libtrtllm_ops.so")
_loaded = False


def register() -> None:
    global _loaded
    if _loaded:
        return
    if not os.path.exists(OPS_LIB_PATH):
        raise ImportError(f"{OPS_LIB_PATH} is missing: build it with tensorrt-llm_b200/csrc/build.sh and "
                          "tensorrt-llm_b200/csrc/build_ops.sh (there is no fallback path)")
    torch.ops.load_library(OPS_LIB_PATH)
    _loaded = True


register()
