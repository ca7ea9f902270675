"""rust_ascend_b200 — host-side mirror of rust-ascend's runtime and `nn` operator surface on top of
libruda_b200.so (hand-written sm_100a CUDA kernels behind a C ABI).

`runtime` mirrors rust-ascend-driver/src/tensor/runtime/mod.rs (AscendRuntime, ComputeClient,
TensorBuffer, RuntimeOptions, CannError); `nn` mirrors src/nn.rs and src/nn/*.rs; `distributed`
mirrors src/distributed.rs with NCCL in place of HCCL.
"""
from . import nn
from .runtime import (B200Device, B200Error, B200Runtime, ComputeClient, DType, InvalidTensor, RotaryLayout,
                      RuntimeOptions, ServerUnhealthy, TensorBuffer, Transpose)

__all__ = ["B200Device", "B200Error", "B200Runtime", "ComputeClient", "DType", "InvalidTensor", "RotaryLayout",
           "RuntimeOptions", "ServerUnhealthy", "TensorBuffer", "Transpose"]
