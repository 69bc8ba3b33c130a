"""trinix_b200 — B200 (sm_100a) backend for Trinix's layer forward hot path.

Hand-written CUDA kernels behind a C ABI (include/trinix_b200.h), reached through
kernel classes with the reference's names (`kernels`), its functional attention entry
point (`functional.triton_attn_func`), mirror modules (`layers`) and `install()`, which
patches an installed Trinix in place. CUDA tensors only; no fallback paths.
"""
from .functional import flash_attn_func, triton_attn_func
from .fusion import FastFusedRMSNormInt8, RowwiseInt8Quant, fuse, register_fusion
from .install import install, uninstall
from .kernels import (
    RowwiseInt8Kernel,
    TritonAttentionKernel,
    TritonFusedResidualLayerNormKernel,
    TritonFusedResidualRMSNormKernel,
    TritonFusedRMSNormActivationKernel,
    TritonGeGLUKernel,
    TritonLayerNormKernel,
    TritonReGLUKernel,
    TritonRMSNormKernel,
    TritonRoPEKernel,
    TritonSwiGLUKernel,
)
from .layers import (
    FastALiBiPositionEmbedding,
    FastBaseAttention,
    FastFusedResidualLayerNorm,
    FastFusedResidualRMSNorm,
    FastFusedRMSNormActivation,
    FastGeGLU,
    FastGroupedQueryAttention,
    FastLayerNorm,
    FastMultiQueryAttention,
    FastReGLU,
    FastRMSNorm,
    FastRoPEPositionEmbedding,
    FastSwiGLU,
)
from .ops import (
    attention,
    attention_status,
    dequantize_rowwise,
    glu,
    glu_backward,
    glu_pair,
    layernorm,
    layernorm_backward,
    quantize_rowwise,
    residual_layernorm,
    residual_rmsnorm,
    residual_rmsnorm_quantize,
    rmsnorm,
    rmsnorm_activation,
    rmsnorm_backward,
    rmsnorm_quantize,
    rope,
)

__version__ = "0.1.0"
