"""alice_train — host-side mirror of the reference crate's BitLinear API over libalice_b200.

Names follow the crate's re-exports (src/lib.rs:130-156): ternary_matvec_backward,
bitlinear_backward, ste_weight_grad, FakeQuantize, QatConfig, QatTrainer, QuantBits,
CalibrationStats, QatEpochResult, pack_ternary, unpack_ternary, quantize_and_pack, dequantize,
blas.ternary_matmul_bt, GpuContext; export_alice_model / read_alice_meta / read_*_layer (src/export.rs:279-683)
and StreamingAliceModel (src/inference.rs:976).  Importing this package never touches a GPU; the first call
that needs one creates the default context and raises if no B200 is present.
"""
from . import _ffi, blas
from .backward import bitlinear_backward, ste_weight_grad, ternary_matvec_backward, ternary_matvec_kernel
from .context import GpuContext, default_context, set_default_context
from .cuda_matmul import CudaMatmul, GpuBackwardEngine, blas_matmul_bt, blas_matmul_nn, init_cuda_blas
from .export import (AliceModelMeta, LayerScales, Qwen35Config, dequantize, export_alice_model, pack_ternary, quantize_and_pack,
                     read_alice_meta, read_deltanet_layer, read_embedding, read_fullattn_layer, read_lm_head, read_output_norm,
                     unpack_ternary)
from .inference import StreamingAliceModel
from .ops import TernaryWeightKernel
from .qat import CalibrationStats, FakeQuantize, QatConfig, QatEpochResult, QatTrainer, QuantBits

__all__ = [
    "GpuContext", "default_context", "set_default_context", "TernaryWeightKernel",
    "ternary_matvec_backward", "ternary_matvec_kernel", "bitlinear_backward", "ste_weight_grad",
    "FakeQuantize", "QatConfig", "QatTrainer", "QuantBits", "CalibrationStats", "QatEpochResult",
    "pack_ternary", "unpack_ternary", "quantize_and_pack", "dequantize", "blas",
    "CudaMatmul", "GpuBackwardEngine", "blas_matmul_bt", "blas_matmul_nn", "init_cuda_blas",
    "Qwen35Config", "AliceModelMeta", "LayerScales", "export_alice_model", "read_alice_meta", "read_embedding",
    "read_output_norm", "read_lm_head", "read_deltanet_layer", "read_fullattn_layer", "StreamingAliceModel",
]
