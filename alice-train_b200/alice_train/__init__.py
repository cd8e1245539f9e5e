"""alice_train — host-side mirror of the reference crate's BitLinear API over libalice_b200.

Names follow the crate's re-exports (src/lib.rs:130-156): ternary_matvec_backward,
bitlinear_backward, ste_weight_grad, FakeQuantize, QatConfig, QatTrainer, QuantBits,
CalibrationStats, QatEpochResult, pack_ternary, unpack_ternary, quantize_and_pack, dequantize,
blas.ternary_matmul_bt, GpuContext.  Importing this package never touches a GPU; the first call
that needs one creates the default context and raises if no B200 is present.
"""
from . import _ffi, blas
from .backward import bitlinear_backward, ste_weight_grad, ternary_matvec_backward, ternary_matvec_kernel
from .context import GpuContext, default_context, set_default_context
from .cuda_matmul import CudaMatmul, GpuBackwardEngine, blas_matmul_bt, blas_matmul_nn, init_cuda_blas
from .export import dequantize, pack_ternary, quantize_and_pack, unpack_ternary
from .ops import TernaryWeightKernel
from .qat import CalibrationStats, FakeQuantize, QatConfig, QatEpochResult, QatTrainer, QuantBits

__all__ = [
    "GpuContext", "default_context", "set_default_context", "TernaryWeightKernel",
    "ternary_matvec_backward", "ternary_matvec_kernel", "bitlinear_backward", "ste_weight_grad",
    "FakeQuantize", "QatConfig", "QatTrainer", "QuantBits", "CalibrationStats", "QatEpochResult",
    "pack_ternary", "unpack_ternary", "quantize_and_pack", "dequantize", "blas",
    "CudaMatmul", "GpuBackwardEngine", "blas_matmul_bt", "blas_matmul_nn", "init_cuda_blas",
]
