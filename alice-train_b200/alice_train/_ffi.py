"""ctypes binding of libalice_b200.so (declarations follow include/alice_b200.h).

Loading fails loudly when the shared object has not been built; creating a context fails
loudly when there is no B200.  There is no CPU path behind this module.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libalice_b200.so")

AB_OK = 0
AB_ERR_NULL, AB_ERR_SHAPE, AB_ERR_ALIGN, AB_ERR_CUDA = 1, 2, 3, 4
AB_ERR_DEVICE_TIMEOUT, AB_ERR_UNSUPPORTED, AB_ERR_NO_DEVICE, AB_ERR_STATE = 5, 6, 7, 8
AB_F32, AB_BF16 = 0, 1
AB_TERNARY, AB_BINARY2, AB_INT4, AB_INT8 = 0, 1, 2, 3
AB_GUARD_INV_ZERO, AB_GUARD_FLOOR = 0, 1
AB_OPT_EXACT_MATVEC, AB_OPT_ASYNC_HOST_STEP, AB_OPT_HOST_INTEGER_MATVEC, AB_OPT_GEMM_OPERAND_FORM = 1, 2, 3, 4
AB_XCHG_ALLREDUCE_F32, AB_XCHG_ALLGATHER, AB_XCHG_REDUCESCATTER_BF16 = 0, 1, 2


class FqReport(C.Structure):
    _fields_ = [("gamma", C.c_float), ("sum_abs", C.c_double), ("n", C.c_uint64),
                ("n_plus", C.c_uint64), ("n_minus", C.c_uint64), ("n_threshold", C.c_uint64),
                ("sum_err", C.c_double), ("dot_wq", C.c_double), ("dot_ww", C.c_double),
                ("dot_qq", C.c_double), ("w_min", C.c_float), ("w_max", C.c_float)]


_vp, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float


class LinearStep(C.Structure):
    """ab_linear_step of the header: one linear of ab_qat_linear_steps."""
    _fields_ = [("w", C.c_void_p), ("w_latent", C.c_void_p), ("x_bf16", C.c_void_p), ("dy_bf16", C.c_void_p),
                ("xq", C.c_void_p), ("scales", C.c_void_p), ("rowsums", C.c_void_p), ("y_bf16", C.c_void_p),
                ("dx_bf16", C.c_void_p), ("dW", C.c_void_p), ("dw_beta", C.c_float), ("dw_multicast", C.c_void_p),
                ("flags_local", C.c_void_p), ("flags_multicast", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/alice_b200.h declares
SIGNATURES = {
    "ab_ctx_create": (_i, [_i, _vp, C.POINTER(_vp)]),
    "ab_ctx_set_option": (_i, [_vp, _i, _i]),
    "ab_ctx_destroy": (_i, [_vp]),
    "ab_ctx_sync": (_i, [_vp]),
    "ab_ctx_stream": (_vp, [_vp]),
    "ab_ctx_last_error": (C.c_char_p, [_vp]),
    "ab_ctx_launch_count": (C.c_uint64, [_vp]),
    "ab_status_str": (C.c_char_p, [_i]),
    "ab_device_count": (_i, []),
    "ab_weights_create": (_i, [_vp, _sz, _sz, C.POINTER(_vp)]),
    "ab_weights_destroy": (_i, [_vp]),
    "ab_weights_out_features": (_sz, [_vp]),
    "ab_weights_in_features": (_sz, [_vp]),
    "ab_weights_words_per_row": (_sz, [_vp]),
    "ab_weights_set_ternary": (_i, [_vp, _vp, _sz]),
    "ab_weights_set_bitplanes": (_i, [_vp, _vp, _vp, _sz]),
    "ab_weights_get_bitplanes": (_i, [_vp, _vp, _vp, _sz]),
    "ab_weights_set_packed2b": (_i, [_vp, _vp, _sz, _f]),
    "ab_weights_get_packed2b": (_i, [_vp, _vp, _sz]),
    "ab_weights_get_ternary": (_i, [_vp, _vp, _sz]),
    "ab_weights_set_gamma": (_i, [_vp, _f]),
    "ab_weights_get_gamma": (_i, [_vp, C.POINTER(_f)]),
    "ab_fq_absmean_pack": (_i, [_vp, _vp, _vp, _vp, _i, _i]),
    "ab_fq_merge_quantize_alpha": (_i, [_vp, _vp, _vp, _vp, _sz, _f, _f, C.POINTER(_f), C.POINTER(C.c_double)]),
    "ab_fq_shard_abs_sum": (_i, [_vp, _vp, _vp, _vp]),
    "ab_fq_shard_pack": (_i, [_vp, _vp, _vp, _vp, _sz, _vp, _i, _i]),
    "ab_sgd_step_fq": (_i, [_vp, _vp, _vp, _sz, _f, _f, _vp, _i, _vp]),
    "ab_adamw_step_fq": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _f, _f, _f, _f, _f, _f, _f, _vp, _i, _vp]),
    "ab_weights_fq_report": (_i, [_vp, C.POINTER(FqReport)]),
    "ab_dp_allreduce_start": (_i, [_vp, _vp, _sz, _vp, _vp, _i, _i, C.c_uint32, _i]),
    "ab_dp_allreduce_wait": (_i, [_vp]),
    "ab_switch_exchange_start": (_i, [_vp, _i, _vp, _vp, _vp, _sz, _vp, _vp, _i, _i, C.c_uint32, _i]),
    "ab_quantize_and_pack_host": (_i, [_vp, _vp, _sz, C.POINTER(_f), _vp]),
    "ab_calibrate_scale": (_i, [_vp, _vp, _sz, _vp]),
    "ab_fake_quantize_forward": (_i, [_vp, _vp, _vp, _sz, _vp, _f, _i]),
    "ab_ste_backward": (_i, [_vp, _vp, _vp, _sz, _f]),
    "ab_calibration_stats": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "ab_calibrate_scale_host": (_i, [_vp, _vp, _sz, C.POINTER(_f)]),
    "ab_fake_quantize_forward_host": (_i, [_vp, _vp, _sz, _vp, _sz, _f, _f, _i]),
    "ab_ste_backward_host": (_i, [_vp, _vp, _sz, _vp, _sz, _f]),
    "ab_calibration_stats_host": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "ab_ternary_matvec": (_i, [_vp, _vp, _vp, _vp]),
    "ab_ternary_matvec_backward": (_i, [_vp, _vp, _vp, _vp]),
    "ab_ternary_matvec_backward_static": (_i, [_vp, _vp, _vp, _vp]),
    "ab_bitlinear_backward": (_i, [_vp, _vp, _vp, _vp, _i, _f, _vp, _vp]),
    "ab_ste_weight_grad": (_i, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "ab_ternary_matmul_bt": (_i, [_vp, _vp, _vp, _f, _vp, _sz]),
    "ab_lm_head_logits": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _sz, _sz, _vp, _i, _sz]),
    "ab_cross_entropy": (_i, [_vp, _vp, _i, _sz, _vp, _sz, _sz, _f, _vp, _vp, _sz, _vp, _sz]),
    "ab_lm_head_backward": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _f]),
    "ab_matmul_bt_dense_host": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, _sz, _sz, _sz]),
    "ab_matmul_nn_dense_host": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, _sz, _sz, _sz]),
    "ab_ternary_matvec_ex": (_i, [_vp, _vp, _vp, _vp, _f, _vp, _i]),
    "ab_ternary_swiglu_ffn_host": (_i, [_vp, _vp, _vp, _f, _vp, _f, _vp, _f, _vp, _vp, _vp, _sz, _sz, _sz]),
    "ab_ternary_swiglu_ffn": (_i, [_vp, _vp, _vp, _f, _vp, _f, _vp, _f, _vp, _vp, _vp, _sz]),
    "ab_ternary_matvec_host": (_i, [_vp, _vp, _vp, _sz, _vp, _sz]),
    "ab_ternary_matvec_backward_host": (_i, [_vp, _vp, _vp, _sz, _vp, _sz]),
    "ab_bitlinear_backward_host": (_i, [_vp, _vp, _vp, _sz, _vp, _sz, _i, _f, _vp, _sz, _vp, _sz]),
    "ab_ste_weight_grad_host": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _sz]),
    "ab_ternary_matmul_bt_host": (_i, [_vp, _vp, _vp, _f, _vp, _sz, _sz, _sz]),
    "ab_act_quant_int8": (_i, [_vp, _vp, _i, _sz, _sz, _sz, _vp, _sz, _vp, _vp]),
    "ab_rmsnorm_act_quant": (_i, [_vp, _vp, _i, _vp, _sz, _sz, _sz, _f, _vp, _i, _sz, _vp, _sz, _vp, _vp]),
    "ab_swiglu_act_quant": (_i, [_vp, _vp, _vp, _i, _sz, _sz, _sz, _vp, _i, _sz, _vp, _sz, _vp, _vp]),
    "ab_rmsnorm_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _f]),
    "ab_swiglu_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz]),
    "ab_bitlinear_fwd": (_i, [_vp, _vp, _vp, _sz, _vp, _vp, _sz, _vp, _i, _sz, _vp]),
    "ab_matmul_bt_host": (_i, [_vp, _vp, _sz, _vp, _vp, _sz, _sz]),
    "ab_matmul_nn_host": (_i, [_vp, _vp, _sz, _vp, _vp, _sz, _sz]),
    "ab_matmul_tn_host": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, _sz, _sz, _sz]),
    "ab_bitlinear_fwd_bf16": (_i, [_vp, _vp, _vp, _sz, _sz, _vp, _i, _sz, _f]),
    "ab_bitlinear_dx": (_i, [_vp, _vp, _vp, _sz, _sz, _vp, _i, _sz, _f]),
    "ab_ste_dw": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _sz, _sz, _vp, _sz, _f]),
    "ab_bitlinear_step_host": (_i, [_vp, _vp, _vp, _vp, _sz, _vp, _vp, _vp]),
    "ab_qat_linear_steps": (_i, [_vp, _vp, _sz, _sz, _i, _i, _i, C.c_uint32, _i]),
    "ab_tensor_peak_probe": (_i, [_vp, _i, _i, C.POINTER(C.c_double)]),
    "ab_selftest_bounded_wait": (_i, [_vp, C.c_uint32]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with "
                               f"`python alice-train_b200/build.py` (no CPU fallback exists)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class AliceB200Error(RuntimeError):
    def __init__(self, status: int, detail: str = ""):
        self.status = status
        msg = load().ab_status_str(status).decode()
        super().__init__(f"alice_b200 status {status} ({msg})" + (f": {detail}" if detail else ""))


def check(status: int, ctx=None):
    if status != AB_OK:
        detail = ""
        if ctx is not None and status in (AB_ERR_CUDA, AB_ERR_DEVICE_TIMEOUT):
            detail = load().ab_ctx_last_error(ctx).decode()
        raise AliceB200Error(status, detail)
