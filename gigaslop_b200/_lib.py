"""ctypes binding of libgigaslop_b200.so -- the only way the Python host code
reaches the device kernels.  There is no fallback: a missing library is an error."""
import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GIGASLOP_B200_LIB") or os.path.join(_PKG, "libgigaslop_b200.so")

OK = 0
ERRORS = {-1: "bad argument", -2: "unsupported shape", -3: "device is not sm_100"}

F16, F32 = 0, 1
FLAG_SCALAR_SCALE_B = 4
FLAG_OWN_ROW_BLOCKS = 8

_i32, _i64, _p = C.c_int32, C.c_int64, C.c_void_p

SIGNATURES = {
    "gsb200_version": (C.c_char_p, []),
    "gsb200_init": (_i32, []),
    "gsb200_device_status": (_i32, [C.POINTER(C.c_uint32)]),
    "gsb200_set_spin_budget": (_i32, [C.c_uint32]),
    "gsb200_set_sm_limit": (_i32, [_i32]),
    "gsb200_set_gemm_variant": (_i32, [_i32, _i32]),
    "gsb200_selftest_wait_timeout": (_i32, [_p]),
    "gsb200_tensor_peak_probe": (_i32, [_i32, _i32, _i32, _p, C.POINTER(C.c_int32), _p]),
    "gsb200_tensor_map_encodes": (_i64, []),
    "gsb200_ptq_int8": (_i32, [_p, _i32, _i64, _p, _i64, _p, _i64, _i32, _p]),
    "gsb200_ptq_fp8": (_i32, [_p, _i32, _i64, _p, _i64, _p, _i64, _i32, _i32, _p]),
    "gsb200_gemm_i8_i32": (_i32, [_p, _i64, _p, _i64, _p, _i64, _i64, _i32, _i32, _p]),
    "gsb200_gemm_i8_f16": (_i32, [_p, _i64, _p, _i64, _p, _i64, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "gsb200_gemm_i8_rotary_f16": (_i32, [_p, _i64, _p, _i64, _p, _i64, _p, _p, _p, _p, _i64, _i32, _i32,
                                         _i32, _i32, _i32, _i32, _i64, _i32, _p]),
    "gsb200_ptq_gemm_i8_rotary_f16": (_i32, [_p, _i64, _p, _i64, _p, _i64, _p, _p, _p, _p, _i64, _i32, _i32,
                                             _i32, _i32, _i32, _i32, _i64, _i32, _p]),
    "gsb200_dual_gemm_i8_silu_f16": (_i32, [_p, _i64, _p, _p, _i64, _p, _i64, _p, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "gsb200_gemm_fp8_f16": (_i32, [_p, _i64, _p, _i64, _p, _i64, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "gsb200_gemm_fp8_rotary_f16": (_i32, [_p, _i64, _p, _i64, _p, _i64, _p, _p, _p, _p, _i64, _i32, _i32,
                                          _i32, _i32, _i32, _i32, _i64, _i32, _p]),
    "gsb200_gemm_f16_f16": (_i32, [_p, _i64, _p, _i64, _p, _i64, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "gsb200_module_cuda_init": (None, [_p]),
    "gsb200_module_cuda_load_to_device": (None, [_p]),
    "gsb200_fac_gemm_fp8_f16": (_i32, [_p, _i64, _p, _p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i32, _i32, _i32, _p]),
    "gsb200_factored_lstm_step": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "gsb200_mx_tiled_scale_bytes": (_i64, [_i64, _i32]),
    "gsb200_mx_scales_to_tiled": (_i32, [_p, _i64, _i64, _i32, _p, _p]),
    "gsb200_gemm_mxfp8_f16": (_i32, [_p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i32, _i32, _p]),
    "gsb200_dual_gemm_mxfp8_silu_f16": (_i32, [_p, _i64, _p, _p, _p, _i64, _p, _p, _p, _i64, _i64, _i32, _i32, _p]),
    "gsb200_lstm_scratch_bytes": (_i64, [_i64, _i32]),
    "gsb200_lstm_layer_fp8": (_i32, [_p, _i64, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32, _i32, _p, _i64, _p]),
    "gsb200_lstm_layer_fp8_static": (_i32, [_p, _i64, _p, _i64, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32, _i32, _p]),
    "gsb200_lstm_stack_workspace_bytes": (_i64, [_i64, _i64, _i32, _i32]),
    "gsb200_lstm_stack_fp8": (_i32, [_p, _i64, _p, _i32, _p, _i32, _i32, _p, _i64, _i64, _i32, _i32, _p, _i64, _p, _p]),
    "gsb200_ptq_mxfp8": (_i32, [_p, _i32, _i64, _p, _i64, _p, _i64, _i64, _i32, _p]),
    "gsb200_dual_gemm_fp8_silu_mxfp8": (_i32, [_p, _i64, _p, _p, _i64, _p, _i64, _p, _i64, _p, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "gsb200_dual_gemm_fp8_silu_f16": (_i32, [_p, _i64, _p, _p, _i64, _p, _i64, _p, _p, _p, _i64, _i32, _i32, _i32, _p]),
}



class LstmLayer(C.Structure):
    """``gsb200_lstm_layer_t``: the weights of one layer of the LSTM stack (device pointers)."""
    _fields_ = [("w_ih", _p), ("ld_w_ih", _i64), ("s_ih", _p), ("w_hh", _p), ("ld_w_hh", _i64), ("s_hh", _p),
                ("bias", _p)]


_lib = None


def lib():
    """The loaded library (loads on first use; raises if it was never built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m gigaslop_b200.build` "
                "(nvcc, sm_100a). gigaslop_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)      # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status, what):
    if status == OK:
        return
    if status < 0:
        raise RuntimeError(f"gigaslop_b200.{what}: {ERRORS.get(status, 'error')} (status {status})")
    raise RuntimeError(f"gigaslop_b200.{what}: CUDA error {status}")


def device_status():
    """Read-and-clear the device status word: (flags, where, spin_budget, reserved)."""
    buf = (C.c_uint32 * 4)()
    check(lib().gsb200_device_status(buf), "device_status")
    return tuple(int(v) for v in buf)
