"""ctypes loader of libsp_moe_b200.so (the C ABI in include/sp_engine/moe_backend.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libsp_moe_b200.so")

# every symbol include/sp_engine/moe_backend.h declares
EXPORTS = ("sp_last_error", "sp_set_error", "sp_moe_open", "sp_moe_close", "sp_moe_upload_layer",
           "sp_moe_upload_layer_dev", "sp_moe_device_bytes", "sp_moe_forward", "sp_moe_forward_dev",
           "sp_moe_status", "gemma4_moe_ffn_q4b_cuda", "sp_moe_q4b_quantize_dev",
           "sp_moe_q4b_dequantize_dev", "sp_moe_gemv_q4b_dev", "sp_moe_gemv_q4b_static_dev", "sp_moe_gelu_mul_dev", "sp_moe_kernel_launches",
           "sp_moe_ep_route_dev", "sp_moe_ep_recv_layout_dev", "sp_moe_ep_shared_dev", "sp_moe_ep_experts_dev", "sp_moe_ep_finish_dev",
           "sp_moe_ext_open", "sp_moe_ext_close", "sp_moe_ext_upload_experts", "sp_moe_ext_moe",
           "sp_frob_matmul_q8_dev", "sp_frob_matmul_q4_dev", "sp_moe_decode_timing", "sp_moe_debug_wait_timeout", "sp_moe_set_router_bias_dev", "sp_moe_load_sp_model",
           "sp_moe_ep_forward_dev", "sp_moe_ep_last_rows", "sp_moe_ep_timing", "sp_moe_ep_unique_id", "sp_moe_ep_comm_create", "sp_moe_ep_comm_destroy")


class SpMoeConfig(C.Structure):
    _fields_ = [("E", C.c_int32), ("NE", C.c_int32), ("NU", C.c_int32), ("FFE", C.c_int32),
                ("FFS", C.c_int32), ("n_layers", C.c_int32), ("max_tokens", C.c_int32),
                ("device", C.c_int32), ("eps", C.c_float), ("max_expert_rows", C.c_int32),
                ("reserved", C.c_int32 * 6)]


_PTR_FIELDS = ("router_w", "router_scale", "router_bias", "ffn_norm", "post_ffw1", "pre_ffw2",
               "post_ffw2", "post_ffw", "dexps_scale", "gu_codes", "gu_bs", "dn_codes", "dn_bs",
               "sg_codes", "sg_bs", "su_codes", "su_bs", "sd_codes", "sd_bs")


class SpMoeLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in _PTR_FIELDS]


class SpMoeTiming(C.Structure):
    _fields_ = [("wait_us", C.c_float * 3), ("prologue_us", C.c_float * 3), ("rows_us", C.c_float * 3),
                ("layer_us", C.c_float), ("raw_us", (C.c_float * 16) * 3)]


class SpMoeError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"sp_moe error {code}: {text}")
        self.code = code
        self.text = text


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m kairos_engine_b200.build` "
                               "(there is no fallback implementation)")
        L = C.CDLL(LIB_PATH)
        L.sp_last_error.restype = C.c_char_p
        L.sp_set_error.argtypes = [C.c_char_p]
        L.sp_moe_open.argtypes = [C.POINTER(SpMoeConfig), C.POINTER(C.c_void_p)]
        L.sp_moe_close.argtypes = [C.c_void_p]
        L.sp_moe_upload_layer.argtypes = [C.c_void_p, C.c_int, C.POINTER(SpMoeLayerWeights)]
        L.sp_moe_upload_layer_dev.argtypes = [C.c_void_p, C.c_int, C.POINTER(SpMoeLayerWeights)]
        L.sp_moe_device_bytes.argtypes = [C.c_void_p]
        L.sp_moe_device_bytes.restype = C.c_size_t
        L.sp_moe_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sp_moe_forward_dev.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sp_moe_status.argtypes = [C.c_void_p]
        L.gemma4_moe_ffn_q4b_cuda.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float] + [C.c_void_p] * 9
        L.sp_moe_q4b_quantize_dev.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sp_moe_q4b_dequantize_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
        L.sp_moe_gemv_q4b_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sp_moe_gemv_q4b_static_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sp_moe_gelu_mul_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
        L.sp_moe_kernel_launches.argtypes = [C.c_void_p]
        L.sp_moe_ep_route_dev.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 8 + [C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.sp_moe_ep_recv_layout_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sp_moe_ep_shared_dev.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.sp_moe_ep_experts_dev.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 5
        L.sp_moe_ep_finish_dev.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 5
        L.sp_moe_kernel_launches.restype = C.c_uint64
        L.sp_moe_ext_open.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
        L.sp_moe_ext_close.argtypes = [C.c_void_p]
        L.sp_moe_ext_upload_experts.argtypes = [C.c_void_p, C.c_char_p] + [C.c_void_p] * 6 + [C.c_int] * 3
        L.sp_moe_ext_moe.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.sp_frob_matmul_q8_dev.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
        L.sp_frob_matmul_q4_dev.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p]
        L.sp_moe_decode_timing.argtypes = [C.c_void_p, C.POINTER(SpMoeTiming)]
        L.sp_moe_debug_wait_timeout.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.sp_moe_set_router_bias_dev.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.sp_moe_load_sp_model.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
        L.sp_moe_ep_forward_dev.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 6 + [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.sp_moe_ep_last_rows.argtypes = [C.c_void_p]
        L.sp_moe_ep_last_rows.restype = C.c_longlong
        L.sp_moe_ep_timing.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
        L.sp_moe_ep_timing.restype = C.c_int
        L.sp_moe_ep_unique_id.argtypes = [C.c_void_p]
        L.sp_moe_ep_comm_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        L.sp_moe_ep_comm_destroy.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise SpMoeError(rc, (lib().sp_last_error() or b"").decode("utf-8", "replace"))
