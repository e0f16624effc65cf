"""ctypes binding of libb200i.so, the CUDA library behind this package.

There is no CPU fallback: if the library is missing, or no CUDA device is
visible when a computation is asked for, the call raises. The C ABI is
declared in include/b200i.h.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
#: MOJOLEARN_B200_LIB overrides the in-tree library (a differently built libb200i.so with the same ABI).
LIB_PATH = os.environ.get("MOJOLEARN_B200_LIB") or os.path.join(_HERE, "csrc", "libb200i.so")
ERR_CAP = 512

_lib = None


class NativeError(RuntimeError):
    """The CUDA library refused a call or a CUDA runtime call failed."""


def lib():
    """The loaded library. Raises if it has not been built (python -m mojolearn_b200.csrc.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeError(
                "mojolearn_b200: %s is missing; build it with `python -m mojolearn_b200.csrc.build` "
                "(there is no CPU fallback)" % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


I64, VP, CP, F64 = ctypes.c_int64, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_double

#: name -> argument types, as declared in include/b200i.h (all return int64 unless noted)
SIGNATURES = {
    "b200i_abi": [],
    "b200i_numeric_mode": [],
    "b200i_profile_version": [],
    "b200i_lowbit_profile_version": [],
    "b200i_device_count": [],
    "b200i_launch_count": [],
    "b200i_workspace_bytes": [I64, I64, I64],
    "b200i_plan_workspace_bytes": [I64, I64, I64, I64, I64],
    "b200i_kernel_timing": [I64],
    "b200i_kernel_timing_read": [VP, VP],
    "b200i_decode_plan_fits": [I64, I64, I64, I64, I64],
    "b200i_gemm_f32": [I64, VP, VP, VP, VP, I64, I64, I64, I64, VP, I64, VP, I64],
    "b200i_gemm_f32_noalloc": [I64, VP, VP, VP, VP, I64, I64, I64, I64, VP, I64],
    "b200i_gemm_w": [I64, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, VP, I64, VP, I64],
    "b200i_gemm_w_epilogue": [I64, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, VP, I64, I64, I64, VP, I64, VP, I64],
    "b200i_gemm_w_nodes": [I64, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, VP, I64, VP, I64, VP, VP, I64],
    "b200i_gemm_w_plan": [I64, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, I64, I64, VP, I64, VP, I64],
    "b200i_to_bf16": [I64, VP, VP, VP, I64, VP, I64],
    "b200i_from_bf16": [I64, VP, VP, VP, I64, VP, I64],
    "b200i_quantize_int8": [I64, VP, VP, VP, VP, I64, I64, VP, I64],
    "b200i_dequantize_int8": [I64, VP, VP, VP, VP, I64, I64, VP, I64],
    "b200i_attention_scratch_floats": [I64, I64, I64, I64],
    "b200i_gemm_int8": [I64, VP, VP, VP, VP, VP, VP, I64, I64, I64, VP, I64],
    "b200i_quantize_int15": [I64, VP, VP, VP, VP, VP, I64, I64, VP, I64],
    "b200i_dequantize_int15": [I64, VP, VP, VP, VP, VP, I64, I64, VP, I64],
    "b200i_gemm_int15": [I64, VP, VP, VP, VP, VP, VP, VP, VP, I64, I64, I64, VP, I64],
    "b200i_host_quantize_int15": [I64, VP, VP, VP, VP, I64, I64, VP, I64],
    "b200i_host_dequantize_int15": [I64, VP, VP, VP, VP, I64, I64, VP, I64],
    "b200i_host_gemm_int15": [I64, VP, VP, VP, VP, VP, VP, VP, I64, I64, I64, VP, I64],
    "b200i_host_gemm_w": [I64, VP, VP, VP, VP, I64, I64, I64, I64, I64, VP, I64],
    "b200i_host_to_bf16": [I64, VP, VP, I64, VP, I64],
    "b200i_host_from_bf16": [I64, VP, VP, I64, VP, I64],
    "b200i_host_quantize_int8": [I64, VP, VP, VP, I64, I64, VP, I64],
    "b200i_host_dequantize_int8": [I64, VP, VP, VP, I64, I64, VP, I64],
    "b200i_host_gemm_int8": [I64, VP, VP, VP, VP, VP, I64, I64, I64, VP, I64],
    "b200i_decode_status": [I64],
    "b200i_debug_set_status": [I64, I64],
    "b200i_noalloc_scratch_bytes": [I64, I64, I64],
    "b200i_norm": [I64, VP, VP, VP, VP, VP, I64, I64, F64, I64, VP, I64],
    "b200i_add_norm": [I64, VP, VP, VP, VP, VP, VP, VP, I64, I64, F64, I64, VP, I64],
    "b200i_qkv_rope_cache": [I64, VP, VP, VP, VP, VP, VP, VP, I64, VP, VP, I64, I64, I64, I64, I64, I64, I64, VP, I64, VP, I64],
    "b200i_rope_table_opts": [I64, VP, VP, VP, I64, VP, I64, I64, F64, I64, F64, F64, F64, I64, VP, I64],
    "b200i_rope_table": [I64, VP, VP, VP, I64, I64, I64, F64, VP, I64],
    "b200i_rope_apply": [I64, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, I64, VP, I64],
    "b200i_kv_append": [I64, VP, VP, VP, I64, I64, I64, I64, I64, I64, I64, VP, I64],
    "b200i_attention": [I64, VP, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, I64, I64, I64, F64, VP, I64],
    "b200i_act_mul": [I64, VP, VP, VP, VP, I64, I64, I64, I64, I64, VP, I64],
    "b200i_pair_epilogue_fits": [I64, I64, I64, I64],
    "b200i_add": [I64, VP, VP, VP, VP, I64, VP, I64],
    "b200i_bias_add": [I64, VP, VP, VP, I64, I64, VP, I64],
    "b200i_embedding": [I64, VP, VP, VP, VP, I64, I64, I64, VP, VP, I64],
    "b200i_add_positions": [I64, VP, VP, VP, I64, I64, I64, I64, VP, I64],
    "b200i_argmax": [I64, VP, VP, VP, I64, I64, VP, I64],
    "b200i_rope_table_at": [I64, VP, VP, VP, VP, I64, I64, F64, VP, I64],
    "b200i_kv_append_at": [I64, VP, VP, VP, I64, I64, I64, I64, I64, VP, I64, VP, I64],
    "b200i_attention_at": [I64, VP, VP, VP, VP, VP, VP, I64, I64, I64, I64, I64, I64, VP, I64, F64, VP, I64],
    "b200i_add_positions_at": [I64, VP, VP, VP, I64, I64, VP, I64, VP, I64],
    "b200i_advance_position": [I64, VP, VP, I64, VP, I64],
    "b200i_ffma_probe": [I64, VP, VP, I64, I64, I64, VP, I64],
    "b200i_comm_create": [I64, I64, I64, I64, VP, VP, I64],
    "b200i_comm_export": [VP, VP, I64, VP, I64],
    "b200i_comm_attach": [VP, I64, VP, VP, I64],
    "b200i_comm_attach_local": [VP, I64, VP, VP, I64],
    "b200i_comm_advance": [VP, VP, VP, I64],
    "b200i_comm_gather": [VP, VP, I64, I64, VP, I64, VP, I64, I64, I64, VP, I64],
    "b200i_comm_gather_nodes": [VP, VP, I64, I64, VP, I64, VP, I64, I64, I64, VP, I64, VP, I64],
    "b200i_comm_destroy": [VP],
}
STRING_FUNCTIONS = ["b200i_numerical_profile", "b200i_vendor"]
POINTER_FUNCTIONS = {}


def _declare(l):
    for name, args in SIGNATURES.items():
        fn = getattr(l, name)
        fn.restype = I64
        fn.argtypes = args
    for name in STRING_FUNCTIONS:
        fn = getattr(l, name)
        fn.restype = CP
        fn.argtypes = []
    for name, args in POINTER_FUNCTIONS.items():
        fn = getattr(l, name)
        fn.restype = VP
        fn.argtypes = args


def call(name, *args):
    """Call an entry point whose last two arguments are the error buffer; raise on a refusal."""
    buf = ctypes.create_string_buffer(ERR_CAP)
    status = getattr(lib(), name)(*args, ctypes.cast(buf, VP), ERR_CAP)
    if status != 0:
        raise NativeError(buf.value.decode("utf-8", "replace") or ("%s failed with status %d" % (name, status)))
    return status


def require_device():
    n = lib().b200i_device_count()
    if n <= 0:
        raise NativeError("mojolearn_b200: no CUDA device is visible (there is no CPU fallback)")
    return n
