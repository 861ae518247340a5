"""ctypes binding of ``libxnq.so``.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, os.environ.get("XNQ_LIB_NAME", "libxnq.so"))

XNQ_OK = 0
XNQ_ACT_IMAGE = 100  # x_dtype of an activation image (activations quantized ahead of the matmul)
XNQ_ACT_OPERAND = 101  # the same, in the integer tensor-core kernel's operand layout (2..64 rows, Q8_K activations)
STATUS_NAMES = {0: "XNQ_OK", -1: "XNQ_ERR_NULL", -2: "XNQ_ERR_DTYPE", -3: "XNQ_ERR_SHAPE", -4: "XNQ_ERR_ALIGN",
                -5: "XNQ_ERR_SIZE", -6: "XNQ_ERR_CUDA", -7: "XNQ_ERR_COMM", -8: "XNQ_ERR_UNSUPPORTED"}


class XnqError(RuntimeError):
    """A non-zero status from the C ABI; ``code`` is the xnq_status, the text is xnq_last_error()."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {msg}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing. Build it with `python -m xn_b200.build` (needs nvcc); "
            "this package has no CPU or PyTorch fallback for the quantized matmul path.")
    L = ctypes.CDLL(LIB_PATH)
    vp, i64, ci, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    pvp = ctypes.POINTER(ctypes.c_void_p)
    L.xnq_last_error.restype = ctypes.c_char_p
    L.xnq_version.restype = ci
    L.xnq_init.argtypes = [ci]
    L.xnq_type_size.argtypes = [ci]
    L.xnq_block_size.argtypes = [ci]
    L.xnq_weight_upload.argtypes = [ci, vp, sz, i64, i64, ci, ci, vp, pvp]
    L.xnq_weight_upload_rows.argtypes = [ci, vp, sz, i64, i64, i64, i64, vp, pvp]
    L.xnq_weight_free.argtypes = [vp]
    L.xnq_weight_info.argtypes = [vp, ctypes.POINTER(ci), ctypes.POINTER(i64), ctypes.POINTER(i64), ctypes.POINTER(i64),
                                  ctypes.POINTER(i64), ctypes.POINTER(sz)]
    L.xnq_weight_dequantize.argtypes = [vp, ci, vp, vp]
    L.xnq_weight_canonical_bytes.argtypes = [vp, vp, sz, vp]
    L.xnq_quantize_act.argtypes = [ci, vp, ci, i64, i64, i64, vp, vp]
    L.xnq_act_image_bytes.argtypes = [ci, i64, i64]
    L.xnq_act_image_bytes.restype = sz
    L.xnq_quantize_act_image.argtypes = [ci, vp, ci, i64, i64, i64, vp, vp]
    L.xnq_quantize_weight.argtypes = [ci, vp, i64, i64, vp, vp]
    L.xnq_matmul_workspace_bytes.argtypes = [vp, i64]
    L.xnq_matmul_workspace_bytes.restype = sz
    L.xnq_matmul_t.argtypes = [vp, vp, ci, i64, i64, vp, ci, i64, vp, sz, vp]
    L.xnq_linear_forward_host.argtypes = [vp, vp, i64, vp, vp, vp]
    L.xnq_weight_reserve_host_staging.argtypes = [vp, i64]
    L.xnq_hint_next_weight.argtypes = [vp]
    L.xnq_matvec_normed.argtypes = [vp, vp, vp, ci, vp, ctypes.c_float, vp, vp, ci, vp, vp]
    L.xnq_matmul_t_static.argtypes = [vp, vp, ci, i64, i64, vp, ci, i64, vp]
    L.xnq_comm_create.argtypes = [ci, ci, sz, ci, pvp]
    L.xnq_comm_ipc_handle.argtypes = [vp, vp]
    L.xnq_comm_connect.argtypes = [vp, vp]
    L.xnq_comm_slot.argtypes = [vp, ci, pvp, ctypes.POINTER(sz)]
    L.xnq_matmul_t_gather.argtypes = [vp, vp, ci, ci, vp, ci, i64, i64, ci, vp, sz, vp, pvp]
    L.xnq_comm_gather.argtypes = [vp, ci, vp, ci, i64, i64, i64, vp, pvp]
    L.xnq_comm_set_deferred.argtypes = [vp, ci]
    L.xnq_comm_wait.argtypes = [vp, vp]
    L.xnq_comm_status.argtypes = [vp, ctypes.POINTER(ctypes.c_uint)]
    L.xnq_comm_free.argtypes = [vp]
    fp = ctypes.c_float
    L.xnq_add_rmsnorm.argtypes = [vp, vp, ci, vp, fp, vp, vp, ci, i64, i64, vp]
    L.xnq_act_operand_bytes.argtypes = [i64, i64]
    L.xnq_act_operand_bytes.restype = sz
    L.xnq_swiglu.argtypes = [vp, vp, vp, ci, i64, i64, vp]
    L.xnq_embed_rows.argtypes = [vp, vp, vp, i64, i64, i64, vp]
    L.xnq_argmax_advance.argtypes = [vp, i64, i64, vp, vp, vp]
    L.xnq_rope_kv_store.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, ci, ci, ci, i64, vp]
    L.xnq_attn_decode_workspace_bytes.argtypes = [i64, ci]
    L.xnq_attn_decode_workspace_bytes.restype = sz
    L.xnq_attn_decode.argtypes = [vp, vp, vp, vp, vp, i64, ci, ci, ci, i64, vp, sz, vp]
    L.xnq_rope_attn_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, ci, ci, ci, i64, vp, sz, vp]
    L.xnq_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
    L.xnq_device_check_record.argtypes = [ctypes.POINTER(ctypes.c_ulonglong)]
    L.xnq_set_option.argtypes = [ctypes.c_char_p, ci]
    L.xnq_launch_count.restype = ctypes.c_uint64
    L.xnq_profile_begin.argtypes = [ci]
    L.xnq_profile_end.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ci)]
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != XNQ_OK:
        raise XnqError(rc, lib().xnq_last_error().decode("utf-8", "replace"))
