"""ctypes binding of ``liblattice_q4.so`` (the C ABI declared in ``include/lattice_q4.h``).

There is no CPU fallback: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# LQ4_LIB_PATH selects another build of the same library (a development build, a system-wide install)
LIB_PATH = os.environ.get("LQ4_LIB_PATH") or os.path.join(HERE, "liblattice_q4.so")

# status codes (include/lattice_q4.h)
OK, ERR_NULL, ERR_K, ERR_OVERFLOW, ERR_ALIGN, ERR_DTYPE, ERR_LORA, ERR_ROT, ERR_BAD_BLOCK, ERR_CUDA, \
    ERR_UNSUPPORTED, ERR_DEVICE, ERR_FORMAT, ERR_IO, ERR_SHAPE, ERR_NOSPACE = range(16)
DTYPE_F32, DTYPE_BF16, DTYPE_F64 = 0, 1, 2
QUANT_ASYMMETRIC, QUANT_SYMMETRIC = 0, 1
PATH_AUTO, PATH_GEMV_MMA, PATH_GEMV_GENERIC, PATH_GEMM_TC = 0, 1, 2, 3
OPT_MLP_ONE_LAUNCH, OPT_PDL, OPT_ALLOW_GROW = 1, 2, 3


class LoraDesc(C.Structure):
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("rank", C.c_uint32), ("scale", C.c_float)]


class RotDesc(C.Structure):
    _fields_ = [("signs", C.c_void_p), ("dim", C.c_uint32)]


MAX_PEERS = 8
PEER_HANDLE_BYTES = 64
MAX_TOP_K = 256


class GatherDesc(C.Structure):
    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("bases", C.c_void_p * MAX_PEERS)]


NCCL_ID_BYTES = 128


class StepGroup(C.Structure):
    _fields_ = [("args", C.c_void_p), ("count", C.c_uint32)]


class StepRange(C.Structure):
    _fields_ = [("start", C.c_void_p), ("count", C.c_uint64)]


class StepDesc(C.Structure):
    _fields_ = [("bufs", C.POINTER(GatherDesc)), ("gathered", C.c_void_p), ("n_gathered", C.c_uint32)]


class ShardDesc(C.Structure):
    _fields_ = [("nccl_comm", C.c_void_p), ("world", C.c_uint32), ("rank", C.c_uint32), ("n_total", C.c_uint64),
                ("y_full", C.c_void_p), ("ldy_full", C.c_uint64)]


class LinearArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("m", C.c_uint32), ("n", C.c_uint32),
                ("k", C.c_uint32), ("w", C.c_void_p), ("y", C.c_void_p), ("ldy", C.c_uint64),
                ("lora", C.POINTER(LoraDesc)), ("rot", C.POINTER(RotDesc)), ("path", C.c_int32),
                ("gather", C.POINTER(GatherDesc)), ("wait_gather", C.POINTER(GatherDesc))]


class MlpArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x_dtype", C.c_int32), ("m", C.c_uint32), ("hidden", C.c_uint32),
                ("inter", C.c_uint32), ("w_gate_up", C.c_void_p), ("w_down", C.c_void_p),
                ("lora_gate", C.POINTER(LoraDesc)), ("lora_up", C.POINTER(LoraDesc)),
                ("lora_down", C.POINTER(LoraDesc)), ("gate_up", C.c_void_p), ("y", C.c_void_p),
                ("rot_down", C.POINTER(RotDesc))]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "lq4_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(C.c_void_p)]),
    "lq4_ctx_destroy": (None, [C.c_void_p]),
    "lq4_ctx_reserve": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "lq4_ctx_check": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "lq4_ctx_set_option": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32]),
    "lq4_ctx_launch_count": (C.c_uint64, [C.c_void_p]),
    "lq4_last_error": (C.c_char_p, []),
    "lq4_status_string": (C.c_char_p, [C.c_int32]),
    "lq4_abi_version": (C.c_int32, []),
    "lq4_linear": (C.c_int32, [C.c_void_p, C.POINTER(LinearArgs), C.c_void_p]),
    "lq4_linear_host": (C.c_int32, [C.c_void_p, C.POINTER(LinearArgs), C.c_void_p]),
    "lq4_linear_decode_noalloc": (C.c_int32, [C.POINTER(LinearArgs), C.c_void_p]),
    "lq4_noalloc_check": (C.c_int32, [C.c_void_p]),
    "lq4_linear_group": (C.c_int32, [C.c_void_p, C.POINTER(LinearArgs), C.c_uint32, C.c_void_p]),
    "lq4_step_buf_create": (C.c_int32, [C.c_uint64, C.POINTER(C.c_void_p)]),
    "lq4_decode_step": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(StepDesc), C.c_void_p]),
    "lq4_decode_step_host": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(StepDesc), C.c_void_p]),
    "lq4_peer_buf_create": (C.c_int32, [C.c_uint64, C.POINTER(C.c_void_p)]),
    "lq4_peer_buf_free": (None, [C.c_void_p]),
    "lq4_peer_buf_base": (C.c_void_p, [C.c_void_p]),
    "lq4_peer_buf_payload": (C.c_void_p, [C.c_void_p]),
    "lq4_peer_buf_export": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "lq4_peer_buf_open": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "lq4_peer_buf_close": (C.c_int32, [C.c_void_p]),
    "lq4_gather_wait": (C.c_int32, [C.c_void_p, C.POINTER(GatherDesc), C.c_void_p]),
    "lq4_mlp_block": (C.c_int32, [C.c_void_p, C.POINTER(MlpArgs), C.c_void_p]),
    "lq4_logits_topk": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "lq4_lm_head_topk": (C.c_int32, [C.c_void_p, C.POINTER(LinearArgs), C.c_uint32, C.c_void_p, C.c_void_p]),
    "lq4_lora_apply": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint32, C.c_uint32, C.c_void_p,
                                   C.c_uint32, C.c_uint64, C.POINTER(LoraDesc), C.c_void_p]),
    "lq4_dequant_f32": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "lq4_quantize_f32": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "lq4_quantize_tensor": (C.c_int32, [C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_void_p,
                                        C.c_void_p, C.c_void_p]),
    "lq4_absorb_input_rotation": (C.c_int32, [C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64, C.POINTER(RotDesc), C.c_void_p]),
    "lq4_absorb_output_rotation": (C.c_int32, [C.c_void_p, C.c_int32, C.c_uint64, C.c_uint64, C.POINTER(RotDesc), C.c_void_p]),
    "lq4_q4_file_write": (C.c_int32, [C.c_char_p, C.POINTER(C.c_uint64), C.c_uint32, C.c_uint64, C.c_void_p, C.c_void_p]),
    "lq4_hadamard_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.POINTER(RotDesc), C.c_void_p]),
    "lq4_rot_signs_from_seed": (C.c_int32, [C.c_uint64, C.c_uint32, C.c_void_p, C.c_void_p]),
    "lq4_block_hadamard_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(RotDesc), C.c_void_p]),
    "lq4_cross_head_hadamard_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "lq4_block_rot_signs_from_seed": (C.c_int32, [C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "lq4_weights_upload": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_void_p)]),
    "lq4_weights_load_q4_file": (C.c_int32, [C.c_char_p, C.POINTER(C.c_uint64), C.c_uint32, C.POINTER(C.c_void_p)]),
    "lq4_weights_payload": (C.c_void_p, [C.c_void_p]),
    "lq4_weights_rows": (C.c_uint64, [C.c_void_p]),
    "lq4_weights_cols": (C.c_uint64, [C.c_void_p]),
    "lq4_weights_free": (None, [C.c_void_p]),
    "lq4_lora_upload": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64,
                                    C.c_uint64, C.c_float, C.POINTER(C.c_void_p)]),
    "lq4_lora_desc_for_rows": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(LoraDesc)]),
    "lq4_lora_free": (None, [C.c_void_p]),
    "lq4_nccl_unique_id": (C.c_int32, [C.c_void_p]),
    "lq4_nccl_comm_create": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_void_p)]),
    "lq4_nccl_comm_destroy": (None, [C.c_void_p]),
    "lq4_linear_sharded": (C.c_int32, [C.c_void_p, C.POINTER(LinearArgs), C.POINTER(ShardDesc), C.c_void_p]),
    "lq4_place_slices": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint32, C.c_void_p]),
    "lq4_shard_plan": (C.c_int32, [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64),
                                   C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
}

_lib = None


class Lq4Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"lattice_q4 status {status}: {message}")
        self.status = status


def lib() -> C.CDLL:
    """Loads the CUDA library. Raises if it has not been built: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m lattice_b200.build` "
                              "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise Lq4Error(status, lib().lq4_last_error().decode("utf-8", "replace"))
