"""ctypes front end of the CPU oracle (``lq4_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline legs of ``bench.py``.  The shipped package never imports
it.  Parity status: pinned by the reference's golden ``.q4`` fixtures and
known-answer tests (see ``tests/test_oracle_golden.py``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblq4_oracle.so")

OK, ERR_NONFINITE, ERR_SCALE, ERR_BIAS, ERR_SHAPE, ERR_POW2, ERR_IO, ERR_FORMAT, ERR_VALID_LEN = range(9)


class OracleError(ValueError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: oracle error {code}")
        self.code = code


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "lq4_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "liblq4_oracle.so"])
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        vp, sz, u64 = C.c_void_p, C.c_size_t, C.c_uint64
        L.orc_f32_to_f16_bits.restype = C.c_uint16
        L.orc_f32_to_f16_bits.argtypes = [C.c_float]
        L.orc_f16_bits_to_f32.restype = C.c_float
        L.orc_f16_bits_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16_bits_rne.restype = C.c_uint16
        L.orc_f32_to_bf16_bits_rne.argtypes = [C.c_float]
        L.orc_quantize_block.argtypes = [vp, C.c_int, C.c_int, vp]
        L.orc_quantize_f32_to_q4.argtypes = [vp, sz, C.c_int, vp]
        L.orc_quantize_tensor_q4_0.argtypes = [vp, sz, sz, vp]
        L.orc_quantize_bf16_to_q4.argtypes = [vp, sz, vp]
        L.orc_quantize_f64_to_q4.argtypes = [vp, sz, C.c_int, vp]
        L.orc_dequantize_q4_to_f32.restype = None
        L.orc_dequantize_q4_to_f32.argtypes = [vp, sz, sz, vp]
        L.orc_q4_first_invalid_block.restype = C.c_int64
        L.orc_q4_first_invalid_block.argtypes = [vp, sz]
        L.orc_q4_write_file.argtypes = [C.c_char_p, vp, C.c_uint32, u64, vp, sz]
        L.orc_q4_parse.argtypes = [vp, sz, vp, vp, vp, vp]
        for name in ("orc_matmul_bt", "orc_matmul_bt_scalar", "orc_matmul_bt_tiled_scalar",
                     "orc_matmul_bt_tiled_avx2", "orc_matmul_bt_avx2", "orc_matmul_bt_avx512",
                     "orc_matmul_bt_f64acc"):
            fn = getattr(L, name)
            fn.restype = None
            fn.argtypes = [vp, vp, vp, sz, sz, sz]
        L.orc_matmul_bt_kernel_id.argtypes = [sz, sz, sz]
        L.orc_set_force_scalar.restype = None
        L.orc_set_force_scalar.argtypes = [C.c_int]
        L.orc_effective_scale.restype = C.c_float
        L.orc_effective_scale.argtypes = [sz, C.c_float]
        L.orc_apply_lora.argtypes = [vp, sz, vp, sz, sz, sz, sz, C.c_float, vp, sz, vp, sz]
        L.orc_splitmix64_mix.restype = u64
        L.orc_splitmix64_mix.argtypes = [u64]
        L.orc_signs_from_seed.restype = None
        L.orc_signs_from_seed.argtypes = [u64, sz, vp]
        L.orc_derive_block_seed.restype = u64
        L.orc_derive_block_seed.argtypes = [u64, u64]
        for name in ("orc_walsh_hadamard_f32", "orc_walsh_hadamard_f64",
                     "orc_walsh_hadamard_orthonormal_f32", "orc_walsh_hadamard_orthonormal_f64"):
            getattr(L, name).argtypes = [vp, sz]
        for name in ("orc_rh_apply_f32", "orc_rh_apply_f64", "orc_rh_apply_inverse_f32",
                     "orc_rh_apply_inverse_f64"):
            getattr(L, name).argtypes = [vp, sz, vp]
        for name in ("orc_absorb_input_rotation_f64", "orc_absorb_input_rotation_f32",
                     "orc_absorb_output_rotation_f64", "orc_absorb_output_rotation_f32",
                     "orc_counter_rotate_a", "orc_rotate_b_output_side"):
            getattr(L, name).argtypes = [vp, sz, sz, vp, sz]
        L.orc_q4_linear.argtypes = [vp, vp, vp, vp, sz, sz, sz, vp, vp, sz, C.c_float, vp]
        L.orc_gemv_q4_decode_form.restype = None
        L.orc_gemv_q4_decode_form.argtypes = [vp, vp, vp, sz, sz]
        L.orc_topk.argtypes = [vp, sz, sz, vp, vp]
        L.orc_block_hadamard_check.argtypes = [sz, sz]
        L.orc_silu_mul.argtypes = [vp, sz, vp]
        L.orc_silu_mul.restype = None
        L.orc_cross_head_rotation_f32.argtypes = [vp, sz, sz, vp]
        L.orc_block_hadamard_signs.argtypes = [u64, sz, sz, vp]
        L.orc_block_hadamard_apply_f32.argtypes = [vp, sz, sz, vp, C.c_int]
        L.orc_topk.restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _check(rc: int, what: str) -> None:
    if rc != OK:
        raise OracleError(rc, what)


# ---- f16 -----------------------------------------------------------------
def f32_to_f16_bits(v: float) -> int:
    return int(lib().orc_f32_to_f16_bits(C.c_float(v)))


def f16_bits_to_f32(bits: int) -> float:
    return float(lib().orc_f16_bits_to_f32(C.c_uint16(bits)))


# ---- quantizer / dequantizer ---------------------------------------------
def n_blocks(n_weights: int) -> int:
    return (n_weights + 31) // 32


def quantize_block(vals, valid_len: int = 32, symmetric: bool = False) -> bytes:
    v = _c(vals, np.float32)
    assert v.size == 32
    out = np.zeros(20, np.uint8)
    _check(lib().orc_quantize_block(_p(v), valid_len, int(symmetric), _p(out)), "quantize_block")
    return out.tobytes()


def quantize_f32_to_q4(data, symmetric: bool = False) -> np.ndarray:
    """Flat 32-chunks of the flattened tensor (the reference's ``quantize_f32_to_q4``)."""
    d = _c(data, np.float32).reshape(-1)
    out = np.zeros(n_blocks(d.size) * 20, np.uint8)
    _check(lib().orc_quantize_f32_to_q4(_p(d), d.size, int(symmetric), _p(out)), "quantize_f32_to_q4")
    return out


def quantize_tensor_q4_0(data, rows: int, cols: int) -> np.ndarray:
    d = _c(data, np.float32).reshape(-1)
    if d.size != rows * cols:
        raise OracleError(ERR_SHAPE, "quantize_tensor_q4_0")
    out = np.zeros(rows * n_blocks(cols) * 20, np.uint8)
    _check(lib().orc_quantize_tensor_q4_0(_p(d), rows, cols, _p(out)), "quantize_tensor_q4_0")
    return out


def quantize_bf16_to_q4(bits) -> np.ndarray:
    d = _c(bits, np.uint16).reshape(-1)
    out = np.zeros(n_blocks(d.size) * 20, np.uint8)
    _check(lib().orc_quantize_bf16_to_q4(_p(d), d.size, _p(out)), "quantize_bf16_to_q4")
    return out


def quantize_f64_to_q4(data, symmetric: bool = True) -> np.ndarray:
    d = _c(data, np.float64).reshape(-1)
    out = np.zeros(n_blocks(d.size) * 20, np.uint8)
    _check(lib().orc_quantize_f64_to_q4(_p(d), d.size, int(symmetric), _p(out)), "quantize_f64_to_q4")
    return out


def dequantize_q4_to_f32(payload, original_len: int | None = None) -> np.ndarray:
    p = _c(payload, np.uint8).reshape(-1)
    nb = p.size // 20
    if original_len is None:
        original_len = nb * 32
    out = np.zeros(original_len, np.float32)
    lib().orc_dequantize_q4_to_f32(_p(p), nb, original_len, _p(out))
    return out


def first_invalid_block(payload) -> int:
    p = _c(payload, np.uint8).reshape(-1)
    return int(lib().orc_q4_first_invalid_block(_p(p), p.size // 20))


def q4_file_bytes(shape, original_len: int, payload) -> bytes:
    """Serialise a `.q4` image in memory (same layout orc_q4_write_file puts on disk)."""
    import struct
    head = b"KHQ4" + struct.pack("<II", 2, len(shape))
    head += b"".join(struct.pack("<Q", int(s)) for s in shape) + struct.pack("<Q", original_len)
    return head + _c(payload, np.uint8).tobytes()


def q4_parse(img: bytes):
    buf = np.frombuffer(img, np.uint8)
    ndim = C.c_uint32()
    shape = (C.c_uint64 * 8)()
    olen, off = C.c_uint64(), C.c_uint64()
    _check(lib().orc_q4_parse(_p(buf), buf.size, C.byref(ndim), shape, C.byref(olen), C.byref(off)), "q4_parse")
    return [int(shape[i]) for i in range(ndim.value)], int(olen.value), int(off.value)


# ---- matmul ---------------------------------------------------------------
KERNEL_NAMES = {0: "scalar", 1: "tiled-scalar", 2: "tiled-avx2", 3: "avx2", 4: "avx512"}


def matmul_bt(a, b, m: int, k: int, n: int, variant: str = "dispatch") -> np.ndarray:
    a = _c(a, np.float32).reshape(-1)
    b = _c(b, np.float32).reshape(-1)
    assert a.size >= m * k and b.size >= n * k
    fn = {"dispatch": "orc_matmul_bt", "scalar": "orc_matmul_bt_scalar",
          "tiled_scalar": "orc_matmul_bt_tiled_scalar", "tiled_avx2": "orc_matmul_bt_tiled_avx2",
          "avx2": "orc_matmul_bt_avx2", "avx512": "orc_matmul_bt_avx512"}[variant]
    c = np.zeros(m * n, np.float32)
    getattr(lib(), fn)(_p(a), _p(b), _p(c), m, k, n)
    return c.reshape(m, n)


def matmul_bt_f64acc(a, b, m: int, k: int, n: int) -> np.ndarray:
    a = _c(a, np.float32).reshape(-1)
    b = _c(b, np.float32).reshape(-1)
    c = np.zeros(m * n, np.float64)
    lib().orc_matmul_bt_f64acc(_p(a), _p(b), _p(c), m, k, n)
    return c.reshape(m, n)


def matmul_bt_kernel(m: int, k: int, n: int) -> str:
    return KERNEL_NAMES[lib().orc_matmul_bt_kernel_id(m, k, n)]


def set_force_scalar(on: bool) -> None:
    lib().orc_set_force_scalar(int(on))


# ---- LoRA -------------------------------------------------------------------
def effective_scale(rank: int, alpha: float) -> float:
    return float(lib().orc_effective_scale(rank, C.c_float(alpha)))


def apply_lora(a, b, rank: int, d_in: int, d_out: int, scale: float, x, out) -> bool:
    """In place on ``out`` (float32 ndarray). Returns False for the silent shape-mismatch no-op."""
    a = _c(a, np.float32).reshape(-1)
    b = _c(b, np.float32).reshape(-1)
    x = _c(x, np.float32).reshape(-1)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    return bool(lib().orc_apply_lora(_p(a), a.size, _p(b), b.size, rank, d_in, d_out,
                                     C.c_float(scale), _p(x), x.size, _p(out), out.size))


# ---- Hadamard ---------------------------------------------------------------
def splitmix64_mix(z: int) -> int:
    return int(lib().orc_splitmix64_mix(C.c_uint64(z & (2**64 - 1))))


def signs_from_seed(seed: int, n: int) -> np.ndarray:
    out = np.zeros(n, np.float32)
    lib().orc_signs_from_seed(C.c_uint64(seed & (2**64 - 1)), n, _p(out))
    return out


def derive_block_seed(seed: int, block_index: int) -> int:
    return int(lib().orc_derive_block_seed(C.c_uint64(seed & (2**64 - 1)), C.c_uint64(block_index)))


def walsh_hadamard(data, orthonormal: bool = False) -> np.ndarray:
    d = np.array(data, copy=True)
    if d.dtype not in (np.float32, np.float64):
        d = d.astype(np.float32)
    d = np.ascontiguousarray(d).reshape(-1)
    name = "orc_walsh_hadamard_" + ("orthonormal_" if orthonormal else "") + ("f32" if d.dtype == np.float32 else "f64")
    _check(getattr(lib(), name)(_p(d), d.size), name)
    return d


def rh_apply(signs, data, inverse: bool = False) -> np.ndarray:
    s = _c(signs, np.float32)
    d = np.array(data, copy=True)
    if d.dtype not in (np.float32, np.float64):
        d = d.astype(np.float32)
    d = np.ascontiguousarray(d).reshape(-1)
    if d.size != s.size:
        raise OracleError(ERR_SHAPE, "rh_apply")
    name = "orc_rh_apply_" + ("inverse_" if inverse else "") + ("f32" if d.dtype == np.float32 else "f64")
    _check(getattr(lib(), name)(_p(s), s.size, _p(d)), name)
    return d


def absorb_rotation(w, rows: int, cols: int, signs, side: str = "input") -> np.ndarray:
    s = _c(signs, np.float32)
    d = np.array(w, copy=True)
    assert d.dtype in (np.float32, np.float64)
    d = np.ascontiguousarray(d).reshape(-1)
    name = f"orc_absorb_{side}_rotation_" + ("f32" if d.dtype == np.float32 else "f64")
    _check(getattr(lib(), name)(_p(d), rows, cols, _p(s), s.size), name)
    return d.reshape(rows, cols)


# ---- composed linear ----------------------------------------------------------
def q4_linear(x, payload, m: int, n: int, k: int, lora=None, rot_signs=None, w_f32=None) -> np.ndarray:
    """Reference CPU answer for one projection.  ``lora`` = (A[rank,k], B[n,rank], scale)."""
    x = _c(x, np.float32).reshape(-1)
    p = None if payload is None else _c(payload, np.uint8).reshape(-1)
    wf = None if w_f32 is None else _c(w_f32, np.float32).reshape(-1)
    y = np.zeros(m * n, np.float32)
    a = b = None
    rank, scale = 0, 0.0
    if lora is not None:
        a = _c(lora[0], np.float32).reshape(-1)
        b = _c(lora[1], np.float32).reshape(-1)
        scale = float(lora[2])
        rank = a.size // k
    s = None if rot_signs is None else _c(rot_signs, np.float32)
    _check(lib().orc_q4_linear(_p(x), _p(p), _p(wf), _p(y), m, n, k, _p(a), _p(b), rank,
                               C.c_float(scale), _p(s)), "q4_linear")
    return y.reshape(m, n)


def gemv_q4_decode_form(x, payload, n: int, k: int) -> np.ndarray:
    x = _c(x, np.float32).reshape(-1)
    p = _c(payload, np.uint8).reshape(-1)
    y = np.zeros(n, np.float32)
    lib().orc_gemv_q4_decode_form(_p(x), _p(p), _p(y), n, k)
    return y


def topk(logits, k: int):
    """(logits[k], token_ids[k]) of the k best entries in the reference's candidate order (higher logit
    first, ties to the lower id, NaN never ranks); unused slots hold (-inf, 0xFFFFFFFF)."""
    v = _c(logits, np.float32).reshape(-1)
    out_l = np.zeros(k, np.float32)
    out_i = np.zeros(k, np.uint32)
    lib().orc_topk(_p(v), v.size, k, _p(out_l), _p(out_i))
    return out_l, out_i


def block_hadamard_signs(seed: int, n: int, block: int) -> np.ndarray:
    """The flat sign buffer of BlockHadamard::new(seed, n, block); raises where the constructor refuses."""
    _check(lib().orc_block_hadamard_check(n, block), "block_hadamard_check")
    out = np.zeros(n, np.float32)
    _check(lib().orc_block_hadamard_signs(seed, n, block, _p(out)), "block_hadamard_signs")
    return out


def block_hadamard_apply(signs, data, block: int, inverse: bool = False) -> np.ndarray:
    """BlockHadamard::apply / apply_inverse on one vector of len(signs) f32 values."""
    s = _c(signs, np.float32).reshape(-1)
    d = np.array(data, dtype=np.float32, copy=True).reshape(-1)
    if d.size != s.size:
        raise OracleError(ERR_SHAPE, "block_hadamard_apply")
    _check(lib().orc_block_hadamard_apply_f32(_p(s), s.size, block, _p(d), 1 if inverse else 0), "block_hadamard_apply")
    return d


def cross_head_rotation(signs, data, head_dim: int) -> np.ndarray:
    """The R3 "Hadamard heads" rotation of one [num_heads * head_dim] activation; num_heads = len(signs)."""
    s = _c(signs, np.float32).reshape(-1)
    d = np.array(data, dtype=np.float32, copy=True).reshape(-1)
    if d.size != s.size * head_dim:
        raise OracleError(ERR_SHAPE, "cross_head_rotation")
    _check(lib().orc_cross_head_rotation_f32(_p(s), s.size, head_dim, _p(d)), "cross_head_rotation")
    return d


def silu_mul(gate_up, inter: int) -> np.ndarray:
    """silu_mul_fused on rows of merged gate || up values: [m, 2 * inter] -> [m, inter]."""
    g = _c(gate_up, np.float32).reshape(-1, 2 * inter)
    out = np.zeros((g.shape[0], inter), np.float32)
    for r in range(g.shape[0]):
        row = np.ascontiguousarray(g[r])
        o = np.zeros(inter, np.float32)
        lib().orc_silu_mul(_p(row), inter, _p(o))
        out[r] = o
    return out


def mlp_block(x, w_gate_up_payload, w_down_payload, m: int, hidden: int, inter: int,
              lora_gate=None, lora_up=None, lora_down=None) -> np.ndarray:
    """The dense FFN of encode_mlp_block (inner/layers/mod.rs:93-148): merged gate||up matmul with the
    gate_proj / up_proj adapters on its two halves, silu_mul_fused, down_proj with its adapter."""
    p = _c(w_gate_up_payload, np.uint8).reshape(-1)
    half = inter * (hidden // 32) * 20
    gate = q4_linear(x, p[:half], m, inter, hidden, lora=lora_gate)
    up = q4_linear(x, p[half:2 * half], m, inter, hidden, lora=lora_up)
    h = silu_mul(np.concatenate([gate, up], axis=1), inter)
    return q4_linear(h, w_down_payload, m, hidden, inter, lora=lora_down)
