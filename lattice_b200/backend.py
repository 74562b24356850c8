"""Host-side mirror of the reference's Q4 matmul seam, over the C ABI.

The reference exposes no plugin interface for this path: the seam is a set of methods
on its Metal engine state.  The methods below keep those names, argument meaning and
error behaviour so that call sites (and tests) read like the reference's:

* ``dispatch_matmul_q4`` / ``dispatch_gemm_q4`` / ``dispatch_gemm_q4_at``
  (crates/inference/src/forward/metal_qwen35/inner/dispatch.rs:148-229, 1037-1097)
* ``dispatch_lora_if_active`` (crates/inference/src/forward/metal_qwen35/inner/layers/mod.rs:15-51)
* ``load_lora_adapter`` / ``unload_lora_adapter`` / ``LoraLayerData``
  (crates/inference/src/forward/metal_qwen35.rs:1699-1716, 3806-3986, 4063-4075)
* ``Q4WeightBuf`` (crates/inference/src/forward/metal_qwen35.rs:599-702)

Buffers are torch CUDA tensors (device memory only); ``*_offset`` arguments are byte
offsets into them, as the Metal encoder takes them.  All compute is in the CUDA library;
nothing here falls back to PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import GatherDesc, LinearArgs, LoraDesc, Lq4Error, RotDesc, check


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Q4WeightBuf:
    """Device-resident Q4 payload of one ``[n, k]`` weight in the reference block layout."""

    def __init__(self, handle: int, n: int, k: int):
        self._handle = handle
        self.n, self.k = n, k
        self.payload_ptr = _lib.lib().lq4_weights_payload(handle)
        self.payload_bytes = n * (k // 32) * 20

    @classmethod
    def from_host_payload(cls, payload: np.ndarray, n: int, k: int) -> "Q4WeightBuf":
        """Validates every block's scale/bias on the host, then copies to the device."""
        p = np.ascontiguousarray(payload, dtype=np.uint8).reshape(-1)
        if p.size != n * (k // 32) * 20:
            raise ValueError(f"payload has {p.size} bytes, expected {n * (k // 32) * 20} for [{n}, {k}]")
        h = C.c_void_p()
        check(_lib.lib().lq4_weights_upload(p.ctypes.data_as(C.c_void_p), n, k, C.byref(h)))
        return cls(h.value, n, k)

    @classmethod
    def from_q4_file(cls, path: str, expected_shape: Optional[Tuple[int, int]] = None) -> "Q4WeightBuf":
        h = C.c_void_p()
        if expected_shape is None:
            check(_lib.lib().lq4_weights_load_q4_file(path.encode(), None, 0, C.byref(h)))
        else:
            shp = (C.c_uint64 * len(expected_shape))(*expected_shape)
            check(_lib.lib().lq4_weights_load_q4_file(path.encode(), shp, len(expected_shape), C.byref(h)))
        L = _lib.lib()
        return cls(h.value, int(L.lq4_weights_rows(h)), int(L.lq4_weights_cols(h)))

    @classmethod
    def from_device_payload(cls, payload: torch.Tensor, n: int, k: int) -> "Q4WeightBuf":
        """Wraps bytes that are already on the device (e.g. produced by ``quantize``); not validated."""
        assert payload.is_cuda and payload.dtype == torch.uint8 and payload.numel() >= n * (k // 32) * 20
        self = cls.__new__(cls)
        self._handle = None
        self._keep = payload
        self.n, self.k = n, k
        self.payload_ptr = payload.data_ptr()
        self.payload_bytes = n * (k // 32) * 20
        return self

    def free(self) -> None:
        if getattr(self, "_handle", None):
            _lib.lib().lq4_weights_free(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


@dataclass
class LoraLayerData:
    """Input data for one LoRA projection: A row-major ``(rank, d_in)``, B row-major ``(d_out, rank)``."""
    layer_idx: int
    module: str
    a: np.ndarray
    b: np.ndarray
    rank: int
    d_in: int
    d_out: int


@dataclass
class _LoraProjection:
    handle: int
    rank: int
    d_in: int
    d_out: int


@dataclass
class _LoraAdapter:
    projections: List[Dict[str, _LoraProjection]]
    scale: float
    max_rank: int = 0


class PreparedGroup:
    """Argument block of one ``lq4_linear_group`` call, reusable while its tensors live."""

    def __init__(self, backend: "CudaQ4Backend", arr, count: int, outs: List[torch.Tensor], keep):
        self._be, self._arr, self._count, self.outs, self._keep = backend, arr, count, outs, keep
        self._fn = _lib.lib().lq4_linear_group

    def __call__(self) -> List[torch.Tensor]:
        check(self._fn(self._be._ctx, self._arr, self._count, _stream()))
        return self.outs


class PreparedStep:
    """Argument blocks of one ``lq4_decode_step`` call, reusable while its tensors live."""

    def __init__(self, backend: "CudaQ4Backend", garr, ngroups: int, desc, keep, host: bool = False):
        self._be, self._garr, self._ngroups, self._desc, self._keep = backend, garr, ngroups, desc, keep
        self._fn = _lib.lib().lq4_decode_step_host if host else _lib.lib().lq4_decode_step

    def __call__(self) -> None:
        check(self._fn(self._be._ctx, C.cast(self._garr, C.c_void_p), self._ngroups,
                       C.byref(self._desc) if self._desc is not None else None, _stream()))


class CudaQ4Backend:
    """One instance per device and owning thread, like the reference's GPU state."""

    def __init__(self, device: int = 0, num_hidden_layers: int = 1,
                 projection_shapes: Optional[Dict[str, Tuple[int, int]]] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("CudaQ4Backend needs a CUDA device; there is no CPU path")
        self.device = device
        torch.cuda.set_device(device)
        h = C.c_void_p()
        check(_lib.lib().lq4_ctx_create(device, C.byref(h)))
        self._ctx = h.value
        self.num_hidden_layers = num_hidden_layers
        # module name -> (d_in, d_out); None disables the model-shape check of load_lora_adapter
        self.projection_shapes = projection_shapes
        self.lora: Optional[_LoraAdapter] = None

    def close(self) -> None:
        if self._ctx:
            self.unload_lora_adapter()
            _lib.lib().lq4_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- bookkeeping ------------------------------------------------------
    @property
    def launch_count(self) -> int:
        return int(_lib.lib().lq4_ctx_launch_count(self._ctx))

    def check_device_status(self) -> None:
        """Synchronises the current stream and raises if a kernel gave up on a bounded wait."""
        check(_lib.lib().lq4_ctx_check(self._ctx, _stream()))

    def set_option(self, option: int, value: int) -> None:
        """Per-context switches of the library (``_lib.OPT_*``)."""
        check(_lib.lib().lq4_ctx_set_option(self._ctx, option, int(value)))

    def reserve(self, m: int, n: int, k: int, rank: int = 0) -> None:
        check(_lib.lib().lq4_ctx_reserve(self._ctx, m, n, k, rank))

    # ---- the seam -----------------------------------------------------------
    def _linear(self, x_ptr: int, x_dtype: int, w_ptr: int, y_ptr: int, m: int, n: int, k: int, ldy: int = 0,
                lora: Optional[LoraDesc] = None, rot: Optional[RotDesc] = None, path: int = _lib.PATH_AUTO,
                host: bool = False, gather: Optional[GatherDesc] = None,
                wait_gather: Optional[GatherDesc] = None) -> None:
        args = LinearArgs(x_ptr, x_dtype, m, n, k, w_ptr, y_ptr, ldy,
                          C.pointer(lora) if lora is not None else None,
                          C.pointer(rot) if rot is not None else None, path,
                          C.pointer(gather) if gather is not None else None,
                          C.pointer(wait_gather) if wait_gather is not None else None)
        fn = _lib.lib().lq4_linear_host if host else _lib.lib().lq4_linear
        check(fn(self._ctx, C.byref(args), _stream()))

    @staticmethod
    def _require_k(name: str, k: int) -> None:
        # the reference asserts here: dispatch.rs:185-188
        if k <= 0 or k % 32 != 0:
            raise ValueError(f"{name} requires K to be non-zero and divisible by 32, got {k}")

    @staticmethod
    def _dtype_of(x: torch.Tensor) -> int:
        if x.dtype == torch.float32:
            return _lib.DTYPE_F32
        if x.dtype == torch.bfloat16:
            return _lib.DTYPE_BF16
        raise TypeError(f"activations must be float32 or bfloat16, got {x.dtype}")

    def dispatch_gemm_q4_at(self, x: torch.Tensor, x_offset: int, qw: Q4WeightBuf, qw_extra_offset: int,
                            y: torch.Tensor, y_offset: int, m: int, n: int, k: int, *,
                            lora: Optional[LoraDesc] = None, rot: Optional[RotDesc] = None,
                            ldy: int = 0, path: int = _lib.PATH_AUTO, gather: Optional[GatherDesc] = None,
                            wait_gather: Optional[GatherDesc] = None) -> None:
        """``y[m, n] = x[m, k] . Wq4[n, k]^T`` (overwrites y); ``qw_extra_offset`` bytes into the payload."""
        if m == 0 or n == 0:
            return
        self._require_k("dispatch_gemm_q4_at", k)
        assert x.is_cuda and y.is_cuda and y.dtype == torch.float32
        self._linear(x.data_ptr() + x_offset, self._dtype_of(x), qw.payload_ptr + qw_extra_offset,
                     y.data_ptr() + y_offset, m, n, k, ldy, lora, rot, path, gather=gather, wait_gather=wait_gather)

    def dispatch_gemm_q4(self, x: torch.Tensor, x_offset: int, qw: Q4WeightBuf, y: torch.Tensor, y_offset: int,
                         m: int, n: int, k: int, **kw) -> None:
        if m == 0 or n == 0:
            return
        self._require_k("dispatch_gemm_q4", k)
        self.dispatch_gemm_q4_at(x, x_offset, qw, 0, y, y_offset, m, n, k, **kw)

    def dispatch_matmul_q4(self, x: torch.Tensor, qw: Q4WeightBuf, y: torch.Tensor, m: int, n: int, k: int, **kw) -> None:
        """Decode-step form (m == 1 in the reference)."""
        self.dispatch_gemm_q4(x, 0, qw, y, 0, m, n, k, **kw)

    # ---- LoRA ------------------------------------------------------------------
    # Which side of a projection the residual-stream rotation was absorbed on
    # (crates/inference/src/quant/quarot/plan.rs:935-941, tests at :1483-1514).
    QUAROT_INPUT_SIDE = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "in_proj_qkv", "in_proj_z",
                         "in_proj_b", "in_proj_a")
    QUAROT_OUTPUT_SIDE = ("o_proj", "down_proj", "out_proj")

    def _rotate_adapter_layer(self, layer: LoraLayerData, seed: int, hidden_dim: int):
        """Rotation correction of one adapter projection for a QuaRot base, on the device
        (crates/inference/src/quant/quarot/lora.rs:32-58,150-216): input side ``A <- A R^T`` (R applied to
        every row of A), output side ``B <- R B`` (R applied to every column of B).  Modules outside the
        plan are refused, as in the reference."""
        a = np.ascontiguousarray(layer.a, dtype=np.float32).reshape(layer.rank, layer.d_in)
        b = np.ascontiguousarray(layer.b, dtype=np.float32).reshape(layer.d_out, layer.rank)
        if layer.module in self.QUAROT_INPUT_SIDE:
            if layer.d_in != hidden_dim:
                raise Lq4Error(_lib.ERR_SHAPE, f"rotate_adapter_for_quarot: layer {layer.layer_idx} module "
                                               f"'{layer.module}' has d_in={layer.d_in} but hidden_dim={hidden_dim}")
            signs = self.rot_signs(seed, hidden_dim)
            a = self.hadamard_rows(torch.from_numpy(a).cuda(), signs).cpu().numpy()
        elif layer.module in self.QUAROT_OUTPUT_SIDE:
            if layer.d_out != hidden_dim:
                raise Lq4Error(_lib.ERR_SHAPE, f"rotate_adapter_for_quarot: layer {layer.layer_idx} module "
                                               f"'{layer.module}' has d_out={layer.d_out} but hidden_dim={hidden_dim}")
            signs = self.rot_signs(seed, hidden_dim)
            bt = torch.from_numpy(np.ascontiguousarray(b.T)).cuda()          # columns of B as rows
            b = np.ascontiguousarray(self.hadamard_rows(bt, signs).cpu().numpy().T)
        else:
            raise Lq4Error(_lib.ERR_LORA, f"rotate_adapter_for_quarot: layer {layer.layer_idx} targets module "
                                          f"'{layer.module}' which is not in the rotation plan")
        return a, b

    def load_lora_adapter(self, layers: List[LoraLayerData], scale: float, quarot_seed: Optional[int] = None,
                          quarot_hidden_dim: Optional[int] = None) -> None:
        """Copies the adapter to the device after the reference's load-time checks.  With ``quarot_seed`` (and
        the hidden dimension the base was rotated in) the factors are first corrected for the rotated base."""
        if self.lora is not None:
            raise Lq4Error(_lib.ERR_LORA, "LoRA adapter already loaded; call unload_lora_adapter first")
        if len(layers) == 0:
            raise Lq4Error(_lib.ERR_LORA, "load_lora_adapter: layers must not be empty")
        if not math.isfinite(scale):
            raise Lq4Error(_lib.ERR_LORA, f"load_lora_adapter: scale must be finite, got {scale}")
        if quarot_seed is not None:
            if quarot_hidden_dim is None or quarot_hidden_dim <= 0 or quarot_hidden_dim & (quarot_hidden_dim - 1):
                raise Lq4Error(_lib.ERR_ROT, "quarot_hidden_dim must be a power of two")
        projections: List[Dict[str, _LoraProjection]] = [dict() for _ in range(self.num_hidden_layers)]
        max_rank = 0
        try:
            for layer in layers:
                if layer.rank == 0:
                    raise Lq4Error(_lib.ERR_LORA, f"load_lora_adapter: layer {layer.layer_idx} module "
                                                  f"'{layer.module}' has rank=0")
                if layer.d_in == 0 or layer.d_out == 0:
                    raise Lq4Error(_lib.ERR_LORA, f"load_lora_adapter: layer {layer.layer_idx} module "
                                                  f"'{layer.module}' has zero dimension")
                if layer.layer_idx >= self.num_hidden_layers:
                    raise Lq4Error(_lib.ERR_SHAPE, f"load_lora_adapter: layer_idx {layer.layer_idx} >= "
                                                   f"num_hidden_layers {self.num_hidden_layers}")
                if self.projection_shapes is not None:
                    if layer.module not in self.projection_shapes:
                        raise Lq4Error(_lib.ERR_LORA, f"unknown LoRA module '{layer.module}'")
                    exp = self.projection_shapes[layer.module]
                    if (layer.d_in, layer.d_out) != exp:
                        raise Lq4Error(_lib.ERR_SHAPE, f"load_lora_adapter: layer {layer.layer_idx} module "
                                                       f"'{layer.module}' has (d_in={layer.d_in}, d_out={layer.d_out}) "
                                                       f"but model expects (d_in={exp[0]}, d_out={exp[1]})")
                if layer.module in projections[layer.layer_idx]:
                    raise Lq4Error(_lib.ERR_LORA, f"load_lora_adapter: duplicate projection for layer "
                                                  f"{layer.layer_idx} module '{layer.module}'")
                if quarot_seed is not None:
                    if np.asarray(layer.a).size != layer.rank * layer.d_in or np.asarray(layer.b).size != layer.d_out * layer.rank:
                        raise Lq4Error(_lib.ERR_SHAPE, f"load_lora_adapter: layer {layer.layer_idx} module "
                                                       f"'{layer.module}' factor sizes do not match its shape")
                    a, b = self._rotate_adapter_layer(layer, quarot_seed, quarot_hidden_dim)
                    a, b = a.reshape(-1), b.reshape(-1)
                else:
                    a = np.ascontiguousarray(layer.a, dtype=np.float32).reshape(-1)
                    b = np.ascontiguousarray(layer.b, dtype=np.float32).reshape(-1)
                h = C.c_void_p()
                # A/B length, overflow and u32 checks happen in the library
                check(_lib.lib().lq4_lora_upload(a.ctypes.data_as(C.c_void_p), a.size, b.ctypes.data_as(C.c_void_p),
                                                 b.size, layer.rank, layer.d_in, layer.d_out, scale, C.byref(h)))
                projections[layer.layer_idx][layer.module] = _LoraProjection(h.value, layer.rank, layer.d_in, layer.d_out)
                max_rank = max(max_rank, layer.rank)
        except Exception:
            for d in projections:
                for pr in d.values():
                    _lib.lib().lq4_lora_free(pr.handle)
            raise
        self.lora = _LoraAdapter(projections, float(scale), max_rank)

    def load_lora_adapter_file(self, path: str, quarot_seed: Optional[int] = None,
                               quarot_hidden_dim: Optional[int] = None) -> "PeftAdapter":   # noqa: F821
        """Reads a PEFT or MLX ``.safetensors`` adapter (bounded read, the reference's key grammar and refusals,
        ``lattice_b200/lora_safetensors.py``) and loads it with scale ``alpha / rank``."""
        from .lora_safetensors import load_peft_safetensors
        adapter = load_peft_safetensors(path)
        self.load_lora_adapter(adapter.layers, adapter.scale, quarot_seed, quarot_hidden_dim)
        return adapter

    def unload_lora_adapter(self) -> None:
        if self.lora is not None:
            for d in self.lora.projections:
                for pr in d.values():
                    _lib.lib().lq4_lora_free(pr.handle)
            self.lora = None

    def has_lora_adapter(self) -> bool:
        return self.lora is not None

    def get_projection(self, layer_idx: int, module: str) -> Optional[_LoraProjection]:
        if self.lora is None or layer_idx >= len(self.lora.projections):
            return None
        return self.lora.projections[layer_idx].get(module)

    def lora_desc(self, layer_idx: int, module: str, n0: int = 0, n1: Optional[int] = None) -> Optional[LoraDesc]:
        """Descriptor to pass as ``lora=`` so the delta is added inside the matmul launch."""
        pr = self.get_projection(layer_idx, module)
        if pr is None:
            return None
        d = LoraDesc()
        check(_lib.lib().lq4_lora_desc_for_rows(pr.handle, n0, pr.d_out if n1 is None else n1, C.byref(d)))
        return d

    def dispatch_lora_if_active(self, x: torch.Tensor, x_byte_offset: int, y: torch.Tensor, y_byte_offset: int,
                                layer_idx: int, module: str, m: int = 1, ldy: int = 0) -> None:
        """``y[0..d_out] += scale * B (A x)``; no-op without an adapter or a projection for this module."""
        pr = self.get_projection(layer_idx, module)
        if pr is None:
            return
        d = self.lora_desc(layer_idx, module)
        check(_lib.lib().lq4_lora_apply(self._ctx, x.data_ptr() + x_byte_offset, self._dtype_of(x), m, pr.d_in,
                                        y.data_ptr() + y_byte_offset, pr.d_out, ldy, C.byref(d), _stream()))

    # ---- helpers on device tensors ------------------------------------------------
    def dequantize(self, payload: torch.Tensor, n_blocks: int) -> torch.Tensor:
        out = torch.empty(n_blocks * 32, dtype=torch.float32, device=payload.device)
        check(_lib.lib().lq4_dequant_f32(payload.data_ptr(), n_blocks, out.data_ptr(), _stream()))
        return out

    def quantize(self, data: torch.Tensor, symmetric: bool = False) -> torch.Tensor:
        """Flat 32-chunk quantizer on the device; raises if a block was not representable."""
        assert data.is_cuda and data.dtype == torch.float32 and data.is_contiguous()
        n = data.numel()
        out = torch.empty(((n + 31) // 32) * 20, dtype=torch.uint8, device=data.device)
        st = torch.zeros(1, dtype=torch.int32, device=data.device)
        check(_lib.lib().lq4_quantize_f32(data.data_ptr(), n, int(symmetric), out.data_ptr(), st.data_ptr(), _stream()))
        if int(st.item()) != 0:
            raise Lq4Error(_lib.ERR_BAD_BLOCK, "a block had a non-finite value or unrepresentable scale/bias")
        return out

    _QUANT_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16, torch.float64: _lib.DTYPE_F64}

    def quantize_tensor(self, data: torch.Tensor, symmetric: bool = False, per_row: bool = False) -> torch.Tensor:
        """The reference's other quantizer entry points on the device, chosen by ``data``'s dtype: f32 flat
        (``quantize_f32_to_q4``) or per row (``quantize_tensor_q4_0``), bf16 (``quantize_bf16_to_q4``), f64
        (``quantize_f64_to_q4_mode``; ``symmetric=True`` is ``quantize_f64_to_q4``).  ``data`` is 1-D or 2-D."""
        assert data.is_cuda and data.is_contiguous() and data.dtype in self._QUANT_DTYPES
        rows, cols = (1, data.numel()) if data.dim() == 1 else (data.shape[0], data.shape[1])
        nb = rows * ((cols + 31) // 32) if per_row else (rows * cols + 31) // 32
        out = torch.empty(nb * 20, dtype=torch.uint8, device=data.device)
        st = torch.zeros(1, dtype=torch.int32, device=data.device)
        check(_lib.lib().lq4_quantize_tensor(data.data_ptr(), self._QUANT_DTYPES[data.dtype], rows, cols, int(per_row),
                                             int(symmetric), out.data_ptr(), st.data_ptr(), _stream()))
        if int(st.item()) != 0:
            raise Lq4Error(_lib.ERR_BAD_BLOCK, "a block had a non-finite value or unrepresentable scale/bias")
        return out

    def absorb_rotation(self, w: torch.Tensor, signs: torch.Tensor, side: str = "input") -> torch.Tensor:
        """``absorb_input_rotation{,_f64}`` (``W <- W R^T``) or ``absorb_output_rotation{,_f64}`` (``W <- R W``)
        in place on a 2-D f32 / f64 device tensor (crates/inference/src/quant/quarot/rotation.rs:86-195)."""
        assert w.is_cuda and w.is_contiguous() and w.dim() == 2 and w.dtype in (torch.float32, torch.float64)
        rot = self.rot_desc(signs)
        fn = _lib.lib().lq4_absorb_input_rotation if side == "input" else _lib.lib().lq4_absorb_output_rotation
        check(fn(w.data_ptr(), self._QUANT_DTYPES[w.dtype], w.shape[0], w.shape[1], C.byref(rot), _stream()))
        return w

    def save_q4_file(self, path: str, payload: torch.Tensor, shape) -> None:
        """``save_q4_file`` (q4_weights.rs:623-645) for a device payload of ``prod(shape)`` weights."""
        assert payload.is_cuda and payload.dtype == torch.uint8
        shp = (C.c_uint64 * len(shape))(*shape)
        n = int(np.prod(shape)) if len(shape) else 0
        assert payload.numel() >= ((n + 31) // 32) * 20
        check(_lib.lib().lq4_q4_file_write(str(path).encode(), shp, len(shape), n, payload.data_ptr(), _stream()))

    def rot_signs(self, seed: int, dim: int) -> torch.Tensor:
        s = torch.empty(dim, dtype=torch.float32, device=f"cuda:{self.device}")
        check(_lib.lib().lq4_rot_signs_from_seed(seed & (2 ** 64 - 1), dim, s.data_ptr(), _stream()))
        return s

    def block_rot_signs(self, seed: int, n: int, block: int) -> torch.Tensor:
        """The flat sign buffer of ``BlockHadamard::new(seed, n, block)`` (hadamard.rs:358-414)."""
        s = torch.empty(max(n, 1), dtype=torch.float32, device=f"cuda:{self.device}")
        check(_lib.lib().lq4_block_rot_signs_from_seed(seed & (2 ** 64 - 1), n, block, s.data_ptr(), _stream()))
        return s[:n]

    @staticmethod
    def rot_desc(signs: torch.Tensor, block: Optional[int] = None) -> RotDesc:
        """``block=None``: one rotation over ``len(signs)`` entries; else the block-diagonal rotation with that
        block size (``signs`` still holds one entry per activation column)."""
        assert signs.is_cuda and signs.dtype == torch.float32
        return RotDesc(signs.data_ptr(), signs.numel() if block is None else block)

    def block_hadamard_rows(self, x: torch.Tensor, signs: torch.Tensor, block: int) -> torch.Tensor:
        """``BlockHadamard::apply`` on every row of ``x`` (``[rows, n]``, ``n = len(signs)``)."""
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        out = torch.empty_like(x)
        rot = self.rot_desc(signs, block)
        n = signs.numel()
        check(_lib.lib().lq4_block_hadamard_rows(x.data_ptr(), out.data_ptr(), x.numel() // max(n, 1), n, C.byref(rot), _stream()))
        return out

    def hadamard_rows(self, x: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        out = torch.empty_like(x)
        rot = self.rot_desc(signs)
        check(_lib.lib().lq4_hadamard_rows(x.data_ptr(), out.data_ptr(), x.numel() // signs.numel(), C.byref(rot), _stream()))
        return out

    def cross_head_hadamard_rows(self, x: torch.Tensor, signs: torch.Tensor, head_dim: int) -> torch.Tensor:
        """The R3 "Hadamard heads" rotation of every row of ``x`` (``[rows, num_heads * head_dim]``,
        ``num_heads = len(signs)``): mixes across heads at each within-head channel."""
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        nh = signs.numel()
        out = torch.empty_like(x)
        check(_lib.lib().lq4_cross_head_hadamard_rows(x.data_ptr(), out.data_ptr(), x.numel() // max(nh * head_dim, 1),
                                                      nh, head_dim, signs.data_ptr(), _stream()))
        return out

    def linear(self, x: torch.Tensor, qw: Q4WeightBuf, *, lora: Optional[LoraDesc] = None,
               rot: Optional[RotDesc] = None, path: int = _lib.PATH_AUTO, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Convenience wrapper: ``x`` is ``[m, k]`` on the device, returns ``[m, n]`` f32."""
        m, k = x.shape
        y = out if out is not None else torch.empty((m, qw.n), dtype=torch.float32, device=x.device)
        self.dispatch_gemm_q4(x.contiguous(), 0, qw, y, 0, m, qw.n, k, lora=lora, rot=rot, path=path)
        return y

    # ---- dense MLP block ------------------------------------------------------------------
    def mlp_block(self, x: torch.Tensor, w_gate_up: Q4WeightBuf, w_down: Q4WeightBuf, *,
                  lora_gate: Optional[LoraDesc] = None, lora_up: Optional[LoraDesc] = None,
                  lora_down: Optional[LoraDesc] = None, gate_up: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None, rot_down: Optional[RotDesc] = None) -> torch.Tensor:
        """The FFN half of the reference's ``encode_mlp_block`` for dense layers: merged gate||up projection
        (``w_gate_up`` is ``[2 * inter, hidden]``), ``silu(gate) * up``, ``down_proj``; ``x`` is ``[m, hidden]``."""
        from ._lib import MlpArgs
        x = x.contiguous()
        m, hidden = x.shape
        inter = w_gate_up.n // 2
        self._require_k("mlp_block", hidden)
        self._require_k("mlp_block", inter)
        if w_gate_up.k != hidden or w_gate_up.n != 2 * inter or w_down.k != inter or w_down.n != hidden:
            raise ValueError("mlp_block: w_gate_up must be [2 * inter, hidden] and w_down [hidden, inter]")
        y = out if out is not None else torch.empty((m, hidden), dtype=torch.float32, device=x.device)
        args = MlpArgs(x.data_ptr(), self._dtype_of(x), m, hidden, inter, w_gate_up.payload_ptr, w_down.payload_ptr,
                       C.pointer(lora_gate) if lora_gate is not None else None,
                       C.pointer(lora_up) if lora_up is not None else None,
                       C.pointer(lora_down) if lora_down is not None else None,
                       gate_up.data_ptr() if gate_up is not None else None, y.data_ptr(),
                       C.pointer(rot_down) if rot_down is not None else None)
        check(_lib.lib().lq4_mlp_block(self._ctx, C.byref(args), _stream()))
        return y

    # ---- lm_head: vocabulary projection + exact top-k --------------------------------------
    @staticmethod
    def _split_candidates(cand: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``cand`` is ``[top_k, 2]`` int32 holding (logit bits, token id) pairs."""
        return cand[:, 0].view(torch.float32), cand[:, 1]        # strided views: no copy kernels

    def logits_topk(self, logits: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Top ``top_k`` of a device logit row in the reference's candidate order (higher logit first, ties to
        the lower token id, NaN never ranks).  Returns ``(logits[top_k] f32, token_ids[top_k] int32)``; token
        ids of unused slots are -1 (0xFFFFFFFF) with logit -inf."""
        if logits.dtype != torch.float32 or logits.dim() != 1:
            raise TypeError("logits must be a 1-D float32 device tensor")
        logits = logits.contiguous()
        cand = torch.empty((max(top_k, 1), 2), dtype=torch.int32, device=logits.device)
        check(_lib.lib().lq4_logits_topk(self._ctx, logits.data_ptr(), logits.numel(), top_k, cand.data_ptr(), _stream()))
        return self._split_candidates(cand)

    def lm_head_topk(self, x: torch.Tensor, qw: Q4WeightBuf, top_k: int, *, lora: Optional[LoraDesc] = None,
                     rot: Optional[RotDesc] = None, logits_out: Optional[torch.Tensor] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
        """One token's vocabulary projection followed by the exact top-k (the reference's two-stage lm_head
        path).  ``x`` is ``[1, k]`` or ``[k]``; ``logits_out`` (``[n]`` f32), when given, also receives the
        full logit row, otherwise it stays in the context's workspace."""
        x = x.reshape(1, -1).contiguous()
        k = x.shape[1]
        self._require_k("lm_head_topk", k)
        if k != qw.k:
            raise ValueError(f"x has {k} columns, the weights have {qw.k}")
        cand = torch.empty((max(top_k, 1), 2), dtype=torch.int32, device=x.device)
        args = LinearArgs(x.data_ptr(), self._dtype_of(x), 1, qw.n, k, qw.payload_ptr,
                          logits_out.data_ptr() if logits_out is not None else None, 0,
                          C.pointer(lora) if lora is not None else None,
                          C.pointer(rot) if rot is not None else None, _lib.PATH_AUTO, None, None)
        check(_lib.lib().lq4_lm_head_topk(self._ctx, C.byref(args), top_k, cand.data_ptr(), _stream()))
        return self._split_candidates(cand)

    def prepare_group(self, problems, outs: Optional[List[torch.Tensor]] = None,
                      gather: Optional[GatherDesc] = None, wait_gather: Optional[GatherDesc] = None) -> "PreparedGroup":
        """Builds the argument block of a grouped call once; calling the result launches it.

        ``problems`` is a list of ``(x, qw)`` or ``(x, qw, lora)`` with ``x`` ``[m, k]`` on the device.  The
        tensors are referenced, not copied: refill ``x`` in place between calls.  No output may alias
        another problem's input."""
        n_prob = len(problems)
        arr = (LinearArgs * max(n_prob, 1))()
        keep, ys = [], []
        for i, pr in enumerate(problems):
            x, qw = pr[0], pr[1]
            lora = pr[2] if len(pr) > 2 else None
            m, k = x.shape
            self._require_k("linear_group", k)
            assert x.is_cuda and x.is_contiguous(), "activations are contiguous [m, k] device tensors"
            y = outs[i] if outs is not None else torch.empty((m, qw.n), dtype=torch.float32, device=x.device)
            assert y.is_cuda and y.dtype == torch.float32
            assert y.shape == (m, qw.n) and y.stride(1) == 1, "outputs are [m, n] with unit column stride"
            keep.append((x, qw, lora))
            ys.append(y)
            ldy = y.stride(0) if m > 1 or y.stride(0) >= qw.n else qw.n      # row pitch of a column slice
            arr[i] = LinearArgs(x.data_ptr(), self._dtype_of(x), m, qw.n, k, qw.payload_ptr, y.data_ptr(), ldy,
                                C.pointer(lora) if lora is not None else None, None, _lib.PATH_AUTO,
                                C.pointer(gather) if gather is not None else None,
                                C.pointer(wait_gather) if wait_gather is not None else None)
        keep += [gather, wait_gather]
        return PreparedGroup(self, arr, n_prob, ys, keep)

    def prepare_step(self, groups, step_buffer=None, gathered=None, host: bool = False) -> "PreparedStep":
        """Builds the argument blocks of one ``lq4_decode_step`` call; calling the result launches it.

        ``groups`` is a list of groups, each a list of ``(x, qw, lora, y)`` with ``x`` ``[1, k]`` or ``[k]`` and
        ``y`` ``[n]`` (or ``[1, n]``) device tensors.  A later group's ``x`` may be a slice of
        ``step_buffer.payload`` where earlier groups' ``y`` slices lie.  ``gathered`` lists the payload slices
        that must be complete on this rank when the launch completes.  ``host=True`` makes the call
        ``lq4_decode_step_host``: inputs and outputs may then be pinned host tensors (``pin_memory=True``); the
        inputs are staged in by a kernel chained in front of the step kernel, the outputs are stored by the step
        kernel itself, and the caller synchronises before it reads them."""
        from ._lib import StepDesc, StepGroup, StepRange
        keep, garr = [], (StepGroup * max(len(groups), 1))()
        for gi, grp in enumerate(groups):
            arr = (LinearArgs * max(len(grp), 1))()
            for i, (x, qw, lora, y) in enumerate(grp):
                k = x.numel()
                self._require_k("decode_step", k)
                assert (x.is_cuda or (host and x.is_pinned())) and (y.is_cuda or (host and y.is_pinned()))
                assert y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
                assert k == qw.k and y.numel() == qw.n
                arr[i] = LinearArgs(x.data_ptr(), self._dtype_of(x), 1, qw.n, k, qw.payload_ptr, y.data_ptr(), 0,
                                    C.pointer(lora) if lora is not None else None, None, _lib.PATH_AUTO, None, None)
                keep.append((x, qw, lora, y))
            keep.append(arr)
            garr[gi] = StepGroup(C.cast(arr, C.c_void_p).value, len(grp))
        desc = None
        if step_buffer is not None:
            rng = (StepRange * max(len(gathered or []), 1))()
            for i, t in enumerate(gathered or []):
                assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()
                rng[i] = StepRange(t.data_ptr(), t.numel())
            desc = StepDesc(C.pointer(step_buffer.desc), C.cast(rng, C.c_void_p).value, len(gathered or []))
            keep += [rng, step_buffer, gathered]
        return PreparedStep(self, garr, len(groups), desc, keep, host)

    def gather_wait(self, gather: GatherDesc) -> None:
        """Stream-ordered wait until every peer's results of the gathered launches issued so far are here."""
        check(_lib.lib().lq4_gather_wait(self._ctx, C.byref(gather), _stream()))

    def linear_group(self, problems, outs: Optional[List[torch.Tensor]] = None,
                     gather: Optional[GatherDesc] = None, wait_gather: Optional[GatherDesc] = None) -> List[torch.Tensor]:
        """Several independent projections in one call (one persistent launch for decode shapes);
        returns the list of ``[m, n]`` f32 outputs."""
        if len(problems) == 0:
            return []
        problems = [(pr[0].contiguous(),) + tuple(pr[1:]) for pr in problems]
        return self.prepare_group(problems, outs, gather, wait_gather)()

    def linear_host(self, x: np.ndarray, qw: Q4WeightBuf, y: np.ndarray, *, lora: Optional[LoraDesc] = None,
                    rot: Optional[RotDesc] = None) -> None:
        """End-to-end call with HOST activations and output (copies inside the call, waits for y)."""
        m, k = x.shape
        self._require_k("linear_host", k)
        dt = _lib.DTYPE_F32 if x.dtype == np.float32 else _lib.DTYPE_BF16
        self._linear(x.ctypes.data, dt, qw.payload_ptr, y.ctypes.data, m, qw.n, k, 0, lora, rot, host=True)
