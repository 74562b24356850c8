"""PEFT / MLX safetensors adapters -> ``LoraLayerData`` for ``CudaQ4Backend.load_lora_adapter``.

Mirrors the reference's importer (crates/tune/src/lora/safetensors.rs:36-375,449-520):

* key grammar (``parse_peft_key``, :36-83): optional ``.weight`` suffix, ``.lora_A`` / ``.lora_B`` (PEFT) or
  ``.lora_a`` / ``.lora_b`` (MLX, stored transposed), a ``.layers.{i}.`` segment, the module is the last path
  segment; every other key is ignored;
* tensors are F32, F16 or BF16, converted to f32, any non-finite value is refused (:88-150);
* MLX tensors are transposed to the PEFT orientation A ``(rank, d_in)``, B ``(d_out, rank)`` (:207-232);
* every A needs its B and the reverse, both 2-D, equal ranks inside a pair and ONE rank across the file,
  element counts equal to the shapes (:253-345);
* ``alpha`` comes from the header metadata (a finite float) and defaults to the rank (:347-367);
* files are read through a size bound (10 GiB) before anything is parsed (:449-503).

The container itself is the published safetensors layout (the reference uses the ``safetensors`` crate, which
is not vendored in its tree): an 8-byte little-endian header length, that many bytes of JSON mapping tensor
names to ``{"dtype", "shape", "data_offsets": [begin, end]}`` plus an optional ``"__metadata__"`` string map,
then the tensor bytes.  The parser here checks what that crate checks: header length within the file and a
100 MB cap, offsets inside the buffer, ``end - begin`` equal to the shape's byte size, no overlapping or
uncovered ranges.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

MAX_LORA_SIZE = 10 * 1024 * 1024 * 1024          # safetensors.rs:449
MAX_HEADER_SIZE = 100_000_000                    # the safetensors format's header cap

_DTYPE_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1,
                "U16": 2, "U32": 4, "U64": 8, "F8_E5M2": 1, "F8_E4M3": 1}


class LoraFileError(ValueError):
    """A malformed, incomplete or inconsistent adapter file (the reference's ``TuneError::Serialization`` /
    ``TuneError::Io``)."""


@dataclass(frozen=True)
class PeftKey:
    layer_idx: int
    module: str
    matrix: str            # "A" or "B"
    transposed: bool       # MLX layout: A = (d_in, rank), B = (rank, d_out)


def parse_peft_key(key: str) -> Optional[PeftKey]:
    """``None`` for every key that is not a LoRA factor of a numbered layer."""
    if key.endswith(".weight"):
        key = key[:-len(".weight")]
    for suffix, matrix, mlx in ((".lora_A", "A", False), (".lora_B", "B", False), (".lora_a", "A", True), (".lora_b", "B", True)):
        if key.endswith(suffix):
            key = key[:-len(suffix)]
            break
    else:
        return None
    marker = ".layers."
    pos = key.find(marker)
    if pos < 0:
        return None
    after = key[pos + len(marker):]
    dot = after.find(".")
    if dot < 0:
        return None
    idx = after[:dot]
    if idx.startswith("+"):                       # Rust's usize::from_str takes one leading '+'
        idx = idx[1:]
    if not (idx.isascii() and idx.isdigit()) or int(idx) >= 2 ** 64:
        return None
    module = after[dot + 1:].rsplit(".", 1)[-1]
    if not module:
        return None
    return PeftKey(int(idx), module, matrix, mlx)


@dataclass
class _TensorInfo:
    dtype: str
    shape: List[int]
    begin: int
    end: int


def _parse_container(data: bytes) -> Tuple[Dict[str, _TensorInfo], Dict[str, str], int]:
    """Header checks of the safetensors format; returns (tensors, metadata, offset of the byte buffer)."""
    if len(data) < 8:
        raise LoraFileError("failed to parse safetensors: header too small")
    (n,) = struct.unpack("<Q", data[:8])
    if n > MAX_HEADER_SIZE:
        raise LoraFileError("failed to parse safetensors: header too large")
    if 8 + n > len(data):
        raise LoraFileError("failed to parse safetensors: invalid header length")
    try:
        header = json.loads(data[8:8 + n].decode("utf-8"))
    except (UnicodeDecodeError, ValueError) as e:
        raise LoraFileError(f"failed to parse safetensors: invalid header: {e}")
    if not isinstance(header, dict):
        raise LoraFileError("failed to parse safetensors: header is not an object")
    metadata: Dict[str, str] = {}
    tensors: Dict[str, _TensorInfo] = {}
    for name, info in header.items():
        if name == "__metadata__":
            if not isinstance(info, dict) or not all(isinstance(k, str) and isinstance(v, str) for k, v in info.items()):
                raise LoraFileError("failed to parse safetensors: __metadata__ is not a string map")
            metadata = info
            continue
        try:
            dtype, shape, (begin, end) = info["dtype"], info["shape"], info["data_offsets"]
        except (TypeError, KeyError, ValueError):
            raise LoraFileError(f"failed to parse safetensors: malformed entry for tensor '{name}'")
        if dtype not in _DTYPE_BYTES or not isinstance(shape, list) or \
                not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape) or \
                not all(isinstance(o, int) and not isinstance(o, bool) and o >= 0 for o in (begin, end)):
            raise LoraFileError(f"failed to parse safetensors: malformed entry for tensor '{name}'")
        tensors[name] = _TensorInfo(dtype, shape, begin, end)
    buf_len = len(data) - 8 - n
    covered = 0
    for name, t in sorted(tensors.items(), key=lambda kv: kv[1].begin):
        if t.begin != covered or t.end < t.begin:
            raise LoraFileError(f"failed to parse safetensors: invalid offsets for tensor '{name}'")
        numel = 1
        for d in t.shape:
            numel *= d
        if t.end - t.begin != numel * _DTYPE_BYTES[t.dtype]:
            raise LoraFileError(f"failed to parse safetensors: tensor '{name}' byte size does not match its shape")
        covered = t.end
    if covered != buf_len:
        raise LoraFileError("failed to parse safetensors: metadata incomplete buffer")
    return tensors, metadata, 8 + n


def _read_tensor_f32(data: bytes, base: int, name: str, t: _TensorInfo) -> Tuple[np.ndarray, List[int]]:
    raw = data[base + t.begin: base + t.end]
    if t.dtype == "F32":
        vals = np.frombuffer(raw, dtype="<f4").astype(np.float32)
    elif t.dtype == "F16":
        vals = np.frombuffer(raw, dtype="<f2").astype(np.float32)
    elif t.dtype == "BF16":
        vals = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
    else:
        raise LoraFileError(f"tensor '{name}' has unsupported dtype {t.dtype}, expected F32/F16/BF16")
    bad = np.flatnonzero(~np.isfinite(vals))
    if bad.size:
        raise LoraFileError(f"tensor '{name}' contains non-finite value at index {int(bad[0])}: {vals[bad[0]]}")
    return vals, list(t.shape)


@dataclass
class PeftAdapter:
    """What ``load_peft_safetensors_bytes`` returns: the factor pairs plus the adapter-level configuration."""
    layers: list                       # List[LoraLayerData], sorted by (layer, module)
    rank: int
    alpha: float
    target_modules: List[str]          # sorted, as the reference's BTreeSet yields them
    metadata: Dict[str, str]

    @property
    def scale(self) -> float:
        """``alpha / rank`` (the reference's effective scale, crates/tune/src/lora/mod.rs:87-101)."""
        return float(np.float32(self.alpha) / np.float32(self.rank))


def load_peft_safetensors_bytes(data: bytes) -> PeftAdapter:
    from .backend import LoraLayerData
    tensors, metadata, base = _parse_container(data)
    a_t: Dict[Tuple[int, str], Tuple[np.ndarray, List[int]]] = {}
    b_t: Dict[Tuple[int, str], Tuple[np.ndarray, List[int]]] = {}
    modules = set()
    for name, info in tensors.items():
        pk = parse_peft_key(name)
        if pk is None:
            continue
        vals, shape = _read_tensor_f32(data, base, name, info)
        modules.add(pk.module)
        if pk.transposed and len(shape) == 2:
            vals = np.ascontiguousarray(vals.reshape(shape[0], shape[1]).T).reshape(-1)
            shape = [shape[1], shape[0]]
        (a_t if pk.matrix == "A" else b_t)[(pk.layer_idx, pk.module)] = (vals, shape)
    if not a_t and not b_t:
        raise LoraFileError("LoRA adapter contains no lora_A/lora_B tensors")
    rank: Optional[int] = None
    layers = []
    for key in sorted(a_t):
        a, a_shape = a_t[key]
        if key not in b_t:
            raise LoraFileError(f"LoRA adapter has lora_A for layer {key[0]} module '{key[1]}' but no matching lora_B")
        b, b_shape = b_t[key]
        if len(a_shape) != 2 or len(b_shape) != 2:
            raise LoraFileError(f"LoRA matrices for layer {key[0]} module '{key[1]}' must be 2D, got A={a_shape} B={b_shape}")
        a_rank, d_in = a_shape
        d_out, b_rank = b_shape
        if a_rank != b_rank:
            raise LoraFileError(f"LoRA rank mismatch for layer {key[0]} module '{key[1]}': A rank={a_rank}, B rank={b_rank}")
        if rank is None:
            rank = a_rank
        elif rank != a_rank:
            raise LoraFileError(f"inconsistent LoRA ranks: first seen rank={rank}, layer {key[0]} module '{key[1]}' has rank={a_rank}")
        if a.size != a_rank * d_in:
            raise LoraFileError(f"LoRA A data size mismatch for layer {key[0]} module '{key[1]}': expected {a_rank * d_in}, got {a.size}")
        if b.size != d_out * b_rank:
            raise LoraFileError(f"LoRA B data size mismatch for layer {key[0]} module '{key[1]}': expected {d_out * b_rank}, got {b.size}")
        layers.append(LoraLayerData(key[0], key[1], a.reshape(a_rank, d_in), b.reshape(d_out, b_rank), a_rank, d_in, d_out))
    for key in b_t:
        if key not in a_t:
            raise LoraFileError(f"LoRA adapter has lora_B for layer {key[0]} module '{key[1]}' but no matching lora_A")
    rank = rank or 0
    if "alpha" in metadata:
        try:
            text = metadata["alpha"]
            if "_" in text or text != text.strip():           # accepted by Python's float(), not by Rust's f32::from_str
                raise ValueError("invalid float literal")
            alpha = float(np.float32(float(text)))
        except ValueError as e:
            raise LoraFileError(f"invalid LoRA alpha metadata '{metadata['alpha']}': {e}")
        if not np.isfinite(alpha):
            raise LoraFileError(f"LoRA alpha metadata must be finite, got '{metadata['alpha']}'")
    else:
        alpha = float(rank)
    if rank == 0 or not np.isfinite(np.float32(alpha) / np.float32(rank)):
        raise LoraFileError("LoRA adapter needs a non-zero rank and a finite alpha / rank")      # LoraAdapter::new
    return PeftAdapter(layers, rank, alpha, sorted(modules), dict(metadata))


def read_lora_file_bounded(path: str, max_bytes: int = MAX_LORA_SIZE) -> bytes:
    """Two-stage bound (safetensors.rs:452-503): the size on disk is checked before anything is allocated, and
    the read itself stops at the bound, so a file that grows in between is still refused."""
    try:
        size = os.stat(path).st_size
    except OSError as e:
        raise LoraFileError(f"failed to read metadata for {path}: {e}")
    if size > max_bytes:
        raise LoraFileError(f"LoRA file {path} is {size} bytes, exceeds maximum of {max_bytes} bytes")
    try:
        with open(path, "rb") as f:
            data = f.read(max_bytes + 1)
    except OSError as e:
        raise LoraFileError(f"failed to read {path}: {e}")
    if len(data) > max_bytes:
        raise LoraFileError(f"LoRA file {path} grew past the maximum of {max_bytes} bytes while being read")
    return data


def load_peft_safetensors(path: str, max_bytes: int = MAX_LORA_SIZE) -> PeftAdapter:
    return load_peft_safetensors_bytes(read_lora_file_bounded(path, max_bytes))


def _block_of(module: str) -> str:
    """The transformer block a module's key is written under (safetensors.rs:526-530)."""
    return "mlp" if module in ("gate_proj", "up_proj", "down_proj") else "self_attn"


def save_peft_safetensors(path: str, layers, rank: int, alpha: float, target_modules: Optional[List[str]] = None,
                          extra_metadata: Optional[Dict[str, str]] = None) -> None:
    """PEFT-compatible export (safetensors.rs:505-585): F32 tensors ``base_model.model.model.layers.{i}.{block}.
    {module}.lora_A.weight`` ``(rank, d_in)`` and ``...lora_B.weight`` ``(d_out, rank)``, header metadata ``rank``,
    ``alpha`` and ``target_modules``; layers whose factors are empty are skipped."""
    entries = []
    for l in sorted(layers, key=lambda l: (l.layer_idx, l.module)):
        a = np.ascontiguousarray(l.a, dtype="<f4")
        b = np.ascontiguousarray(l.b, dtype="<f4")
        if a.size == 0 or b.size == 0:
            continue
        if a.size != l.rank * l.d_in or b.size != l.d_out * l.rank:
            raise LoraFileError(f"layer {l.layer_idx} module '{l.module}': factor sizes do not match rank, d_in, d_out")
        stem = f"base_model.model.model.layers.{l.layer_idx}.{_block_of(l.module)}.{l.module}"
        entries.append((stem + ".lora_A.weight", [l.rank, l.d_in], a.tobytes()))
        entries.append((stem + ".lora_B.weight", [l.d_out, l.rank], b.tobytes()))
    if target_modules is None:
        target_modules = sorted({l.module for l in layers})
    meta = {"rank": str(rank), "alpha": str(np.float32(alpha)) if float(alpha) != int(alpha) else str(int(alpha)),      # f32 Display
            "target_modules": ",".join(target_modules)}
    meta.update(extra_metadata or {})
    header: Dict[str, object] = {"__metadata__": meta}
    blob = bytearray()
    for name, shape, raw in sorted(entries):                    # tensors in name order, offsets back to back
        header[name] = {"dtype": "F32", "shape": shape, "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * ((8 - len(h) % 8) % 8)                          # the format pads the header to 8 bytes with spaces
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + bytes(blob))
