"""``quantize_index.json``: the per-tensor manifest beside a Q4 checkpoint's ``.q4`` files.

Mirrors the bounded, fail-closed reader of the reference
(crates/inference/src/quant/q4_manifest.rs:154-279).  Two writers exist upstream:

* ``bin/quantize_q4.rs`` writes a bare JSON array of tensor entries (flavor ``"quantize_q4"``);
* the QuaRot converter writes ``{"quarot_seed": u64 | null, "tensors": [...]}`` (flavor ``"quarot"``),
  so that a loader recovers the rotation seed without any other file.

A manifest that is absent is a valid, degraded input (``None``); one that is present but oversized,
unreadable, a dangling symlink, not JSON, or of neither shape is an error.  ``load_q4_directory``
then uploads every quantized 2-D tensor through the C library's ``.q4`` loader, which repeats the
reference's header, extent, shape and per-block checks.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

MAX_QUANTIZE_INDEX_LEN = 16 * 1024 * 1024      # q4_manifest.rs:52
MANIFEST_NAME = "quantize_index.json"


class ManifestError(ValueError):
    """``kind`` is one of ``unreadable``, ``too_large``, ``invalid_json``, ``invalid_shape``
    (the reference's ``Q4ManifestError`` variants, q4_manifest.rs:63-84)."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


@dataclass
class ManifestEntry:
    name: str
    file: str
    quantized: Optional[bool] = None
    shape: Optional[List[int]] = None
    numel: Optional[int] = None


@dataclass
class Manifest:
    flavor: str                       # "quantize_q4" (bare array) or "quarot" (object form)
    quarot_seed: Optional[int]
    tensors: List[ManifestEntry]


def read_manifest_bytes_bounded(path: str) -> Optional[bytes]:
    """``None`` only if there is no directory entry at ``path``; at most 16 MiB are ever read."""
    try:
        os.lstat(path)                 # does not follow symlinks: a dangling link is "present"
    except FileNotFoundError:
        return None
    except OSError as e:
        raise ManifestError("unreadable", f"{path}: failed to stat {MANIFEST_NAME}: {e}")
    try:
        size = os.stat(path).st_size
    except OSError as e:
        raise ManifestError("unreadable", f"{path}: {MANIFEST_NAME} entry exists but is unreadable "
                                          f"(broken symlink or permission error): {e}")
    if size > MAX_QUANTIZE_INDEX_LEN:
        raise ManifestError("too_large", f"{path}: {MANIFEST_NAME} too large: {size} bytes exceeds cap of "
                                         f"{MAX_QUANTIZE_INDEX_LEN} bytes")
    try:
        with open(path, "rb") as f:
            buf = f.read(MAX_QUANTIZE_INDEX_LEN + 1)      # a file swapped for a larger one is still bounded
    except OSError as e:
        raise ManifestError("unreadable", f"{path}: failed to read {MANIFEST_NAME}: {e}")
    if len(buf) > MAX_QUANTIZE_INDEX_LEN:
        raise ManifestError("too_large", f"{path}: {MANIFEST_NAME} too large: read exceeds cap of "
                                         f"{MAX_QUANTIZE_INDEX_LEN} bytes")
    return buf


def _entry(obj, where: str) -> ManifestEntry:
    if not isinstance(obj, dict):
        raise ManifestError("invalid_shape", f"{where}: tensor entry is not an object")
    for key in ("name", "file"):
        if not isinstance(obj.get(key), str):
            raise ManifestError("invalid_shape", f"{where}: missing field `{key}`")
    quantized = obj.get("quantized")
    if quantized is not None and not isinstance(quantized, bool):
        raise ManifestError("invalid_shape", f"{where}: `quantized` is not a boolean")
    shape = obj.get("shape")
    if shape is not None and not (isinstance(shape, list) and all(isinstance(d, int) and not isinstance(d, bool) and d >= 0
                                                                   for d in shape)):
        raise ManifestError("invalid_shape", f"{where}: `shape` is not a list of non-negative integers")
    numel = obj.get("numel")
    if numel is not None and not (isinstance(numel, int) and not isinstance(numel, bool) and numel >= 0):
        raise ManifestError("invalid_shape", f"{where}: `numel` is not a non-negative integer")
    return ManifestEntry(obj["name"], obj["file"], quantized, shape, numel)


def parse_manifest(data: bytes, path: str = MANIFEST_NAME) -> Manifest:
    try:
        value = json.loads(data)
    except (ValueError, UnicodeDecodeError) as e:
        raise ManifestError("invalid_json", f"{path} is not valid JSON: {e}")
    if isinstance(value, list):
        return Manifest("quantize_q4", None,
                        [_entry(v, f"{path}: invalid bare-array (quantize_q4) manifest") for v in value])
    if isinstance(value, dict):
        where = f"{path}: invalid object-form (quantize_quarot) manifest"
        tensors = value.get("tensors")
        if not isinstance(tensors, list):
            raise ManifestError("invalid_shape", f"{where}: missing field `tensors`")
        seed = value.get("quarot_seed")
        if seed is not None and not (isinstance(seed, int) and not isinstance(seed, bool) and 0 <= seed < 2 ** 64):
            raise ManifestError("invalid_shape", f"{where}: `quarot_seed` is not a u64")
        return Manifest("quarot", seed, [_entry(v, where) for v in tensors])
    raise ManifestError("invalid_shape", f"{path}: expected {MANIFEST_NAME} to be either a bare array of tensor "
                                         f"entries (quantize_q4) or an object with a \"tensors\" array (quantize_quarot)")


def load_manifest(directory: str) -> Optional[Manifest]:
    path = os.path.join(directory, MANIFEST_NAME)
    data = read_manifest_bytes_bounded(path)
    return None if data is None else parse_manifest(data, path)


def load_q4_directory(directory: str, names: Optional[List[str]] = None) -> Dict[str, "Q4WeightBuf"]:   # noqa: F821
    """Uploads the quantized 2-D tensors the manifest lists (all of them, or ``names``) and returns them by
    tensor name.  Entries kept in f16 (``quantized == false``) and non-2-D tensors are skipped; a file
    name that leaves the directory is refused."""
    from .backend import Q4WeightBuf
    manifest = load_manifest(directory)
    if manifest is None:
        raise ManifestError("unreadable", f"{directory}: no {MANIFEST_NAME}")
    out: Dict[str, Q4WeightBuf] = {}
    try:
        for e in manifest.tensors:
            if names is not None and e.name not in names:
                continue
            if e.quantized is False or not e.file.endswith(".q4"):
                continue
            if e.shape is not None and len(e.shape) != 2:
                continue
            if os.path.isabs(e.file) or ".." in e.file.replace("\\", "/").split("/"):
                raise ManifestError("invalid_shape", f"{directory}: entry '{e.name}' points outside the directory")
            out[e.name] = Q4WeightBuf.from_q4_file(os.path.join(directory, e.file),
                                                   tuple(e.shape) if e.shape is not None else None)
    except Exception:
        for qw in out.values():
            qw.free()
        raise
    return out
