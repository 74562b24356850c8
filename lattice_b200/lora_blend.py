"""Exact blending of several LoRA adapters into one adapter of the summed rank.

Mirrors ``blend_lora_adapters`` (crates/tune/src/lora/blend.rs:28-123) and its per-projection
helper (:126-200): for every ``(layer_idx, module)`` that any source adapter targets, the A blocks are
stacked vertically and the B blocks horizontally after each source's mixture weight and its own
``alpha / rank`` scale have been folded into B, so that

    sum_i w_i * s_i * B_i (A_i x)  ==  B_blend (A_blend x)         with scale exactly 1.

The result is loaded with ``load_lora_adapter(layers, scale=1.0)``; the decode kernels take ranks up to
128 on the fast path, larger blended ranks fall back to the generic kernel.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import numpy as np

from .backend import LoraLayerData

MAX_BLEND_RANK_TOTAL = 4096          # crates/fann/src/lora.rs:141


def blend_lora_layer_data(adapters: Sequence[Tuple[Sequence[LoraLayerData], float, float]]) -> List[LoraLayerData]:
    """``adapters`` is a sequence of ``(layers, scale, mixture_weight)``; returns the blended layers
    (to be loaded with scale 1.0).  Raises ``ValueError`` where the reference returns a validation error."""
    if len(adapters) == 0:
        raise ValueError("blend_lora_adapters: adapters slice must not be empty")
    for idx, (layers, scale, weight) in enumerate(adapters):
        if not math.isfinite(weight):
            raise ValueError(f"blend_lora_adapters: adapters[{idx}] mixture weight must be finite, got {weight}")
        if not math.isfinite(scale):
            raise ValueError(f"blend_lora_adapters: adapters[{idx}] scale must be finite, got {scale}")
        if len(layers) == 0:
            raise ValueError(f"blend_lora_adapters: adapters[{idx}] has no layers")
    grouped: Dict[Tuple[int, str], List[Tuple[LoraLayerData, float]]] = {}
    for layers, scale, weight in adapters:
        for layer in layers:
            grouped.setdefault((layer.layer_idx, layer.module), []).append((layer, float(weight) * float(scale)))
    out: List[LoraLayerData] = []
    for (layer_idx, module), entries in sorted(grouped.items()):
        first = entries[0][0]
        d_in, d_out = first.d_in, first.d_out
        rank_total = 0
        for i, (layer, _) in enumerate(entries):
            if (layer.d_in, layer.d_out) != (d_in, d_out):
                raise ValueError(f"blend_lora_adapters: layer {layer_idx} module '{module}' source {i} has "
                                 f"(d_in={layer.d_in}, d_out={layer.d_out}) but the first source has "
                                 f"(d_in={d_in}, d_out={d_out})")
            if layer.rank == 0:
                raise ValueError(f"blend_lora_adapters: layer {layer_idx} module '{module}' source {i} has rank 0")
            a_len, b_len = np.asarray(layer.a).size, np.asarray(layer.b).size
            if a_len != layer.rank * d_in or b_len != d_out * layer.rank:
                raise ValueError(f"blend_layer_entries: source {i} buffer lengths (A {a_len}, B {b_len}) do not match "
                                 f"rank {layer.rank} x (d_in {d_in}, d_out {d_out})")
            rank_total += layer.rank
        if rank_total > MAX_BLEND_RANK_TOTAL:
            raise ValueError(f"blend_layer_entries: summed rank {rank_total} exceeds "
                             f"MAX_BLEND_RANK_TOTAL={MAX_BLEND_RANK_TOTAL}")
        a = np.concatenate([np.asarray(l.a, np.float32).reshape(l.rank, d_in) for l, _ in entries], axis=0)
        b = np.concatenate([np.float32(eff) * np.asarray(l.b, np.float32).reshape(d_out, l.rank) for l, eff in entries],
                           axis=1)
        out.append(LoraLayerData(layer_idx, module, np.ascontiguousarray(a), np.ascontiguousarray(b), rank_total, d_in, d_out))
    return out
