"""Adapter blending (crates/tune/src/lora/blend.rs): the blended adapter applied with scale 1 equals the
weighted sum of the sources, checked with the oracle's apply_lora."""
import numpy as np
import pytest

import oracle

pytest.importorskip("torch")
from lattice_b200 import LoraLayerData                      # noqa: E402
from lattice_b200.lora_blend import MAX_BLEND_RANK_TOTAL, blend_lora_layer_data      # noqa: E402


def layer(rng, idx, module, rank, d_in, d_out):
    return LoraLayerData(idx, module, rng.standard_normal((rank, d_in), dtype=np.float32) * 0.1,
                         rng.standard_normal((d_out, rank), dtype=np.float32) * 0.1, rank, d_in, d_out)


def test_blend_equals_weighted_sum_of_the_sources():
    rng = np.random.default_rng(3)
    d_in, d_out = 64, 48
    a1 = [layer(rng, 0, "q_proj", 4, d_in, d_out), layer(rng, 1, "q_proj", 4, d_in, d_out)]
    a2 = [layer(rng, 0, "q_proj", 8, d_in, d_out), layer(rng, 0, "v_proj", 2, d_in, d_out)]
    sources = [(a1, 2.0, 0.75), (a2, 0.5, -0.25)]
    blended = {(l.layer_idx, l.module): l for l in blend_lora_layer_data(sources)}
    assert set(blended) == {(0, "q_proj"), (1, "q_proj"), (0, "v_proj")}      # union of the targets
    assert blended[(0, "q_proj")].rank == 12 and blended[(1, "q_proj")].rank == 4 and blended[(0, "v_proj")].rank == 2
    x = rng.standard_normal(d_in, dtype=np.float32)
    for key, bl in blended.items():
        want = np.zeros(d_out, np.float32)
        for layers, scale, weight in sources:
            for l in layers:
                if (l.layer_idx, l.module) == key:
                    assert oracle.apply_lora(l.a, l.b, l.rank, d_in, d_out, weight * scale, x, want)
        got = np.zeros(d_out, np.float32)
        assert oracle.apply_lora(bl.a, bl.b, bl.rank, d_in, d_out, 1.0, x, got)
        assert np.max(np.abs(got - want)) <= 1e-5 * max(1.0, float(np.max(np.abs(want))))


def test_blend_rejects_what_the_reference_rejects():
    rng = np.random.default_rng(4)
    ok = [layer(rng, 0, "q_proj", 4, 32, 16)]
    with pytest.raises(ValueError):
        blend_lora_layer_data([])
    with pytest.raises(ValueError):
        blend_lora_layer_data([(ok, 1.0, float("nan"))])
    with pytest.raises(ValueError):
        blend_lora_layer_data([([], 1.0, 1.0)])
    with pytest.raises(ValueError):                       # same projection, different shape
        blend_lora_layer_data([(ok, 1.0, 1.0), ([layer(rng, 0, "q_proj", 4, 32, 24)], 1.0, 1.0)])
    bad = layer(rng, 0, "q_proj", 4, 32, 16)
    bad.a = bad.a[:3]                                     # A shorter than rank * d_in
    with pytest.raises(ValueError):
        blend_lora_layer_data([([bad], 1.0, 1.0)])
    big = [layer(rng, 0, "q_proj", MAX_BLEND_RANK_TOTAL // 2 + 1, 4, 4)]
    with pytest.raises(ValueError):                       # summed rank above the cap
        blend_lora_layer_data([(big, 1.0, 1.0), (big, 1.0, 1.0)])
