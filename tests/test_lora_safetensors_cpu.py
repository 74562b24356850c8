"""PEFT / MLX safetensors ingestion: the reference's key grammar, conversions and refusals
(crates/tune/src/lora/safetensors.rs:36-375,449-520).  Files are written with the `safetensors` Python
package, an independent writer of the container format."""
import json
import struct

import numpy as np
import pytest

from lattice_b200 import lora_safetensors as ls

st_numpy = pytest.importorskip("safetensors.numpy")


def _factors(rng, rank=4, d_in=32, d_out=24):
    return rng.standard_normal((rank, d_in)).astype(np.float32), rng.standard_normal((d_out, rank)).astype(np.float32)


def test_key_grammar():
    k = ls.parse_peft_key("base_model.model.model.layers.3.self_attn.q_proj.lora_A.weight")
    assert (k.layer_idx, k.module, k.matrix, k.transposed) == (3, "q_proj", "A", False)
    k = ls.parse_peft_key("model.layers.17.mlp.gate_proj.lora_b")
    assert (k.layer_idx, k.module, k.matrix, k.transposed) == (17, "gate_proj", "B", True)
    k = ls.parse_peft_key("x.layers.0.linear_attn.in_proj_qkv.lora_B")
    assert (k.layer_idx, k.module, k.matrix) == (0, "in_proj_qkv", "B")
    for bad in ("model.layers.3.self_attn.q_proj.weight", "model.embed.lora_A.weight", "model.layers.x.q_proj.lora_A",
                "model.layers.3.lora_A", "lora_A", "model.layers..q_proj.lora_A"):
        assert ls.parse_peft_key(bad) is None, bad


def test_peft_file_round_trip(tmp_path):
    rng = np.random.default_rng(1)
    tensors, expect = {}, {}
    for layer, module, blk in ((0, "q_proj", "self_attn"), (0, "down_proj", "mlp"), (5, "v_proj", "self_attn")):
        a, b = _factors(rng, 4, 32 + layer, 24)
        tensors[f"base_model.model.model.layers.{layer}.{blk}.{module}.lora_A.weight"] = a
        tensors[f"base_model.model.model.layers.{layer}.{blk}.{module}.lora_B.weight"] = b
        expect[(layer, module)] = (a, b)
    tensors["base_model.model.model.embed_tokens.weight"] = np.zeros((3, 3), np.float32)      # ignored
    path = tmp_path / "adapter_model.safetensors"
    st_numpy.save_file(tensors, str(path), metadata={"alpha": "8", "adapter_id": "demo"})
    ad = ls.load_peft_safetensors(str(path))
    assert ad.rank == 4 and ad.alpha == 8.0 and ad.scale == 2.0
    assert ad.target_modules == ["down_proj", "q_proj", "v_proj"] and ad.metadata["adapter_id"] == "demo"
    assert [(l.layer_idx, l.module) for l in ad.layers] == sorted(expect)
    for l in ad.layers:
        a, b = expect[(l.layer_idx, l.module)]
        assert np.array_equal(l.a, a) and np.array_equal(l.b, b)
        assert (l.rank, l.d_in, l.d_out) == (4, a.shape[1], 24)


def test_mlx_layout_is_transposed_and_alpha_defaults_to_rank(tmp_path):
    rng = np.random.default_rng(2)
    a, b = _factors(rng, 8, 16, 12)
    path = tmp_path / "adapters.safetensors"
    st_numpy.save_file({"model.layers.2.self_attn.o_proj.lora_a": np.ascontiguousarray(a.T),
                        "model.layers.2.self_attn.o_proj.lora_b": np.ascontiguousarray(b.T)}, str(path))
    ad = ls.load_peft_safetensors(str(path))
    assert ad.rank == 8 and ad.alpha == 8.0 and ad.scale == 1.0
    assert np.array_equal(ad.layers[0].a, a) and np.array_equal(ad.layers[0].b, b)


def _raw_file(entries, metadata=None):
    """Hand-written container: entries = [(name, dtype, shape, bytes)]."""
    header, blob = {}, b""
    for name, dtype, shape, raw in entries:
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    if metadata is not None:
        header["__metadata__"] = metadata
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + blob


def test_f16_and_bf16_tensors_convert_exactly():
    a = np.array([[1.0, -2.5, 0.15625, 6.1e-5]], np.float32)            # exact in f16
    b = np.array([[3.0], [-0.5]], np.float32)
    a16 = a.astype(np.float16).tobytes()
    bbf = (b.view(np.uint32) >> 16).astype(np.uint16).tobytes()
    data = _raw_file([("m.layers.0.mlp.up_proj.lora_A.weight", "F16", [1, 4], a16),
                      ("m.layers.0.mlp.up_proj.lora_B.weight", "BF16", [2, 1], bbf)])
    ad = ls.load_peft_safetensors_bytes(data)
    assert np.array_equal(ad.layers[0].a, a.astype(np.float16).astype(np.float32)) and np.array_equal(ad.layers[0].b, b)


def test_refusals():
    f = lambda arr: arr.astype("<f4").tobytes()
    a, b = np.ones((2, 4), np.float32), np.ones((3, 2), np.float32)
    A, B = "m.layers.0.mlp.up_proj.lora_A.weight", "m.layers.0.mlp.up_proj.lora_B.weight"
    ok = [(A, "F32", [2, 4], f(a)), (B, "F32", [3, 2], f(b))]
    ls.load_peft_safetensors_bytes(_raw_file(ok))
    cases = {
        "no factors": [("m.embed.weight", "F32", [1], f(np.ones(1)))],
        "A without B": ok[:1],
        "B without A": ok[1:],
        "not 2-D": [(A, "F32", [8], f(np.ones(8))), ok[1]],
        "rank mismatch in a pair": [ok[0], (B, "F32", [2, 3], f(np.ones((2, 3))))],
        "two ranks in one file": ok + [("m.layers.1.mlp.up_proj.lora_A", "F32", [3, 4], f(np.ones((3, 4)))),
                                      ("m.layers.1.mlp.up_proj.lora_B", "F32", [3, 3], f(np.ones((3, 3))))],
        "non-finite": [(A, "F32", [2, 4], f(np.array([[1, np.nan, 1, 1], [1, 1, 1, 1]]))), ok[1]],
        "integer dtype": [(A, "I32", [2, 4], np.ones(8, "<i4").tobytes()), ok[1]],
    }
    for why, entries in cases.items():
        with pytest.raises(ls.LoraFileError):
            ls.load_peft_safetensors_bytes(_raw_file(entries))
        assert why
    for meta in ({"alpha": "abc"}, {"alpha": "inf"}, {"alpha": "nan"}, {"alpha": " 4"}, {"alpha": "1_6"}):
        with pytest.raises(ls.LoraFileError):
            ls.load_peft_safetensors_bytes(_raw_file(ok, meta))
    assert ls.load_peft_safetensors_bytes(_raw_file(ok, {"alpha": "1e1"})).alpha == 10.0


def test_container_checks_and_size_bound(tmp_path):
    good = _raw_file([("m.layers.0.q_proj.lora_A", "F32", [1, 2], np.ones(2, "<f4").tobytes()),
                      ("m.layers.0.q_proj.lora_B", "F32", [2, 1], np.ones(2, "<f4").tobytes())])
    for bad in (b"", good[:7], struct.pack("<Q", 10 ** 9) + good[8:], struct.pack("<Q", len(good)) + good[8:],
                good[:-1], good + b"\0", struct.pack("<Q", 2) + b"[]"):
        with pytest.raises(ls.LoraFileError):
            ls.load_peft_safetensors_bytes(bad)
    # a shape whose byte size disagrees with its offsets
    h = {"m.layers.0.q_proj.lora_A": {"dtype": "F32", "shape": [1, 3], "data_offsets": [0, 8]}}
    hb = json.dumps(h).encode()
    with pytest.raises(ls.LoraFileError):
        ls.load_peft_safetensors_bytes(struct.pack("<Q", len(hb)) + hb + b"\0" * 8)
    path = tmp_path / "a.safetensors"
    path.write_bytes(good)
    assert ls.load_peft_safetensors(str(path)).rank == 1
    with pytest.raises(ls.LoraFileError):
        ls.read_lora_file_bounded(str(path), max_bytes=len(good) - 1)
    with pytest.raises(ls.LoraFileError):
        ls.read_lora_file_bounded(str(tmp_path / "missing.safetensors"))


def test_key_known_answers_of_the_reference_tests():
    # crates/tune/src/lora/safetensors.rs:623-720
    kat = {
        "base_model.model.model.layers.5.self_attn.q_proj.lora_A.weight": (5, "q_proj", "A", False),
        "base_model.model.model.layers.12.mlp.gate_proj.lora_B.weight": (12, "gate_proj", "B", False),
        "model.layers.0.self_attn.v_proj.lora_A.weight": (0, "v_proj", "A", False),
        "base_model.model.model.layers.3.mlp.up_proj.lora_B": (3, "up_proj", "B", False),
        "model.layers.3.self_attn.q_proj.lora_a": (3, "q_proj", "A", True),
        "model.layers.7.mlp.down_proj.lora_b": (7, "down_proj", "B", True),
    }
    for key, (layer, module, matrix, mlx) in kat.items():
        k = ls.parse_peft_key(key)
        assert (k.layer_idx, k.module, k.matrix, k.transposed) == (layer, module, matrix, mlx), key
    for key in ("model.layers.0.self_attn.q_proj.weight", "some_random_tensor", ""):
        assert ls.parse_peft_key(key) is None
    for block, module in (("self_attn", "q_proj"), ("self_attn", "k_proj"), ("self_attn", "v_proj"), ("self_attn", "o_proj"),
                          ("mlp", "gate_proj"), ("mlp", "up_proj"), ("mlp", "down_proj")):
        k = ls.parse_peft_key(f"base_model.model.model.layers.7.{block}.{module}.lora_A.weight")
        assert (k.layer_idx, k.module) == (7, module)


def test_export_round_trips_and_is_readable_by_an_independent_reader(tmp_path):
    from lattice_b200 import LoraLayerData
    rng = np.random.default_rng(5)
    layers = []
    for layer, module in ((0, "q_proj"), (0, "down_proj"), (3, "in_proj_qkv")):
        a, b = _factors(rng, 4, 16, 8)
        layers.append(LoraLayerData(layer, module, a, b, 4, 16, 8))
    path = tmp_path / "out.safetensors"
    ls.save_peft_safetensors(str(path), layers, rank=4, alpha=8.0)
    ad = ls.load_peft_safetensors(str(path))
    assert ad.rank == 4 and ad.alpha == 8.0 and ad.metadata["target_modules"] == "down_proj,in_proj_qkv,q_proj"
    got = {(l.layer_idx, l.module): l for l in ad.layers}
    for l in layers:
        assert np.array_equal(got[(l.layer_idx, l.module)].a, l.a) and np.array_equal(got[(l.layer_idx, l.module)].b, l.b)
    other = st_numpy.load_file(str(path))
    assert np.array_equal(other["base_model.model.model.layers.0.mlp.down_proj.lora_A.weight"], layers[1].a)
    assert np.array_equal(other["base_model.model.model.layers.3.self_attn.in_proj_qkv.lora_B.weight"], layers[2].b)
