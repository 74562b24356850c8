"""quantize_index.json reader: both writer flavours, bounded and fail-closed
(crates/inference/src/quant/q4_manifest.rs:154-279 and its tests)."""
import os

import pytest

from lattice_b200 import manifest as mf


def write(tmp_path, text):
    (tmp_path / mf.MANIFEST_NAME).write_text(text)


def test_absent_manifest_is_none(tmp_path):
    assert mf.load_manifest(str(tmp_path)) is None


def test_bare_array_is_the_quantize_q4_flavor(tmp_path):
    write(tmp_path, '[{"name":"foo","file":"foo.q4","quantized":true,"shape":[2,2],"numel":4}]')
    m = mf.load_manifest(str(tmp_path))
    assert m.flavor == "quantize_q4" and m.quarot_seed is None
    assert len(m.tensors) == 1 and m.tensors[0].name == "foo" and m.tensors[0].shape == [2, 2]


def test_object_form_is_the_quarot_flavor_with_seed(tmp_path):
    write(tmp_path, '{"quarot_seed":42,"tensors":[{"name":"foo","file":"foo.q4","quantized":true,"shape":[2],"numel":2}]}')
    m = mf.load_manifest(str(tmp_path))
    assert m.flavor == "quarot" and m.quarot_seed == 42 and len(m.tensors) == 1
    write(tmp_path, '{"quarot_seed":null,"tensors":[]}')
    assert mf.load_manifest(str(tmp_path)).quarot_seed is None
    write(tmp_path, '{"tensors":[{"name":"a","file":"a.q4"}]}')          # minimal entries are tolerated
    m = mf.load_manifest(str(tmp_path))
    assert m.quarot_seed is None and m.tensors[0].quantized is None and m.tensors[0].shape is None


@pytest.mark.parametrize("text,kind", [
    ("not json", "invalid_json"),
    ("42", "invalid_shape"),
    ('"a string"', "invalid_shape"),
    ('{"quarot_seed":1}', "invalid_shape"),                      # object form needs `tensors`
    ('[{"name":"foo"}]', "invalid_shape"),                        # entry without `file`
    ('{"tensors":[{"file":"foo.q4"}]}', "invalid_shape"),         # entry without `name`
    ('{"quarot_seed":-1,"tensors":[]}', "invalid_shape"),
    ('{"quarot_seed":"7","tensors":[]}', "invalid_shape"),
    ('[{"name":"a","file":"a.q4","shape":"2x2"}]', "invalid_shape"),
])
def test_malformed_manifests_are_refused_with_their_reason(tmp_path, text, kind):
    write(tmp_path, text)
    with pytest.raises(mf.ManifestError) as e:
        mf.load_manifest(str(tmp_path))
    assert e.value.kind == kind


def test_dangling_symlink_and_oversized_file_fail_closed(tmp_path):
    link = tmp_path / mf.MANIFEST_NAME
    os.symlink(str(tmp_path / "missing-target.json"), str(link))
    with pytest.raises(mf.ManifestError) as e:
        mf.load_manifest(str(tmp_path))
    assert e.value.kind == "unreadable"           # present but broken is not "absent"
    link.unlink()
    with open(link, "wb") as f:
        f.truncate(mf.MAX_QUANTIZE_INDEX_LEN + 1)   # sparse: nothing is written
    with pytest.raises(mf.ManifestError) as e:
        mf.load_manifest(str(tmp_path))
    assert e.value.kind == "too_large"
    with open(link, "wb") as f:
        f.truncate(mf.MAX_QUANTIZE_INDEX_LEN)       # exactly at the cap is read (and is not JSON)
    with pytest.raises(mf.ManifestError) as e:
        mf.load_manifest(str(tmp_path))
    assert e.value.kind == "invalid_json"
