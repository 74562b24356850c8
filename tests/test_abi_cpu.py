"""No-GPU checks of the C ABI: the library loads, exports every symbol the header declares,
and rejects bad arguments before touching the device."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

import oracle
from lattice_b200 import _lib, build as lq4_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    lq4_build.build()
    return _lib.lib()


def test_header_symbols_all_exported(L):
    hdr = open(os.path.join(ROOT, "include", "lattice_q4.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)          # declarations only, not prose
    declared = set(re.findall(r"\b(lq4_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert getattr(L, name) is not None
    assert L.lq4_abi_version() >= 1


def test_shard_plan(L):
    n0, n1, off = C.c_uint64(), C.c_uint64(), C.c_uint64()
    for n, k in [(17408, 5120), (5120, 17408), (1024, 5120), (11008, 4096), (3584, 1024), (100, 64)]:
        prev = 0
        for world in (1, 2, 4, 8):
            prev = 0
            for r in range(world):
                assert L.lq4_shard_plan(n, k, world, r, C.byref(n0), C.byref(n1), C.byref(off)) == _lib.OK
                assert n0.value == prev and n1.value == n * (r + 1) // world
                assert off.value == n0.value * (k // 32) * 20
                prev = n1.value
            assert prev == n
    assert L.lq4_shard_plan(64, 64, 0, 0, C.byref(n0), C.byref(n1), C.byref(off)) == _lib.ERR_SHAPE
    assert L.lq4_shard_plan(64, 64, 2, 2, C.byref(n0), C.byref(n1), C.byref(off)) == _lib.ERR_SHAPE
    assert L.lq4_shard_plan(64, 48, 2, 0, C.byref(n0), C.byref(n1), C.byref(off)) == _lib.ERR_K
    assert L.lq4_shard_plan(64, 64, 2, 0, None, C.byref(n1), C.byref(off)) == _lib.ERR_NULL


def test_lora_upload_validation_happens_before_any_copy(L):
    a = np.zeros(8, np.float32)
    b = np.zeros(8, np.float32)
    h = C.c_void_p()
    pa, pb = a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p)
    up = L.lq4_lora_upload
    assert up(pa, 8, pb, 8, 0, 4, 4, 1.0, C.byref(h)) == _lib.ERR_LORA           # rank 0
    assert up(pa, 8, pb, 8, 2, 0, 4, 1.0, C.byref(h)) == _lib.ERR_LORA           # zero dim
    assert up(pa, 8, pb, 8, 2, 4, 4, float("nan"), C.byref(h)) == _lib.ERR_LORA  # non-finite scale
    assert up(pa, 7, pb, 8, 2, 4, 4, 1.0, C.byref(h)) == _lib.ERR_LORA           # A length
    assert up(pa, 8, pb, 9, 2, 4, 4, 1.0, C.byref(h)) == _lib.ERR_LORA           # B length
    assert up(pa, 8, pb, 8, 2 ** 33, 4, 4, 1.0, C.byref(h)) == _lib.ERR_OVERFLOW
    assert up(None, 8, pb, 8, 2, 4, 4, 1.0, C.byref(h)) == _lib.ERR_NULL
    assert h.value is None
    assert b"rank" in L.lq4_last_error() or L.lq4_last_error() != b""


def test_weights_upload_rejects_bad_blocks_on_the_host(L):
    w = (np.random.default_rng(0).standard_normal(64 * 4) * 0.02).astype(np.float32)
    p = oracle.quantize_f32_to_q4(w)
    h = C.c_void_p()
    bad = p.copy()
    bad[2 * 20:2 * 20 + 2] = 0                      # scale == 0
    assert L.lq4_weights_upload(bad.ctypes.data_as(C.c_void_p), 4, 64, C.byref(h)) == _lib.ERR_BAD_BLOCK
    bad = p.copy()
    bad[5 * 20 + 2:5 * 20 + 4] = np.frombuffer((0x7E00).to_bytes(2, "little"), np.uint8)   # bias NaN
    assert L.lq4_weights_upload(bad.ctypes.data_as(C.c_void_p), 4, 64, C.byref(h)) == _lib.ERR_BAD_BLOCK
    assert b"block 5" in L.lq4_last_error()
    bad = p.copy()
    bad[20:22] = np.frombuffer((0xBC00).to_bytes(2, "little"), np.uint8)                   # scale -1
    assert L.lq4_weights_upload(bad.ctypes.data_as(C.c_void_p), 4, 64, C.byref(h)) == _lib.ERR_BAD_BLOCK
    assert L.lq4_weights_upload(p.ctypes.data_as(C.c_void_p), 4, 48, C.byref(h)) == _lib.ERR_K
    assert L.lq4_weights_upload(None, 4, 64, C.byref(h)) == _lib.ERR_NULL
    assert h.value is None


def test_q4_file_loader_rejects_malformed_files(L, tmp_path, golden_dir):
    import json
    fx = json.load(open(os.path.join(golden_dir, "reference_q4_fixtures.json")))["k_proj"]
    img = bytes.fromhex(fx["hex"])
    h = C.c_void_p()

    def load(data, shape=None):
        p = tmp_path / "t.q4"
        p.write_bytes(data)
        if shape is None:
            return L.lq4_weights_load_q4_file(str(p).encode(), None, 0, C.byref(h))
        arr = (C.c_uint64 * len(shape))(*shape)
        return L.lq4_weights_load_q4_file(str(p).encode(), arr, len(shape), C.byref(h))

    assert load(b"KHQ5" + img[4:]) == _lib.ERR_FORMAT
    assert load(img[:4] + (1).to_bytes(4, "little") + img[8:]) == _lib.ERR_FORMAT      # legacy v1
    assert load(img[:4] + (3).to_bytes(4, "little") + img[8:]) == _lib.ERR_FORMAT
    assert load(img[:-1]) == _lib.ERR_FORMAT and b"truncated" in L.lq4_last_error()
    assert load(img + b"\0") == _lib.ERR_FORMAT and b"trailing" in L.lq4_last_error()
    assert load(img, (1, 64)) == _lib.ERR_SHAPE
    assert load(img, (32,)) == _lib.ERR_SHAPE
    bad = bytearray(img)
    bad[36:38] = (0).to_bytes(2, "little")                                              # scale == 0
    assert load(bytes(bad)) == _lib.ERR_BAD_BLOCK
    assert L.lq4_weights_load_q4_file(b"/nonexistent/x.q4", None, 0, C.byref(h)) == _lib.ERR_IO
    assert h.value is None


def test_entry_points_reject_null_and_bad_shapes_without_a_device(L):
    assert L.lq4_linear(None, None, None) == _lib.ERR_NULL
    assert L.lq4_ctx_reserve(None, 1, 1, 32, 0) == _lib.ERR_NULL
    assert L.lq4_ctx_check(None, None) == _lib.ERR_NULL
    assert L.lq4_dequant_f32(None, 4, None, None) == _lib.ERR_NULL
    assert L.lq4_dequant_f32(None, 0, None, None) == _lib.OK
    assert L.lq4_quantize_f32(None, 0, 0, None, None, None) == _lib.OK
    assert L.lq4_quantize_f32(None, 32, 0, None, None, None) == _lib.ERR_NULL
    assert L.lq4_status_string(_lib.ERR_K).startswith(b"k must")
    assert L.lq4_ctx_launch_count(None) == 0


def test_group_gather_and_peer_buffer_entry_points_validate_without_a_device(L):
    assert L.lq4_abi_version() >= 2
    assert L.lq4_linear_group(None, None, 0, None) == _lib.ERR_NULL
    args = (_lib.LinearArgs * 2)()
    # a context is needed before anything else is looked at; NULL is refused
    assert L.lq4_linear_group(None, args, 2, None) == _lib.ERR_NULL
    assert L.lq4_gather_wait(None, None, None) == _lib.ERR_NULL
    h = C.c_void_p()
    assert L.lq4_peer_buf_create(0, C.byref(h)) == _lib.ERR_SHAPE and h.value is None
    assert L.lq4_peer_buf_create(16, None) == _lib.ERR_NULL
    buf = (C.c_uint8 * _lib.PEER_HANDLE_BYTES)()
    assert L.lq4_peer_buf_export(None, buf) == _lib.ERR_NULL
    assert L.lq4_peer_buf_open(None, C.byref(h)) == _lib.ERR_NULL
    assert L.lq4_peer_buf_open(buf, None) == _lib.ERR_NULL
    assert L.lq4_peer_buf_close(None) == _lib.OK
    assert L.lq4_peer_buf_base(None) is None and L.lq4_peer_buf_payload(None) is None
    L.lq4_peer_buf_free(None)
    # the argument block carries the two gather descriptors after `path` (ABI version 2)
    names = [f[0] for f in _lib.LinearArgs._fields_]
    assert names[-3:] == ["path", "gather", "wait_gather"]
    assert C.sizeof(_lib.GatherDesc) == 8 + 8 * _lib.MAX_PEERS


def test_topk_entry_points_validate_without_a_device(L):
    out = (C.c_uint64 * 4)()
    logits = (C.c_float * 4)()
    assert L.lq4_logits_topk(None, logits, 4, 2, out, None) == _lib.ERR_NULL
    args = _lib.LinearArgs()
    assert L.lq4_lm_head_topk(None, C.byref(args), 2, out, None) == _lib.ERR_NULL
    assert _lib.MAX_TOP_K == 256


def test_block_rotation_entry_points_refuse_what_the_reference_constructor_refuses(L):
    # BlockHadamard::new, quant/quarot/hadamard.rs:358-400: checked before anything touches a device
    buf = (C.c_float * 4)()
    for n, b in ((0, 64), ((1 << 24) + 64, 64), (100, 64), (96, 48), (64, 0), (1 << 24, 1)):
        assert L.lq4_block_rot_signs_from_seed(1, n, b, buf, None) == _lib.ERR_ROT, (n, b)
    assert L.lq4_block_rot_signs_from_seed(1, 128, 64, None, None) == _lib.ERR_NULL
    rot = _lib.RotDesc(C.cast(buf, C.c_void_p).value, 48)
    assert L.lq4_block_hadamard_rows(buf, buf, 1, 96, C.byref(rot), None) == _lib.ERR_ROT
    assert L.lq4_block_hadamard_rows(None, buf, 1, 96, C.byref(rot), None) == _lib.ERR_NULL


def test_mlp_block_validates_without_a_device(L):
    assert L.lq4_mlp_block(None, None, None) == _lib.ERR_NULL
    args = _lib.MlpArgs()
    assert L.lq4_mlp_block(None, C.byref(args), None) == _lib.ERR_NULL


def test_converter_entry_points_validate_without_a_device(L, tmp_path):
    buf = (C.c_float * 64)()
    ptr = C.cast(buf, C.c_void_p).value
    # empty tensors are no-ops; NULL and unknown dtypes are refused before any launch
    assert L.lq4_quantize_tensor(None, _lib.DTYPE_F32, 0, 32, 0, 0, None, None, None) == _lib.OK
    assert L.lq4_quantize_tensor(None, _lib.DTYPE_F32, 2, 32, 0, 0, None, None, None) == _lib.ERR_NULL
    assert L.lq4_quantize_tensor(ptr, 7, 2, 32, 0, 0, ptr, None, None) == _lib.ERR_DTYPE
    assert L.lq4_quantize_tensor(ptr, _lib.DTYPE_F32, 1 << 40, 1 << 40, 0, 0, ptr, None, None) == _lib.ERR_OVERFLOW
    # rotation absorption: the reference's shape check (rotation.rs:55-80) comes first
    rot = _lib.RotDesc(ptr, 64)
    assert L.lq4_absorb_input_rotation(ptr, _lib.DTYPE_F64, 4, 32, C.byref(rot), None) == _lib.ERR_ROT
    assert b"rotation.dim()=64 but weight.cols=32" in L.lq4_last_error()
    assert L.lq4_absorb_output_rotation(ptr, _lib.DTYPE_F32, 32, 4, C.byref(rot), None) == _lib.ERR_ROT
    assert b"weight.rows=32" in L.lq4_last_error()
    bad = _lib.RotDesc(ptr, 48)
    assert L.lq4_absorb_input_rotation(ptr, _lib.DTYPE_F32, 4, 48, C.byref(bad), None) == _lib.ERR_ROT
    assert L.lq4_absorb_input_rotation(ptr, _lib.DTYPE_BF16, 4, 64, C.byref(rot), None) == _lib.ERR_DTYPE
    assert L.lq4_absorb_input_rotation(ptr, _lib.DTYPE_F32, 4, 64, None, None) == _lib.ERR_NULL
    # the writer: header rules without a device (an empty tensor has no payload to fetch)
    shp = (C.c_uint64 * 2)(0, 32)
    path = tmp_path / "empty.q4"
    assert L.lq4_q4_file_write(str(path).encode(), shp, 2, 0, None, None) == _lib.OK
    assert path.read_bytes() == oracle.q4_file_bytes([0, 32], 0, np.zeros(0, np.uint8))
    shp = (C.c_uint64 * 2)(4, 32)
    assert L.lq4_q4_file_write(str(path).encode(), shp, 2, 127, None, None) == _lib.ERR_SHAPE
    assert L.lq4_q4_file_write(str(path).encode(), shp, 0, 128, None, None) == _lib.ERR_SHAPE
    assert L.lq4_q4_file_write(None, shp, 2, 128, None, None) == _lib.ERR_NULL
    assert L.lq4_q4_file_write(str(path).encode(), shp, 2, 128, None, None) == _lib.ERR_NULL


def test_kernel_attribute_bookkeeping_is_per_device(tmp_path):
    """The shared-memory opt-in of a kernel is a per-device attribute: the bookkeeping that decides whether
    to repeat it must answer per device, not per process (a process may drive several GPUs)."""
    import subprocess
    src = tmp_path / "once.cc"
    src.write_text('''
#include "lq4_once.h"
#include <cstdio>
#include <initializer_list>
int main() {
    static lq4::DeviceOnce once;
    int bad = 0;
    for (int d : {0, 1, 63, 64, 255}) bad += !once.needs(d);
    once.mark(0);
    bad += once.needs(0);              // device 0 is done ...
    bad += !once.needs(1);             // ... device 1 is not
    once.mark(64); once.mark(255);
    bad += once.needs(64) + once.needs(255) + !once.needs(63) + !once.needs(65);
    bad += !once.needs(-1) + !once.needs(256);      // outside the table: always repeat (harmless)
    once.mark(256); once.mark(-1);
    once.reset();
    bad += !once.needs(0) + !once.needs(64);
    std::printf("%d\\n", bad);
    return bad;
}
''')
    exe = tmp_path / "once"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "lattice_b200", "csrc"), str(src), "-o", str(exe)],
                   check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0 and res.stdout.strip() == "0"


def test_step_shares_cover_every_work_unit_once(tmp_path):
    """The cut of a projection's work units into CTA shares (lq4_step_share.h): contiguous, monotone, complete,
    and the owner function agrees with the cuts - for every charge, also where shares come out empty."""
    src = tmp_path / "share.cpp"
    src.write_text('''
#include "lq4_step_share.h"
#include <cstdio>
#include <initializer_list>
using namespace lq4;
int main() {
    long bad = 0, checks = 0;
    for (uint32_t tiles : {1u, 2u, 3u, 8u, 40u, 136u})
        for (uint32_t kg : {1u, 2u, 5u, 40u, 136u})
            for (uint32_t charge : {0u, 1u, 3u, 5u, 9u})
                for (uint32_t count = 1; count <= 148 && count <= tiles * kg; count += (count < 12 ? 1 : 7)) {
                    const uint64_t total = (uint64_t)tiles * kg;
                    bad += step_share_begin(0, tiles, kg, charge, count) != 0;
                    bad += step_share_begin(count, tiles, kg, charge, count) != total;
                    for (uint32_t c = 0; c < count; ++c)
                        bad += step_share_begin(c, tiles, kg, charge, count) > step_share_begin(c + 1, tiles, kg, charge, count);
                    for (uint64_t p = 0; p < total; ++p, ++checks) {
                        const uint32_t o = step_share_owner(p, tiles, kg, charge, count);
                        bad += !(o < count && step_share_begin(o, tiles, kg, charge, count) <= p &&
                                 p < step_share_begin(o + 1, tiles, kg, charge, count));
                    }
                    if (step_share_fits32(tiles, kg, charge, count))
                        for (uint32_t c = 0; c <= count; ++c)
                            bad += step_share_begin_t<uint32_t>(c, tiles, kg, charge, count) != step_share_begin(c, tiles, kg, charge, count);
                    for (uint32_t tile = 0; tile < tiles; ++tile) {      // the walk from a tile's first CTA to its last
                        const uint64_t first = (uint64_t)tile * kg, last = first + kg - 1;
                        const uint32_t f = step_share_owner(first, tiles, kg, charge, count);
                        bad += step_share_last_t<uint64_t>(f, last, tiles, kg, charge, count) != step_share_owner(last, tiles, kg, charge, count);
                        bad += step_share_last_t<uint32_t>(f, (uint32_t)last, tiles, kg, charge, count) != step_share_owner(last, tiles, kg, charge, count);
                    }
                    if (charge == 0)      // no charge: the even cut of the other decode kernels
                        for (uint32_t c = 0; c <= count; ++c) bad += step_share_begin(c, tiles, kg, 0, count) != c * total / count;
                }
    // a CTA that starts a tile gets `charge` units less than one that does not (17408 -> 5120: 40 tiles x 136)
    uint64_t with_start = 0, without = 0;
    for (uint32_t c = 0; c < 61; ++c) {
        const uint64_t r0 = step_share_begin(c, 40, 136, 5, 61), r1 = step_share_begin(c + 1, 40, 136, 5, 61);
        const bool starts = (r0 % 136 == 0) || (r0 / 136 != (r1 - 1) / 136);
        (starts ? with_start : without) = r1 - r0;
    }
    bad += !(without > with_start && without - with_start <= 6);
    std::printf("%ld %ld\\n", bad, checks);
    return bad != 0;
}
''')
    exe = tmp_path / "share"
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "lattice_b200", "csrc"), str(src), "-o", str(exe)],
                   check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0 and res.stdout.split()[0] == "0", res.stdout


def test_step_sharded_and_option_entry_points_validate_without_a_device(L):
    assert L.lq4_decode_step(None, None, 0, None, None) == _lib.ERR_NULL
    assert L.lq4_decode_step_host(None, None, 0, None, None) == _lib.ERR_NULL
    assert L.lq4_linear_sharded(None, None, None, None) == _lib.ERR_NULL
    assert L.lq4_ctx_set_option(None, _lib.OPT_PDL, 0) == _lib.ERR_NULL
    assert L.lq4_noalloc_check is not None
    h = C.c_void_p()
    assert L.lq4_step_buf_create(0, C.byref(h)) == _lib.ERR_SHAPE and h.value is None
    assert L.lq4_step_buf_create(1 << 31, C.byref(h)) == _lib.ERR_OVERFLOW
    assert L.lq4_step_buf_create(16, None) == _lib.ERR_NULL
    buf = (C.c_float * 8)()
    ptr = C.cast(buf, C.c_void_p).value
    assert L.lq4_place_slices(None, ptr, 0, 1, 8, 2, None) == _lib.ERR_NULL
    assert L.lq4_place_slices(ptr, ptr, 4, 1, 8, 2, None) == _lib.ERR_SHAPE       # row pitch below n_total
    assert L.lq4_place_slices(ptr, ptr, 0, 1, 8, 0, None) == _lib.ERR_SHAPE       # world 0
    assert L.lq4_place_slices(ptr, ptr, 0, 0, 8, 2, None) == _lib.OK              # nothing to place
    assert L.lq4_nccl_comm_create(None, 2, 0, C.byref(h)) == _lib.ERR_NULL
    ident = (C.c_uint8 * _lib.NCCL_ID_BYTES)()
    assert L.lq4_nccl_comm_create(ident, 2, 2, C.byref(h)) == _lib.ERR_SHAPE      # rank >= world
    L.lq4_nccl_comm_destroy(None)
    # argument blocks of the step call
    assert C.sizeof(_lib.StepGroup) == 16 and C.sizeof(_lib.StepRange) == 16 and C.sizeof(_lib.ShardDesc) == 40
