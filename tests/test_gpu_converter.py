"""GPU parity of the converter side: the quantizer entry points for bf16 / f64 / per-row input, rotation
absorption into weights (f32 and f64, both sides), the `.q4` writer, and the reference's composed
QuaRot gate with the device doing absorb + quantize + dequantize.  Everything here is bit-exact."""
import json
import os

import numpy as np
import pytest

import oracle
from lattice_b200 import _lib, synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def be():
    from lattice_b200 import CudaQ4Backend
    b = CudaQ4Backend(0)
    yield b
    b.check_device_status()
    b.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _edge_values(rng, n):
    w = (rng.standard_normal(n) * 0.02).astype(np.float64)
    w[32 * 5:32 * 6] = 0.0                                      # zero-range block
    w[32 * 9:32 * 10] = 1e-38                                   # range underflows f16
    w[32 * 11] = 7.0; w[32 * 11 + 1] = -7.0
    w[32 * 13:32 * 14] = 0.5 * np.arange(-16, 16)               # exact .5 ties
    return w


def test_quantize_bf16_bit_exact(be):
    rng = np.random.default_rng(21)
    w = _edge_values(rng, 32 * 3000 + 5).astype(np.float32)
    bits = (w.view(np.uint32) >> 16).astype(np.uint16)          # any bf16 pattern of finite values
    got = be.quantize_tensor(dev(bits).view(torch.bfloat16)).cpu().numpy()
    assert got.tobytes() == oracle.quantize_bf16_to_q4(bits).tobytes()
    bad = bits.copy(); bad[77] = 0x7F80                         # +inf
    with pytest.raises(_lib.Lq4Error):
        be.quantize_tensor(dev(bad).view(torch.bfloat16))


@pytest.mark.parametrize("symmetric", [True, False])
def test_quantize_f64_bit_exact_with_the_cast_inside(be, symmetric):
    rng = np.random.default_rng(22)
    w = _edge_values(rng, 32 * 3000 + 9)
    w[200:300] += rng.standard_normal(100) * 1e-12              # not f32-representable: the cast must round
    w[40] = 0.1 + 2.0 ** -30
    got = be.quantize_tensor(dev(w), symmetric=symmetric).cpu().numpy()
    assert got.tobytes() == oracle.quantize_f64_to_q4(w, symmetric=symmetric).tobytes()
    bad = w.copy(); bad[3] = 1e300                              # finite in f64, infinite after `as f32`
    with pytest.raises(_lib.Lq4Error):
        be.quantize_tensor(dev(bad), symmetric=symmetric)
    bad = w.copy(); bad[3] = np.nan
    with pytest.raises(_lib.Lq4Error):
        be.quantize_tensor(dev(bad), symmetric=symmetric)


@pytest.mark.parametrize("rows,cols", [(7, 33), (5, 100), (3, 64), (1, 31), (64, 4097)])
def test_quantize_per_row_when_cols_is_not_a_multiple_of_32(be, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    got = be.quantize_tensor(dev(w), per_row=True).cpu().numpy()
    want = oracle.quantize_tensor_q4_0(w, rows, cols)
    assert got.tobytes() == want.tobytes()
    # the flat entry point on the same data crosses row ends instead
    flat = be.quantize_tensor(dev(w)).cpu().numpy()
    assert flat.tobytes() == oracle.quantize_f32_to_q4(w.reshape(-1)).tobytes()
    if cols % 32 and rows > 1:
        assert flat.size != got.size or flat.tobytes() != got.tobytes()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("rows,cols", [(5, 32), (11, 4096), (3, 16384), (128, 2), (6, 1)])
def test_absorb_input_rotation_bit_exact(be, dtype, rows, cols):
    signs = oracle.signs_from_seed(synth.QUAROT_DEFAULT_SEED ^ cols, cols)
    rng = np.random.default_rng(cols + rows)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(dtype)
    got = be.absorb_rotation(dev(w), dev(signs), "input").cpu().numpy()
    want = oracle.absorb_rotation(w, rows, cols, signs, "input")
    assert got.dtype == want.dtype and got.tobytes() == want.tobytes()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("rows,cols", [(32, 5), (4096, 9), (1024, 130), (2, 7), (1, 3), (16, 1)])
def test_absorb_output_rotation_bit_exact(be, dtype, rows, cols):
    signs = oracle.signs_from_seed(synth.QUAROT_DEFAULT_SEED ^ rows, rows)
    rng = np.random.default_rng(cols * 7 + rows)
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(dtype)
    got = be.absorb_rotation(dev(w), dev(signs), "output").cpu().numpy()
    want = oracle.absorb_rotation(w, rows, cols, signs, "output")
    assert got.tobytes() == want.tobytes()


def test_absorb_refuses_what_the_reference_refuses(be):
    signs = dev(oracle.signs_from_seed(1, 64))
    w = torch.zeros((8, 32), device="cuda")
    with pytest.raises(_lib.Lq4Error) as e:
        be.absorb_rotation(w, signs, "input")                    # rotation.dim()=64 but weight.cols=32
    assert e.value.status == _lib.ERR_ROT
    with pytest.raises(_lib.Lq4Error) as e:
        be.absorb_rotation(w, signs, "output")
    assert e.value.status == _lib.ERR_ROT


def test_q4_writer_reproduces_the_golden_files_and_round_trips(be, golden_dir, tmp_path):
    from lattice_b200 import Q4WeightBuf
    fxs = json.load(open(os.path.join(golden_dir, "reference_q4_fixtures.json")))
    for name in ("gate_proj", "k_proj"):
        fx = fxs[name]
        n = int(np.prod(fx["shape"]))
        vals = np.array([float(((i * 37 + fx["seed"] * 13) % 200) - 100) / 4.0 for i in range(n)], np.float32)
        bits = (vals.view(np.uint32) >> 16).astype(np.uint16)     # the generator truncates to bf16
        payload = be.quantize_tensor(dev(bits).view(torch.bfloat16))
        path = tmp_path / f"{name}.q4"
        be.save_q4_file(path, payload, fx["shape"])
        assert path.read_bytes() == bytes.fromhex(fx["hex"])       # the reference's file, byte for byte
    # a device-quantized 2-D tensor written here loads through the library's own loader
    w = synth.weights(1, 64, 256)
    payload = be.quantize(dev(w).reshape(-1))
    path = tmp_path / "w.q4"
    be.save_q4_file(path, payload, [64, 256])
    assert path.read_bytes() == oracle.q4_file_bytes([64, 256], 64 * 256, payload.cpu().numpy())
    qw = Q4WeightBuf.from_q4_file(str(path), (64, 256))
    got = be.dequantize(torch.from_numpy(np.frombuffer(path.read_bytes()[36:], np.uint8).copy()).cuda(), 64 * 8)
    assert np.array_equal(got.cpu().numpy(), oracle.dequantize_q4_to_f32(payload.cpu().numpy()))
    assert (qw.n, qw.k) == (64, 256)
    qw.free()
    import ctypes as C
    shp = (C.c_uint64 * 2)(64, 256)                               # shape product != original_len: refused
    assert _lib.lib().lq4_q4_file_write(str(tmp_path / "bad.q4").encode(), shp, 2, 64 * 256 - 1, payload.data_ptr(), None) == _lib.ERR_SHAPE


def _lcg_f64(n, seed):
    out, state = [], seed
    for _ in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        out.append((state >> 32) / 4294967295.0 * 2.0 - 1.0)
    return np.array(out, np.float64)


def test_composed_quarot_gate_with_the_device_pipeline(be):
    """The reference's composed gate (crates/inference/src/weights/q4_weights.rs:2487-2672): rotate in f64,
    symmetric Q4, dequantize, matvec against an independent restatement, bound 1e-5, same seeds and shapes -
    here absorb + quantize + dequantize all run on the device, and must also equal the oracle bit for bit."""
    H, QR, OR = 32, 2, 32
    q = _lcg_f64(QR * H, 0x1111111111111111).reshape(QR, H)
    o = _lcg_f64(OR * H, 0x2222222222222222).reshape(OR, H)
    xq = _lcg_f64(H, 0x3333333333333333)
    xo = _lcg_f64(H, 0x4444444444444444)
    signs = oracle.signs_from_seed(0x32000001, H)
    sd = be.rot_signs(0x32000001, H)
    assert np.array_equal(sd.cpu().numpy(), signs)

    def device_pipeline(w, side):
        wr = be.absorb_rotation(dev(w), sd, side)
        payload = be.quantize_tensor(wr, symmetric=True)
        return payload, be.dequantize(payload, payload.numel() // 20).cpu().numpy().astype(np.float64).reshape(w.shape)

    pq, q_deq = device_pipeline(q, "input")
    po, o_deq = device_pipeline(o, "output")
    assert pq.cpu().numpy().tobytes() == oracle.quantize_f64_to_q4(oracle.absorb_rotation(q, QR, H, signs, "input")).tobytes()
    assert po.cpu().numpy().tobytes() == oracle.quantize_f64_to_q4(oracle.absorb_rotation(o, OR, H, signs, "output")).tobytes()

    def ref_dequant(data):      # numpy restatement, independent of the C code and of the device
        out = []
        for chunk in data.reshape(-1, 32):
            f = chunk.astype(np.float32)
            amax = np.float32(np.max(np.abs(f)))
            scale = np.float32(1.0) if amax == 0 else amax / np.float32(7.0)
            bias = np.float32(-8.0) * scale
            sdq, bdq = np.float32(np.float16(scale)), np.float32(np.float16(bias))
            t = f * (np.float32(1.0) / scale)
            r = np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))
            nib = np.clip(r + np.float32(8.0), 0, 15).astype(np.uint8).astype(np.float32)
            out.append((nib * sdq + bdq).astype(np.float64))
        return np.concatenate(out)

    q_ref = np.stack([oracle.rh_apply(signs, r) for r in q])
    o_ref = np.stack([oracle.rh_apply(signs, c) for c in o.T]).T
    assert np.max(np.abs(q_deq @ xq - ref_dequant(q_ref).reshape(QR, H) @ xq)) <= 1e-5
    assert np.max(np.abs(o_deq @ xo - ref_dequant(o_ref).reshape(OR, H) @ xo)) <= 1e-5


def test_config5_weights_from_the_device_converter(be):
    """The QuaRot layer's (K=4096) weight preparation at its real row length on a slice of rows: f32 weights -> f64 ->
    absorb_input_rotation_f64 (default converter seed) -> symmetric Q4, device against oracle, byte for byte."""
    n, k = 344, 4096
    w = synth.weights(5, n, k).astype(np.float64)
    signs = oracle.signs_from_seed(synth.QUAROT_DEFAULT_SEED, k)
    sd = be.rot_signs(synth.QUAROT_DEFAULT_SEED, k)
    got = be.quantize_tensor(be.absorb_rotation(dev(w), sd, "input"), symmetric=True).cpu().numpy()
    want = oracle.quantize_f64_to_q4(oracle.absorb_rotation(w, n, k, signs, "input"), symmetric=True)
    assert got.tobytes() == want.tobytes()
