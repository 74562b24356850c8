"""GPU parity: every result of the CUDA library, called through its C ABI, against the CPU oracle.

Bit-exact for bytes and dequantized weights; |y - y_ref| <= 1e-3 * (|y_ref| + rms(y_ref)) for outputs.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from lattice_b200 import _lib, synth
from tests._cases import make_case, tol_ratio

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def be():
    from lattice_b200 import CudaQ4Backend
    b = CudaQ4Backend(0)
    yield b
    b.check_device_status()
    b.close()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def run_case(be, case, path=_lib.PATH_AUTO, bf16=False, repeat=1):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
    x = dev(case["x"]).to(torch.bfloat16) if bf16 else dev(case["x"])
    keep = []
    lora = None
    if case["lora"] is not None:
        a, b, s = case["lora"]
        ad, bd = dev(a), dev(b)
        keep += [ad, bd]
        lora = LoraDesc(ad.data_ptr(), bd.data_ptr(), case["rank"], s)
    rot = None
    if case["signs"] is not None:
        sd = dev(case["signs"])
        keep.append(sd)
        rot = be.rot_desc(sd)
    ys = []
    for _ in range(repeat):
        y = torch.full((case["m"], case["n"]), float("nan"), dtype=torch.float32, device="cuda")
        be.dispatch_gemm_q4(x, 0, qw, y, 0, case["m"], case["n"], case["k"], lora=lora, rot=rot, path=path)
        ys.append(y.cpu().numpy())
    be.check_device_status()
    qw.free()
    return ys if repeat > 1 else ys[0]


# ---------------------------------------------------------------- bytes and integers
def test_dequant_bit_exact(be):
    w = synth.weights(1, 3584, 1024)
    p = oracle.quantize_f32_to_q4(w)
    got = be.dequantize(dev(p), p.size // 20).cpu().numpy()
    want = oracle.dequantize_q4_to_f32(p)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # arbitrary nibbles with edge metadata: subnormal scale, negative bias, largest finite values
    rng = np.random.default_rng(7)
    raw = rng.integers(0, 256, size=(4096, 20), dtype=np.uint8)
    scales = np.array([0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x2E66], np.uint16)
    biases = np.array([0x0000, 0x8000, 0xFBFF, 0x7BFF, 0x8001, 0xB800], np.uint16)
    meta = np.stack([scales[rng.integers(0, 6, 4096)], biases[rng.integers(0, 6, 4096)]], 1)
    raw[:, :4] = meta.view(np.uint8).reshape(4096, 4)
    got = be.dequantize(dev(raw.reshape(-1)), 4096).cpu().numpy()
    want = oracle.dequantize_q4_to_f32(raw.reshape(-1))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("symmetric", [False, True])
def test_quantize_bit_exact(be, symmetric):
    rng = np.random.default_rng(11)
    w = (rng.standard_normal(32 * 4000 + 7) * 0.02).astype(np.float32)      # ragged tail of 7
    w[32 * 5:32 * 6] = 0.0                                                    # zero-range block
    w[32 * 9:32 * 10] = np.float32(1e-38)                                     # underflowing range
    w[32 * 11] = 7.0; w[32 * 11 + 1] = -7.0
    w[32 * 13:32 * 14] = np.float32(0.5) * np.arange(-16, 16, dtype=np.float32)   # exact .5 ties
    got = be.quantize(dev(w), symmetric).cpu().numpy()
    want = oracle.quantize_f32_to_q4(w, symmetric)
    assert got.tobytes() == want.tobytes()
    bad = w.copy(); bad[100] = np.inf
    with pytest.raises(_lib.Lq4Error):
        be.quantize(dev(bad), symmetric)
    big = np.zeros(64, np.float32); big[3] = 1.0e7                            # scale overflows f16
    with pytest.raises(_lib.Lq4Error):
        be.quantize(dev(big), symmetric)


def test_golden_q4_files_from_device_quantizer(be, golden_dir):
    import json, os
    fxs = json.load(open(os.path.join(golden_dir, "reference_q4_fixtures.json")))
    for name in ("gate_proj", "k_proj"):
        fx = fxs[name]
        n = int(np.prod(fx["shape"]))
        vals = np.array([float(((i * 37 + fx["seed"] * 13) % 200) - 100) / 4.0 for i in range(n)], np.float32)
        vals = ((vals.view(np.uint32) >> 16) << 16).view(np.float32)
        payload = be.quantize(dev(vals)).cpu().numpy()
        assert oracle.q4_file_bytes(fx["shape"], n, payload) == bytes.fromhex(fx["hex"])


def test_hadamard_and_signs_bit_exact(be):
    for dim, rows in [(32, 3), (4096, 5), (16384, 2), (2, 1)]:
        signs = oracle.signs_from_seed(synth.QUAROT_DEFAULT_SEED ^ dim, dim)
        sd = be.rot_signs(synth.QUAROT_DEFAULT_SEED ^ dim, dim)
        assert np.array_equal(sd.cpu().numpy(), signs)
        x = synth.activations(5, rows, dim, extra=dim)
        got = be.hadamard_rows(dev(x), sd).cpu().numpy()
        want = np.stack([oracle.rh_apply(signs, r) for r in x])
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# ---------------------------------------------------------------- the linear layer
def test_config1_decode_no_lora(be):
    case = make_case(1, 1, 1024, 3584)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


@pytest.mark.parametrize("m", [1, 8])
def test_config2_lora_r16(be, m):
    case = make_case(2, m, 1024, 3584, rank=16, alpha=32.0)
    ys = run_case(be, case, repeat=3)
    for y in ys:
        assert tol_ratio(y, case["y_ref"]) <= 1.0
    assert all(np.array_equal(ys[0], y) for y in ys[1:]), "repeated launches must be bit-identical"


@pytest.mark.parametrize("m", [1, 4, 16])
@pytest.mark.parametrize("k,n", [(5120, 1024), (17408, 640), (5120, 2176)])
def test_config3_large_layers_lora(be, m, k, n):
    case = make_case(3, m, k, n, rank=16, alpha=32.0, extra=k // 7 + n)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_config3_full_size_up_projection(be):
    case = make_case(3, 1, 5120, 17408, rank=16, alpha=32.0)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


@pytest.mark.parametrize("m", [1, 3, 8])
def test_config5_quarot_decode(be, m):
    case = make_case(5, m, 4096, 1376, quarot=True)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    # the rotation must matter: without it the answer is far away
    plain = dict(case, signs=None)
    assert tol_ratio(run_case(be, plain), case["y_ref"]) > 10.0


def test_quarot_with_rotated_adapter(be):
    case = make_case(5, 2, 1024, 256, rank=8, alpha=16.0, quarot=True, extra=3)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


@pytest.mark.parametrize("m,k,n,rank", [(1, 128, 1, 0), (1, 128, 130, 4), (2, 256, 127, 0), (4, 16384, 128, 16),
                                         (3, 2048, 300, 5), (5, 384, 129, 128), (16, 128, 257, 3), (9, 640, 64, 0)])
def test_ragged_shapes_and_split_k(be, m, k, n, rank):
    case = make_case(9, m, k, n, rank=rank, alpha=2.0 * rank, extra=m * 1000 + n)
    for path in (_lib.PATH_AUTO, _lib.PATH_GEMV_GENERIC):
        y = run_case(be, case, path=path)
        assert tol_ratio(y, case["y_ref"]) <= 1.0, path


@pytest.mark.parametrize("m,k,n,rank", [(1, 32, 5, 0), (3, 96, 37, 3), (2, 160, 64, 0), (20, 64, 40, 2)])
def test_generic_path_takes_any_k_multiple_of_32(be, m, k, n, rank):
    case = make_case(8, m, k, n, rank=rank, alpha=4.0, extra=k)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_bf16_activations_decode(be):
    case = make_case(4, 4, 1024, 512, rank=16, alpha=32.0, bf16_x=True)
    y = run_case(be, case, bf16=True)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_edge_scale_activations(be):
    # the reference's +-500 activation case (metal_qwen35.rs:23530-23692): relative error far below 2 %
    case = make_case(7, 2, 1024, 256, x_scale=500.0)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    assert np.max(np.abs(y - case["y_ref"])) / np.max(np.abs(case["y_ref"])) < 0.02


def test_row_slice_addressing_and_strided_output(be):
    """dispatch_gemm_q4_at: a byte offset into the payload selects a row range (an N-shard)."""
    from lattice_b200 import Q4WeightBuf
    case = make_case(6, 2, 1024, 512)
    qw = Q4WeightBuf.from_host_payload(case["payload"], 512, 1024)
    x = dev(case["x"])
    y = torch.zeros((2, 512), dtype=torch.float32, device="cuda")
    row_bytes = (1024 // 32) * 20
    # two halves written into one output with ldy = 512 (the fused gate||up pattern)
    be.dispatch_gemm_q4_at(x, 0, qw, 0, y, 0, 2, 256, 1024, ldy=512)
    be.dispatch_gemm_q4_at(x, 0, qw, 256 * row_bytes, y, 256 * 4, 2, 256, 1024, ldy=512)
    assert tol_ratio(y.cpu().numpy(), case["y_ref"]) <= 1.0
    # x offset: second token only
    y1 = torch.zeros((1, 512), dtype=torch.float32, device="cuda")
    be.dispatch_gemm_q4(x, 1024 * 4, qw, y1, 0, 1, 512, 1024)
    assert tol_ratio(y1.cpu().numpy(), case["y_ref"][1:2]) <= 1.0
    be.check_device_status()


def test_call_site_contract(be):
    from lattice_b200 import Q4WeightBuf
    case = make_case(6, 1, 128, 16)
    qw = Q4WeightBuf.from_host_payload(case["payload"], 16, 128)
    x = dev(case["x"])
    y = torch.full((1, 16), 5.0, dtype=torch.float32, device="cuda")
    be.dispatch_gemm_q4(x, 0, qw, y, 0, 0, 16, 128)          # m == 0: no-op
    be.dispatch_gemm_q4(x, 0, qw, y, 0, 1, 0, 128)           # n == 0: no-op
    assert torch.all(y == 5.0)
    for bad_k in (0, 48, 100):
        with pytest.raises(ValueError, match="divisible by 32"):
            be.dispatch_gemm_q4(x, 0, qw, y, 0, 1, 16, bad_k)
    # the C entry point itself reports the same condition as a status, never aborts
    args = _lib.LinearArgs(x.data_ptr(), 0, 1, 16, 48, qw.payload_ptr, y.data_ptr(), 0, None, None, 0)
    assert _lib.lib().lq4_linear(be._ctx, C.byref(args), None) == _lib.ERR_K
    args = _lib.LinearArgs(x.data_ptr(), 0, 1, 16, 128, qw.payload_ptr, y.data_ptr(), 8, None, None, 0)
    assert _lib.lib().lq4_linear(be._ctx, C.byref(args), None) == _lib.ERR_SHAPE   # ldy < n
    be.dispatch_matmul_q4(x, qw, y, 1, 16, 128)              # overwrites, does not accumulate
    assert tol_ratio(y.cpu().numpy(), case["y_ref"]) <= 1.0


def test_lora_adapter_lifecycle_and_standalone_dispatch(be):
    from lattice_b200 import LoraLayerData
    k, n, r = 256, 96, 4
    a, b = synth.lora_factors(2, r, k, n, extra=1)
    layers = [LoraLayerData(0, "q_proj", a, b, r, k, n)]
    with pytest.raises(_lib.Lq4Error, match="must not be empty"):
        be.load_lora_adapter([], 2.0)
    with pytest.raises(_lib.Lq4Error, match="finite"):
        be.load_lora_adapter(layers, float("inf"))
    with pytest.raises(_lib.Lq4Error, match="rank=0"):
        be.load_lora_adapter([LoraLayerData(0, "q_proj", a, b, 0, k, n)], 2.0)
    with pytest.raises(_lib.Lq4Error):
        be.load_lora_adapter([LoraLayerData(0, "q_proj", a[:-1], b, r, k, n)], 2.0)      # A length
    with pytest.raises(_lib.Lq4Error, match="duplicate"):
        be.load_lora_adapter(layers + layers, 2.0)
    with pytest.raises(_lib.Lq4Error, match="num_hidden_layers"):
        be.load_lora_adapter([LoraLayerData(3, "q_proj", a, b, r, k, n)], 2.0)
    assert not be.has_lora_adapter()
    be.load_lora_adapter(layers, 2.0)
    with pytest.raises(_lib.Lq4Error, match="already loaded"):
        be.load_lora_adapter(layers, 2.0)
    x = synth.activations(2, 3, k, extra=5)
    y0 = synth.activations(2, 3, n, extra=6)
    y = dev(y0)
    be.dispatch_lora_if_active(dev(x), 0, y, 0, 0, "k_proj", m=3)      # no projection: no-op
    assert np.array_equal(y.cpu().numpy(), y0)
    be.dispatch_lora_if_active(dev(x), 0, y, 0, 0, "q_proj", m=3)
    want = y0.copy()
    for i in range(3):
        oracle.apply_lora(a, b, r, k, n, 2.0, x[i], want[i])
    assert np.max(np.abs(y.cpu().numpy() - want)) < 1e-5
    be.unload_lora_adapter()
    be.dispatch_lora_if_active(dev(x), 0, y, 0, 0, "q_proj", m=3)      # unloaded: no-op
    assert np.max(np.abs(y.cpu().numpy() - want)) < 1e-5


def test_host_buffer_entry_point_matches_device_path(be):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    case = make_case(2, 1, 1024, 3584, rank=16, alpha=32.0)
    qw = Q4WeightBuf.from_host_payload(case["payload"], 3584, 1024)
    a, b, s = case["lora"]
    ad, bd = dev(a), dev(b)
    lora = LoraDesc(ad.data_ptr(), bd.data_ptr(), 16, s)
    xh = torch.from_numpy(case["x"]).pin_memory()
    yh = torch.empty((1, 3584), dtype=torch.float32).pin_memory()
    be.linear_host(xh.numpy(), qw, yh.numpy(), lora=lora)
    y_dev = be.linear(dev(case["x"]), qw, lora=lora).cpu().numpy()
    assert np.array_equal(yh.numpy(), y_dev)
    assert tol_ratio(yh.numpy(), case["y_ref"]) <= 1.0


def test_q4_file_round_trip_to_device(be, tmp_path):
    from lattice_b200 import Q4WeightBuf
    case = make_case(1, 1, 256, 64)
    path = tmp_path / "w.q4"
    path.write_bytes(oracle.q4_file_bytes([64, 256], 64 * 256, case["payload"]))
    qw = Q4WeightBuf.from_q4_file(str(path), (64, 256))
    assert (qw.n, qw.k) == (64, 256)
    y = be.linear(dev(case["x"]), qw).cpu().numpy()
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    with pytest.raises(_lib.Lq4Error):
        Q4WeightBuf.from_q4_file(str(path), (64, 128))


def test_launches_are_counted(be):
    from lattice_b200 import Q4WeightBuf
    case = make_case(1, 1, 128, 16)
    qw = Q4WeightBuf.from_host_payload(case["payload"], 16, 128)
    before = be.launch_count
    be.linear(dev(case["x"]), qw)
    assert be.launch_count == before + 1      # m = 1 runs as a single fused kernel


# ---------------------------------------------------------------- prefill (tensor-core) path
@pytest.mark.parametrize("m,k,n,rank,bf16", [(17, 128, 128, 0, False), (64, 256, 256, 0, False),
                                              (200, 1024, 300, 16, False), (300, 512, 520, 64, True),
                                              (33, 1024, 129, 5, True), (1024, 1024, 640, 64, True)])
def test_prefill_gemm_matches_oracle(be, m, k, n, rank, bf16):
    case = make_case(4, m, k, n, rank=rank, alpha=2.0 * rank, bf16_x=bf16, extra=m + n)
    # the tensor-core kernel explicitly (a few dozen tokens take the decode kernel in chunks by default)
    y = run_case(be, case, bf16=bf16, path=_lib.PATH_GEMM_TC)
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    y = run_case(be, case, bf16=bf16)
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    # the decode kernel, forced onto the same inputs in chunks of 16 tokens, agrees as well
    if m <= 64:
        y2 = run_case(be, case, bf16=bf16, path=_lib.PATH_GEMV_MMA)
        assert tol_ratio(y2, case["y_ref"]) <= 1.0


def test_config5_quarot_prefill(be):
    case = make_case(5, 512, 4096, 1376, quarot=True)
    y = run_case(be, case)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_config4_shape_slice_prefill_lora64(be):
    # config 4 (M=2048, K=5120, LoRA r=64, bf16 activations) on a 640-row slice of the 17408 outputs
    case = make_case(4, 2048, 5120, 640, rank=64, alpha=128.0, bf16_x=True)
    y = run_case(be, case, bf16=True)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_prefill_edge_scale_activations(be):
    # +-500 activations (reference: metal_qwen35.rs:23530-23692, relative error bound 2 %)
    case = make_case(7, 72, 512, 48, x_scale=500.0)
    y = run_case(be, case)
    assert np.max(np.abs(y - case["y_ref"])) / np.max(np.abs(case["y_ref"])) < 0.02
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_config4_full_size_sampled_output_features(be):
    """The prefill GEMM at its full size (M=2048, K=5120, N=17408, LoRA r=64, bf16 activations): the GPU result
    is checked on a sample of output features, each against the oracle run on that feature's own Q4 row."""
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    m, k, n, r = 2048, 5120, 17408, 64
    g = torch.Generator(device="cuda"); g.manual_seed(4)
    w = torch.randn((n, k), generator=g, device="cuda") * 0.02
    payload = be.quantize(w.reshape(-1))
    del w
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    a = torch.randn((r, k), generator=g, device="cuda") * 0.02
    b = torch.randn((n, r), generator=g, device="cuda") * 0.02
    qw = Q4WeightBuf.from_device_payload(payload, n, k)
    y = be.linear(x, qw, lora=LoraDesc(a.data_ptr(), b.data_ptr(), r, 2.0))
    be.check_device_status()
    sel = np.unique(np.concatenate([np.arange(0, 8), np.arange(120, 136), np.arange(n - 8, n),
                                    np.random.default_rng(0).integers(0, n, 64)]))
    row_bytes = (k // 32) * 20
    rows = payload.view(n, row_bytes)[torch.from_numpy(sel).cuda()].cpu().numpy().reshape(-1)
    assert oracle.first_invalid_block(rows) == -1
    y_ref = oracle.q4_linear(x.float().cpu().numpy(), rows, m, len(sel), k,
                             lora=(a.cpu().numpy(), b.cpu().numpy()[sel], 2.0))
    got = y[:, torch.from_numpy(sel).cuda()].cpu().numpy()
    assert tol_ratio(got, y_ref) <= 1.0
    # every output was written (the buffer is NaN-free) and the adapter term is present
    assert bool(torch.isfinite(y).all())
    y0 = be.linear(x, qw)
    assert float((y - y0).abs().max()) > 0.1


# ---------------------------------------------------------------- grouped decode launch
def _run_group(be, cases, bf16=False):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    keep, problems, qws = [], [], []
    for case in cases:
        qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
        qws.append(qw)
        x = dev(case["x"]).to(torch.bfloat16) if bf16 else dev(case["x"])
        lora = None
        if case["lora"] is not None:
            a, b, s = case["lora"]
            ad, bd = dev(a), dev(b)
            keep += [ad, bd]
            lora = LoraDesc(ad.data_ptr(), bd.data_ptr(), case["rank"], s)
        problems.append((x, qw, lora))
    outs = [torch.full((c["m"], c["n"]), float("nan"), dtype=torch.float32, device="cuda") for c in cases]
    before = be.launch_count
    be.linear_group(problems, outs)
    launches = be.launch_count - before
    be.check_device_status()
    ys = [o.cpu().numpy() for o in outs]
    for qw in qws:
        qw.free()
    return ys, launches


@pytest.mark.parametrize("m", [1, 2, 4])
def test_group_decode_set_matches_oracle(be, m):
    # the four shapes of the large-layer decode set, scaled down 4x, each with its own adapter
    shapes = [(1280, 1280), (1280, 256), (1280, 4352), (4352, 1280)]
    cases = [make_case(3, m, k, n, 16, 32.0, extra=10 + i) for i, (k, n) in enumerate(shapes)]
    ys, launches = _run_group(be, cases)
    # one token: a single launch (the adapters are projected inside it); more tokens: one
    # preparation launch (activation limbs, adapter projections) and one decode launch
    assert launches == (1 if m == 1 else 2)
    for y, c in zip(ys, cases):
        assert not np.isnan(y).any()
        assert tol_ratio(y, c["y_ref"]) <= 1.0


def test_group_mixed_adapters_ragged_rows_eight_problems(be):
    spec = [(1024, 300, 0), (2048, 129, 8), (128, 1000, 16), (1024, 128, 0), (3072, 77, 4), (1024, 2000, 0),
            (512, 640, 128), (1024, 1, 2)]
    cases = [make_case(2, 3, k, n, r, 2.0 * r, extra=30 + i) for i, (k, n, r) in enumerate(spec)]
    ys, launches = _run_group(be, cases)
    assert launches == 2
    for y, c in zip(ys, cases):
        assert not np.isnan(y).any()
        assert tol_ratio(y, c["y_ref"]) <= 1.0


def test_group_without_adapters_is_one_launch_and_repeatable(be):
    cases = [make_case(1, 1, 1024, 3584, extra=50), make_case(1, 1, 1024, 512, extra=51)]
    ys1, launches = _run_group(be, cases, bf16=False)
    ys2, _ = _run_group(be, cases, bf16=False)
    assert launches == 1
    for y1, y2, c in zip(ys1, ys2, cases):
        assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32))     # fixed summation order
        assert tol_ratio(y1, c["y_ref"]) <= 1.0


def test_group_that_cannot_share_a_launch_runs_problem_by_problem(be):
    # different token counts, an odd k and a rotated problem: served through the single-problem path
    cases = [make_case(2, 1, 1024, 256, 16, 32.0, extra=60), make_case(2, 8, 1024, 256, 16, 32.0, extra=61),
             make_case(2, 2, 96, 200, extra=62)]
    ys, launches = _run_group(be, cases)
    assert launches >= 3
    for y, c in zip(ys, cases):
        assert tol_ratio(y, c["y_ref"]) <= 1.0
    # nine one-token projections: more than the grouped kernel takes, one group of the step kernel
    many = [make_case(1, 1, 256, 128, extra=70 + i) for i in range(9)]
    ys, launches = _run_group(be, many)
    assert launches == 1
    for y, c in zip(ys, many):
        assert tol_ratio(y, c["y_ref"]) <= 1.0
    # nine two-token projections: more problems than one launch takes
    many = [make_case(1, 2, 256, 128, extra=80 + i) for i in range(9)]
    ys, launches = _run_group(be, many)
    assert launches >= 9
    for y, c in zip(ys, many):
        assert tol_ratio(y, c["y_ref"]) <= 1.0
    assert be.linear_group([]) == []


# ---------------------------------------------------------------- dense decode kernel (2..16 tokens)
@pytest.mark.parametrize("m,k,n,rank", [(2, 1024, 3584, 16), (5, 1024, 3584, 16), (12, 2048, 640, 0), (16, 1024, 3584, 64),
                                        (13, 128, 130, 3), (16, 5120, 384, 16), (4, 17408, 256, 16), (16, 17408, 200, 128)])
def test_dense_decode_tokens_and_long_rows(be, m, k, n, rank):
    case = make_case(2, m, k, n, rank, 2.0 * rank, extra=200 + m)
    y = run_case(be, case, path=_lib.PATH_GEMV_MMA)
    assert not np.isnan(y).any()
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    y2 = run_case(be, case)                     # automatic dispatch takes the same kernel for m <= 16
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))


def test_dense_decode_bf16_activations_and_rotation(be):
    case = make_case(2, 8, 1024, 512, 16, 32.0, bf16_x=True, extra=210)
    y = run_case(be, case, bf16=True)
    assert tol_ratio(y, case["y_ref"]) <= 1.0
    rot = make_case(5, 6, 1024, 300, quarot=True, extra=211)
    y = run_case(be, rot)
    assert tol_ratio(y, rot["y_ref"]) <= 1.0


def test_dense_decode_more_than_sixteen_tokens_in_chunks(be):
    case = make_case(2, 37, 256, 200, 8, 16.0, extra=212)
    y = run_case(be, case, path=_lib.PATH_GEMV_MMA)
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_group_sixteen_tokens(be):
    shapes = [(1280, 1280), (1280, 256), (1280, 4352), (4352, 1280)]
    cases = [make_case(3, 16, k, n, 16, 32.0, extra=220 + i) for i, (k, n) in enumerate(shapes)]
    ys, launches = _run_group(be, cases)
    assert launches == 2
    for y, c in zip(ys, cases):
        assert not np.isnan(y).any()
        assert tol_ratio(y, c["y_ref"]) <= 1.0


# ---------------------------------------------------------------- all-gather fused into the epilogue
def _peer_pair():
    """Two peer buffers on this GPU standing in for two ranks' output buffers."""
    L = _lib.lib()
    bufs = []
    for _ in range(2):
        h = C.c_void_p()
        _lib.check(L.lq4_peer_buf_create(16 * 8192 * 4, C.byref(h)))
        bufs.append(h.value)
    bases = [L.lq4_peer_buf_base(b) for b in bufs]
    return bufs, bases


def _as_tensor(ptr, shape):
    from lattice_b200.sharded import _DeviceArray
    return torch.as_tensor(_DeviceArray(ptr, shape, None), device="cuda")


@pytest.mark.parametrize("m", [1, 4, 16])
def test_fused_all_gather_writes_every_peer_and_signals(be, m):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import GatherDesc, LoraDesc
    L = _lib.lib()
    bufs, bases = _peer_pair()
    try:
        n_total, k = 1024 + 384, 1024
        cases = [make_case(2, m, k, 1024, 16, 32.0, extra=300), make_case(2, m, k, 384, 16, 32.0, extra=301)]
        full = [_as_tensor(L.lq4_peer_buf_payload(b), (m, n_total)) for b in bufs]
        for f in full:
            f.fill_(float("nan"))
        ctrl = [_as_tensor(bs, (64,)).view(torch.int64) for bs in bases]
        # "rank 0" computes columns [0, 1024), "rank 1" columns [1024, 1408); each writes both buffers
        col0 = [0, 1024]
        keep = []
        for r, case in enumerate(cases):
            desc = GatherDesc(2, r, (C.c_void_p * _lib.MAX_PEERS)(*bases))
            qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
            a, b, s = case["lora"]
            ad, bd = dev(a), dev(b)
            lora = LoraDesc(ad.data_ptr(), bd.data_ptr(), 16, s)
            keep += [qw, ad, bd, desc]
            out = full[r][:, col0[r]:col0[r] + case["n"]]
            be.linear_group([(dev(case["x"]), qw, lora), (dev(case["x"]), qw, lora)], [out, out], gather=desc) \
                if r == 0 else be.dispatch_gemm_q4(dev(case["x"]), 0, qw, out, 0, m, case["n"], k, lora=lora,
                                                   ldy=n_total, gather=desc)
        # both "ranks" have launched once: each one's wait finds the other's 256 arrivals
        for desc in (keep[3], keep[7]):
            be.gather_wait(desc)
        be.check_device_status()
        want = np.concatenate([c["y_ref"] for c in cases], axis=1)
        for f in full:
            got = f.cpu().numpy()
            assert not np.isnan(got).any()
            assert tol_ratio(got, want) <= 1.0
        assert np.array_equal(full[0].cpu().numpy().view(np.uint32), full[1].cpu().numpy().view(np.uint32))
        # each gathered launch adds exactly 256 to the peer's arrival counter and to its own sequence counter
        assert [int(c[0]) for c in ctrl] == [256, 256] and [int(c[1]) for c in ctrl] == [256, 256]
        assert [int(c[2]) for c in ctrl] == [256, 256]      # the CTAs of each launch counted themselves
        # a launch whose input depends on gathered results waits inside the kernel: all arrivals are
        # there already, so it goes straight through and computes the same values
        y2 = torch.full((m, cases[1]["n"]), float("nan"), device="cuda")
        be.dispatch_gemm_q4(dev(cases[1]["x"]), 0, keep[4], y2, 0, m, cases[1]["n"], k, lora=LoraDesc(keep[5].data_ptr(), keep[6].data_ptr(), 16, cases[1]["lora"][2]),
                            wait_gather=keep[7])
        be.check_device_status()
        assert tol_ratio(y2.cpu().numpy(), cases[1]["y_ref"]) <= 1.0
        # a prefill-sized consumer of gathered activations gets the stand-alone wait in front of its kernels
        big_case = make_case(2, 64, k, 256, extra=302)
        qwb = Q4WeightBuf.from_host_payload(big_case["payload"], 256, k)
        yb = torch.full((64, 256), float("nan"), device="cuda")
        before = be.launch_count
        be.dispatch_gemm_q4(dev(big_case["x"]), 0, qwb, yb, 0, 64, 256, k, wait_gather=keep[7])
        be.check_device_status()
        assert be.launch_count - before >= 2          # the wait kernel and the GEMM's kernels
        assert tol_ratio(yb.cpu().numpy(), big_case["y_ref"]) <= 1.0
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            L.lq4_peer_buf_free(b)


@pytest.mark.parametrize("m,bf16", [(40, False), (300, True)])
def test_fused_all_gather_from_the_tensor_core_epilogue(be, m, bf16):
    """Prefill shapes: two peer buffers on one GPU stand in for two ranks; each "rank" runs the tensor-core kernel
    on its rows of the weight and its epilogue stores the slice into BOTH buffers; a signal kernel behind it
    advances the arrival counters that lq4_gather_wait reads."""
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import GatherDesc, LoraDesc
    L = _lib.lib()
    n_total, k, r = 512 + 384, 512, 8
    bufs, bases = [], []
    for _ in range(2):
        h = C.c_void_p()
        _lib.check(L.lq4_peer_buf_create(m * n_total * 4, C.byref(h)))
        bufs.append(h.value)
        bases.append(L.lq4_peer_buf_base(h.value))
    try:
        case = make_case(4, m, k, n_total, r, 2.0 * r, bf16_x=bf16, extra=310)
        a, b, s = case["lora"]
        ad = dev(a)
        full = [_as_tensor(L.lq4_peer_buf_payload(bf), (m, n_total)) for bf in bufs]
        for f in full:
            f.fill_(float("nan"))
        ctrl = [_as_tensor(bs, (64,)).view(torch.int64) for bs in bases]
        x = dev(case["x"]).to(torch.bfloat16) if bf16 else dev(case["x"])
        keep, descs = [], []
        for rk, (n0, n1) in enumerate([(0, 512), (512, n_total)]):
            desc = GatherDesc(2, rk, (C.c_void_p * _lib.MAX_PEERS)(*bases))
            off = n0 * (k // 32) * 20
            qw = Q4WeightBuf.from_host_payload(case["payload"][off: off + (n1 - n0) * (k // 32) * 20], n1 - n0, k)
            bd = dev(b[n0:n1])
            keep += [qw, bd]
            descs.append(desc)
            out = full[rk][:, n0:n1]
            be.dispatch_gemm_q4(x, 0, qw, out, 0, m, n1 - n0, k, lora=LoraDesc(ad.data_ptr(), bd.data_ptr(), r, s),
                                ldy=n_total, gather=desc)
        for desc in descs:
            be.gather_wait(desc)
        be.check_device_status()
        for f in full:
            got = f.cpu().numpy()
            assert not np.isnan(got).any()
            assert tol_ratio(got, case["y_ref"]) <= 1.0
        assert np.array_equal(full[0].cpu().numpy().view(np.uint32), full[1].cpu().numpy().view(np.uint32))
        assert [int(c[0]) for c in ctrl] == [256, 256] and [int(c[1]) for c in ctrl] == [256, 256]
        # an adapter too wide to ride along in the tensor-core kernel is applied in a second pass: no fused gather
        wide_a, wide_b = torch.zeros((160, k), device="cuda"), torch.zeros((512, 160), device="cuda")
        with pytest.raises(_lib.Lq4Error):
            be.dispatch_gemm_q4(x, 0, keep[0], full[0][:, 0:512], 0, m, 512, k,
                                lora=LoraDesc(wide_a.data_ptr(), wide_b.data_ptr(), 160, 1.0), ldy=n_total, gather=descs[0])
    finally:
        torch.cuda.synchronize()
        for bf in bufs:
            L.lq4_peer_buf_free(bf)


def test_wide_adapter_takes_the_second_pass_on_prefill_shapes_and_the_decode_kernels_below(be):
    """A blend of adapters adds their ranks: rank 192 runs inside the decode kernels (m <= 16) and, for prefill
    shapes, as the tensor-core product followed by the adapter pass."""
    for m in (1, 4, 40):
        case = make_case(3, m, 512, 384, 192, 384.0, extra=320 + m)
        y = run_case(be, case)
        assert tol_ratio(y, case["y_ref"]) <= 1.0


@pytest.mark.parametrize("k", [256, 2048, 4096, 8192, 16384])
def test_rotation_in_the_decode_prologue_all_row_lengths(be, k):
    # k < 2048 takes the level-by-level transform, longer rows the register/shuffle one
    case = make_case(5, 1, k, 384, quarot=True, extra=400 + k // 256)
    y = run_case(be, case, path=_lib.PATH_GEMV_MMA)
    assert not np.isnan(y).any()
    assert tol_ratio(y, case["y_ref"]) <= 1.0


def test_adapter_rotation_for_a_quarot_base_at_load_time():
    """Input side A <- A R^T, output side B <- R B, unknown modules refused
    (crates/inference/src/quant/quarot/lora.rs:150-216 and its tests)."""
    from lattice_b200 import CudaQ4Backend, LoraLayerData
    hidden, inter, rank, seed = 256, 512, 4, 0xC0FFEE
    rng = np.random.default_rng(5)
    a_q = rng.standard_normal((rank, hidden), dtype=np.float32) * 0.1
    b_q = rng.standard_normal((inter, rank), dtype=np.float32) * 0.1
    a_o = rng.standard_normal((rank, inter), dtype=np.float32) * 0.1
    b_o = rng.standard_normal((hidden, rank), dtype=np.float32) * 0.1
    be2 = CudaQ4Backend(0, num_hidden_layers=1)
    try:
        be2.load_lora_adapter([LoraLayerData(0, "gate_proj", a_q, b_q, rank, hidden, inter),
                               LoraLayerData(0, "down_proj", a_o, b_o, rank, inter, hidden)], scale=2.0,
                              quarot_seed=seed, quarot_hidden_dim=hidden)
        signs = oracle.signs_from_seed(seed, hidden)
        h = rng.standard_normal((1, hidden), dtype=np.float32)
        # input side: the delta on the rotated activation R h equals the oracle's with its rotated A,
        # and equals the unrotated delta on h (B A R^T R h = B A h)
        rh = oracle.rh_apply(signs, h.reshape(-1)).reshape(1, hidden)
        y = torch.zeros((1, inter), device="cuda")
        be2.dispatch_lora_if_active(dev(rh), 0, y, 0, 0, "gate_proj")
        a_rot = oracle.absorb_rotation(a_q, rank, hidden, signs, "input")
        want = np.zeros(inter, np.float32)
        assert oracle.apply_lora(a_rot, b_q, rank, hidden, inter, 2.0, rh, want)
        assert np.max(np.abs(y.cpu().numpy().reshape(-1) - want)) <= 1e-5 * max(1.0, float(np.max(np.abs(want))))
        plain = np.zeros(inter, np.float32)
        assert oracle.apply_lora(a_q, b_q, rank, hidden, inter, 2.0, h, plain)
        assert np.max(np.abs(want - plain)) <= 1e-4
        # output side: the delta comes out in the rotated basis, R (B A x)
        xi = rng.standard_normal((1, inter), dtype=np.float32)
        y2 = torch.zeros((1, hidden), device="cuda")
        be2.dispatch_lora_if_active(dev(xi), 0, y2, 0, 0, "down_proj")
        b_rot = oracle.absorb_rotation(b_o, hidden, rank, signs, "output")
        want2 = np.zeros(hidden, np.float32)
        assert oracle.apply_lora(a_o, b_rot, rank, inter, hidden, 2.0, xi, want2)
        assert np.max(np.abs(y2.cpu().numpy().reshape(-1) - want2)) <= 1e-5 * max(1.0, float(np.max(np.abs(want2))))
        plain2 = np.zeros(hidden, np.float32)
        assert oracle.apply_lora(a_o, b_o, rank, inter, hidden, 2.0, xi, plain2)
        assert np.max(np.abs(want2 - oracle.rh_apply(signs, plain2))) <= 1e-4
        be2.unload_lora_adapter()
        with pytest.raises(_lib.Lq4Error):       # not in the rotation plan
            be2.load_lora_adapter([LoraLayerData(0, "conv1d", a_q, b_q, rank, hidden, inter)], 2.0,
                                  quarot_seed=seed, quarot_hidden_dim=hidden)
        with pytest.raises(_lib.Lq4Error):       # input-side module whose d_in is not the hidden dimension
            be2.load_lora_adapter([LoraLayerData(0, "q_proj", a_o, b_o, rank, inter, hidden)], 2.0,
                                  quarot_seed=seed, quarot_hidden_dim=hidden)
        assert not be2.has_lora_adapter()
    finally:
        be2.close()


def test_resident_decode_bf16_activations_with_adapter_long_row(be):
    # one token, bf16 activations: the in-kernel adapter projection takes its element-wise path, and a
    # 17408-long row is cut into six k pieces per dot product
    for k, n, rank in [(1024, 384, 16), (17408, 256, 8)]:
        case = make_case(3, 1, k, n, rank=rank, alpha=2.0 * rank, bf16_x=True, extra=500 + rank)
        y = run_case(be, case, bf16=True)
        assert tol_ratio(y, case["y_ref"]) <= 1.0
    # unaligned adapter factors (4-byte aligned only) also take the element-wise path
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    case = make_case(3, 1, 1024, 384, rank=16, alpha=32.0, extra=520)
    qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
    a, b, s = case["lora"]
    abuf = torch.zeros(a.size + 1, device="cuda")
    abuf[1:] = dev(a).reshape(-1)
    bd = dev(b)
    y = be.linear(dev(case["x"]), qw, lora=LoraDesc(abuf.data_ptr() + 4, bd.data_ptr(), 16, s))
    be.check_device_status()
    assert tol_ratio(y.cpu().numpy(), case["y_ref"]) <= 1.0
    qw.free()


def test_checkpoint_directory_through_its_manifest(be, tmp_path):
    """quantize_index.json (QuaRot flavour) -> uploaded weights by tensor name -> a projection that matches the oracle."""
    import json
    from lattice_b200 import manifest as mf
    cases = {"model.layers.0.mlp.gate_proj.weight": make_case(2, 1, 256, 384, extra=600),
             "model.layers.0.mlp.up_proj.weight": make_case(2, 1, 256, 128, extra=601)}
    entries = []
    for i, (name, c) in enumerate(cases.items()):
        fname = f"t{i}.q4"
        (tmp_path / fname).write_bytes(oracle.q4_file_bytes([c["n"], c["k"]], c["n"] * c["k"], c["payload"]))
        entries.append({"name": name, "file": fname, "quantized": True, "shape": [c["n"], c["k"]], "numel": c["n"] * c["k"]})
    entries.append({"name": "model.norm.weight", "file": "norm.f16", "quantized": False, "shape": [256], "numel": 256})
    (tmp_path / mf.MANIFEST_NAME).write_text(json.dumps({"quarot_seed": 7, "tensors": entries}))
    assert mf.load_manifest(str(tmp_path)).quarot_seed == 7
    weights = mf.load_q4_directory(str(tmp_path))
    try:
        assert set(weights) == set(cases)            # the f16 tensor is skipped
        for name, c in cases.items():
            y = be.linear(dev(c["x"]), weights[name])
            assert tol_ratio(y.cpu().numpy(), c["y_ref"]) <= 1.0
    finally:
        for qw in weights.values():
            qw.free()
    # a shape in the manifest that contradicts the file is refused by the library's loader
    entries[0]["shape"] = [c["n"], c["k"] * 2]
    (tmp_path / mf.MANIFEST_NAME).write_text(json.dumps(entries))
    with pytest.raises(_lib.Lq4Error):
        mf.load_q4_directory(str(tmp_path))
    entries[0]["shape"] = None
    entries[0]["file"] = "../escape.q4"
    (tmp_path / mf.MANIFEST_NAME).write_text(json.dumps(entries))
    with pytest.raises(mf.ManifestError):
        mf.load_q4_directory(str(tmp_path))


# ---------------------------------------------------------------- lm_head: projection + exact top-k
def _topk_ids(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("n", [1, 37, 1024, 1025, 5000, 248320])
@pytest.mark.parametrize("k", [1, 8, 50, 256])
def test_logits_topk_is_exact_index_work(be, n, k):
    # coarse values: most of the order is decided by the tie rule, and the result must be identical
    rng = np.random.default_rng(n * 1000 + k)
    logits = rng.integers(-300, 300, n).astype(np.float32) * np.float32(0.125)
    if n > 40:
        logits[rng.integers(0, n, 20)] = np.nan
        logits[rng.integers(0, n, 5)] = -np.inf
        logits[rng.integers(0, n, 3)] = np.inf
    vals, ids = be.logits_topk(dev(logits), k)
    rv, ri = oracle.topk(logits, k)
    assert np.array_equal(_topk_ids(ids), ri)
    assert np.array_equal(vals.cpu().numpy(), rv)
    be.check_device_status()


def test_logits_topk_all_winners_in_one_block(be):
    # the reference's adversarial case (metal_qwen35.rs:24967-25040): every global winner sits in one
    # 1024-row block; a block-local argmax or a truncated local list would drop some of them
    n, k = 20000, 64
    rng = np.random.default_rng(7)
    logits = rng.standard_normal(n).astype(np.float32)
    block = 5
    winners = block * 1024 + rng.permutation(1024)[:k]
    logits[winners] = 50.0 + rng.standard_normal(k).astype(np.float32)
    vals, ids = be.logits_topk(dev(logits), k)
    rv, ri = oracle.topk(logits, k)
    assert set(ri.tolist()) == set(winners.tolist())
    assert np.array_equal(_topk_ids(ids), ri) and np.array_equal(vals.cpu().numpy(), rv)


def test_logits_topk_rejects_bad_requests(be):
    from lattice_b200._lib import Lq4Error
    t = dev(np.zeros(16, np.float32))
    for k in (0, 257):
        with pytest.raises(Lq4Error) as e:
            be.logits_topk(t, k)
        assert e.value.status == _lib.ERR_SHAPE


def _assert_topk_agrees(ref_logits, ids, vals, k):
    """The reference's acceptance rule for GPU-vs-CPU lm_head top-k (topk_set_agreement_or_boundary_tie,
    metal_qwen35.rs:37488-37570): the sets are equal, or every differing token lies within epsilon of the
    boundary logit.  On top of it: each returned logit is that row's logit within the output tolerance,
    and the list is sorted in candidate order."""
    ids = ids.astype(np.int64)
    assert len(set(ids.tolist())) == k and ids.min() >= 0 and ids.max() < ref_logits.size
    rms = float(np.sqrt(np.mean(ref_logits.astype(np.float64) ** 2)))
    eps = 2e-3 * (float(np.max(np.abs(ref_logits))) + rms)
    assert np.all(np.abs(vals - ref_logits[ids]) <= 1e-3 * (np.abs(ref_logits[ids]) + rms))
    assert np.all((vals[:-1] > vals[1:]) | ((vals[:-1] == vals[1:]) & (ids[:-1] < ids[1:])))
    rv, ri = oracle.topk(ref_logits, k)
    diff = set(ri.tolist()) ^ set(ids.tolist())
    assert all(abs(float(ref_logits[t]) - float(rv[-1])) <= eps for t in diff), sorted(diff)


@pytest.mark.parametrize("n,k_dim,top_k,rank", [(4096 + 37, 1024, 8, 0), (4096 + 37, 1024, 50, 16), (32000, 2048, 64, 0)])
def test_lm_head_topk_agrees_with_full_logits(be, n, k_dim, top_k, rank):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    case = make_case(3, 1, k_dim, n, rank=rank, alpha=2.0 * rank)
    qw = Q4WeightBuf.from_host_payload(case["payload"], n, k_dim)
    lora, keep = None, []
    if rank:
        a, b, s = case["lora"]
        keep = [dev(a), dev(b)]
        lora = LoraDesc(keep[0].data_ptr(), keep[1].data_ptr(), rank, s)
    x = dev(case["x"])
    full = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    vals, ids = be.lm_head_topk(x, qw, top_k, lora=lora, logits_out=full)
    vals2, ids2 = be.lm_head_topk(x, qw, top_k, lora=lora)          # logit row kept in the workspace only
    be.check_device_status()
    ref = case["y_ref"].reshape(-1)
    _assert_topk_agrees(ref, _topk_ids(ids), vals.cpu().numpy(), top_k)
    assert np.array_equal(_topk_ids(ids), _topk_ids(ids2)) and np.array_equal(vals.cpu().numpy(), vals2.cpu().numpy())
    # the selection itself is exact on the logits the projection produced
    rv, ri = oracle.topk(full.cpu().numpy(), top_k)
    assert np.array_equal(_topk_ids(ids), ri) and np.array_equal(vals.cpu().numpy(), rv)
    assert tol_ratio(full.cpu().numpy().reshape(1, -1), case["y_ref"]) <= 1.0
    qw.free()


def test_lm_head_topk_takes_one_token(be):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LinearArgs, Lq4Error, check
    case = make_case(1, 2, 256, 128)
    qw = Q4WeightBuf.from_host_payload(case["payload"], 128, 256)
    x = dev(case["x"])
    cand = torch.empty((4, 2), dtype=torch.int32, device="cuda")
    args = LinearArgs(x.data_ptr(), _lib.DTYPE_F32, 2, 128, 256, qw.payload_ptr, None, 0, None, None, _lib.PATH_AUTO, None, None)
    with pytest.raises(Lq4Error) as e:
        check(_lib.lib().lq4_lm_head_topk(be._ctx, C.byref(args), 4, cand.data_ptr(), None))
    assert e.value.status == _lib.ERR_SHAPE
    qw.free()


# ---------------------------------------------------------------- block-diagonal rotation (R4 in front of down_proj)
@pytest.mark.parametrize("n,block", [(3584, 128), (17408, 256), (17408, 128), (4096, 4096), (96, 32)])
def test_block_rotation_signs_and_rows_bit_exact(be, n, block):
    seed = 0x5EED0000 + n + block
    signs = be.block_rot_signs(seed, n, block)
    ref_signs = oracle.block_hadamard_signs(seed, n, block)
    assert np.array_equal(signs.cpu().numpy(), ref_signs)
    rng = np.random.default_rng(n)
    x = rng.standard_normal((3, n)).astype(np.float32)
    y = be.block_hadamard_rows(dev(x), signs, block).cpu().numpy()
    for r in range(3):
        ref = oracle.block_hadamard_apply(ref_signs, x[r], block)
        assert np.array_equal(y[r].view(np.uint32), ref.view(np.uint32))
    be.check_device_status()


@pytest.mark.parametrize("m,k,n,block,rank,bf16", [(1, 3584, 1024, 128, 0, False), (1, 17408, 2560, 256, 16, False),
                                                   (4, 3584, 1024, 128, 16, False), (40, 3584, 512, 128, 0, True)])
def test_projection_with_block_rotation_in_front(be, m, k, n, block, rank, bf16):
    # the R4 recipe: down_proj rows were rotated block by block offline; the activations get the same rotation online
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    case = make_case(5, m, k, n, rank=rank, alpha=2.0 * rank, bf16_x=bf16)
    signs_h = oracle.block_hadamard_signs(0xB10C, k, block)
    xr = np.stack([oracle.block_hadamard_apply(signs_h, case["x"][i], block) for i in range(m)])
    y_ref = oracle.q4_linear(xr, None, m, n, k, lora=None, w_f32=case["w_deq"])
    if rank:
        a, b, s = case["lora"]
        # the adapter sees the rotated activations too (one x for both products, as in the fused call)
        y_ref = oracle.q4_linear(xr, None, m, n, k, lora=case["lora"], w_f32=case["w_deq"])
    qw = Q4WeightBuf.from_host_payload(case["payload"], n, k)
    signs = dev(signs_h)
    lora, keep = None, []
    if rank:
        keep = [dev(a), dev(b)]
        lora = LoraDesc(keep[0].data_ptr(), keep[1].data_ptr(), rank, s)
    x = dev(case["x"]).to(torch.bfloat16) if bf16 else dev(case["x"])
    y = be.linear(x, qw, lora=lora, rot=be.rot_desc(signs, block))
    be.check_device_status()
    assert tol_ratio(y.cpu().numpy(), y_ref) <= 1.0
    qw.free()


def test_rotation_descriptor_must_divide_k(be):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import Lq4Error
    case = make_case(1, 1, 384, 64)
    qw = Q4WeightBuf.from_host_payload(case["payload"], 64, 384)
    signs = dev(np.ones(384, np.float32))
    for block in (256, 48, 512):
        with pytest.raises(Lq4Error) as e:
            be.linear(dev(case["x"]), qw, rot=be.rot_desc(signs, block))
        assert e.value.status == _lib.ERR_ROT
    y = be.linear(dev(case["x"]), qw, rot=be.rot_desc(signs, 128))       # all-plus signs, block 128: accepted
    be.check_device_status()
    qw.free()


@pytest.mark.parametrize("nh,dh", [(8, 256), (16, 128), (32, 128), (2, 64), (128, 8), (1, 32)])
def test_cross_head_rotation_bit_exact(be, nh, dh):
    # R3 in front of o_proj: H_nh (x) I_dh on the gated attention output
    signs_h = oracle.signs_from_seed(0x703 + nh, nh)
    rng = np.random.default_rng(nh * dh)
    x = rng.standard_normal((5, nh * dh)).astype(np.float32)
    y = be.cross_head_hadamard_rows(dev(x), dev(signs_h), dh).cpu().numpy()
    for r in range(5):
        ref = oracle.cross_head_rotation(signs_h, x[r], dh)
        assert np.array_equal(y[r].view(np.uint32), ref.view(np.uint32))
    be.check_device_status()
    from lattice_b200._lib import Lq4Error
    if nh == 8:
        with pytest.raises(Lq4Error) as e:
            be.cross_head_hadamard_rows(dev(np.zeros((1, 6 * 4), np.float32)), dev(np.ones(6, np.float32)), 4)
        assert e.value.status == _lib.ERR_ROT


# ---------------------------------------------------------------- dense MLP block: gate||up -> silu*up -> down
@pytest.mark.parametrize("m,hidden,inter,rank", [(1, 1024, 3584, 0), (1, 1024, 3584, 16), (1, 2048, 6144, 16),
                                                 (4, 1024, 3584, 16), (24, 1024, 3584, 16), (1, 1024, 96, 8)])
def test_mlp_block_matches_the_three_step_reference(be, m, hidden, inter, rank):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    x = synth.activations(3, m, hidden, 0)
    wgu = synth.weights(3, 2 * inter, hidden, 1)
    wd = synth.weights(3, hidden, inter, 2)
    p_gu, p_d = oracle.quantize_f32_to_q4(wgu), oracle.quantize_f32_to_q4(wd)
    loras, descs, keep = [None] * 3, [None] * 3, []
    if rank:
        for i, (k_in, n_out) in enumerate(((hidden, inter), (hidden, inter), (inter, hidden))):
            a, b = synth.lora_factors(3, rank, k_in, n_out, 10 + i)
            loras[i] = (a, b, oracle.effective_scale(rank, 2.0 * rank))
            ad, bd = dev(a), dev(b)
            keep += [ad, bd]
            descs[i] = LoraDesc(ad.data_ptr(), bd.data_ptr(), rank, loras[i][2])
    y_ref = oracle.mlp_block(x, p_gu, p_d, m, hidden, inter, *loras)
    qgu = Q4WeightBuf.from_host_payload(p_gu, 2 * inter, hidden)
    qd = Q4WeightBuf.from_host_payload(p_d, hidden, inter)
    before = be.launch_count
    y = be.mlp_block(dev(x), qgu, qd, lora_gate=descs[0], lora_up=descs[1], lora_down=descs[2])
    launches = be.launch_count - before
    be.check_device_status()
    # Decode shapes keep the single-projection bound end to end.  With more than 16 tokens both projections
    # run on the tensor-core kernel, which rounds the dequantized weights to f16 once and uses most of the
    # single-projection bound by itself; two of them in a row get the sum of their bounds.
    bound = 1.0 if m <= 16 else 2.0
    ratio = tol_ratio(y.cpu().numpy(), y_ref)
    assert ratio <= bound, f"tolerance ratio {ratio}"
    if m == 1 and inter % 128 == 0 and hidden % 128 == 0:
        assert launches == 1          # the whole block as ONE persistent launch (down_proj reads silu(gate) * up through the mailbox)
        # switched off: gate and up rows in one grouped launch; down_proj gates its own input
        be.set_option(_lib.OPT_MLP_ONE_LAUNCH, 0)
        before = be.launch_count
        y1 = be.mlp_block(dev(x), qgu, qd, lora_gate=descs[0], lora_up=descs[1], lora_down=descs[2])
        be.set_option(_lib.OPT_MLP_ONE_LAUNCH, 1)
        assert be.launch_count - before == 2
        be.check_device_status()
        assert tol_ratio(y1.cpu().numpy(), y_ref) <= bound
    # with a caller-provided scratch (one token: gate||up launch, then down_proj gating its own input) the
    # result holds the same bound; for more tokens the two forms are the same code path
    scratch = torch.empty((m, 2 * inter), dtype=torch.float32, device="cuda")
    before = be.launch_count
    y2 = be.mlp_block(dev(x), qgu, qd, lora_gate=descs[0], lora_up=descs[1], lora_down=descs[2], gate_up=scratch)
    if m == 1 and inter % 128 == 0:
        assert be.launch_count - before == 2
    be.check_device_status()
    assert tol_ratio(y2.cpu().numpy(), y_ref) <= bound
    if m > 1:
        diff = float(np.abs(y2.cpu().numpy() - y.cpu().numpy()).max())
        assert diff == 0.0, f"scratch given vs workspace: max abs difference {diff}"
    qgu.free()
    qd.free()


def test_adapter_from_a_safetensors_file_drives_the_fused_projection(be, tmp_path):
    st_numpy = pytest.importorskip("safetensors.numpy")
    from lattice_b200 import Q4WeightBuf
    k, n, r = 1024, 512, 8
    case = make_case(2, 1, k, n)
    a, b = synth.lora_factors(2, r, k, n, extra=3)
    path = tmp_path / "adapter_model.safetensors"
    st_numpy.save_file({"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": a,
                        "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": b},
                       str(path), metadata={"alpha": "16"})
    adapter = be.load_lora_adapter_file(str(path))
    try:
        assert adapter.rank == r and adapter.scale == 2.0 and be.has_lora_adapter()
        qw = Q4WeightBuf.from_host_payload(case["payload"], n, k)
        y = be.linear(dev(case["x"]), qw, lora=be.lora_desc(0, "q_proj"))
        be.check_device_status()
        y_ref = oracle.q4_linear(case["x"], None, 1, n, k, lora=(a, b, 2.0), w_f32=case["w_deq"])
        assert tol_ratio(y.cpu().numpy(), y_ref) <= 1.0
        qw.free()
    finally:
        be.unload_lora_adapter()


def test_vocabulary_sharded_lm_head_topk_merges_to_the_global_topk(be):
    # two vocabulary shards on one GPU (the N-sharded lm_head of a 2-GPU group): local top-k per shard on the
    # device, candidates merged as ShardedLmHead does after its exchange
    from lattice_b200 import Q4WeightBuf
    from lattice_b200.sharded import merge_topk_candidates, shard_plan
    vocab, k, top_k = 6000 + 37, 1024, 40
    case = make_case(3, 1, k, vocab)
    x = dev(case["x"])
    vals, ids, rows = [], [], []
    for r in range(2):
        n0, n1, off = shard_plan(vocab, k, 2, r)
        shard = case["payload"][off: off + (n1 - n0) * (k // 32) * 20]
        qw = Q4WeightBuf.from_host_payload(shard, n1 - n0, k)
        full = torch.empty(n1 - n0, device="cuda")
        v, i = be.lm_head_topk(x, qw, top_k, logits_out=full)
        i = i.to(torch.int64) & 0xFFFFFFFF
        vals.append(v.clone())
        ids.append(torch.where(i == 0xFFFFFFFF, i, i + n0))
        rows.append(full.cpu().numpy())
        qw.free()
    be.check_device_status()
    mv, mi = merge_topk_candidates(torch.cat(vals), torch.cat(ids), top_k)
    rv, ri = oracle.topk(np.concatenate(rows), top_k)               # exact on the logits the shards produced
    assert np.array_equal(mi.cpu().numpy(), ri.astype(np.int64)) and np.array_equal(mv.cpu().numpy(), rv)
    _assert_topk_agrees(case["y_ref"].reshape(-1), ri, rv, top_k)


def test_mlp_block_checks_all_three_projections_before_launching(be):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc, Lq4Error
    hidden, inter = 256, 128
    p_gu = oracle.quantize_f32_to_q4(synth.weights(1, 2 * inter, hidden, 1))
    p_d = oracle.quantize_f32_to_q4(synth.weights(1, hidden, inter, 2))
    qgu, qd = Q4WeightBuf.from_host_payload(p_gu, 2 * inter, hidden), Q4WeightBuf.from_host_payload(p_d, hidden, inter)
    a = dev(np.zeros((4, inter), np.float32))
    b = dev(np.zeros((hidden, 4), np.float32))
    bad = LoraDesc(a.data_ptr(), b.data_ptr(), 0, 1.0)           # rank 0 on down_proj
    before = be.launch_count
    with pytest.raises(Lq4Error) as e:
        be.mlp_block(dev(synth.activations(1, 1, hidden, 0)), qgu, qd, lora_down=bad)
    assert e.value.status == _lib.ERR_LORA and be.launch_count == before
    qgu.free()
    qd.free()


def test_group_of_one_runs_the_single_projection_on_the_grouped_kernel(be):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    case = make_case(2, 1, 2048, 1536, rank=16, alpha=32.0)
    qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
    a, b, s = case["lora"]
    ad, bd = dev(a), dev(b)
    before = be.launch_count
    (y,) = be.linear_group([(dev(case["x"]), qw, LoraDesc(ad.data_ptr(), bd.data_ptr(), 16, s))])
    assert be.launch_count == before + 1
    be.check_device_status()
    assert tol_ratio(y.cpu().numpy(), case["y_ref"]) <= 1.0
    qw.free()


@pytest.mark.parametrize("m", [1, 3])
def test_mlp_block_with_the_r4_rotation_in_front_of_down_proj(be, m):
    # down_proj's rows were rotated block by block offline; the gated activations get the same rotation online
    from lattice_b200 import Q4WeightBuf
    hidden, inter, block = 1024, 3584, 128
    x = synth.activations(4, m, hidden, 0)
    p_gu = oracle.quantize_f32_to_q4(synth.weights(4, 2 * inter, hidden, 1))
    p_d = oracle.quantize_f32_to_q4(synth.weights(4, hidden, inter, 2))
    signs_h = oracle.block_hadamard_signs(0xD0, inter, block)
    half = inter * (hidden // 32) * 20
    gate = oracle.q4_linear(x, p_gu[:half], m, inter, hidden)
    up = oracle.q4_linear(x, p_gu[half:], m, inter, hidden)
    h = oracle.silu_mul(np.concatenate([gate, up], axis=1), inter)
    hr = np.stack([oracle.block_hadamard_apply(signs_h, h[i], block) for i in range(m)])
    y_ref = oracle.q4_linear(hr, p_d, m, hidden, inter)
    qgu, qd = Q4WeightBuf.from_host_payload(p_gu, 2 * inter, hidden), Q4WeightBuf.from_host_payload(p_d, hidden, inter)
    signs = dev(signs_h)
    y = be.mlp_block(dev(x), qgu, qd, rot_down=be.rot_desc(signs, block))
    be.check_device_status()
    assert tol_ratio(y.cpu().numpy(), y_ref) <= 1.0
    qgu.free()
    qd.free()
