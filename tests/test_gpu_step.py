"""GPU parity of lq4_decode_step: several groups of one-token projections in one persistent launch, later
groups reading what earlier groups wrote through the step buffer's mailbox."""
import ctypes as C

import numpy as np
import pytest

import oracle
from lattice_b200 import _lib
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


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _problem(case):
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LoraDesc
    qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
    lora, keep = None, [qw]
    if case["lora"] is not None:
        a, b, s = case["lora"]
        ad, bd = dev(a), dev(b)
        keep += [ad, bd]
        lora = LoraDesc(ad.data_ptr(), bd.data_ptr(), case["rank"], s)
    return qw, lora, keep


def test_independent_groups_without_a_step_buffer(be):
    """Three groups that do not depend on one another: one launch, every output against the oracle."""
    spec = [[(1024, 300, 16), (1024, 128, 0)], [(2048, 640, 8), (512, 1000, 16), (1024, 77, 4)], [(3072, 256, 16)]]
    groups, checks, keep = [], [], []
    e = 0
    for grp in spec:
        g = []
        for (k, n, r) in grp:
            case = make_case(3, 1, k, n, r, 2.0 * r, extra=200 + e)
            e += 1
            qw, lora, kp = _problem(case)
            keep += kp
            y = torch.full((n,), float("nan"), device="cuda")
            g.append((dev(case["x"]), qw, lora, y))
            checks.append((y, case))
        groups.append(g)
    step = be.prepare_step(groups)
    before = be.launch_count
    step()
    assert be.launch_count - before == 1
    be.check_device_status()
    for y, case in checks:
        assert tol_ratio(y.cpu().numpy().reshape(1, -1), case["y_ref"]) <= 1.0
    first = [y.clone() for y, _ in checks]
    step()                                                  # the same bits on a second launch
    be.check_device_status()
    assert all(torch.equal(a, y) for a, (y, _) in zip(first, checks))


def _chain_reference(cases, x0, links):
    """Oracle for a chain: problem i's input is x0 (link None) or the concatenated outputs listed in links[i]."""
    outs = []
    for case, link in zip(cases, links):
        x = x0[case["k"]] if link is None else np.concatenate([outs[j] for j in link]).reshape(1, -1)
        outs.append(oracle.q4_linear(x.astype(np.float32), case["payload"], 1, case["n"], case["k"], lora=case["lora"])[0])
    return outs


@pytest.mark.parametrize("rank", [0, 16])
def test_chained_groups_read_earlier_outputs_through_the_mailbox(be, rank):
    """group 0: A 1024->1280 and B 1024->768; group 1: C 2048->512 whose input is [A | B]'s row and D 1280->300
    whose input is A's row; group 2: E 512->1024 on C's row.  The GPU chain is compared with the oracle run on
    the GPU's own intermediate rows (same inputs), and end to end with a looser sanity bound."""
    from lattice_b200.sharded import StepBuffer
    shapes = [(1024, 1280), (1024, 768), (2048, 512), (1280, 300), (512, 1024)]
    cases = [make_case(3, 1, k, n, rank, 2.0 * rank, extra=300 + i) for i, (k, n) in enumerate(shapes)]
    probs = [_problem(c) for c in cases]
    buf = StepBuffer(4096)
    p = buf.payload
    ya, yb, yc, yd, ye = p[0:1280], p[1280:2048], p[2048:2560], p[2560:2860], p[3072:4096]
    x0 = dev(cases[0]["x"])
    groups = [[(x0, probs[0][0], probs[0][1], ya), (x0, probs[1][0], probs[1][1], yb)],
              [(p[0:2048], probs[2][0], probs[2][1], yc), (p[0:1280], probs[3][0], probs[3][1], yd)],
              [(p[2048:2560], probs[4][0], probs[4][1], ye)]]
    step = be.prepare_step(groups, buf, gathered=[])
    for rep in range(3):                                    # alternates the mailbox halves, reuses every slot
        p.fill_(float("nan"))
        before = be.launch_count
        step()
        assert be.launch_count - before == 1
        be.check_device_status()
        got = [t.cpu().numpy() for t in (ya, yb, yc, yd, ye)]
        assert all(np.isfinite(g).all() for g in got)
        # each projection against the oracle on the inputs the GPU actually had
        x_in = [cases[0]["x"], cases[0]["x"], np.concatenate([got[0], got[1]]).reshape(1, -1), got[0].reshape(1, -1),
                got[2].reshape(1, -1)]
        for c, x, g in zip(cases, x_in, got):
            ref = oracle.q4_linear(x.astype(np.float32), c["payload"], 1, c["n"], c["k"], lora=c["lora"])
            assert tol_ratio(g.reshape(1, -1), ref) <= 1.0
    # end to end against the pure oracle chain (errors of the stages compound; an order-of-magnitude check)
    outs = _chain_reference(cases, {1024: cases[0]["x"]}, [None, None, (0, 1), (0,), (2,)])
    assert tol_ratio(got[4].reshape(1, -1), outs[4].reshape(1, -1)) <= 8.0
    buf.close()


def test_step_publishes_into_every_rank_mailbox(be):
    """Two step buffers on one GPU stand in for two ranks' buffers: rank 0's launch writes its outputs into both
    mailboxes (plain stores, as it would over NVLink), tagged with the step; only its own columns are handed
    back here, so nothing waits for the absent second rank."""
    from lattice_b200.sharded import StepBuffer
    L = _lib.lib()
    case = make_case(3, 1, 1024, 256, 8, 16.0, extra=400)
    qw, lora, keep = _problem(case)
    own, peer = StepBuffer(1024), StepBuffer(1024)
    desc = _lib.GatherDesc(2, 0, (C.c_void_p * _lib.MAX_PEERS)(own.desc.bases[0], peer.desc.bases[0]))

    class Two:                                              # what prepare_step needs of a buffer
        pass
    two = Two()
    two.desc = desc
    y = own.payload[128:384]
    step = be.prepare_step([[(dev(case["x"]), qw, lora, y)]], two, gathered=[y])
    for launch in (1, 2):
        step()
        be.check_device_status()
        assert tol_ratio(y.cpu().numpy().reshape(1, -1), case["y_ref"]) <= 1.0
        # the peer's mailbox half for this step holds the same values with the step's tag
        half = launch & 1
        mbox_off = 256 + 1024 * 4                           # control block + payload (a multiple of 256 bytes)
        base = peer.desc.bases[0]
        from lattice_b200.sharded import _DeviceArray
        src = base + mbox_off + (half * 1024 + 128) * 8
        raw = torch.as_tensor(_DeviceArray(src, (512,), peer), device="cuda").view(torch.int32)
        raw = raw.cpu().numpy().reshape(256, 2)
        assert np.array_equal(raw[:, 0].view(np.float32), y.cpu().numpy())
        assert (raw[:, 1] == launch).all()
    own.close()
    peer.close()


def test_step_refuses_what_it_cannot_order(be):
    from lattice_b200.sharded import StepBuffer
    case = make_case(3, 1, 1024, 1024, 0, 0.0, extra=500)
    qw, lora, keep = _problem(case)
    buf = StepBuffer(2048)
    p = buf.payload
    x = dev(case["x"])
    # a projection reading what the same group writes
    with pytest.raises(_lib.Lq4Error) as e:
        be.prepare_step([[(x, qw, None, p[0:1024]), (p[0:1024], qw, None, p[1024:2048])]], buf, gathered=[])()
    assert e.value.status == _lib.ERR_SHAPE
    # an input taken from an earlier group that does not live in a step buffer
    y0 = torch.empty(1024, device="cuda")
    with pytest.raises(_lib.Lq4Error) as e:
        be.prepare_step([[(x, qw, None, y0)], [(y0, qw, None, p[0:1024])]], buf, gathered=[])()
    assert e.value.status == _lib.ERR_SHAPE
    # more than one token, a rotation: not a step
    args = _lib.LinearArgs(x.data_ptr(), 0, 2, 1024, 1024, qw.payload_ptr, p.data_ptr(), 0, None, None, 0, None, None)
    grp = _lib.StepGroup(C.cast(C.pointer(args), C.c_void_p).value, 1)
    assert _lib.lib().lq4_decode_step(be._ctx, C.byref(grp), 1, None, None) == _lib.ERR_SHAPE
    assert _lib.lib().lq4_decode_step(be._ctx, C.byref(grp), 9, None, None) == _lib.ERR_NOSPACE
    assert _lib.lib().lq4_decode_step(None, C.byref(grp), 1, None, None) == _lib.ERR_NULL
    buf.close()


def test_host_step_reads_pinned_inputs_and_writes_pinned_outputs(be):
    """lq4_decode_step_host: inputs in page-locked host memory (staged in by a kernel chained in front of the
    step kernel), outputs stored straight to page-locked host memory; the same bits as the device-buffer call,
    also after the host has changed the inputs between two launches, and with a chained second group."""
    from lattice_b200.sharded import StepBuffer
    spec = [[(1024, 300, 16), (2048, 640, 8)], [(1024, 512, 4), (2048, 77, 0)]]
    cases = [[make_case(3, 1, k, n, r, 2.0 * r, extra=400 + 10 * gi + i) for i, (k, n, r) in enumerate(grp)] for gi, grp in enumerate(spec)]
    # both groups share one input per k, as the projections of a layer do (staged once per distinct pointer)
    hx = {k: torch.from_numpy(np.ascontiguousarray(cases[0][i]["x"].reshape(-1))).pin_memory() for i, (k, _, _) in enumerate(spec[0])}
    dx = {k: v.cuda() for k, v in hx.items()}
    dev_groups, host_groups, outs, keep = [], [], [], []
    for gi, grp in enumerate(spec):
        dg, hg = [], []
        for i, (k, n, r) in enumerate(grp):
            qw, lora, kp = _problem(cases[gi][i])
            keep += kp
            yd = torch.full((n,), float("nan"), device="cuda")
            yh = torch.full((n,), float("nan")).pin_memory()
            dg.append((dx[k], qw, lora, yd))
            hg.append((hx[k], qw, lora, yh))
            outs.append((yd, yh))
        dev_groups.append(dg)
        host_groups.append(hg)
    on_dev, on_host = be.prepare_step(dev_groups), be.prepare_step(host_groups, host=True)
    on_dev()
    before = be.launch_count
    on_host()
    assert be.launch_count - before == 2                    # stage-in kernel + step kernel
    be.check_device_status()
    for yd, yh in outs:
        assert torch.equal(yd.cpu(), yh)
    for i in range(2):                                      # group 0 runs on its own cases' inputs: against the oracle
        assert tol_ratio(outs[i][1].numpy().reshape(1, -1), cases[0][i]["y_ref"]) <= 1.0
    # new activations written by the host between launches are what the next launch reads
    for k in hx:
        hx[k].mul_(-0.5)
        dx[k].copy_(hx[k])
    on_dev()
    on_host()
    be.check_device_status()
    for yd, yh in outs:
        assert torch.equal(yd.cpu(), yh)
    # a chained step: group 1 reads group 0's output through the step buffer; its own output goes to the host
    c0 = make_case(3, 1, 1024, 512, 16, 32.0, extra=470)
    c1 = make_case(3, 1, 512, 200, 8, 16.0, extra=471)
    q0, l0, k0 = _problem(c0)
    q1, l1, k1 = _problem(c1)
    sb = StepBuffer(512)
    hx0 = torch.from_numpy(np.ascontiguousarray(c0["x"].reshape(-1))).pin_memory()
    mid = sb.payload[:512]
    y_host = torch.full((200,), float("nan")).pin_memory()
    y_dev = torch.full((200,), float("nan"), device="cuda")
    chained_host = be.prepare_step([[(hx0, q0, l0, mid)], [(mid, q1, l1, y_host)]], sb, gathered=[], host=True)
    chained_dev = be.prepare_step([[(hx0.cuda(), q0, l0, mid)], [(mid, q1, l1, y_dev)]], sb, gathered=[])
    chained_dev()
    chained_host()
    be.check_device_status()
    assert torch.equal(y_dev.cpu(), y_host)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_steps_match_the_oracle(be, seed):
    """Seeded random steps (1-3 groups of 1-4 projections, ragged n, k from one to 34 granules per tile, adapters of
    rank 0-64): every output against the oracle.  Exercises the cut of the work units into CTA shares where tiles
    are few, shares are a handful of units and some CTAs get nothing."""
    rng = np.random.default_rng(seed)
    groups, checks, keep = [], [], []
    e = 0
    for _ in range(int(rng.integers(1, 4))):
        g = []
        for _ in range(int(rng.integers(1, 5))):
            k = 128 * int(rng.choice([1, 2, 3, 8, 17, 34]))
            n = int(rng.choice([1, 77, 128, 129, 640, 1000, 2500]))
            r = int(rng.choice([0, 4, 16, 64]))
            case = make_case(3, 1, k, n, r, 2.0 * max(r, 1), extra=600 + 37 * seed + e)
            e += 1
            qw, lora, kp = _problem(case)
            keep += kp
            y = torch.full((n,), float("nan"), device="cuda")
            g.append((dev(case["x"]), qw, lora, y))
            checks.append((y, case))
        groups.append(g)
    step = be.prepare_step(groups)
    step()
    be.check_device_status()
    for y, case in checks:
        assert tol_ratio(y.cpu().numpy().reshape(1, -1), case["y_ref"]) <= 1.0, (case["n"], case["k"], case["rank"])
    first = [y.clone() for y, _ in checks]
    step()
    be.check_device_status()
    assert all(torch.equal(a, y) for a, (y, _) in zip(first, checks))


def test_a_group_of_twelve_projections_is_one_launch(be):
    """lq4_linear_group with 9 to 24 one-token projections runs them as one group of the step kernel: ONE launch,
    every output against the oracle; a group that does not qualify (a rotated member) still runs problem by
    problem with the same results."""
    shapes = [(1024, 300, 16), (1024, 128, 0), (2048, 640, 8), (512, 1000, 16), (1024, 77, 4), (3072, 256, 16),
              (1024, 512, 0), (2048, 129, 64), (512, 2500, 4), (1024, 640, 16), (2048, 300, 0), (1024, 1000, 8)]
    problems, outs, checks, keep = [], [], [], []
    for i, (k, n, r) in enumerate(shapes):
        case = make_case(3, 1, k, n, r, 2.0 * max(r, 1), extra=700 + i)
        qw, lora, kp = _problem(case)
        keep += kp
        y = torch.full((1, n), float("nan"), device="cuda")
        problems.append((dev(case["x"]), qw, lora))
        outs.append(y)
        checks.append((y, case))
    before = be.launch_count
    be.linear_group(problems, outs)
    assert be.launch_count - before == 1
    be.check_device_status()
    for y, case in checks:
        assert tol_ratio(y.cpu().numpy().reshape(1, -1), case["y_ref"]) <= 1.0


def test_host_step_refuses_pageable_memory(be):
    """A pointer the device cannot address must not reach a kernel: pageable host tensors are refused."""
    from lattice_b200 import _lib as L
    from lattice_b200._lib import LinearArgs, StepGroup
    case = make_case(3, 1, 1024, 128, 0, 0.0, extra=480)
    qw, _, keep = _problem(case)
    x_pinned = torch.from_numpy(np.ascontiguousarray(case["x"].reshape(-1))).pin_memory()
    x_pageable = torch.from_numpy(np.ascontiguousarray(case["x"].reshape(-1)).copy())
    y_pinned = torch.zeros(128).pin_memory()
    y_pageable = torch.zeros(128)
    for x, y in ((x_pageable, y_pinned), (x_pinned, y_pageable)):
        arr = (LinearArgs * 1)()
        arr[0] = LinearArgs(x.data_ptr(), L.DTYPE_F32, 1, 128, 1024, qw.payload_ptr, y.data_ptr(), 0, None, None, L.PATH_AUTO, None, None)
        grp = (StepGroup * 1)()
        grp[0] = StepGroup(C.cast(arr, C.c_void_p).value, 1)
        rc = L.lib().lq4_decode_step_host(be._ctx, C.cast(grp, C.c_void_p), 1, None, None)
        assert rc == L.ERR_UNSUPPORTED
    be.check_device_status()


def test_repeated_step_reuses_its_plan_and_a_changed_argument_replans(be):
    """The library keeps the last step's argument block: the same call again gives the same bits, and a call that
    differs in one pointer, one adapter scale or one group size is planned afresh (checked against the oracle)."""
    from lattice_b200._lib import LoraDesc
    c0 = make_case(3, 1, 1024, 300, 16, 32.0, extra=800)
    c1 = make_case(3, 1, 2048, 640, 8, 16.0, extra=801)
    q0, l0, k0 = _problem(c0)
    q1, l1, k1 = _problem(c1)
    x0, x1 = dev(c0["x"]), dev(c1["x"])
    ya, yb = torch.zeros(300, device="cuda"), torch.zeros(640, device="cuda")
    step = be.prepare_step([[(x0, q0, l0, ya), (x1, q1, l1, yb)]])
    step(); step()
    be.check_device_status()
    assert tol_ratio(ya.cpu().numpy().reshape(1, -1), c0["y_ref"]) <= 1.0
    assert tol_ratio(yb.cpu().numpy().reshape(1, -1), c1["y_ref"]) <= 1.0
    # another output pointer for the first problem
    ya2 = torch.full((300,), float("nan"), device="cuda")
    be.prepare_step([[(x0, q0, l0, ya2), (x1, q1, l1, yb)]])()
    be.check_device_status()
    assert torch.equal(ya2, ya)
    # the same pointers, the adapter's scale doubled in place: the result must follow
    a, b, s = c0["lora"]
    l0.scale = 2.0 * s
    ya.fill_(float("nan"))
    step()
    be.check_device_status()
    ref = oracle.q4_linear(c0["x"], None, 1, 300, 1024, lora=(a, b, 2.0 * s), w_f32=c0["w_deq"])
    assert tol_ratio(ya.cpu().numpy().reshape(1, -1), ref) <= 1.0
    l0.scale = s
    # the same two problems as two groups of one
    ya.fill_(float("nan")); yb.fill_(float("nan"))
    be.prepare_step([[(x0, q0, l0, ya)], [(x1, q1, l1, yb)]])()
    be.check_device_status()
    assert tol_ratio(ya.cpu().numpy().reshape(1, -1), c0["y_ref"]) <= 1.0
    assert tol_ratio(yb.cpu().numpy().reshape(1, -1), c1["y_ref"]) <= 1.0
