"""GPU: bit-exact parity of every kernel family with the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import int4linear_b200 as L
from conftest import golden_files, make_case
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def run_device(cuda, xp, wp, k, path=L.PATH_AUTO, tile_n=0, direct=False, pairs=-1, two_pass=0):
    """Upload packed operands, run one blocking launch through the C ABI, download Y."""
    import torch
    xd = torch.from_numpy(xp).to(cuda)
    wd = torch.from_numpy(wp).to(cuda)
    m, n = xp.shape[0], wp.shape[0]
    yd = torch.full((m, n), -12345, dtype=torch.int32, device=cuda)
    prev = L.set_path(path)
    L.set_tuning(tile_n, direct, pairs)
    L.set_two_pass(two_pass)
    try:
        L.linear_v21_launch(xd, wd, yd, m, n, k)
    finally:
        L.set_path(prev)
        L.set_tuning(0, False, -1)
        L.set_two_pass(-1)
    return yd.cpu().numpy()


VARIANTS = [
    ("tcgen05-256-tma", dict(path=L.PATH_TCGEN05, tile_n=256, direct=False)),
    ("tcgen05-256-direct", dict(path=L.PATH_TCGEN05, tile_n=256, direct=True)),
    ("tcgen05-128-tma", dict(path=L.PATH_TCGEN05, tile_n=128, direct=False)),
    ("tcgen05-64-direct", dict(path=L.PATH_TCGEN05, tile_n=64, direct=True)),
    ("tcgen05-pairs-tma", dict(path=L.PATH_TCGEN05, pairs=1)),
    ("tcgen05-pairs-direct", dict(path=L.PATH_TCGEN05, pairs=1, direct=True)),
    ("two-pass-tma", dict(path=L.PATH_TCGEN05, two_pass=1)),
    ("two-pass-direct", dict(path=L.PATH_TCGEN05, two_pass=1, direct=True)),
    ("legacy", dict(path=L.PATH_LEGACY)),
    ("auto", dict(path=L.PATH_AUTO)),
]


@pytest.mark.parametrize("vname,variant", VARIANTS, ids=[v[0] for v in VARIANTS])
@pytest.mark.parametrize("path", golden_files(), ids=lambda p: p.split("/")[-1][:-4])
def test_golden_vectors(cuda, path, vname, variant):
    g = np.load(path)
    k = g["x"].shape[1]
    if k % 32:
        pytest.skip("k % 32 != 0 is outside the device contract")
    xp = g["x_packed"].view(np.uint8).reshape(g["x"].shape[0], -1)
    wp = g["w_packed"].view(np.uint8).reshape(g["w"].shape[0], -1)
    y = run_device(cuda, xp, wp, k, **variant)
    assert O.is_same(y, g["y"])


# (m, n, k): M/N/K tails around every tile size, the reference's edge cases
# (rows predicated at tile edges, K tail at 32-element granularity) and odd N.
TAIL_SHAPES = [
    (1, 2, 32), (16, 130, 96), (17, 14, 128), (255, 258, 160), (257, 130, 32),
    (128, 256, 128), (129, 257, 224), (300, 77, 416), (64, 1000, 1056), (384, 512, 2048),
    # several output chunks of the last tile fall outside Y (staging-buffer rotation)
    (1024, 1024, 1024), (520, 36, 256),
]


@pytest.mark.parametrize("vname,variant", VARIANTS, ids=[v[0] for v in VARIANTS])
@pytest.mark.parametrize("shape", TAIL_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tail_shapes(cuda, shape, vname, variant):
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=m + n + k)
    y = run_device(cuda, xp, wp, k, **variant)
    ref = O.linear_ref(x.astype(np.int32), w.astype(np.int32))
    assert O.is_same(y, ref)


@pytest.mark.parametrize("shape", [(1, 8, 32), (16, 14336, 4096), (7, 100, 992), (32, 520, 1024), (64, 264, 2048), (48, 8, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_skinny_kernel(cuda, shape):
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=9)
    # up to 32 rows the register kernels (from 17 rows on only while the weights are small)
    assert L.path_for(m, n, k) == (L.PATH_SKINNY if m <= 32 else L.PATH_TCGEN05)
    y = run_device(cuda, xp, wp, k, path=L.PATH_SKINNY)
    ref = O.linear_ref_sgemm(x, w) if m * n * k > 2e8 else O.linear_ref(x.astype(np.int32), w.astype(np.int32))
    assert O.is_same(y, ref)
    # the tensor-memory family must agree on the same inputs
    y2 = run_device(cuda, xp, wp, k, path=L.PATH_TCGEN05)
    assert O.is_same(y2, ref)


def test_extreme_values_closed_form(cuda):
    """All -8 times all -8 is the largest accumulator the format can produce: 64*K per element."""
    for k in (128, 8192, 65536, 131040):  # 131040 is the largest K the 256-fold scaled accumulator allows
        m, n = 130, 72
        xp = np.full((m, k // 2), 0x88, dtype=np.uint8)
        wp = np.full((n, k // 2), 0x88, dtype=np.uint8)
        for path in (L.PATH_TCGEN05, L.PATH_LEGACY):
            y = run_device(cuda, xp, wp, k, path=path)
            assert (y == 64 * k).all()
        wp7 = np.full((n, k // 2), 0x77, dtype=np.uint8)
        y = run_device(cuda, xp, wp7, k, path=L.PATH_TCGEN05)
        assert (y == -56 * k).all()


def test_single_nonzero_positions(cuda):
    """One non-zero per row at varying K positions: any K permutation that differs between
    the operands, or a swizzle slip, shows up as a wrong or missing product."""
    m, n, k = 128, 256, 512
    x = np.zeros((m, k), np.int8)
    w = np.zeros((n, k), np.int8)
    for i in range(m):
        x[i, (37 * i + 11) % k] = (i % 15) - 7 or 3
    for j in range(n):
        w[j, (37 * j + 11) % k] = -8 if j % 2 else 7
    ref = x.astype(np.int32) @ w.astype(np.int32).T
    for path in (L.PATH_TCGEN05, L.PATH_LEGACY):
        y = run_device(cuda, L.pack_bytes(x), L.pack_bytes(w), k, path=path)
        assert O.is_same(y, ref)


def test_repeatable(cuda):
    """Integer arithmetic: two runs must agree bit for bit, anything else is a race."""
    m, n, k = 512, 768, 1024
    x, w, xp, wp = make_case(m, n, k, seed=4)
    a = run_device(cuda, xp, wp, k)
    b = run_device(cuda, xp, wp, k)
    assert O.is_same(a, b)


def test_host_buffer_entry_point(cuda):
    m, n, k = 100, 300, 256
    x, w, xp, wp = make_case(m, n, k, seed=2)
    ref = O.linear_ref(x.astype(np.int32), w.astype(np.int32))
    before = L.launch_count()
    y = L.linear_host(xp, wp, k)
    assert O.is_same(y, ref)
    # weights declared resident: same result without re-uploading them
    x2 = L.uniform_s4(77, m, k)
    y2 = L.linear_host(L.pack_bytes(x2), wp, k, w_resident=True)
    assert O.is_same(y2, O.linear_ref(x2.astype(np.int32), w.astype(np.int32)))
    assert L.launch_count() == before + 2


def test_host_buffer_entry_point_pipelined(cuda):
    """Large host-buffer calls run as row blocks on three streams (upload / GEMM / download); the
    last block here is ragged and the weights are declared resident on the second call."""
    m, n, k = 2148, 2048, 256
    x, w, xp, wp = make_case(m, n, k, seed=14)
    y = L.linear_host(xp, wp, k)
    assert O.is_same(y, O.linear_ref_sgemm(x, w))
    x2 = L.uniform_s4(78, m, k)
    y2 = L.linear_host(L.pack_bytes(x2), wp, k, w_resident=True)
    assert O.is_same(y2, O.linear_ref_sgemm(x2, w))
    assert L.last_status() == 0


@pytest.mark.parametrize("m,n,k", [(2148, 2500, 256), (1100, 4099, 128), (4096, 1024, 128)])
def test_host_buffer_entry_point_chunked_start(cuda, m, n, k):
    """With weights to upload, the first row block is computed in four column chunks of W (compact
    slabs, strided download): ragged last chunk, odd n, the smallest n that is chunked."""
    x, w, xp, wp = make_case(m, n, k, seed=15)
    y = L.linear_host(xp, wp, k)
    assert O.is_same(y, O.linear_ref_sgemm(x, w))
    assert L.last_status() == 0


def test_host_buffer_entry_point_with_two_pass(cuda):
    """The host-buffer entry point must work when the dispatcher takes the two-pass path (it keeps
    its own staging lock while the two-pass scratch is looked up)."""
    m, n, k = 300, 264, 256
    x, w, xp, wp = make_case(m, n, k, seed=8)
    L.set_two_pass(1)
    try:
        y = L.linear_host(xp, wp, k)
    finally:
        L.set_two_pass(-1)
    assert O.is_same(y, O.linear_ref(x.astype(np.int32), w.astype(np.int32)))


def test_tensor_front_end(cuda):
    import torch
    m, n, k = 96, 160, 384
    x, w, xp, wp = make_case(m, n, k, seed=6)
    y = L.linear(torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda))
    torch.cuda.synchronize()
    assert L.last_status() == 0
    assert O.is_same(y.cpu().numpy(), O.linear_ref(x.astype(np.int32), w.astype(np.int32)))


@pytest.mark.parametrize("mode", [1, 2])
def test_overlapped_launches_stay_exact(cuda, mode):
    """Back-to-back decode launches with programmatic dependent launch enabled: every launch of the
    chain must still produce the exact result (distinct weights per launch, one shared Y buffer that
    each launch overwrites, and a result snapshot taken between launches on the same stream)."""
    import torch
    m, n, k = 16, 2368, 4096
    x = L.uniform_s4(31, m, k)
    xd = torch.from_numpy(L.pack_bytes(x)).to(cuda)
    ws = [L.uniform_s4(40 + i, n, k) for i in range(4)]
    wds = [torch.from_numpy(L.pack_bytes(w)).to(cuda) for w in ws]
    yd = torch.empty((m, n), dtype=torch.int32, device=cuda)
    prev = L.set_overlap(mode)
    try:
        outs = []
        for rep in range(3):
            for wd in wds:
                L.linear(xd, wd, out=yd)
                outs.append(yd.clone())
        torch.cuda.synchronize()
    finally:
        L.set_overlap(prev)
    assert L.last_status() == 0
    refs = [O.linear_ref_sgemm(x, w) for w in ws]
    for i, out in enumerate(outs):
        assert O.is_same(out.cpu().numpy(), refs[i % 4]), f"launch {i}"


@pytest.mark.parametrize("shape,variant", [
    ((300, 520, 256), dict(path=L.PATH_TCGEN05, pairs=1)),
    ((300, 520, 256), dict(path=L.PATH_TCGEN05, pairs=1, direct=True)),
    ((200, 77, 160), dict(path=L.PATH_TCGEN05, pairs=0)),
    ((16, 1000, 4096), dict(path=L.PATH_SKINNY)),
    ((40, 264, 1024), dict(path=L.PATH_SKINNY)),
    ((9, 64, 96), dict(path=L.PATH_SKINNY)),
    ((130, 70, 128), dict(path=L.PATH_LEGACY)),
], ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else "-".join(f"{k}{x}" for k, x in v.items()))
def test_fused_bias_is_exact(cuda, shape, variant):
    import torch
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=21)
    bias = (np.arange(n, dtype=np.int64) * 7919 % 200001 - 100000).astype(np.int32)
    prev = L.set_path(variant.get("path", L.PATH_AUTO))
    L.set_tuning(0, variant.get("direct", False), variant.get("pairs", -1))
    try:
        y = L.linear(torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda), bias=torch.from_numpy(bias).to(cuda))
        torch.cuda.synchronize()
    finally:
        L.set_path(prev)
        L.set_tuning(0, False, -1)
    assert L.last_status() == 0
    want = O.linear_ref(x.astype(np.int32), w.astype(np.int32)) + bias[None, :]
    assert O.is_same(y.cpu().numpy(), want)


@pytest.mark.parametrize("shape", [(300, 520, 256), (128, 256, 128), (1024, 1024, 1024), (100, 77, 96), (513, 130, 1056), (16, 264, 512)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("direct", [False, True], ids=["tma", "direct"])
def test_prepared_weights_path(cuda, shape, direct):
    """Weights expanded once by int4_linear_prepare_weights, then used in place of the packed ones."""
    import torch
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=33)
    wd = torch.from_numpy(wp).to(cuda)
    we = L.prepare_weights(wd)
    torch.cuda.synchronize()
    # the expansion itself: 16 even elements then 16 odd ones of every 32, each times 16
    w32 = w.reshape(n, k // 32, 32).astype(np.int16) * 16
    want_bytes = np.concatenate([w32[:, :, 0::2], w32[:, :, 1::2]], axis=2).reshape(n, k).astype(np.int8)
    assert np.array_equal(we.cpu().numpy().view(np.int8), want_bytes)
    bias = (np.arange(n, dtype=np.int32) % 97) - 48
    L.set_tuning(0, direct, -1)
    try:
        y = L.linear_prepared(torch.from_numpy(xp).to(cuda), we)
        yb = L.linear_prepared(torch.from_numpy(xp).to(cuda), we, bias=torch.from_numpy(bias).to(cuda))
        torch.cuda.synchronize()
    finally:
        L.set_tuning(0, False, -1)
    assert L.last_status() == 0
    ref = O.linear_ref(x.astype(np.int32), w.astype(np.int32))
    assert O.is_same(y.cpu().numpy(), ref)
    assert O.is_same(yb.cpu().numpy(), ref + bias[None, :])


@pytest.mark.parametrize("shape", [(300, 520, 256), (1024, 1024, 512), (64, 72, 96), (257, 130, 1056), (4096, 4096, 1024), (515, 1096, 128),
                                   # decode shapes: the streaming kernels write the scaled output themselves
                                   (16, 1024, 4096), (8, 264, 2048), (16, 512, 8192), (32, 520, 256), (5, 77, 96)],
                         ids=lambda s: "x".join(map(str, s)))
def test_scaled_bf16_epilogue(cuda, shape):
    """Dequantising epilogue: bf16(float(acc) * row_scale * col_scale + bias).  The integer part is
    exact, so the only freedom is the float arithmetic (one multiply, one fused multiply-add) and
    the final rounding to bfloat16: tolerance one bf16 unit in the last place (2^-7 relative)."""
    import torch
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=51)
    rng = np.random.default_rng(7)
    rs = rng.uniform(0.01, 0.1, size=m).astype(np.float32)
    cs = rng.uniform(0.005, 0.05, size=n).astype(np.float32)
    b = rng.uniform(-1, 1, size=n).astype(np.float32)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    acc = O.linear_ref_sgemm(x, w).astype(np.float32)
    for use in [(True, True, True), (False, True, False), (False, False, False)]:
        args = [torch.from_numpy(v).to(cuda) if u else None for v, u in zip((rs, cs, b), use)]
        y = L.linear_scaled(xd, wd, *args)
        torch.cuda.synchronize()
        assert L.last_status() == 0
        ref = acc * (rs[:, None] if use[0] else 1.0) * (cs[None, :] if use[1] else 1.0) + (b[None, :] if use[2] else 0.0)
        got = y.float().cpu().numpy()
        tol = np.abs(ref) * 2.0 ** -7 + 1e-6
        assert np.all(np.abs(got - ref) <= tol), float(np.max(np.abs(got - ref) / (np.abs(ref) + 1e-6)))
    # unscaled: bf16 of the exact integers (all |acc| here are exactly representable up to rounding)
    exact = torch.from_numpy(acc).to(torch.bfloat16).float().numpy()
    assert np.array_equal(got, exact)
    # The per-thread-store epilogue (forced here; taken by itself when n % 8 != 0) and the
    # TMA-store one do the same arithmetic, so their results must be identical.
    full = [torch.from_numpy(v).to(cuda) for v in (rs, cs, b)]
    y_tma = L.linear_scaled(xd, wd, *full)
    L.set_tuning(0, True, -1)
    try:
        y_direct = L.linear_scaled(xd, wd, *full)
        torch.cuda.synchronize()
    finally:
        L.set_tuning(0, False, -1)
    assert torch.equal(y_tma, y_direct)
    # Whatever kernel family the dispatcher picks (decode shapes go to the streaming kernels), the
    # tensor-memory family must give the same bits.
    L.set_path(L.PATH_TCGEN05)
    try:
        y_tc = L.linear_scaled(xd, wd, *full)
        torch.cuda.synchronize()
    finally:
        L.set_path(L.PATH_AUTO)
    assert torch.equal(y_tma, y_tc)
    # IEEE half output: same arithmetic, rounding to 11 significant bits instead of 8.
    y_half = L.linear_scaled(xd, wd, *full, dtype=torch.float16)
    torch.cuda.synchronize()
    ref = acc * rs[:, None] * cs[None, :] + b[None, :]
    got = y_half.float().cpu().numpy()
    assert y_half.dtype == torch.float16
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -10 + 1e-3), float(np.max(np.abs(got - ref)))


def test_bounded_wait_reports_and_recovers(cuda):
    """Failure handling without a fault: a wait that can never be satisfied runs out after its
    budget, the kernel returns, the status word says so once, and the next launch works."""
    import time
    import torch
    from int4linear_b200 import _lib
    lib = _lib.load()
    assert lib.int4_linear_last_status() == 0
    t0 = time.perf_counter()
    assert lib.int4_linear_selftest_timeout(20) == 0
    assert time.perf_counter() - t0 < 2.0           # came back by itself, promptly
    assert lib.int4_linear_last_status() == 5       # INT4L_ERR_DEVICE_TIMEOUT, reported ...
    assert lib.int4_linear_selftest_timeout(0) == 1 # (argument check)
    m, n, k = 200, 136, 160
    x, w, xp, wp = make_case(m, n, k, seed=3)
    y = L.linear(torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda))
    torch.cuda.synchronize()
    assert lib.int4_linear_last_status() == 0       # ... once; the device is still usable
    assert O.is_same(y.cpu().numpy(), O.linear_ref(x.astype(np.int32), w.astype(np.int32)))


def test_random_shapes_through_the_dispatcher(cuda):
    """Seeded random shapes through the automatic path/tile choice (pairs, the three single-CTA
    tile widths, tail splitting, the decode kernels, TMA and per-thread stores), each bit-exact
    against the oracle."""
    rng = np.random.default_rng(20240607)
    shapes = []
    for _ in range(48):
        m = int(rng.choice([rng.integers(1, 40), rng.integers(40, 300), rng.integers(300, 1400)]))
        n = int(rng.choice([rng.integers(1, 64), rng.integers(64, 600), rng.integers(600, 2600)]))
        k = 32 * int(rng.integers(1, 48))
        shapes.append((m, n, k))
    for i, (m, n, k) in enumerate(shapes):
        x, w, xp, wp = make_case(m, n, k, seed=200 + i)
        y = run_device(cuda, xp, wp, k)
        ref = O.linear_ref_sgemm(x, w) if m * n * k > 2e8 else O.linear_ref(x.astype(np.int32), w.astype(np.int32))
        assert O.is_same(y, ref), (m, n, k)
    assert L.last_status() == 0


def test_concurrent_host_threads_on_their_own_streams(cuda):
    """Four host threads launch different shapes on their own streams at the same time (shared
    per-device context, tensor-map cache and launch counter behind the library's locks); every
    result must be exact."""
    import threading
    import torch
    shapes = [(300, 520, 256), (16, 1024, 4096), (1024, 1024, 512), (257, 130, 1056)]
    cases = []
    for i, (m, n, k) in enumerate(shapes):
        x, w, xp, wp = make_case(m, n, k, seed=300 + i)
        ref = O.linear_ref_sgemm(x, w) if m * n * k > 2e8 else O.linear_ref(x.astype(np.int32), w.astype(np.int32))
        cases.append((torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda), k, ref))
    torch.cuda.synchronize()
    errors = []

    def worker(idx):
        try:
            xd, wd, k, ref = cases[idx]
            stream = torch.cuda.Stream(device=cuda)
            with torch.cuda.stream(stream):
                for _ in range(25):
                    y = L.linear(xd, wd, k=k)
                stream.synchronize()
            if not O.is_same(y.cpu().numpy(), ref):
                errors.append(f"thread {idx}: wrong result")
        except Exception as e:  # noqa: BLE001
            errors.append(f"thread {idx}: {e!r}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(cases))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert L.last_status() == 0


@pytest.mark.parametrize("shape", [(300, 520, 256), (1024, 1024, 1024), (64, 72, 96)], ids=lambda s: "x".join(map(str, s)))
def test_both_operands_pre_expanded(cuda, shape):
    """int4_linear_launch_expanded_async: X and W expanded once by the prepare call, then the
    pure 8-bit GEMM; same bits as the packed path."""
    import torch
    m, n, k = shape
    x, w, xp, wp = make_case(m, n, k, seed=31)
    xd, wd = torch.from_numpy(xp).to(cuda), torch.from_numpy(wp).to(cuda)
    xe, we = L.prepare_weights(xd), L.prepare_weights(wd)
    assert xe.shape == (m, k) and we.shape == (n, k)
    y = L.linear_expanded(xe, we)
    torch.cuda.synchronize()
    assert L.last_status() == 0
    assert O.is_same(y.cpu().numpy(), O.linear_ref(x.astype(np.int32), w.astype(np.int32)))


def test_empty_shard_returns_an_empty_result(cuda):
    """A rank whose shard of W has no rows (more ranks than 256-row units) gets an [m, 0] result
    and launches nothing."""
    import torch
    xd = torch.zeros((64, 64), dtype=torch.uint8, device=cuda)
    wd = torch.zeros((0, 64), dtype=torch.uint8, device=cuda)
    before = L.launch_count()
    y = L.linear(xd, wd)
    assert tuple(y.shape) == (64, 0) and y.dtype == torch.int32
    assert L.launch_count() == before


@pytest.mark.parametrize("promises", [(False, False), (True, False), (True, True)], ids=["none", "weights", "weights+x"])
def test_decode_launches_with_per_call_promises(cuda, promises):
    """int4_linear_decode_launch_async: the launch-overlap promise given per call instead of through
    the process-wide switch.  A chain of launches over distinct weights into one Y buffer, a
    snapshot after each: every result exact, with a bias, and X produced on the same stream just
    before the first launch when X is not promised."""
    import torch
    weights_stationary, x_not_pending = promises
    m, n, k = 12, 3080, 4096
    x = L.uniform_s4(51, m, k)
    ws = [L.uniform_s4(60 + i, n, k) for i in range(3)]
    wds = [torch.from_numpy(L.pack_bytes(w)).to(cuda) for w in ws]
    bias = torch.from_numpy(((np.arange(n) * 13) % 801 - 400).astype(np.int32)).to(cuda)
    x_src = torch.from_numpy(L.pack_bytes(x)).to(cuda)
    xd = torch.zeros_like(x_src)
    yd = torch.empty((m, n), dtype=torch.int32, device=cuda)
    if x_not_pending:
        xd.copy_(x_src)
        torch.cuda.synchronize()
    outs = []
    for rep in range(3):
        if not x_not_pending:
            xd.copy_(x_src)  # X is written by work queued right in front of the launch
        for wd in wds:
            L.linear_decode(xd, wd, out=yd, bias=bias, weights_stationary=weights_stationary, x_not_pending=x_not_pending)
            outs.append(yd.clone())
    torch.cuda.synchronize()
    assert L.last_status() == 0
    refs = [O.linear_ref_sgemm(x, w) + bias.cpu().numpy()[None, :] for w in ws]
    for i, out in enumerate(outs):
        assert O.is_same(out.cpu().numpy(), refs[i % 3]), f"launch {i}"
    lib = _lib_for_args()
    p = xd.data_ptr()
    assert lib.int4_linear_decode_launch_async(p, p, None, p, 8, 8, 32, 2, None) == 1   # X promised without W
    assert lib.int4_linear_decode_launch_async(p, p, None, p, 8, 8, 32, 4, None) == 1


def _lib_for_args():
    from int4linear_b200 import _lib
    return _lib.load()


@pytest.mark.parametrize("m", [33, 64, 96, 128])
@pytest.mark.parametrize("n,k", [(264, 1024), (264, 4096), (14336, 1024), (14336, 4096)])
def test_a_few_dozen_rows(cuda, m, n, k):
    """33 <= M <= 128 (a batch of decode requests, a short prefill): a single row block of tiles.
    Automatic dispatch and the forced tile widths."""
    x, w, xp, wp = make_case(m, n, k, seed=17)
    ref = O.linear_ref_sgemm(x, w) if m * n * k > 2e8 else O.linear_ref(x.astype(np.int32), w.astype(np.int32))
    assert L.path_for(m, n, k) == L.PATH_TCGEN05
    assert O.is_same(run_device(cuda, xp, wp, k), ref)
    for tile_n in (128, 256):
        assert O.is_same(run_device(cuda, xp, wp, k, path=L.PATH_TCGEN05, tile_n=tile_n), ref), f"tile_n={tile_n}"
