"""Each kernel alone against its plain reference (tests/kernel_refs.py), at
sizes other than the engine's tiny configurations: widths and vocabularies
that are no power of two, head sizes in steps of 16, several head groupings.
Where random data would hide a fault the inputs are made so that it shows: one
far key that takes all the softmax weight, a key just inside and just outside
a window, keys on both sides of a page's edge, scrambled page tables."""

from __future__ import annotations

import math

import pytest
import torch

import kernel_refs as R

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def K():
    from litinfer_b200 import kernels
    return kernels


def dev():
    return torch.device("cuda:0")


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(dev())


def close(got, ref, dtype, what="", f32_tol=2e-5, scale=None):
    got, ref = got.float(), ref.float()
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    s = float(ref.abs().max()) if scale is None else scale
    tol = f32_tol * max(s, 1.0) if dtype == torch.float32 else (2.0 ** -7) * max(s, 1e-3)
    err = float((got - ref).abs().max())
    assert err <= tol, f"{what}: max |diff| {err:.3e} > {tol:.3e} (scale {s:.3f})"


# --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    V, H, T = 77, 100, 9
    table = rnd(V, H, dtype=dtype, seed=1)
    ids = torch.tensor([0, 76, 5, 5, 31, 2, 76, 0, 40], dtype=torch.int32, device=dev())
    out = torch.empty(T, H, dtype=torch.float32, device=dev())
    K().embedding(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [80, 1536, 3000])
def test_rmsnorm_family(dtype, H):
    T = 7
    x = rnd(T, H, seed=2, scale=3.0)
    w = 1 + 0.1 * rnd(H, seed=3)
    eps = 1e-5
    out = torch.empty(T, H, dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    K().rmsnorm(x, w, eps, out)
    R.rmsnorm(x, w, eps, ref)
    close(out, ref, dtype, "rmsnorm")
    delta = rnd(T, H, dtype=dtype, seed=4)
    x1, x2 = x.clone(), x.clone()
    K().add_rmsnorm(x1, delta, w, eps, out)
    R.add_rmsnorm(x2, delta, w, eps, ref)
    close(x1, x2, torch.float32, "add_rmsnorm residual")
    close(out, ref, dtype, "add_rmsnorm output")
    rows = torch.tensor([6, 0, 3, 3], dtype=torch.int32, device=dev())
    out = torch.empty(4, H, dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    K().gather_rmsnorm(x, rows, w, eps, out)
    R.gather_rmsnorm(x, rows, w, eps, ref)
    close(out, ref, dtype, "gather_rmsnorm")
    x1, x2 = x.clone(), x.clone()
    K().residual_add(x1, delta)
    R.residual_add(x2, delta)
    assert torch.equal(x1, x2)


def test_table_gather_applies_changes_and_copies_rows():
    """The resident block tables: changes of the step's slots applied (others' and out-of-range ones ignored, the last
    row never written), each sequence's row copied out, the sink page beyond the row's width; twice gives the same."""
    g = torch.Generator().manual_seed(12)
    rows, cols, trash = 9, 37, 500
    resident = torch.randint(0, 400, (rows, cols), generator=g, dtype=torch.int32)
    resident[rows - 1] = trash
    slots = torch.tensor([3, 0, 8, 3, 5, 77], dtype=torch.int32)
    triples = [(3, 0, 11), (3, 36, 12), (0, 5, 13), (4, 2, 14), (5, 40, 15), (8, 1, 16), (5, 7, 17), (3, 9, trash)]
    cap = 12
    updates = torch.zeros(1 + 3 * cap, dtype=torch.int32)
    updates[0] = len(triples)
    updates[1:1 + 3 * len(triples)] = torch.tensor(triples, dtype=torch.int32).reshape(-1)
    for mb in (5, 37, 50):
        want_res, want_out = resident.clone(), torch.empty(len(slots), mb, dtype=torch.int32)
        R.table_gather(want_res, updates, slots, want_out, trash)
        got_res, got_out = resident.clone().to(dev()), torch.empty(len(slots), mb, dtype=torch.int32, device=dev())
        for _ in range(2):
            K().table_gather(got_res, updates.to(dev()), slots.to(dev()), got_out, trash)
            assert torch.equal(got_out.cpu(), want_out) and torch.equal(got_res.cpu(), want_res)
        assert int(want_res[4, 2]) == int(resident[4, 2]), "a slot that is not in the step is left alone"
        assert torch.equal(want_out[2], torch.full((mb,), trash, dtype=torch.int32)), "the padding sequences' row is all sink page"


def test_gather_rows_scale_and_logit_cap():
    k = K()
    g = torch.Generator().manual_seed(9)
    src = torch.randn(37, 4099, generator=g).to(dev())
    rows = torch.tensor([36, 0, 5, 5, 17], dtype=torch.int32, device=dev())
    out = torch.empty(5, 4099, dtype=torch.float32, device=dev())
    k.gather_rows(src, rows, out)
    assert torch.equal(out, src[rows.long()])
    x = src.clone()
    k.scale_inplace(x, 3.0)
    assert torch.equal(x, src * 3.0)
    y = (src * 4).clone()
    k.logit_cap(y, 2.5)
    ref = (src * 4).clone()
    R.logit_cap(ref, 2.5)
    assert (y - ref).abs().max() < 1e-6 and float(y.abs().max()) <= 2.5


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    T, I = 5, 272
    gu = rnd(T, 2 * I, dtype=dtype, seed=5, scale=2.0)
    out = torch.empty(T, I, dtype=dtype, device=dev())
    ref = torch.empty_like(out)
    K().swiglu(gu, out)
    R.swiglu(gu, ref)
    close(out, ref, dtype, "swiglu")


LINEAR_SHAPES = [(1, 64, 64), (5, 100, 72), (33, 389, 96), (130, 200, 272), (64, 1536, 1536), (3, 1000, 8960), (300, 136, 40)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LINEAR_SHAPES)
def test_linear(dtype, shape):
    M, N, Kd = shape
    a = rnd(M, Kd, dtype=dtype, seed=6)
    w = rnd(N, Kd, dtype=dtype, seed=7, scale=0.05)
    b = rnd(N, seed=8)
    for bias in (None, b):
        for out_dtype in ({dtype, torch.float32}):
            out = torch.empty(M, N, dtype=out_dtype, device=dev())
            ref = torch.empty_like(out)
            K().linear(a, w, bias, out)
            R.linear(a, w, bias, ref)
            close(out, ref, out_dtype, f"linear {shape} bias={bias is not None} out={out_dtype}", f32_tol=1e-5 * math.sqrt(Kd))


GEMV_SHAPES = [(1, 64, 64), (8, 2048, 1536), (5, 100, 72), (16, 1536, 8960), (9, 389, 96), (33, 1000, 272), (64, 1536, 1536),
               (3, 17920, 1536), (2, 151936, 1536), (40, 30, 40)]


@pytest.mark.parametrize("which", ["gemv", "gemv_tcgen05"])
@pytest.mark.parametrize("shape", GEMV_SHAPES)
def test_linear_weight_streaming_kernel(shape, which):
    M, N, Kd = shape
    a = rnd(M, Kd, dtype=torch.bfloat16, seed=16)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=17, scale=0.05)
    b = rnd(N, seed=18)
    for bias in (None, b):
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.empty(M, N, dtype=out_dtype, device=dev())
            ref = torch.empty_like(out)
            K().linear_with(which, a, w, bias, out)
            R.linear(a, w, bias, ref)
            close(out, ref, out_dtype, f"{which} {shape} bias={bias is not None} out={out_dtype}", f32_tol=1e-5 * math.sqrt(Kd))
    # a token's result does not depend on the batch it is in, nor on the call (split-k partial sums are added in fixed
    # order).  The swapped tcgen05 kernel splits k by token tile (16, 32, 64): there the smaller batch is one of the same tile.
    full = torch.empty(M, N, dtype=torch.float32, device=dev())
    K().linear_with(which, a, w, None, full)
    few = 1 if which == "gemv" else (33 if M > 32 else (17 if M > 16 else 1))
    part = torch.empty(few, N, dtype=torch.float32, device=dev())
    K().linear_with(which, a[M - few:M].contiguous(), w, None, part)
    assert torch.equal(part[few - 1], full[M - 1])
    torch.cuda.synchronize()
    assert K().library().li_tcgen05_status() == 0, "a wait inside a tcgen05 kernel ran out"


TC_SHAPES = [(128, 128, 64), (128, 128, 512), (256, 384, 1536), (2048, 2048, 1536), (17, 100, 72), (130, 200, 272), (300, 136, 40),
             (1000, 389, 96), (64, 1536, 8960), (2048, 1536, 8960), (5, 151936, 1536)]


@pytest.fixture(params=[1, 2, 3, 4, 5, 6, 7, 8, 9], ids=["tile128", "tile256", "tile256x128", "tile512pair", "tile256pair", "persistent", "tile256x192pair",
                                                   "tile128x64", "tile128x32"])
def forced_tile(request):
    """Every tile size of the tcgen05 kernel, whatever it would choose for the shape itself."""
    lib = K().library()
    lib.li_tcgen05_force_tile(request.param)
    yield request.param
    lib.li_tcgen05_force_tile(0)


@pytest.fixture(params=[0, 3], ids=["ksplit_by_shape", "ksplit3"])
def forced_ksplit(request):
    """The tcgen05 kernel with k split over three CTAs a tile, whatever it would choose for the shape itself."""
    lib = K().library()
    lib.li_tcgen05_force_ksplit(request.param)
    yield request.param
    lib.li_tcgen05_force_ksplit(0)


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_linear_tcgen05_kernel(shape, forced_tile, forced_ksplit):
    M, N, Kd = shape
    a = rnd(M, Kd, dtype=torch.bfloat16, seed=26)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=27, scale=0.05)
    b = rnd(N, seed=28)
    for bias in (None, b):
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev())
            ref = torch.empty_like(out)
            K().linear_with("tcgen05", a, w, bias, out)
            torch.cuda.synchronize()
            assert K().library().li_tcgen05_status() == 0, "a wait inside the kernel ran out"
            R.linear(a, w, bias, ref)
            close(out, ref, out_dtype, f"tcgen05 {shape} bias={bias is not None} out={out_dtype}", f32_tol=1e-5 * math.sqrt(Kd))


@pytest.mark.parametrize("which,shape", [("gemv", (1, 256, 64)), ("gemv", (8, 17920, 1536)), ("gemv", (40, 544, 96)), ("gemv", (16, 352, 80)),
                                         ("gemv_tcgen05", (1, 256, 64)), ("gemv_tcgen05", (8, 17920, 1536)), ("gemv_tcgen05", (40, 544, 96)),
                                         ("gemv_tcgen05", (16, 352, 80)), ("gemv_tcgen05", (64, 3072, 8960)),
                                         ("tcgen05", (128, 256, 64)), ("tcgen05", (300, 544, 96)), ("tcgen05", (2048, 17920, 1536)),
                                         ("tcgen05", (77, 352, 80)), ("tcgen05", (65, 48, 40))])
def test_linear_swiglu_epilogue(which, shape, forced_tile, forced_ksplit):
    """gate and up rows interleaved in groups of 8; the product's epilogue applies up * silu(gate)."""
    if which != "tcgen05" and (forced_tile != 1 or forced_ksplit):
        pytest.skip("tile size and forced splits are properties of the tcgen05 kernel")
    M, N, Kd = shape
    I = N // 2
    a = rnd(M, Kd, dtype=torch.bfloat16, seed=36)
    gate = rnd(I, Kd, dtype=torch.bfloat16, seed=37, scale=0.1)
    up = rnd(I, Kd, dtype=torch.bfloat16, seed=38, scale=0.1)
    w = K().interleave_gate_up(gate, up)
    assert torch.equal(w, R.interleave_gate_up(gate, up))
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=dev())
    K().linear_with(which, a, w, None, out, epilogue="swiglu")
    g, u = a.float() @ gate.float().t(), a.float() @ up.float().t()
    ref = u * (g / (1 + torch.exp(-g)))
    close(out, ref, torch.bfloat16, f"{which} swiglu {shape}")
    ref2 = torch.empty_like(out)
    R.linear(a, w, None, ref2, epilogue="swiglu")
    close(out, ref2, torch.bfloat16, f"{which} swiglu {shape} against the reference of the fused call")


@pytest.mark.parametrize("forced", [2, 3, 16])
def test_gemv_tcgen05_forced_splits_fit_the_workspace(forced):
    """The measurement switch for splits of k: more splits than the fixed workspace of partial sums holds are cut down
    to what fits (140 tiles of gate|up: three), and the result is the product whatever was asked for."""
    lib = K().library()
    M, N, Kd = 8, 17920, 1536
    a = rnd(M, Kd, dtype=torch.bfloat16, seed=46)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=47, scale=0.05)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    ref = torch.empty_like(out)
    lib.li_gemv_tcgen05_force_ksplit(forced)
    try:
        K().linear_with("gemv_tcgen05", a, w, None, out)
        torch.cuda.synchronize()
    finally:
        lib.li_gemv_tcgen05_force_ksplit(0)
    R.linear(a, w, None, ref)
    close(out, ref, torch.bfloat16, f"swapped tcgen05 kernel with {forced} splits asked for")
    assert lib.li_tcgen05_status() == 0


@pytest.mark.parametrize("shape", LINEAR_SHAPES)
def test_linear_simt_rows_do_not_depend_on_batch(shape):
    """float32: a row's result is the same bits whether it runs alone or among others."""
    M, N, Kd = shape
    a = rnd(M, Kd, seed=6)
    w = rnd(N, Kd, seed=7, scale=0.05)
    full = torch.empty(M, N, device=dev())
    K().linear(a, w, None, full)
    one = torch.empty(1, N, device=dev())
    K().linear(a[M - 1:M].contiguous(), w, None, one)
    assert torch.equal(one[0], full[M - 1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cfg", [(4, 2, 16, 16), (3, 1, 32, 32), (6, 2, 48, 32), (12, 2, 128, 128), (5, 5, 64, 32)])
def test_rope_kv_write(dtype, cfg):
    nh, nkv, dh, rot = cfg
    T, pages, page = 11, 9, 16
    qkv = rnd(T, (nh + 2 * nkv) * dh, dtype=dtype, seed=9)
    positions = torch.tensor([0, 1, 2, 15, 16, 17, 100, 1000, 4000, 31, 32], dtype=torch.int32, device=dev())
    theta = 10000.0
    denom = torch.pow(torch.tensor(theta), torch.arange(rot // 2, dtype=torch.float32) * 2.0 / rot).to(dev())
    g = torch.Generator().manual_seed(10)
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32).to(dev())
    kc = torch.zeros(pages, nkv, page, dh, dtype=dtype, device=dev())
    vc = torch.zeros(pages, nkv, dh, page, dtype=dtype, device=dev())
    kc2, vc2, qkv2 = kc.clone(), vc.clone(), qkv.clone()
    K().rope_kv_write(qkv, positions, denom, rot, slots, kc, vc, nh, nkv, dh, True)
    R.rope_kv_write(qkv2, positions, denom, rot, slots, kc2, vc2, nh, nkv, dh, True)
    # angles up to 4000 rad: float32 sine and cosine of such arguments differ by ~1e-4 between libraries
    close(qkv, qkv2, dtype, "rope q", f32_tol=5e-4)
    close(kc, kc2, dtype, "rope k cache", f32_tol=5e-4)
    assert torch.equal(vc, vc2)
    # without writing: q rotated, caches untouched
    kc3, vc3, qkv3 = torch.zeros_like(kc), torch.zeros_like(vc), qkv2.clone()
    K().rope_kv_write(qkv3, positions, denom, rot, slots, kc3, vc3, nh, nkv, dh, False)
    assert not kc3.any() and not vc3.any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cfg", [(4, 2, 16), (12, 2, 128), (6, 2, 48)])
@pytest.mark.parametrize("page", [16, 64])
def test_rope_kv_write_many_tokens(dtype, cfg, page):
    """Prefill sizes: values take the path that writes the transposed cache page-wise.  Runs of 16 tokens in
    consecutive slots of one page (in scrambled page order), a run that starts in the middle of a page, and
    tokens scattered one by one."""
    nh, nkv, dh = cfg
    pages = 640 // page + 6
    T = 16 * 6 + 16 + 13
    qkv = rnd(T, (nh + 2 * nkv) * dh, dtype=dtype, seed=61)
    positions = torch.arange(T, dtype=torch.int32, device=dev()) + 7
    g = torch.Generator().manual_seed(62)
    free16 = torch.randperm(pages * page // 16, generator=g).tolist()          # 16-slot pieces of the cache, in scrambled order
    slots = []
    for i in range(6):
        slots += [free16[i] * 16 + j for j in range(16)]
    base = free16[6] * 16 + 8                                                   # starts at slot 8 of a piece: crosses into the next one
    slots += [base + j for j in range(8)] + [free16[7] * 16 + j for j in range(8)]
    rest = [free16[8 + i] * 16 + (3 * i) % 16 for i in range(13)]
    slots += rest
    assert len(set(slots)) == T
    slots = torch.tensor(slots, dtype=torch.int32, device=dev())
    denom = torch.pow(torch.tensor(10000.0), torch.arange(dh // 2, dtype=torch.float32) * 2.0 / dh).to(dev())
    kc = torch.zeros(pages, nkv, page, dh, dtype=dtype, device=dev())
    vc = torch.zeros(pages, nkv, dh, page, dtype=dtype, device=dev())
    kc2, vc2, qkv2 = kc.clone(), vc.clone(), qkv.clone()
    K().rope_kv_write(qkv, positions, denom, dh, slots, kc, vc, nh, nkv, dh, True)
    R.rope_kv_write(qkv2, positions, denom, dh, slots, kc2, vc2, nh, nkv, dh, True)
    close(qkv, qkv2, dtype, "rope q", f32_tol=5e-5)
    close(kc, kc2, dtype, "rope k cache", f32_tol=5e-5)
    assert torch.equal(vc, vc2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cfg", [(4, 2, 16, 64, 5), (12, 2, 128, 1536, 8), (3, 1, 32, 96, 1), (6, 2, 48, 80, 20), (14, 2, 80, 136, 64), (12, 2, 128, 1536, 70),
                                 (12, 2, 128, 1536, 2048), (12, 2, 128, 1536, 1111), (28, 4, 128, 264, 600), (12, 2, 128, 1536, 300),
                                 (12, 2, 128, 1536, 130), (28, 4, 128, 264, 200)])
def test_linear_rope_kv_fused(dtype, cfg):
    """Projection, rotation and cache write as one call; for few bfloat16 tokens one kernel, the rotation in the
    product's epilogue.  Against the reference, and against the same call forced through separate kernels."""
    nh, nkv, dh, H, T = cfg
    N = (nh + 2 * nkv) * dh
    pages, page = max(9, -(-T // 16) + 2), 16
    a = rnd(T, H, dtype=dtype, seed=51)
    w = rnd(N, H, dtype=dtype, seed=52, scale=0.1)
    b = rnd(N, seed=53, scale=0.5)
    g = torch.Generator().manual_seed(54)
    positions = torch.randint(0, 3000, (T,), generator=g).to(torch.int32).to(dev())
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32).to(dev())
    denom = torch.pow(torch.tensor(10000.0), torch.arange(dh // 2, dtype=torch.float32) * 2.0 / dh).to(dev())

    def run(fn, **kw):
        qkv = torch.zeros(T, N, dtype=dtype, device=dev())
        kc = torch.zeros(pages, nkv, page, dh, dtype=dtype, device=dev())
        vc = torch.zeros(pages, nkv, dh, page, dtype=dtype, device=dev())
        fn(a, w, b, qkv, positions, denom, dh, slots, kc, vc, nh, nkv, dh, True, **kw)
        return qkv[:, :nh * dh].clone(), kc, vc

    # long steps: with the step's table of angles the tensor-memory product rotates and writes the cache in its epilogue
    table = None
    if T > 64:
        table = torch.empty(T, dh // 2, 2, dtype=torch.float32, device=dev())
        K().rope_table(positions, denom, table)
        ref_table = torch.empty_like(table)
        R.rope_table(positions, denom, ref_table)
        close(table, ref_table, torch.float32, "rope table", f32_tol=2e-3)      # sincosf of angles up to 3000 rad
    q1, k1, v1 = run(K().linear_rope_kv, cos_sin=table)
    q2, k2, v2 = run(K().linear_rope_kv, fused=False)
    q3, k3, v3 = run(R.linear_rope_kv)
    for got, ref, what in ((q1, q3, "q"), (k1, k3, "k cache"), (v1, v3, "v cache"), (q2, q3, "q unfused"), (k2, k3, "k unfused")):
        close(got, ref, dtype, f"linear_rope_kv {what} {cfg}", f32_tol=5e-4)
    # with a factor per token on the product
    if dtype == torch.bfloat16 and T <= 64:
        rs = ((rnd(T, 7, seed=55).abs() * 30.0 + 1.0).contiguous(), H, 1e-5)
        q4, k4, v4 = run(K().linear_rope_kv, row_scale=rs)
        q5, k5, v5 = run(R.linear_rope_kv, row_scale=rs)
        for got, ref, what in ((q4, q5, "q"), (k4, k5, "k cache"), (v4, v5, "v cache")):
            close(got, ref, dtype, f"linear_rope_kv scaled {what} {cfg}")
    # without writing: caches untouched
    kc = torch.zeros(pages, nkv, page, dh, dtype=dtype, device=dev())
    vc = torch.zeros(pages, nkv, dh, page, dtype=dtype, device=dev())
    qkv = torch.zeros(T, N, dtype=dtype, device=dev())
    K().linear_rope_kv(a, w, b, qkv, positions, denom, dh, slots, kc, vc, nh, nkv, dh, False, cos_sin=table)
    assert not kc.any() and not vc.any()
    close(qkv[:, :nh * dh], q3, dtype, "q without cache write", f32_tol=5e-4)


ADD_SCALED = [(1, 1536, 1536, False), (8, 1536, 1536, True), (8, 1536, 8960, False), (16, 1536, 8960, False), (3, 136, 200, True),
              (5, 4100, 264, False), (13, 12288, 1536, False), (33, 1536, 1536, True), (64, 1536, 8960, False), (40, 264, 4608, True),
              (8, 1532, 4096, True)]


@pytest.mark.parametrize("cfg", ADD_SCALED)
def test_linear_add_scaled(cfg):
    """The product into the residual stream with the next norm half done: x32 += a w^T (+ b), h' = bfloat16(w_norm x32)
    and partial sums of x32^2, through whichever of the two weight-streaming kernels the sizes choose; then the factor
    per token, applied to h' itself.  Against product, add and norm as separate references; twice in a row, since the
    split of k leaves counters behind."""
    M, N, Kd, with_bias = cfg
    dtype = torch.bfloat16
    a = rnd(M, Kd, dtype=dtype, seed=61)
    w = rnd(N, Kd, dtype=dtype, seed=62, scale=0.05)
    b = rnd(N, seed=63, scale=0.5) if with_bias else None
    x0 = rnd(M, N, seed=64)
    nw = (1.0 + 0.1 * rnd(N, seed=65)).contiguous()
    eps = 3e-6
    x_ref = x0.clone()
    o_ref = torch.zeros(M, N, dtype=dtype, device=dev())
    delta = torch.zeros(M, N, dtype=torch.float32, device=dev())
    R.linear(a, w, b, delta)
    R.add_rmsnorm(x_ref, delta, nw, eps, o_ref)
    for rep in range(2):
        x = x0.clone()
        h = torch.zeros(M, N, dtype=dtype, device=dev())
        parts = K().linear_add_scaled_parts(a, w, x, h)
        assert parts > 0, f"no kernel for {cfg}"
        ssq = torch.full((M, parts), float("nan"), dtype=torch.float32, device=dev())
        K().linear_add_scaled(a, w, b, x, nw, h, ssq)
        close(x, x_ref, dtype, f"stream {cfg} run {rep}")
        close(ssq.sum(1), (x_ref * x_ref).sum(-1), torch.float32, f"sums of squares {cfg}", f32_tol=1e-4)
        out = torch.zeros(M, N, dtype=dtype, device=dev())
        K().apply_row_scale(h, ssq, N, eps, out)
        close(out, o_ref, dtype, f"normalised {cfg} run {rep}")
    # a token's results do not depend on the others in the batch
    if M >= 2:
        x1 = x0[:1].clone()
        h1 = torch.zeros(1, N, dtype=dtype, device=dev())
        ssq1 = torch.zeros(1, K().linear_add_scaled_parts(a[:1].contiguous(), w, x1, h1), dtype=torch.float32, device=dev())
        K().linear_add_scaled(a[:1].contiguous(), w, b, x1, nw, h1, ssq1)
        if M <= 32:                       # the same kernel for 1 and for M tokens
            assert torch.equal(x1[0], x[0]) and torch.equal(h1[0], h[0]) and torch.equal(ssq1[0], ssq[0])


@pytest.mark.parametrize("epilogue", [None, "swiglu"])
@pytest.mark.parametrize("cfg", [(1, 2048, 1536, 12, True), (8, 2048, 1536, 96, True), (8, 17920, 1536, 12, False), (16, 17920, 1536, 96, False),
                                 (5, 272, 200, 1, True), (40, 1536, 8960, 140, False), (64, 4608, 264, 33, True), (9, 640, 4096, 200, False)])
def test_linear_row_scale(cfg, epilogue):
    """A factor per token, from partial sums of squares, on the rows of the product before bias and epilogue."""
    M, N, Kd, parts, with_bias = cfg
    dtype = torch.bfloat16
    a = rnd(M, Kd, dtype=dtype, seed=71)
    w = rnd(N, Kd, dtype=dtype, seed=72, scale=0.05)
    b = rnd(N, seed=73, scale=0.5) if (with_bias and epilogue is None) else None
    ssq = (rnd(M, parts, seed=74).abs() * 50.0 + 1.0).contiguous()
    width, eps = 777, 2e-5
    if epilogue == "swiglu":
        w = K().interleave_gate_up(w[:N // 2].contiguous(), w[N // 2:].contiguous())
    n_out = N // 2 if epilogue else N
    out = torch.zeros(M, n_out, dtype=dtype, device=dev())
    ref = torch.zeros(M, n_out, dtype=dtype, device=dev())
    assert K().linear_scaled_accepts(a, w, out)
    K().linear(a, w, b, out, epilogue=epilogue, row_scale=(ssq, width, eps))
    R.linear(a, w, b, ref, epilogue=epilogue, row_scale=(ssq, width, eps))
    close(out, ref, dtype, f"scaled product {cfg} {epilogue}")
    if M >= 2 and M <= 8:
        one = torch.zeros(1, n_out, dtype=dtype, device=dev())
        K().linear(a[:1].contiguous(), w, b, one, epilogue=epilogue, row_scale=(ssq[:1].contiguous(), width, eps))
        assert torch.equal(one[0], out[0])


def test_linear_row_scale_refused():
    """Products that no weight-streaming kernel takes cannot apply the factor: said, not ignored."""
    a = rnd(100, 64, dtype=torch.bfloat16, seed=1)
    w = rnd(32, 64, dtype=torch.bfloat16, seed=2)
    out = torch.zeros(100, 32, dtype=torch.bfloat16, device=dev())
    assert not K().linear_scaled_accepts(a, w, out)
    with pytest.raises(Exception, match="at most 64"):
        K().linear(a, w, None, out, row_scale=(torch.ones(100, 1, device=dev()), 64, 1e-6))


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------

def decode_cut(pairs, max_ctx, ctx, dh):
    """How the decode attention kernel cuts the context ``ctx`` of a sequence in a step with ``pairs`` pairs of
    (sequence, kv head) whose longest context is ``max_ctx`` (restating the choice in csrc/attention_decode.cu): the keys
    a CTA takes, or None for a whole context per CTA.  A sequence's result is the same bit for bit only between steps
    that cut it alike."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    unit = (32 if dh <= 128 else 16) * 8
    most = -(-max(max_ctx, 1) // unit)
    want = 1 if pairs >= sms else sms // pairs
    if want == 1 and most > 1:
        return None
    if want >= most:
        return unit
    return unit * max(1, -(-(-(-ctx // unit)) // want))


def make_attention_case(q_lens, ctx_lens, nh, nkv, dh, page, dtype, seed=0, extra_pages=5):
    """A ragged batch with scrambled page tables.  Returns the kernel arguments and the
    logical (per sequence) keys and values so that tests can plant special ones."""
    S = len(q_lens)
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // page) for c in ctx_lens]
    pages = sum(blocks) + extra_pages
    perm = torch.randperm(pages, generator=g).tolist()
    mb = max(blocks) + 1
    bt = torch.full((S, mb), pages - 1, dtype=torch.int32)
    it = iter(perm)
    for s in range(S):
        for b in range(blocks[s]):
            bt[s, b] = next(it)
    T = sum(q_lens)
    qkv = (torch.randn(T, (nh + 2 * nkv) * dh, generator=g)).to(dtype)
    keys = [torch.randn(c, nkv, dh, generator=g).to(dtype) for c in ctx_lens]
    vals = [torch.randn(c, nkv, dh, generator=g).to(dtype) for c in ctx_lens]
    q_start = [0]
    for n in q_lens:
        q_start.append(q_start[-1] + n)
    seq_of, pos = [], []
    for s, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        seq_of += [s] * n
        pos += list(range(c - n, c))
    return dict(S=S, T=T, pages=pages, page=page, bt=bt, qkv=qkv, keys=keys, vals=vals, q_start=q_start, seq_of=seq_of, pos=pos,
                ctx_lens=list(ctx_lens), q_lens=list(q_lens), nh=nh, nkv=nkv, dh=dh, dtype=dtype)


def run_attention_case(c, window, implementation=None, old_lens=None, singles=0, dense_reference=False, work_budget=None):
    """``work_budget``: run with the attention work list that the step function would pack for this budget."""
    d = dev()
    page, nkv, dh = c["page"], c["nkv"], c["dh"]
    kc = torch.zeros(c["pages"], nkv, page, dh, dtype=c["dtype"])
    vc = torch.zeros(c["pages"], nkv, dh, page, dtype=c["dtype"])
    for s in range(c["S"]):
        t = torch.arange(c["ctx_lens"][s])
        pages, offs = c["bt"][s].long()[t // page], t % page
        kc[pages, :, offs] = c["keys"][s][:len(t)]
        vc[pages, :, :, offs] = c["vals"][s][:len(t)]
    args = dict(
        qkv=c["qkv"].to(d), k_cache=kc.to(d), v_cache=vc.to(d), block_table=c["bt"].to(d),
        q_start=torch.tensor(c["q_start"], dtype=torch.int32, device=d), ctx_lens=torch.tensor(c["ctx_lens"], dtype=torch.int32, device=d),
        seq_of_token=torch.tensor(c["seq_of"], dtype=torch.int32, device=d), positions=torch.tensor(c["pos"], dtype=torch.int32, device=d))
    out = torch.empty(c["T"], c["nh"] * dh, dtype=c["dtype"], device=d)
    ref = torch.empty_like(out)
    scale = 1.0 / math.sqrt(dh)
    tail = (c["nh"], nkv, dh, scale, window, max(c["q_lens"]), max(c["ctx_lens"]))
    more = {}
    if work_budget is not None:
        from litinfer_b200.engine.batch import attention_units

        units = attention_units(c["q_lens"], c["ctx_lens"], work_budget)
        more = dict(units=torch.from_numpy(units).to(d), unit_slots=(int(units[0]), int(units[1])))
    K().paged_attention(args["qkv"], out, args["k_cache"], args["v_cache"], args["block_table"], args["q_start"], args["ctx_lens"],
                        args["seq_of_token"], args["positions"], *tail, implementation=implementation,
                        old_lens=None if old_lens is None else torch.tensor(old_lens, dtype=torch.int32, device=d), singles=singles, **more)
    reference = R.paged_attention_dense if dense_reference else R.paged_attention
    reference(args["qkv"], ref, args["k_cache"], args["v_cache"], args["block_table"], args["q_start"], args["ctx_lens"],
              args["seq_of_token"], args["positions"], *tail)
    return out, ref


HEADS = [(4, 2, 16), (3, 1, 32), (6, 2, 48), (12, 2, 128), (8, 8, 64), (14, 2, 80)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads", HEADS)
@pytest.mark.parametrize("window", [None, 24])
def test_attention_mixed_batch(dtype, heads, window):
    nh, nkv, dh = heads
    # a whole prompt, a portion with history, single tokens (one at a page's first slot, one at its last), a two-token portion
    q_lens = [37, 20, 1, 1, 2, 1]
    ctx_lens = [37, 75, 33, 48, 130, 1]
    c = make_attention_case(q_lens, ctx_lens, nh, nkv, dh, 16, dtype, seed=nh * 100 + dh)
    out, ref = run_attention_case(c, window)
    close(out, ref, dtype, f"attention heads={heads} window={window}", f32_tol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads", [(4, 2, 16), (12, 2, 128), (6, 2, 48)])
def test_attention_decode_batch(dtype, heads):
    nh, nkv, dh = heads
    ctx_lens = [1, 16, 17, 300, 777, 64, 255, 256, 257]
    c = make_attention_case([1] * len(ctx_lens), ctx_lens, nh, nkv, dh, 16, dtype, seed=3)
    out, ref = run_attention_case(c, None)
    close(out, ref, dtype, f"decode attention heads={heads}")
    out, ref = run_attention_case(c, 100)
    close(out, ref, dtype, f"decode attention heads={heads} window=100")


@pytest.mark.parametrize("heads", [(4, 2, 16), (3, 1, 32), (6, 2, 48), (12, 2, 128), (8, 8, 64), (14, 2, 80), (16, 1, 96), (28, 4, 128)])
@pytest.mark.parametrize("page", [16, 64])
def test_attention_decode_kernel_alone(heads, page):
    nh, nkv, dh = heads
    ctx_lens = [1, 16, 17, 300, 777, 64, 255, 256, 257, 1025]
    c = make_attention_case([1] * len(ctx_lens), ctx_lens, nh, nkv, dh, page, torch.bfloat16, seed=31)
    for window in (None, 100, 300):
        out, ref = run_attention_case(c, window, implementation="decode")
        close(out, ref, torch.bfloat16, f"decode kernel heads={heads} page={page} window={window}")
    # alone or in the batch: the same bits, as long as the contexts are cut the same way
    out_all, _ = run_attention_case(c, None, implementation="decode")
    c1 = make_attention_case([1] * len(ctx_lens), ctx_lens, nh, nkv, dh, page, torch.bfloat16, seed=31)
    for key in ("q_lens", "ctx_lens"):
        c1[key] = c1[key][4:5]
    c1.update(S=1, T=1, bt=c1["bt"][4:5], qkv=c1["qkv"][4:5], keys=c1["keys"][4:5], vals=c1["vals"][4:5], q_start=[0, 1], seq_of=[0],
              pos=[ctx_lens[4] - 1])
    out_one, _ = run_attention_case(c1, None, implementation="decode")
    if decode_cut(len(ctx_lens) * nkv, max(ctx_lens), ctx_lens[4], dh) == decode_cut(nkv, ctx_lens[4], ctx_lens[4], dh):
        assert torch.equal(out_one[0], out_all[4])
    else:
        close(out_one[0:1], out_all[4:5], torch.bfloat16, f"a sequence alone and in a batch that is cut differently, heads={heads}")


@pytest.mark.parametrize("heads", [(4, 2, 16), (12, 2, 128)])
def test_attention_decode_kernel_tokens_of_one_request(heads):
    """A portion of a prompt as single tokens: sequences that share one block table and end one key after the other,
    with the count of keys that were cached before the step (old_lens) given."""
    nh, nkv, dh = heads
    first, n = 283, 40                                   # keys before the portion, tokens of the portion
    c = make_attention_case([1] * n, [first + n] * n, nh, nkv, dh, 16, torch.bfloat16, seed=7)
    c["bt"] = c["bt"][:1].repeat(n, 1)
    c["keys"] = [c["keys"][0]] * n
    c["vals"] = [c["vals"][0]] * n
    c["ctx_lens"] = [first + j + 1 for j in range(n)]
    c["pos"] = [first + j for j in range(n)]
    for window in (None, 100):
        out, ref = run_attention_case(c, window, implementation="decode", old_lens=[first] * n)
        close(out, ref, torch.bfloat16, f"decode kernel, tokens of one request, heads={heads} window={window}")
        again, _ = run_attention_case(c, window, implementation="decode")
        assert torch.equal(out, again)


@pytest.mark.parametrize("heads", [(4, 2, 16), (6, 2, 48), (12, 2, 128), (8, 8, 64), (28, 4, 128)])
@pytest.mark.parametrize("many", [False, True])
def test_attention_single_tokens_beside_portions(heads, many):
    """A step of portions and single tokens in two launches: the decode kernel finds the sequences of one token by
    q_start wherever they stand in the batch, the kernel for portions leaves them out.  `many`: enough sequences for the
    decode kernel that walks a whole context per CTA."""
    nh, nkv, dh = heads
    if many:
        q_lens = [1] * 33 + [80, 1, 2, 5] + [1] * 30 + [64]
        ctx_lens = [17 + 23 * i for i in range(33)] + [200, 1, 130, 5] + [300 - 7 * i for i in range(30)] + [64]
    else:
        q_lens = [1, 1, 37, 1, 70, 1, 2, 1]
        ctx_lens = [300, 17, 37, 1, 200, 256, 130, 777]
    c = make_attention_case(q_lens, ctx_lens, nh, nkv, dh, 16, torch.bfloat16, seed=nh + dh)
    n1 = sum(1 for q in q_lens if q == 1)
    for window in (None, 24, 100):
        for count in (n1, -1):
            out, ref = run_attention_case(c, window, singles=count)
            close(out, ref, torch.bfloat16, f"attention, single tokens beside portions, heads={heads} window={window} singles={count}")
        out, ref = run_attention_case(c, window, implementation="prefill", singles=n1)
        close(out, ref, torch.bfloat16, f"attention, single tokens beside portions (mma.sync tiles), heads={heads} window={window}")
        if dh in (64, 128):
            out, ref = run_attention_case(c, window, implementation="prefill_tcgen05", singles=n1)
            close(out, ref, torch.bfloat16, f"attention, single tokens beside portions (tcgen05 tiles), heads={heads} window={window}")
    # a single token alone in a step of singles, or beside portions: the same kernel, the same bits
    alone = make_attention_case([1] * len(q_lens), ctx_lens, nh, nkv, dh, 16, torch.bfloat16, seed=nh + dh)
    tok0 = c["q_start"][0]
    alone["qkv"][0] = c["qkv"][tok0]
    alone["keys"], alone["vals"], alone["bt"] = c["keys"], c["vals"], c["bt"]
    out_alone, _ = run_attention_case(alone, None, implementation="decode")
    out_mixed, _ = run_attention_case(c, None, singles=n1)
    # (how the contexts are cut depends on how many single tokens there are: the sums then come in another order)
    if decode_cut(len(q_lens) * nkv, max(ctx_lens), ctx_lens[0], dh) == decode_cut(n1 * nkv, max(ctx_lens), ctx_lens[0], dh):
        assert torch.equal(out_alone[0], out_mixed[tok0])
    else:
        close(out_mixed[tok0:tok0 + 1], out_alone[0:1], torch.bfloat16, "a single token alone and beside portions, through different kernels")


@pytest.mark.parametrize("heads", [(4, 2, 16), (3, 1, 32), (6, 2, 48), (12, 2, 128), (8, 8, 64), (14, 2, 80), (28, 4, 128)])
@pytest.mark.parametrize("page", [16, 32])
def test_attention_prefill_kernel_alone(heads, page):
    nh, nkv, dh = heads
    # whole prompts (one longer than a 64-token tile, one of 64 exactly), portions with history, single tokens, two tokens
    q_lens = [37, 20, 1, 150, 2, 1, 64, 17]
    ctx_lens = [37, 75, 33, 150, 130, 1, 64, 300]
    c = make_attention_case(q_lens, ctx_lens, nh, nkv, dh, page, torch.bfloat16, seed=41)
    for window in (None, 24, 100):
        out, ref = run_attention_case(c, window, implementation="prefill")
        close(out, ref, torch.bfloat16, f"prefill kernel heads={heads} page={page} window={window}")


@pytest.mark.parametrize("heads", [(12, 2, 128), (8, 8, 64), (28, 4, 128), (3, 1, 64)])
@pytest.mark.parametrize("page", [16, 32])
def test_attention_tcgen05_kernel_alone(heads, page):
    """The prefill kernel on tcgen05 (128 tokens x 128 keys a tile): whole prompts shorter and longer than a tile and of
    exactly one and two tiles, portions with history (ending inside a key tile and on its edge), single tokens, windows."""
    nh, nkv, dh = heads
    q_lens = [37, 300, 1, 128, 2, 256, 64, 17, 129]
    ctx_lens = [37, 300, 33, 128, 130, 256, 384, 300, 513]
    c = make_attention_case(q_lens, ctx_lens, nh, nkv, dh, page, torch.bfloat16, seed=43)
    for window in (None, 24, 100, 200):
        out, ref = run_attention_case(c, window, implementation="prefill_tcgen05")
        close(out, ref, torch.bfloat16, f"tcgen05 prefill kernel heads={heads} page={page} window={window}")
    assert K().library().li_tcgen05_status() == 0


def test_attention_tcgen05_far_key_and_window_edge():
    """One key far back carries the answer (a lost page or a wrong tile would change everything); the key at
    p - window + 1 is the oldest one seen, the one at p - window is not."""
    nh, nkv, dh = 12, 2, 128
    for far in (0, 15, 16, 127, 128, 255, 256, 383):
        c = make_attention_case([200], [600], nh, nkv, dh, 16, torch.bfloat16, seed=far)
        _plant(c, 0, 1, far, 199)
        out, ref = run_attention_case(c, None, implementation="prefill_tcgen05")
        close(out, ref, torch.bfloat16, f"far key {far}")
        v = c["vals"][0][far, 1].float().to(out.device)
        got = out[199].float().view(nh, dh)[6]
        assert (got - v).abs().max() < 0.1 * v.abs().max() + 0.05
    W = 140
    for key_pos, visible in ((599 - W + 1, True), (599 - W, False)):
        c = make_attention_case([200], [600], nh, nkv, dh, 16, torch.bfloat16, seed=key_pos)
        _plant(c, 0, 0, key_pos, 199)
        out, ref = run_attention_case(c, W, implementation="prefill_tcgen05")
        close(out, ref, torch.bfloat16, f"window edge key {key_pos}")
        v = c["vals"][0][key_pos, 0].float().to(out.device)
        got = out[199].float().view(nh, dh)[0]
        near = (got - v).abs().max() < 0.1 * v.abs().max() + 0.05
        assert bool(near) == visible, f"key {key_pos} should be {'visible' if visible else 'hidden'}"


def _planted_value_comes_out(c, out, s, h_kv, key_pos, q_token, what):
    nh, nkv, dh = c["nh"], c["nkv"], c["dh"]
    v = c["vals"][s][key_pos, h_kv].float().to(out.device)
    got = out[q_token].float().view(nh, dh)[h_kv * (nh // nkv)]
    assert (got - v).abs().max() < 0.1 * v.abs().max() + 0.05, f"{what}: the planted key {key_pos} of sequence {s} did not carry the answer"


def test_the_two_reference_attentions_agree():
    c = make_attention_case([37, 20, 1, 2], [37, 75, 33, 130], 6, 2, 48, 16, torch.float32, seed=8)
    for window in (None, 24):
        _, a = run_attention_case(c, window)
        _, b = run_attention_case(c, window, dense_reference=True)
        assert (a - b).abs().max() < 1e-5


@pytest.mark.parametrize("heads", [(12, 2, 128), (28, 4, 128)])
@pytest.mark.parametrize("many", [False, True], ids=["split_context", "whole_context"])
def test_attention_decode_at_benchmark_lengths(heads, many):
    """Contexts of 2,049 to 4,096 keys, where the benchmark decodes: nine to sixteen splits of 256 keys merged by the CTA
    that finishes last (few sequences), or a CTA walking a whole context (from 120 sequence x kv-head pairs on).  One
    planted key in a split from the ninth on and one in the last, ragged split carry the answer of their sequences."""
    nh, nkv, dh = heads
    ctx_lens = [2049, 2304, 4095, 4096, 2074, 3000]
    if many:
        g = torch.Generator().manual_seed(6)
        ctx_lens += torch.randint(1, 2600, (128 // nkv - 2,), generator=g).tolist()
    S = len(ctx_lens)
    assert (S * nkv >= 120) == many
    c = make_attention_case([1] * S, ctx_lens, nh, nkv, dh, 16, torch.bfloat16, seed=61)
    plants = [(0, 0, 2048), (1, nkv - 1, 2100), (2, 0, 4090), (3, nkv - 1, 2305), (5, 0, 2999)]
    for s, h, key in plants:
        _plant(c, s, h, key, s)
    for window in (None, 1000):
        out, ref = run_attention_case(c, window, implementation="decode", dense_reference=True)
        close(out, ref, torch.bfloat16, f"decode at long contexts heads={heads} many={many} window={window}")
        for s, h, key in plants:
            if window is None or ctx_lens[s] - 1 - key < window:
                _planted_value_comes_out(c, out, s, h, key, s, f"heads={heads} many={many} window={window}")
    out32, ref32 = run_attention_case(make_attention_case([1] * 6, ctx_lens[:6], nh, nkv, dh, 16, torch.float32, seed=62), None, dense_reference=True)
    close(out32, ref32, torch.float32, f"general kernel at long contexts heads={heads}", f32_tol=2e-5)


@pytest.mark.parametrize("heads", [(12, 2, 128), (28, 4, 128)])
def test_attention_tcgen05_at_benchmark_lengths(heads):
    """A whole prompt of 2,048 tokens (sixteen token tiles against up to sixteen key tiles) and a portion of 512 tokens
    behind 1,536 cached keys, with a planted key in the tenth key tile and beyond."""
    nh, nkv, dh = heads
    for q_lens, ctx_lens, plants in (([2048], [2048], [(0, 0, 1300, 1500), (0, nkv - 1, 1999, 2047)]),
                                     ([512, 3], [2048, 700], [(0, 0, 1200, 0), (0, nkv - 1, 1700, 400), (1, 0, 690, 514)])):
        c = make_attention_case(q_lens, ctx_lens, nh, nkv, dh, 16, torch.bfloat16, seed=71)
        for s, h, key, tok in plants:
            _plant(c, s, h, key, tok)
        for window, impl in ((None, "prefill_tcgen05"), (900, "prefill_tcgen05"), (None, None)):
            out, ref = run_attention_case(c, window, implementation=impl, dense_reference=True)
            close(out, ref, torch.bfloat16, f"prefill at 2,048 keys heads={heads} q={q_lens} window={window} {impl}")
            for s, h, key, tok in plants:
                pos = c["pos"][tok]
                if window is None or pos - key < window:
                    _planted_value_comes_out(c, out, s, h, key, tok, f"heads={heads} q={q_lens} window={window}")
    assert K().library().li_tcgen05_status() == 0


@pytest.mark.parametrize("heads", [(12, 2, 128), (4, 4, 64), (28, 4, 128)])
def test_attention_tcgen05_with_a_work_list(heads):
    """The kernel for long portions driven by the step's work list: a portion behind a long context whose key tiles are
    shared out among several CTAs (with a planted key in a late part, a window that cuts parts away, two portions at
    once, single tokens beside them), and lists that share nothing out.  Twice in a row: the counters of the shared
    tiles are left ready for the next launch."""
    from litinfer_b200.engine.batch import attention_units

    nh, nkv, dh = heads
    budget = 148 // nh
    c = make_attention_case([384], [3500], nh, nkv, dh, 16, torch.bfloat16, seed=81)
    _plant(c, 0, nkv - 1, 2900, 200)
    units = attention_units(c["q_lens"], c["ctx_lens"], budget)
    assert (units[0] > 3) == (6 <= budget) and units[0] <= max(budget, 3), "three tiles of tokens, shared out where the budget allows"
    for window, b in ((None, budget), (None, budget), (700, budget), (None, 0), (130, budget)):
        out, ref = run_attention_case(c, window, implementation="prefill_tcgen05", dense_reference=True, work_budget=b)
        close(out, ref, torch.bfloat16, f"work list heads={heads} window={window} budget={b}")
        if window is None:
            _planted_value_comes_out(c, out, 0, nkv - 1, 2900, 200, f"work list heads={heads} budget={b}")
    c = make_attention_case([130, 1, 70, 1, 1], [1500, 900, 70, 2048, 1], nh, nkv, dh, 16, torch.bfloat16, seed=82)
    for singles in (0, 3):
        out, ref = run_attention_case(c, None, implementation="prefill_tcgen05", dense_reference=True, work_budget=budget, singles=singles)
        close(out, ref, torch.bfloat16, f"work list, portions beside single tokens, heads={heads} singles={singles}")
    out, ref = run_attention_case(c, None, dense_reference=True, work_budget=budget, singles=3)
    close(out, ref, torch.bfloat16, f"work list through the dispatcher, heads={heads}")
    assert K().library().li_tcgen05_status() == 0


@pytest.mark.parametrize("heads", [(12, 2, 128), (4, 2, 16), (6, 2, 48), (8, 8, 64)])
def test_attention_decode_large_batch(heads):
    """From 120 (sequence, kv head) pairs on, a CTA takes a whole context instead of a 128-key split."""
    nh, nkv, dh = heads
    S = 128 // nkv + 3
    g = torch.Generator().manual_seed(5)
    ctx_lens = torch.randint(1, 700, (S,), generator=g).tolist()
    ctx_lens[:6] = [1, 16, 17, 255, 256, 257]
    c = make_attention_case([1] * S, ctx_lens, nh, nkv, dh, 16, torch.bfloat16, seed=33)
    for window in (None, 100):
        out, ref = run_attention_case(c, window, implementation="decode")
        close(out, ref, torch.bfloat16, f"decode, large batch, heads={heads} window={window}")
    # one far key carries the answer
    c = make_attention_case([1] * S, [650] * S, nh, nkv, dh, 16, torch.bfloat16, seed=34)
    _plant(c, 7, nkv - 1, 3, 7)
    out, ref = run_attention_case(c, None, implementation="decode")
    close(out, ref, torch.bfloat16, "decode, large batch, far key")
    v = c["vals"][7][3, nkv - 1].float().to(out.device)
    got = out[7].float().view(nh, dh)[(nkv - 1) * (nh // nkv)]
    assert (got - v).abs().max() < 0.1 * v.abs().max() + 0.05


def _plant(c, s, h_kv, key_pos, q_token, strength=30.0):
    """Make key ``key_pos`` of sequence s point along the query of ``q_token`` (all heads
    of that key head), so that it takes nearly all the softmax weight if it is visible."""
    nh, nkv, dh = c["nh"], c["nkv"], c["dh"]
    group = nh // nkv
    q = c["qkv"][q_token, (h_kv * group) * dh:(h_kv * group + 1) * dh].float()
    c["keys"][s][key_pos, h_kv] = (q / q.norm() * strength).to(c["dtype"])
    # all heads of the group share the direction of the first one
    for g in range(1, group):
        c["qkv"][q_token, (h_kv * group + g) * dh:(h_kv * group + g + 1) * dh] = c["qkv"][q_token, (h_kv * group) * dh:(h_kv * group + 1) * dh]


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_far_key_among_hundreds(dtype):
    """One key far back carries the answer: skipping it (a lost page, a wrong split) changes everything."""
    nh, nkv, dh = 12, 2, 128
    for far in (0, 3, 15, 16, 255, 256, 511):
        c = make_attention_case([1, 5], [700, 640], nh, nkv, dh, 16, dtype, seed=far)
        _plant(c, 0, 1, far, 0)
        _plant(c, 1, 0, far, 5)              # last token of the 5-token portion
        out, ref = run_attention_case(c, None)
        close(out, ref, dtype, f"far key {far}")
        # the planted key dominates: the output of that head is close to its value
        v = c["vals"][0][far, 1].float().to(out.device)
        got = out[0].float().view(nh, dh)[6]
        assert (got - v).abs().max() < 0.1 * v.abs().max() + 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(dtype):
    """The key at p - window + 1 is the oldest one seen; the one at p - window is not."""
    nh, nkv, dh, W = 4, 2, 32, 40
    for q_lens, ctx in (([1], [200]), ([3], [200])):
        p_last = ctx[0] - 1
        for key_pos, visible in ((p_last - W + 1, True), (p_last - W, False)):
            c = make_attention_case(q_lens, ctx, nh, nkv, dh, 16, dtype, seed=key_pos)
            _plant(c, 0, 0, key_pos, q_lens[0] - 1)
            out, ref = run_attention_case(c, W)
            close(out, ref, dtype, f"window edge key {key_pos}")
            v = c["vals"][0][key_pos, 0].float().to(out.device)
            got = out[-1].float().view(nh, dh)[0]
            near = (got - v).abs().max() < 0.1 * v.abs().max() + 0.05
            assert bool(near) == visible, f"key {key_pos} should be {'visible' if visible else 'hidden'}"


def test_a_bounded_wait_that_runs_out_raises_the_status_and_leaves_the_device_usable():
    """Every wait in the tcgen05 kernels has a limit; when it runs out the kernel raises a status word in mapped host
    memory and returns, and the launches after it refuse to run until the word is cleared.  Exercised here without any
    kernel at fault: one thread waits a millisecond on a barrier that nobody arrives on."""
    import ctypes

    k = K()
    lib = k.library()
    assert lib.li_tcgen05_status() == 0
    a = rnd(200, 256, dtype=torch.bfloat16, seed=1).to(dev())
    w = rnd(384, 256, dtype=torch.bfloat16, seed=2, scale=0.05).to(dev())
    out = torch.empty(200, 384, dtype=torch.bfloat16, device=dev())
    k.linear_with("tcgen05", a, w, None, out)
    want = out.clone()
    rc = lib.li_tcgen05_wait_selftest(ctypes.c_int(1000), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.li_tcgen05_status() == 99
    with pytest.raises(k.KernelError, match="gave up waiting"):
        k.linear_with("tcgen05", a, w, None, out)
    lib.li_tcgen05_clear_status()
    assert lib.li_tcgen05_status() == 0
    out.zero_()
    k.linear_with("tcgen05", a, w, None, out)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert lib.li_tcgen05_wait_selftest(ctypes.c_int(0), ctypes.c_void_p(0)) != 0          # a limit outside the range is refused


@pytest.mark.parametrize("dtype", DTYPES)
def test_fill_normal_gives_the_bits_of_the_host_restatement(dtype):
    """Random weights drawn on the device by the library's kernel equal, bit for bit, those the host draws for a model
    folder (NumPy in the package, checked against tests/plain_random.py on the CPU): float32 and rounded to bfloat16, odd
    and even sizes, a size beyond one block, other means and deviations; integer tables too."""
    import numpy as np

    import plain_random as PR
    from litinfer_b200.weights.loader import ParamSpec
    from litinfer_b200.weights.random_init import random_tensor

    for name, shape, init, std in (("a.weight", (7, 9), "normal", 0.02), ("b.weight", (64,), "ones_normal", 0.02), ("c", (1001,), "normal", 0.5),
                                   ("big", (1025, 513), "normal", 0.02)):
        p = ParamSpec(name, shape, init=init, std=std)
        on_device = random_tensor(p, 11, dev(), dtype)
        on_host = random_tensor(p, 11, "cpu", dtype)
        assert on_device.dtype == dtype and on_device.is_cuda
        assert torch.equal(on_device.cpu(), on_host), f"{name}: {(on_device.cpu().float() - on_host.float()).abs().max()}"
        if dtype == torch.float32 and on_host.numel() < 2000:
            mean, sd = (1.0, 0.1) if init == "ones_normal" else (0.0, std)
            want = PR.normal(PR.tensor_key(11, name), on_host.numel(), mean, sd)
            assert np.array_equal(on_device.cpu().numpy().reshape(-1), want)
    t = ParamSpec("t", (1000,), role="table", init="randint")
    assert torch.equal(random_tensor(t, 3, dev()).cpu(), random_tensor(t, 3, "cpu"))


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

def test_argmax_first_maximum():
    V = 1000
    lg = rnd(5, V, seed=11)
    lg[0, 17] = lg[0, 900] = 50.0          # tie: the first wins
    lg[1, 999] = 60.0
    lg[2, 0] = 60.0
    out = torch.empty(5, dtype=torch.int32, device=dev())
    ref = torch.empty_like(out)
    K().argmax(lg, out)
    R.argmax(lg, ref)
    assert out.tolist() == ref.tolist()
    assert out.tolist()[:3] == [17, 999, 0]
    big = rnd(3, 151936, seed=12)
    out = torch.empty(3, dtype=torch.int32, device=dev())
    K().argmax(big, out)
    assert out.tolist() == big.argmax(dim=1).tolist()
    # few rows of a large vocabulary are cut into pieces: ties across pieces (the first wins), a maximum in the last,
    # ragged piece, a row without any finite value; twice, since a counter per row stays behind
    for V in (151936, 16384, 50001):
        lg = rnd(8, V, seed=13)
        lg[0, 5] = lg[0, V - 1] = lg[0, V // 2] = 70.0
        lg[1, V - 1] = 70.0
        lg[2, V // 16 + 3] = lg[2, V // 16 - 3] = 70.0
        lg[3, :] = float("-inf")
        lg[4, V - 7:] = 70.0
        for _ in range(2):
            out = torch.full((8,), -1, dtype=torch.int32, device=dev())
            K().argmax(lg, out)
            want = lg.argmax(dim=1).tolist()
            want[0], want[2], want[3], want[4] = 5, V // 16 - 3, 0, V - 7
            assert out.tolist() == want, f"V={V}: {out.tolist()} vs {want}"


def _params(rows):
    t = torch.empty(len(rows), 6, dtype=torch.int32)
    f = t.view(torch.float32)
    for r, (temp, k, p, seed, idx) in enumerate(rows):
        f[r, 0] = temp
        t[r, 1] = k
        f[r, 2] = p
        t[r, 3] = seed & 0x7FFFFFFF
        t[r, 4] = (seed >> 32) & 0x7FFFFFFF
        t[r, 5] = idx
    return t.to(dev())


def test_sample_matches_reference_and_is_batch_independent():
    V = 389
    lg = rnd(6, V, seed=13, scale=2.0)
    rows = [(0.8, 0, 1.0, 5, 0), (1.0, 10, 1.0, 6, 3), (0.7, 0, 0.9, 7, 1), (1.3, 20, 0.5, 8, 2), (0.0, 0, 1.0, 9, 0), (1.0, 1, 1.0, 1, 0)]
    out = torch.empty(6, dtype=torch.int32, device=dev())
    K().sample(lg, _params(rows), out)
    for r, (temp, k, p, seed, idx) in enumerate(rows):
        tok, kept = R.sample_row(lg[r], temp, k, p, seed, idx)
        assert out[r].item() == tok, f"row {r}"
    # the same row alone gives the same token
    for r in (1, 3):
        one = torch.empty(1, dtype=torch.int32, device=dev())
        K().sample(lg[r:r + 1].contiguous(), _params([rows[r]]), one)
        assert one.item() == out[r].item()


@pytest.mark.parametrize("V", [4097, 20011])
def test_sample_large_vocabulary_matches_reference(V):
    # (20,011 tokens also take the path that cuts a row with temperature alone over many CTAs)
    """Above 4,096 tokens the thresholds come from a radix selection and the rest happens on the gathered candidates in
    shared memory: top-k alone, top-p alone (peaked: the gathered tokens hold the mass; flat: they do not, and the row
    is bisected), both, ties at the k-th value, k larger than fits."""
    g = torch.Generator().manual_seed(V)
    peaked = (torch.randn(V, generator=g) * 4.0)
    flat = (torch.randn(V, generator=g) * 0.05)
    ties = peaked.clone()
    ties[torch.randperm(V, generator=g)[:300]] = float(peaked.topk(40).values[-1])         # 300 copies of the 40th largest value
    cases = [(peaked, 0.8, 50, 1.0), (peaked, 1.0, 0, 0.9), (peaked, 0.7, 40, 0.8), (flat, 1.0, 0, 0.9), (flat, 1.0, 64, 0.5),
             (ties, 1.0, 40, 1.0), (ties, 0.9, 40, 0.7), (peaked, 1.0, 5000, 0.95), (peaked, 1.3, 3, 0.999), (peaked, 0.5, 0, 0.3),
             (peaked, 0.9, 0, 1.0), (flat, 1.4, 0, 1.0), (peaked, 0.0, 0, 1.0), (flat, 1.0, 1, 0.5)]
    lg = torch.stack([c[0] for c in cases]).to(dev())
    for rep in range(2):
        rows = [(t, k, p, 77 + i, rep * 5 + i) for i, (_, t, k, p) in enumerate(cases)]
        out = torch.empty(len(cases), dtype=torch.int32, device=dev())
        K().sample(lg, _params(rows), out)
        for i, (temp, k, p, seed, idx) in enumerate(rows):
            tok, kept = R.sample_row(lg[i], temp, k, p, seed, idx)
            assert out[i].item() == tok, f"case {i} {cases[i][1:]}: {out[i].item()} vs {tok} ({len(kept)} candidates)"


def test_sample_stays_in_candidates_and_follows_distribution():
    V = 50
    lg = rnd(1, V, seed=14, scale=1.5)
    n = 4000
    rows = [(1.0, 8, 0.95, 1000 + i, i) for i in range(n)]
    out = torch.empty(n, dtype=torch.int32, device=dev())
    K().sample(lg.expand(n, V).contiguous(), _params(rows), out)
    import plain_qwen2 as P
    ids, pr = P.plain_candidates(lg[0].cpu(), 1.0, 8, 0.95)
    counts = torch.bincount(out.cpu().long(), minlength=V).float()
    assert counts.sum() == n
    allowed = torch.zeros(V, dtype=torch.bool)
    allowed[ids] = True
    assert counts[~allowed].sum() == 0, "a token outside top-k / top-p was drawn"
    freq = counts[ids] / n
    # 4000 draws: standard error of a frequency is below 0.008
    assert (freq - pr).abs().max() < 0.04
