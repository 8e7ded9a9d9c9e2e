"""The few-row products that finish themselves: the CTA that stores a weight tile's last split sums the splits and does
the step after the product (residual + next norm's weights + sums of squares; bias + rotary + cache write), and the
products that apply a deferred RMSNorm row factor to their accumulators.  Each against torch in float64, at sizes
other than the engine's, twice in a row (the tile counters must be back at zero), and against the separate kernels."""
import math

import pytest
import torch

from emu_backend import EmuBackend

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(dtype)


def rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


SHAPES = [(1, 3584, 3584), (8, 3584, 18944), (8, 3584, 3584), (5, 1000, 192), (64, 3584, 2048), (128, 512, 512), (3, 136, 72),
          (17, 5120, 5120), (33, 896, 4864)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_residual_and_deferred_norm_in_the_products_own_kernel(shape, with_bias):
    from hfcpu_b200 import kernels
    b = kernels.backend()
    assert b.fuse_tails
    M, N, K = shape
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias = rnd(N, dtype=torch.bfloat16, seed=2) if with_bias else None
    norm_w = (1 + 0.1 * rnd(N, seed=3)).to(torch.bfloat16)
    res0 = rnd(M, N, seed=4)
    want = res0.double() + a.double() @ w.double().T + (bias.double() if with_bias else 0)
    eps = 1e-5
    outs = []
    for call in range(2):
        res, y = res0.clone(), torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        before = b.launches
        sumsq = kernels.linear_residual_norm(a, w, bias, res, norm_w, eps, y, defer=True)
        assert sumsq is not None and b.launches - before == 1, "one kernel"
        assert rel(res, want) < 2e-5
        assert rel(y.float(), want * norm_w.double()) < 1e-2
        assert rel(sumsq.double().sum(0), (res.double() ** 2).sum(1)) < 1e-5
        outs.append((res, y.clone(), sumsq.clone()))
    assert all(torch.equal(x, z) for x, z in zip(*outs)), "two calls differ"
    assert int(b._counters.abs().sum()) == 0
    # the rows with their factor are what the separate kernels give
    full = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    res2 = res0.clone()
    assert kernels.linear_residual_norm(a, w, bias, res2, norm_w, eps, full) is None
    assert torch.equal(res2, outs[0][0]) or rel(res2, outs[0][0]) < 1e-6
    kernels.scale_rows(outs[0][1], (outs[0][2], eps))
    assert rel(outs[0][1].float(), full.float()) < 1.6e-2
    # without a norm: plain accumulation, also one kernel
    res3 = res0.clone()
    before = b.launches
    kernels.linear(a, w, bias, res3, True)
    assert b.launches - before == 1 and rel(res3, want) < 2e-5
    kernels.check_device_errors()


@pytest.mark.parametrize("shape", [(8, 37888, 3584), (1, 1000, 192), (64, 9728, 896), (100, 640, 256), (128, 2 * 456, 256)])
def test_swiglu_product_applies_the_row_factor(shape):
    from hfcpu_b200 import kernels
    M, N, K = shape
    x = rnd(M, K, scale=3.0)
    norm_w = 1 + 0.1 * rnd(K, seed=3)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    parts = 7
    eps = 1e-6
    split = torch.rand(parts, M, device=DEV)
    sumsq = ((x.double() ** 2).sum(1)[None, :] * (split / split.sum(0))).float().contiguous()
    y = (x * norm_w).to(torch.bfloat16)                                   # the rows without their factor
    r = 1.0 / torch.sqrt((x.double() ** 2).sum(1) / K + eps)
    ref = (y.double() * r[:, None]) @ w.double().T
    g, u = ref[:, 0::2], ref[:, 1::2]
    want = (g / (1 + torch.exp(-g))) * u
    out = torch.empty(M, N // 2, device=DEV, dtype=torch.bfloat16)
    gu = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    kernels.linear_swiglu(y, w, gu, out, row_scale=(sumsq, eps))
    assert rel(out.float(), want) < 1.5e-2
    again = torch.empty_like(out)
    kernels.linear_swiglu(y, w, gu, again, row_scale=(sumsq, eps))
    assert torch.equal(out, again)
    kernels.check_device_errors()


@pytest.mark.parametrize("geom", [(28, 4, 128, 3584), (14, 2, 64, 896), (6, 3, 32, 192), (4, 2, 16, 64), (40, 8, 128, 5120), (5, 5, 64, 320)])
@pytest.mark.parametrize("M", [1, 8, 33, 128])
@pytest.mark.parametrize("scaled", [False, True])
def test_qkv_product_with_rotary_and_cache_write(geom, M, scaled):
    from hfcpu_b200 import kernels
    H, G, d, E = geom
    b = kernels.backend()
    N = (H + 2 * G) * d
    bs, pages = 16, (M + 15) // 16 + 3
    n_rot = d if d != 32 else 16                                         # a partial rotation too
    npos = 500
    ang = torch.arange(npos, dtype=torch.float64)[:, None] * (10000.0 ** (-2.0 * torch.arange(n_rot // 2, dtype=torch.float64) / n_rot))[None, :]
    cos_sin = torch.stack([ang.cos(), ang.sin()], -1).float().contiguous().to(DEV)
    g = torch.Generator().manual_seed(M)
    positions = torch.randint(0, npos, (M,), generator=g).int().to(DEV)
    slots = torch.randperm(pages * bs, generator=g)[:M].int().to(DEV)
    if M > 2:
        slots[1] = -1                                                      # a token whose keys are not kept
    x = rnd(M, E, scale=2.0)
    norm_w = 1 + 0.1 * rnd(E, seed=3)
    w = rnd(N, E, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    eps = 1e-6
    if scaled:
        a = (x * norm_w).to(torch.bfloat16)
        parts = 5
        split = torch.rand(parts, M, device=DEV)
        row_scale = (((x.double() ** 2).sum(1)[None, :] * (split / split.sum(0))).float().contiguous(), eps)
    else:
        a, row_scale = x.to(torch.bfloat16), None
    outs = []
    for impl in ("native", "native", "emu"):
        q = torch.zeros(M, H * d, device=DEV, dtype=torch.bfloat16)
        kc = torch.zeros(pages, bs, G, d, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        qkv = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        if impl == "native":
            before = b.launches
            kernels.linear_rope_kv(a, w, bias, qkv, cos_sin, n_rot, positions, slots, q, kc, vc, H, G, d, row_scale=row_scale)
            assert b.launches - before == 1, "one kernel"
        else:
            EmuBackend().linear_rope_kv(a.clone(), w, bias, qkv, cos_sin, n_rot, positions, slots, q, kc, vc, H, G, d, row_scale=row_scale)
        outs.append((q, kc, vc))
    assert all(torch.equal(x_, y_) for x_, y_ in zip(outs[0], outs[1])), "two calls differ"
    for x_, y_ in zip(outs[0], outs[2]):
        assert rel(x_.float(), y_.float()) < 1.6e-2
    assert int(b._counters.abs().sum()) == 0
    kernels.check_device_errors()


def test_fused_tails_equal_the_separate_kernels_through_the_engine(tiny_folders):
    """Config C (head size 128, tensor-core sizes) decoded with the tails in the products' kernels and as separate
    kernels: the logits agree to bfloat16 rounding, and generation is the same from run to run."""
    import hfcpu_b200
    from hfcpu_b200 import StepEntry, kernels
    from conftest import make_requests
    b = kernels.backend()
    model = hfcpu_b200.load_model(tiny_folders["C16"], torch.bfloat16, "cuda:0")
    reqs = make_requests("C", [70, 9, 200], seed=3)

    def run(fused):
        b.fuse_tails = fused
        try:
            eng = hfcpu_b200.Engine(model, block_size=16, max_tokens=1024, max_requests=4)
            rows = []
            for r, ids in reqs.items():
                eng.add_request(r)
                rows.append(eng.step([StepEntry(r, ids, [len(ids) - 1])]).clone())
            toks = {r: ids[0] for r, ids in reqs.items()}
            for _ in range(4):
                rows.append(eng.step([StepEntry(r, [toks[r]], [0]) for r in reqs]).clone())
            return torch.cat(rows)
        finally:
            b.fuse_tails = True
    fused, again, apart = run(True), run(True), run(False)
    assert torch.equal(fused, again)
    assert rel(fused, apart) < 2e-2
    kernels.check_device_errors()


@pytest.mark.parametrize("geom", [(28, 4, 128, 16), (14, 2, 64, 16), (8, 2, 128, 32), (16, 1, 64, 8)])
def test_decode_attention_merges_its_own_splits(geom):
    """The decode kernel with the keys split over CTAs: merged by the CTA that stores a tile's last split, it gives
    what the separate merge kernel gives, in one launch, and leaves its counters at zero."""
    from hfcpu_b200 import kernels
    from test_gpu_kernels import _attention_case, _run_attention, _with_tiles
    H, G, d, bs = geom
    b = kernels.backend()
    for lens_kv in ([1, 64, 65, 1000, 2311], [2048] * 8, [700]):
        lens_q = [1] * len(lens_kv)
        for window in (0, 300):
            case = _with_tiles(_attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, window), lens_q, lens_kv, H, G)
            ref = _run_attention(EmuBackend(), case, H, G, d, window)
            before = b.launches
            out = _run_attention(kernels, case, H, G, d, window)
            assert b.launches - before == 1, "one kernel, no separate merge"
            again = _run_attention(kernels, case, H, G, d, window)
            b.fuse_tails = False
            try:
                apart = _run_attention(kernels, case, H, G, d, window)
            finally:
                b.fuse_tails = True
            assert torch.equal(out, again) and rel(out.float(), ref.float()) < 3e-2
            assert rel(out.float(), apart.float()) < 1e-2
            assert int(b._counters.abs().sum()) == 0
    kernels.check_device_errors()
