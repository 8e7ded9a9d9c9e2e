"""Each CUDA kernel alone against its plain torch reference, at sizes other than the engine tests'.

Inputs are built so that faults show: a far key among hundreds with a score that stands out, a key
just outside and just inside a window, keys on both sides of a page's edge, scattered pages.
"""
import math
from types import SimpleNamespace

import pytest
import torch

from emu_backend import EmuBackend

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def native():
    from hfcpu_b200 import kernels
    return kernels


@pytest.fixture
def both_tc_forms():
    """Lets small cases reach the attention kernel with two query tiles per CTA, which otherwise waits for enough
    CTAs to fill the SMs three times."""
    b = native().backend()
    old = b.tc2_min_rounds
    b.tc2_min_rounds = 0
    yield b
    b.tc2_min_rounds = old


def rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    V, E, T = 777, 200, 45
    table = rnd(V, E, dtype=DT[dtype])
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    out = torch.empty(T, E, device=DEV)
    native().embed(ids, table, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("E", [48, 200, 3584, 5000])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm(dtype, E):
    x = rnd(37, E, scale=3.0)
    w = rnd(E, dtype=DT[dtype]) + 1
    rows = torch.tensor([36, 0, 5, 5, 17], device=DEV, dtype=torch.int32)
    for r in (None, rows):
        M = 37 if r is None else 5
        out, ref = torch.empty(M, E, device=DEV, dtype=DT[dtype]), torch.empty(M, E, device=DEV, dtype=DT[dtype])
        native().rmsnorm(x, w, 1e-5, out, r)
        EmuBackend().rmsnorm(x, w, 1e-5, ref, r)
        assert rel(out.float(), ref.float()) < (1e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("E", [64, 1000, 3584, 5000, 8192, 8200])
def test_rmsnorm_many_rows(E):
    """From 64 rows on the bfloat16 form keeps a row in registers (up to 8,192 values): against float64."""
    x = rnd(200, E, scale=3.0)
    w = rnd(E, dtype=torch.bfloat16) + 1
    rows = torch.arange(199, 99, -1, device=DEV, dtype=torch.int32)
    for r in (None, rows):
        src = x if r is None else x[r.long()]
        out = torch.empty(src.shape[0], E, device=DEV, dtype=torch.bfloat16)
        native().rmsnorm(x, w, 1e-6, out, r)
        want = src.double() / torch.sqrt((src.double() ** 2).mean(-1, keepdim=True) + 1e-6) * w.double()
        assert rel(out.double(), want) < 5e-3
        assert torch.equal(out, want.float().to(torch.bfloat16)) or float((out.float() - want.float()).abs().max()) <= float(want.abs().max()) * 2 ** -7


@pytest.mark.parametrize("shape", [(1, 50, 70), (5, 130, 64), (67, 1000, 192), (130, 96, 333), (300, 257, 1030)])
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_linear(dtype, wdtype, shape):
    M, N, K = shape
    a, w = rnd(M, K, dtype=DT[dtype]), rnd(N, K, dtype=DT[wdtype], scale=0.1)
    bias = rnd(N, dtype=DT[wdtype])
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, device=DEV, dtype=DT[dtype])
    native().linear(a, w, bias, out, False)
    assert rel(out, ref + bias.double()) < (1e-5 if dtype == "float32" else 1e-2)
    res = rnd(M, N, seed=5)
    want = res.double() + ref
    native().linear(a, w, None, res, True)
    assert rel(res, want) < 1e-5
    logits = torch.empty(M, N, device=DEV)
    native().linear(a, w, None, logits, False)
    assert rel(logits, ref) < 1e-5


@pytest.mark.parametrize("geom", [(5, 1, 48, 48), (6, 3, 32, 16), (8, 8, 128, 128), (2, 2, 256, 64)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rope_kv_write(dtype, geom):
    H, G, d, n_rot = geom
    T, pages, bs, P = 23, 9, 4, 100
    dt = DT[dtype]
    qkv = rnd(T, (H + 2 * G) * d, dtype=dt)
    ang = torch.rand(P, n_rot // 2, device=DEV, dtype=torch.float64) * 6
    cos_sin = torch.stack([ang.cos(), ang.sin()], -1).float().contiguous()
    positions = torch.randint(0, P, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * bs, device=DEV)[:T].int()
    slots[3] = -1
    outs = []
    for impl in (native(), EmuBackend()):
        q = torch.zeros(T, H * d, device=DEV, dtype=dt)
        kc = torch.zeros(pages, bs, G, d, device=DEV, dtype=dt)
        vc = torch.zeros_like(kc)
        impl.rope_kv_write(qkv, cos_sin, n_rot, positions, slots, q, kc, vc, H, G, d)
        outs.append((q, kc, vc))
    tol = 1e-6 if dtype == "float32" else 1e-2
    for a, b in zip(*outs):
        assert rel(a.float(), b.float()) < tol
    q2 = torch.zeros(T, H * d, device=DEV, dtype=dt)
    kc2 = torch.zeros(pages, bs, G, d, device=DEV, dtype=dt)
    native().rope_kv_write(qkv, cos_sin, n_rot, positions, None, q2, kc2, kc2.clone(), H, G, d)
    assert torch.equal(q2, outs[0][0]) and not kc2.any()


def _attention_case(dtype, H, G, d, bs, lens_q, lens_kv, window, spike=None, seed=0):
    """Builds a paged cache with scattered pages for requests of ``lens_kv`` keys, the last ``lens_q`` of
    them being this step's queries.  ``spike = (request, key position, query offset)`` scales one key and one
    query so that their score stands out."""
    dt = DT[dtype]
    S = len(lens_q)
    MB = max((n + bs - 1) // bs for n in lens_kv)
    pages = sum((n + bs - 1) // bs for n in lens_kv) + 5
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pages, generator=g).tolist()
    table = torch.full((S, MB), -1, dtype=torch.int32)
    kc = rnd(pages, bs, G, d, dtype=dt, seed=seed + 1)
    vc = rnd(pages, bs, G, d, dtype=dt, seed=seed + 2)
    token_seq, positions = [], []
    for s in range(S):
        lo = max(0, lens_kv[s] - lens_q[s] - window + 1) if window > 0 else 0
        for b in range((lens_kv[s] + bs - 1) // bs):
            if b >= lo // bs:                      # blocks a window has passed stay unmapped
                table[s, b] = perm.pop()
        token_seq += [s] * lens_q[s]
        positions += list(range(lens_kv[s] - lens_q[s], lens_kv[s]))
    T = len(token_seq)
    q = rnd(T, H * d, dtype=dt, seed=seed + 3)
    if spike is not None:
        s, key_pos, q_off = spike
        t = sum(lens_q[:s]) + q_off
        page = int(table[s, key_pos // bs])
        assert page >= 0
        direction = torch.ones(d, device=DEV)
        kc[page, key_pos % bs] = (direction * 2).to(dt)
        q.view(T, H, d)[t] = (direction * 2).to(dt)
    meta = SimpleNamespace(block_table=table.to(DEV), block_size=bs, max_blocks=MB)
    ctx = SimpleNamespace(token_seq=torch.tensor(token_seq, dtype=torch.int32, device=DEV),
                          positions=torch.tensor(positions, dtype=torch.int32, device=DEV))
    return q, kc, vc, meta, ctx


def _run_attention(impl, case, H, G, d, window):
    q, kc, vc, meta, ctx = case
    out = torch.empty_like(q)
    impl.paged_attention(q, kc, vc, meta, ctx, H, G, d, window, 1.0 / math.sqrt(d), out, tiles=getattr(ctx, "tiles", None))
    return out


@pytest.mark.parametrize("geom", [(4, 2, 16, 16), (6, 3, 32, 8), (7, 7, 48, 4), (28, 4, 128, 16), (8, 1, 256, 32),
                                  (5, 5, 80, 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_mixed_batch(dtype, geom):
    H, G, d, bs = geom
    lens_q, lens_kv = [1, 40, 1, 7, 2], [300, 40, 1, 133, 64]
    for window in (0, 50):
        case = _attention_case(dtype, H, G, d, bs, lens_q, lens_kv, window)
        out, ref = _run_attention(native(), case, H, G, d, window), _run_attention(EmuBackend(), case, H, G, d, window)
        assert rel(out.float(), ref.float()) < TOL[dtype]
    from hfcpu_b200 import kernels
    kernels.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_far_key_and_page_edges(dtype):
    """One key among hundreds carries nearly all the weight; it sits at a page's first slot, last slot, the
    very first position and the query's own position in turn."""
    H, G, d, bs = 4, 2, 64, 16
    for key_pos in (0, 15, 16, 31, 303, 304, 599):
        case = _attention_case(dtype, H, G, d, bs, [1, 3], [200, 600], 0, spike=(1, key_pos, 2), seed=key_pos)
        out, ref = _run_attention(native(), case, H, G, d, 0), _run_attention(EmuBackend(), case, H, G, d, 0)
        assert rel(out.float(), ref.float()) < TOL[dtype], f"key {key_pos}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(dtype):
    """A key that would take all the weight lies just outside the window (must be ignored), then just inside."""
    H, G, d, bs, window = 4, 4, 32, 8, 40
    n = 100                                   # the single query sits at position 99 and sees keys 60..99
    for key_pos, inside in ((59, False), (60, True), (99, True)):
        # map the block of key 59 too, so that a kernel that reads one key too many finds the spike
        case = _attention_case(dtype, H, G, d, bs, [1], [n], 0, spike=(0, key_pos, 0), seed=7)
        out, ref = _run_attention(native(), case, H, G, d, window), _run_attention(EmuBackend(), case, H, G, d, window)
        assert rel(out.float(), ref.float()) < TOL[dtype], f"key {key_pos}"
        q, kc, vc, meta, ctx = case
        page = int(meta.block_table[0, key_pos // bs])
        spike_v = vc[page, key_pos % bs, 0].float()
        close = rel(out.view(1, H, d)[0, 0].float(), spike_v) < 0.05
        assert close == inside


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    T, F = 33, 999
    gu = rnd(T, 2 * F, dtype=DT[dtype], scale=3)
    out, ref = torch.empty(T, F, device=DEV, dtype=DT[dtype]), torch.empty(T, F, device=DEV, dtype=DT[dtype])
    for inter in (False, True):
        native().swiglu(gu, out, inter)
        EmuBackend().swiglu(gu, ref, inter)
        assert rel(out.float(), ref.float()) < (1e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("V", [151937, 152064, 4096, 4100, 37])
def test_argmax_lowest_index_wins(V):
    """Rows that allow 16-byte reads (a vocabulary that is a multiple of 4) and rows that do not; ties within a
    16-byte piece, across warps, across chunks; a row of equal values; the maximum in the last, short chunk."""
    logits = rnd(9, V)
    logits[2, V // 2] = logits[2, V - 7] = 50.0
    logits[3, 5] = logits[3, 4] = 60.0
    logits[4] = 1.0
    logits[5, V - 1] = 70.0
    logits[6, 33] = logits[6, 32] = logits[6, 31] = 55.0
    out = torch.empty(9, device=DEV, dtype=torch.int32)
    native().argmax(logits, out)
    assert out.tolist() == torch.argmax(logits, -1).tolist()
    assert out[2] == V // 2 and out[3] == 4 and out[4] == 0 and out[5] == V - 1 and out[6] == 31


def test_refuses_unsupported_head_dim():
    from hfcpu_b200.config.base import UnsupportedError
    with pytest.raises(UnsupportedError):
        native().check_head_dim(40)
    with pytest.raises(UnsupportedError):
        native().check_head_dim(512)


TC_SHAPES = [(1, 128, 64), (1, 3584, 3584), (8, 4608, 3584), (8, 3584, 18944), (16, 1000, 192), (17, 320, 72),
             (64, 3584, 2048), (100, 1000, 200), (128, 512, 512), (129, 256, 64), (130, 1000, 192), (300, 777 * 8, 136),
             (2048, 1024, 512), (1000, 4608, 3584), (5, 152064, 256),
             # from 256 rows on, pairs of CTAs share tiles of 256 rows (cta_group::2): edges of the pair's halves
             (256, 96, 64), (257, 136, 192), (384, 1000, 72), (511, 3000, 320), (1024, 208, 128), (640, 37888 // 8, 256),
             # a few hundred rows, few output tiles and a long inner dimension: split over K (one CTA, and pairs; ragged K)
             (192, 512, 4096), (300, 256, 4168), (384, 520, 1096), (512, 3584, 18944),
             # the o product at 2,048 tokens; ragged in every dimension with pairs
             (2048, 3584, 3584), (1100, 2000, 640), (768, 3000, 1096)]


@pytest.mark.parametrize("shape", TC_SHAPES)
def test_linear_tensor_core(shape):
    """bfloat16 x bfloat16 products on the tcgen05 kernel (both operand orders, split-K, ragged edges) against
    float64, and bit-for-bit stable from call to call."""
    from hfcpu_b200 import kernels
    assert kernels.backend().gemm == "tc"
    M, N, K = shape
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.05)
    bias = rnd(N, dtype=torch.bfloat16)
    ref = a.double() @ w.double().T
    scale = float(ref.abs().max())
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    native().linear(a, w, bias, out, False)
    err = float((out.double() - (ref + bias.double())).abs().max()) / float((ref + bias.double()).abs().max())
    assert err < 1e-2, f"bf16 store: {err}"
    logits = torch.empty(M, N, device=DEV)
    native().linear(a, w, None, logits, False)
    assert float((logits.double() - ref).abs().max()) / scale < 2e-5, "float32 store"
    again = torch.empty(M, N, device=DEV)
    native().linear(a, w, None, again, False)
    assert torch.equal(logits, again), "two calls differ"
    res = rnd(M, N, seed=5)
    want = res.double() + ref + bias.double()
    native().linear(a, w, bias, res, True)
    assert float((res.double() - want).abs().max()) / float(want.abs().max()) < 2e-5, "accumulate"
    plain_out = torch.empty(M, N, device=DEV)
    b = kernels.backend()
    b.gemm = "plain"
    try:
        native().linear(a, w, None, plain_out, False)
    finally:
        b.gemm = "tc"
    assert float((logits - plain_out).abs().max()) / scale < 2e-5, "differs from the plain kernel"
    kernels.check_device_errors()


def _with_tiles(case, lens_q, lens_kv, H, G, wide=False):
    """Adds what the tiled kernel needs to a case's context: the tile lists and the step's extents."""
    q, kc, vc, meta, ctx = case
    warps = 1 if max(lens_q) == 1 else (8 if wide else 4)
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)

    def tiling(per):
        t_seq, t_t0, t_nt, t0 = [], [], [], 0
        for s, n in enumerate(lens_q):
            for a in range(0, n, per):
                t_seq.append(s); t_t0.append(t0 + a); t_nt.append(min(per, n - a))
            t0 += n
        return {"seq": dev(t_seq), "t0": dev(t_t0), "nt": dev(t_nt)}
    ctx.tiles = {f"{warps}.{k}": v for k, v in tiling((16 * warps) // (H // G)).items()}
    if wide:                                                      # the kernel with two 128-row tiles per CTA
        ctx.tiles.update({f"16.{k}": v for k, v in tiling(2 * (128 // (H // G))).items()})
    ws = {}

    def buf(name, shape, dtype):
        return ws.setdefault((name, shape, dtype), torch.empty(shape, dtype=dtype, device=DEV))
    ctx.max_q_len, ctx.max_kv_len, ctx.buf = max(lens_q), max(lens_kv), buf
    return case


FAST_GEOMS = [(28, 4, 128, 16), (14, 2, 64, 16), (6, 3, 64, 8), (4, 4, 128, 64), (16, 1, 64, 4), (8, 2, 128, 32)]


@pytest.mark.parametrize("geom", FAST_GEOMS)
@pytest.mark.parametrize("window", [0, 50, 300])
def test_attention_tiled_mixed_and_decode(geom, window):
    """The tiled tensor-core kernel in both forms: portions beside decode tokens (4 warps), and pure decode
    with the keys split over CTAs (1 warp), against the torch reference and against the plain kernel."""
    from hfcpu_b200 import kernels
    H, G, d, bs = geom
    b = kernels.backend()
    for lens_q, lens_kv, wide in (([1, 70, 1, 7, 2, 130], [300, 70, 1, 133, 64, 700], False),
                                  ([1, 70, 1, 7, 2, 130], [300, 70, 1, 133, 64, 700], True),
                                  ([1, 1, 1, 1, 1], [1, 64, 65, 1000, 2311], False)):
        case = _with_tiles(_attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, window), lens_q, lens_kv, H, G, wide)
        b.launches = 0
        out = _run_attention(native(), case, H, G, d, window)
        ref = _run_attention(EmuBackend(), case, H, G, d, window)
        assert rel(out.float(), ref.float()) < TOL["bfloat16"], (lens_q, window)
        b.attention = "plain"
        try:
            plain_out = _run_attention(native(), case, H, G, d, window)
        finally:
            b.attention = "fast"
        assert rel(out.float(), plain_out.float()) < TOL["bfloat16"]
        again = _run_attention(native(), case, H, G, d, window)
        assert torch.equal(out, again), "two calls differ"
    kernels.check_device_errors()


def test_attention_tiled_far_key_window_edge_and_page_edges(both_tc_forms):
    H, G, d, bs = 28, 4, 128, 16
    for lens_q, lens_kv, spike_req in (([1, 1], [200, 600], 1), ([5, 40], [200, 600], 1)):
        for key_pos in (0, 15, 16, 63, 64, 303, 304, 559, 560, 599):
            q_off = lens_q[spike_req] - 1
            if key_pos > lens_kv[spike_req] - lens_q[spike_req] + q_off:
                continue
            for window in (0, 40):
                for wide in (False, True, "single"):  # wide: 128-row tiles, the tcgen05 kernels for prompt portions
                    case = _attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, 0, spike=(spike_req, key_pos, q_off), seed=key_pos)
                    case = _with_tiles(case, lens_q, lens_kv, H, G, bool(wide))
                    native().backend().attention_tc2 = wide != "single"
                    try:
                        out = _run_attention(native(), case, H, G, d, window)
                    finally:
                        native().backend().attention_tc2 = True
                    ref = _run_attention(EmuBackend(), case, H, G, d, window)
                    assert rel(out.float(), ref.float()) < TOL["bfloat16"], (lens_q, key_pos, window, wide)


@pytest.mark.parametrize("shape", [(1, 352, 64), (8, 37888, 3584), (5, 640, 192), (64, 2048, 512), (130, 640, 192),
                                   (300, 2048, 256), (2048, 4096, 512), (7, 352, 70)])
def test_linear_swiglu_fused(shape):
    """The product with the SwiGLU epilogue (both operand orders; odd K falls back to two kernels) against torch."""
    M, N, K = shape
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1)
    gu = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(M, N // 2, device=DEV, dtype=torch.bfloat16)
    native().linear_swiglu(a, w, gu, out)
    y = a.double() @ w.double().T
    g, u = y[:, 0::2], y[:, 1::2]
    ref = (g / (1 + torch.exp(-g))) * u
    assert rel(out, ref) < 1.5e-2


@pytest.mark.parametrize("shape", [(1, 3584, 3584), (8, 3584, 18944), (8, 192, 320), (64, 3584, 512), (128, 1000, 64),
                                   (200, 512, 256), (5, 64, 44), (200, 512, 4096), (512, 200, 4104), (320, 1000, 1032)])
@pytest.mark.parametrize("with_norm", [True, False])
def test_linear_residual_norm_fused(shape, with_norm):
    M, N, K = shape
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1)
    bias, nw = rnd(N, dtype=torch.bfloat16), rnd(N, dtype=torch.bfloat16) + 1
    res = rnd(M, N, seed=3)
    res_ref = res.double() + a.double() @ w.double().T + bias.double()
    xn = torch.empty(M, N, device=DEV, dtype=torch.bfloat16) if with_norm else None
    native().linear_residual_norm(a, w, bias, res, nw if with_norm else None, 1e-6, xn)
    assert rel(res, res_ref) < 2e-5
    if with_norm:
        r = 1 / torch.sqrt((res_ref ** 2).mean(-1, keepdim=True) + 1e-6)
        assert rel(xn, res_ref * r * nw.double()) < 1e-2


@pytest.mark.parametrize("geom", [(28, 4, 128, 3584, 8), (6, 3, 32, 192, 5), (4, 2, 16, 64, 1), (8, 8, 64, 512, 130), (5, 1, 48, 100, 3),
                                  (28, 4, 128, 3584, 512), (4, 2, 64, 4096, 200),
                                  # 256 tokens and more: rotation and cache write in the epilogue of the pair kernel (tiles of
                                  # whole heads; a last tile half outside the row; ragged token counts; head size 64)
                                  (28, 4, 128, 3584, 2048), (6, 2, 128, 256, 257), (14, 2, 64, 896, 300), (5, 5, 64, 136, 640)])
def test_linear_rope_kv_fused(geom):
    from hfcpu_b200 import kernels
    H, G, d, K, T = geom
    N = (H + 2 * G) * d
    a, w, bias = rnd(T, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.1), rnd(N, dtype=torch.bfloat16)
    pages, bs, P = max(40, T // 4 + 8), 4, 64
    ang = torch.rand(P, d // 2, device=DEV, dtype=torch.float64) * 6
    cos_sin = torch.stack([ang.cos(), ang.sin()], -1).float().contiguous()
    positions = torch.randint(0, P, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * bs, device=DEV)[:T].int()
    slots[::7] = -1                                      # tokens that are not cached
    outs = []
    b = kernels.backend()
    for impl, in_epilogue in ((native(), True), (native(), False), (EmuBackend(), False)):
        qkv = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        q = torch.zeros(T, H * d, device=DEV, dtype=torch.bfloat16)
        kc = torch.zeros(pages, bs, G, d, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        b.rope_in_epilogue = in_epilogue
        before = b.launches
        try:
            impl.linear_rope_kv(a, w, bias, qkv, cos_sin, d, positions, slots, q, kc, vc, H, G, d)
        finally:
            b.rope_in_epilogue = True
        if impl is native() and T >= 256 and d in (64, 128):
            assert b.launches - before == (1 if in_epilogue else 2)
        outs.append((q, kc, vc))
    for x, y, z in zip(*outs):
        assert torch.equal(x, y), "the product's epilogue and the separate kernel differ"
        assert rel(x.float(), z.float()) < 1.5e-2
    kernels.check_device_errors()


@pytest.mark.parametrize("geom", [(28, 4, 128, 16), (4, 4, 128, 8), (16, 1, 128, 128), (5, 5, 128, 32),
                                  (14, 2, 64, 16), (6, 3, 64, 8), (8, 8, 64, 64), (3, 1, 64, 128)])
def test_attention_tensor_core_prompt_portions(geom, both_tc_forms):
    """The tcgen05 attention kernels (head_dim 128 in both forms, two query tiles per CTA and one; head_dim 64 in the
    first): long portions over long histories, several requests, windows, against the torch reference and against
    the mma.sync kernel."""
    from hfcpu_b200 import kernels
    H, G, d, bs = geom
    b = kernels.backend()
    assert b.attention_tc and b.attention_tc2
    for lens_q, lens_kv in (([300, 1, 40], [300, 900, 417]), ([130, 64], [700, 64]), ([2, 1], [2, 1])):
        for window in (0, 100):
            case = _with_tiles(_attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, window, seed=len(lens_q)), lens_q, lens_kv, H, G, wide=True)
            out = _run_attention(native(), case, H, G, d, window)          # two query tiles per CTA
            ref = _run_attention(EmuBackend(), case, H, G, d, window)
            assert rel(out.float(), ref.float()) < TOL["bfloat16"], (lens_q, window)
            b.attention_tc2 = False
            try:
                single = _run_attention(native(), case, H, G, d, window)   # one query tile per CTA
            finally:
                b.attention_tc2 = True
            assert rel(single.float(), ref.float()) < TOL["bfloat16"], (lens_q, window)
            b.attention_tc = False
            try:
                other = _run_attention(native(), case, H, G, d, window)
            finally:
                b.attention_tc = True
            assert rel(out.float(), other.float()) < TOL["bfloat16"]
            again = _run_attention(native(), case, H, G, d, window)
            assert torch.equal(out, again)
    kernels.check_device_errors()


@pytest.mark.parametrize("geom", [(28, 4, 128, 16), (14, 2, 64, 16)])
@pytest.mark.parametrize("lens_q", [[1, 1], [1, 300]])
def test_attention_long_context_far_keys(lens_q, geom, both_tc_forms):
    """33,000 cached keys: a decode token (the keys split over many CTAs) and a 300-token portion (hundreds of
    tiles per query tile), with one key made to stand out near the start, in the middle and at the very end."""
    H, G, d, bs = geom
    lens_kv = [700, 33000]
    for key_pos in (3, 16384, 32999 - (lens_q[1] - 1)):
        q_off = 0 if key_pos > 30000 else lens_q[1] - 1
        case = _attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, 0, spike=(1, key_pos, q_off), seed=7)
        case = _with_tiles(case, lens_q, lens_kv, H, G, wide=True)
        out, ref = _run_attention(native(), case, H, G, d, 0), _run_attention(EmuBackend(), case, H, G, d, 0)
        assert rel(out.float(), ref.float()) < TOL["bfloat16"], (lens_q, key_pos)
        t = sum(lens_q[:1]) + q_off
        row = out.view(-1, H, d)[t].float()
        assert rel(row, ref.view(-1, H, d)[t].float()) < TOL["bfloat16"]
    from hfcpu_b200 import kernels
    kernels.check_device_errors()


@pytest.mark.parametrize("geom", [(28, 4, 128, 16), (14, 2, 64, 16), (40, 8, 128, 32), (6, 3, 64, 8)])
def test_attention_short_portions_over_long_context(geom):
    """Portions of 2 to 63 tokens behind thousands of cached keys (the end of a prompt, a prompt behind a shared
    prefix) beside single tokens: their keys are split over CTAs and merged; one key far back made to stand out."""
    from hfcpu_b200 import kernels
    H, G, d, bs = geom
    b = kernels.backend()
    for lens_q, lens_kv in (([9], [3000]), ([2, 33, 1], [9000, 1500, 700]), ([63], [8200])):
        for window, key_pos in ((0, 5), (0, lens_kv[0] - lens_q[0]), (300, lens_kv[0] - lens_q[0] - 250)):
            case = _attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, window, spike=(0, key_pos, lens_q[0] - 1), seed=key_pos)
            case = _with_tiles(case, lens_q, lens_kv, H, G)
            before = b.launches
            out = _run_attention(native(), case, H, G, d, window)
            assert b.launches - before == 2, "the keys were split (attention and merge)"
            ref = _run_attention(EmuBackend(), case, H, G, d, window)
            assert rel(out.float(), ref.float()) < TOL["bfloat16"], (lens_q, window, key_pos)
            assert torch.equal(out, _run_attention(native(), case, H, G, d, window)), "two calls differ"
    kernels.check_device_errors()


@pytest.mark.parametrize("geom", [(28, 4, 128, 16), (14, 2, 64, 16), (8, 2, 128, 32), (16, 1, 64, 8)])
def test_decode_attention_merges_its_own_splits(geom):
    """The decode kernel with the keys split over CTAs: merged by the CTA that stores a tile's last split, it gives
    what the separate merge kernel gives, in one launch, and leaves its counters at zero."""
    from hfcpu_b200 import kernels
    H, G, d, bs = geom
    b = kernels.backend()
    for lens_kv in ([1, 64, 65, 1000, 2311], [2048] * 8, [700]):
        lens_q = [1] * len(lens_kv)
        for window in (0, 300):
            case = _with_tiles(_attention_case("bfloat16", H, G, d, bs, lens_q, lens_kv, window), lens_q, lens_kv, H, G)
            ref = _run_attention(EmuBackend(), case, H, G, d, window)
            before = b.launches
            out = _run_attention(native(), case, H, G, d, window)
            assert b.launches - before == 1, "one kernel, no separate merge"
            again = _run_attention(native(), case, H, G, d, window)
            b.merge_in_kernel = False
            try:
                apart = _run_attention(native(), case, H, G, d, window)
            finally:
                b.merge_in_kernel = True
            assert torch.equal(out, again) and rel(out.float(), ref.float()) < 3e-2
            assert rel(out.float(), apart.float()) < 1e-2
            assert int(b._counters.abs().sum()) == 0
    kernels.check_device_errors()
