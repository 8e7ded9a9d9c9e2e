// Attention over the paged cache for bfloat16, tiled, with tensor-core products (mma.sync m16n8k16).
//
// The same arithmetic as the plain kernel (scores = q.k * scale, causal and window masks by absolute
// position, float32 softmax, weighted values; src/model.c:499-528) in flash-attention form: keys are
// visited in tiles of 64 with a running maximum and sum per row, so no score vector is stored.
// The query heads that share a key/value head are packed into one tile's rows (row = token * r + head
// within the group), so every key and value is read once per group, in decode as in prefill.
//   * WARPS = 4 (64 rows): prompt portions and mixed batches, one CTA per (tile of tokens, kv head).
//   * WARPS = 1 (16 rows): pure decode, one CTA per (request, kv head, split of the keys); the splits'
//     partial results (maximum, sum, unnormalised output) are merged by a second kernel in split order,
//     so the result does not depend on how many CTAs ran at once.
// Keys and values arrive by cp.async (16-byte chunks, zero fill for unmapped or out-of-range keys) into
// swizzled shared memory, double buffered; fragments are read with ldmatrix.
#include "attention_common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

template <int D, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
attention_fast_kernel(AttnParams p, int *err)
{
    HFB_TRACE_ENTRY(12);
    pdl_sync();
    constexpr int BM = 16 * WARPS, CH = D / 8, NT = WARPS * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sq = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sk = sq + BM * D * 2, sv = sk + STAGES * ABN * D * 2;      // K and V: STAGES tiles each
    // tiles late in a prompt see the most keys: hand them out first, so that the last CTAs to start are short ones
    const int tile = gridDim.x - 1 - blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = p.H / p.G;
    const int seq = p.tile_seq[tile], t0 = p.tile_t0[tile], nt = p.tile_nt[tile];
    const int32_t *table = p.block_table + (size_t)seq * p.max_blocks;
    const int pos_first = p.positions[t0], pos_last = p.positions[t0 + nt - 1];
    const int lo_all = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    int kt_lo = lo_all / ABN, kt_hi = pos_last / ABN + 1;                 // key tiles [kt_lo, kt_hi)
    if (p.splits > 1) {
        int per = (kt_hi - kt_lo + p.splits - 1) / p.splits;
        kt_lo = kt_lo + split * per;
        kt_hi = min(kt_hi, kt_lo + per);
    }

    // ---- queries: rows (token, head in group) -> swizzled shared memory -------------------------
    for (int i = threadIdx.x; i < BM * CH; i += NT) {
        int row = i / CH, c = i % CH;
        int tl = row / r, hl = row % r;
        bool valid = tl < nt;
        const __nv_bfloat16 *src = p.q + ((size_t)(t0 + (valid ? tl : 0)) * p.H + g * r + hl) * D + c * 8;
        cp_async16(sq + swz<D>(row, c), src, valid);
    }
    cp_async_commit();

    auto load_kv = [&](int kt, int stage) {
        for (int i = threadIdx.x; i < ABN * CH; i += NT) {
            int kr = i / CH, c = i % CH;
            int key = kt * ABN + kr;
            int blk = key / p.block_size;
            long long page = (key <= pos_last && blk < p.max_blocks) ? table[blk] : -1;
            bool valid = page >= 0 && page < p.num_pages;
            size_t off = valid ? (((size_t)page * p.block_size + key % p.block_size) * p.G + g) * D + c * 8 : 0;
            cp_async16(sk + stage * (ABN * D * 2) + swz<D>(kr, c), p.k_cache + off, valid);
            cp_async16(sv + stage * (ABN * D * 2) + swz<D>(kr, c), p.v_cache + off, valid);
        }
        cp_async_commit();
    };

    // the first STAGES - 1 tiles are requested up front; one commit group per tile, empty where there is none
#pragma unroll
    for (int st = 0; st < STAGES - 1; st++) {
        if (kt_lo + st < kt_hi) load_kv(kt_lo + st, st);
        else cp_async_commit();
    }

    // this thread's two rows of the warp's 16: lane/4 and lane/4 + 8
    const int row0 = warp * 16 + (lane >> 2), row1 = row0 + 8;
    const int tl0 = row0 / r, tl1 = row1 / r;
    const bool v0 = tl0 < nt, v1 = tl1 < nt;
    const int pos0 = v0 ? p.positions[t0 + tl0] : -1, pos1 = v1 ? p.positions[t0 + tl1] : -1;
    const int lo0 = p.window > 0 ? max(0, pos0 - p.window + 1) : 0, lo1 = p.window > 0 ? max(0, pos1 - p.window + 1) : 0;

    const bool warp_active = warp * 16 < nt * r;      // a warp whose 16 rows are all padding only helps with the loads
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t qf[D / 16][4];
    bool q_loaded = false;

    for (int kt = kt_lo; kt < kt_hi; kt++) {
        const int stage = (kt - kt_lo) % STAGES;
        if (kt + STAGES - 1 < kt_hi) load_kv(kt + STAGES - 1, (kt + STAGES - 1 - kt_lo) % STAGES);
        else cp_async_commit();
        cp_async_wait<STAGES - 1>();              // everything but the newest STAGES - 1 groups: tile kt has landed
        __syncthreads();
        if (!warp_active) { __syncthreads(); continue; }
        if (!q_loaded) {
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++)
                ldsm_x4(sq + swz<D>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            q_loaded = true;
        }
        const uint32_t ks = sk + stage * (ABN * D * 2), vs = sv + stage * (ABN * D * 2);
        float s[ABN / 8][4];
#pragma unroll
        for (int i = 0; i < ABN / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
            for (int nj = 0; nj < ABN / 16; nj++) {
                uint32_t b0, b1, b2, b3;
                int mi = lane >> 3;
                ldsm_x4(ks + swz<D>(nj * 16 + (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)), b0, b1, b2, b3);
                mma_bf16(s[2 * nj], qf[kk], b0, b1);
                mma_bf16(s[2 * nj + 1], qf[kk], b2, b3);
            }
        }
        // scale, mask by absolute position, running maximum.  A tile whose keys every row may see (all below the
        // tile's first position and inside every window) needs no per-element test.
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const bool all_visible = v0 && v1 && kt * ABN + ABN - 1 <= pos_first &&
                                 (p.window == 0 || kt * ABN >= max(0, pos_last - p.window + 1));
        if (all_visible) {
#pragma unroll
            for (int i = 0; i < ABN / 8; i++) {
#pragma unroll
                for (int e = 0; e < 4; e++) s[i][e] *= p.scale_log2;
                mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
                mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < ABN / 8; i++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    int key = kt * ABN + i * 8 + (lane & 3) * 2 + e;
                    float a = s[i][e] * p.scale_log2, b = s[i][2 + e] * p.scale_log2;
                    a = (v0 && key >= lo0 && key <= pos0) ? a : -INFINITY;
                    b = (v1 && key >= lo1 && key <= pos1) ? b : -INFINITY;
                    s[i][e] = a; s[i][2 + e] = b;
                    mx0 = fmaxf(mx0, a); mx1 = fmaxf(mx1, b);
                }
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;     // rows with no key yet
        float c0 = fast_exp2(m0 - base0), c1 = fast_exp2(m1 - base1);                                   // exp2(-inf) = 0
        m0 = mn0; m1 = mn1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pf[ABN / 16][4];
#pragma unroll
        for (int i = 0; i < ABN / 8; i++) {
            float p00 = fast_exp2(s[i][0] - base0), p01 = fast_exp2(s[i][1] - base0);
            float p10 = fast_exp2(s[i][2] - base1), p11 = fast_exp2(s[i][3] - base1);
            sum0 += p00 + p01; sum1 += p10 + p11;
            pf[i >> 1][(i & 1) * 2] = pack_bf16(p00, p01);
            pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * c0 + sum0; l1 = l1 * c1 + sum1;
#pragma unroll
        for (int i = 0; i < D / 8; i++) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
#pragma unroll
        for (int kk = 0; kk < ABN / 16; kk++) {
#pragma unroll
            for (int dn = 0; dn < D / 16; dn++) {
                uint32_t b0, b1, b2, b3;
                int mi = lane >> 3;
                ldsm_x4_t(vs + swz<D>(kk * 16 + (mi & 1) * 8 + (lane & 7), dn * 2 + (mi >> 1)), b0, b1, b2, b3);
                mma_bf16(o[2 * dn], pf[kk], b0, b1);
                mma_bf16(o[2 * dn + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();                         // the stage is free for the load after next
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

#pragma unroll
    for (int half = 0; half < 2; half++) {
        const bool valid = half ? v1 : v0;
        if (!valid) continue;
        const int row = half ? row1 : row0;
        const int tok = t0 + row / r, head = g * r + row % r;
        const float l = half ? l1 : l0, m = half ? m1 : m0;
        const size_t th = (size_t)tok * p.H + head;
        if (p.splits > 1) {
            float *po = p.part_o + (th * p.splits + split) * D;
#pragma unroll
            for (int i = 0; i < D / 8; i++)
                *(float2 *)(po + i * 8 + (lane & 3) * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
            if ((lane & 3) == 0) *(float2 *)(p.part_ml + (th * p.splits + split) * 2) = make_float2(m, l);
        } else {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            __nv_bfloat16 *dst = p.out + th * D;
#pragma unroll
            for (int i = 0; i < D / 8; i++)
                *(uint32_t *)(dst + i * 8 + (lane & 3) * 2) = pack_bf16(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
        }
    }
}

// Merges the splits of one (token, head) in split order: out = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s.
// One thread per column; the reads of a column's splits are issued sixteen at a time, because their latency is all
// that this kernel costs.
template <int D>
__global__ void attention_combine_kernel(const float *part_o, const float *part_ml, int splits, __nv_bfloat16 *out)
{
    HFB_TRACE_ENTRY(4);
    pdl_sync();
    const size_t th = blockIdx.x;
    const float2 *ml = (const float2 *)(part_ml + th * splits * 2);
    const float *po = part_o + th * splits * D + threadIdx.x;
    float m = -INFINITY;
    for (int c = 0; c < splits; c += 16) {
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; i++) x[i] = c + i < splits ? ml[c + i].x : -INFINITY;
#pragma unroll
        for (int i = 0; i < 16; i++) m = fmaxf(m, x[i]);
    }
    float denom = 0.f, acc = 0.f;
    for (int c = 0; c < splits; c += 16) {
        float v[16];
        float2 w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const bool in = c + i < splits;
            w[i] = in ? ml[c + i] : make_float2(-INFINITY, 0.f);
            v[i] = in ? po[(size_t)(c + i) * D] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float f = w[i].x == -INFINITY ? 0.f : exp2f(w[i].x - m);
            denom += w[i].y * f;
            acc += v[i] * f;
        }
    }
    out[th * D + threadIdx.x] = __float2bfloat16_rn(acc * (denom > 0.f ? 1.0f / denom : 0.f));
    HFB_TRACE_MARK(4);
}

template <int D, int WARPS, int STAGES>
static int launch_attention(const AttnParams &p, int n_tiles, cudaStream_t st)
{
    constexpr int smem = (16 * WARPS + 2 * STAGES * ABN) * D * 2;
    static bool configured[64] = {false};                 // (the opt-in is a property of the function on one device)
    if (!configured[current_device()]) {
        cudaError_t e = cudaFuncSetAttribute(attention_fast_kernel<D, WARPS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "attention: cannot opt in to %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[current_device()] = true;
    }
    dim3 grid(n_tiles, p.G, p.splits);
    g_launch_err = launch_pdl(attention_fast_kernel<D, WARPS, STAGES>, dim3(grid), dim3(WARPS * 32), smem, st, p, error_word());
    return check_pdl_launch(g_launch_err, "attention_fast");
}

int launch_attention_combine(const AttnParams &p, int T, int d, cudaStream_t st)
{
    const dim3 grid((unsigned)((size_t)T * p.H));
    if (d == 128) g_launch_err = launch_pdl(attention_combine_kernel<128>, grid, dim3(128), 0, st, p.part_o, p.part_ml, p.splits, p.out);
    else g_launch_err = launch_pdl(attention_combine_kernel<64>, grid, dim3(64), 0, st, p.part_o, p.part_ml, p.splits, p.out);
    return check_pdl_launch(g_launch_err, "attention_combine");
}

}  // namespace hfb

using namespace hfb;

// Tokens per tile of the fast kernel with `warps` warps when r query heads share a key/value head (0: not supported).
extern "C" int hfb_attention_fast_tile_tokens(int H, int G, int warps)
{
    if (G <= 0 || H % G) return 0;
    int r = H / G, rows = 16 * warps;
    return r <= rows ? rows / r : 0;
}

// Float32 scratch (bytes) that `splits` > 1 need for T tokens.
extern "C" size_t hfb_attention_fast_scratch(int T, int H, int d, int splits)
{
    return splits > 1 ? (size_t)T * H * splits * (d + 2) * sizeof(float) : 0;
}

extern "C" int hfb_attention_fast(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                                  int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                                  const int32_t *tile_nt, int n_tiles, int warps, int stages, int splits, int block_size,
                                  int64_t num_pages, int window, float scale, void *out, void *scratch, size_t scratch_bytes,
                                  int T, int H, int G, int d, hfb_stream s)
{
    if (n_tiles <= 0) return HFB_OK;
    if (d != 64 && d != 128) return fail(HFB_ENOTSUP, "attention_fast: head_dim %d (64 and 128 only; use the plain kernel)", d);
    if (warps != 1 && warps != 4 && warps != 8) return fail(HFB_EINVAL, "attention_fast: 1, 4 or 8 warps");
    if (block_size <= 0 || ABN % block_size) return fail(HFB_ENOTSUP, "attention_fast: block size %d does not divide %d", block_size, ABN);
    if (hfb_attention_fast_tile_tokens(H, G, warps) == 0) return fail(HFB_ENOTSUP, "attention_fast: %d heads per key/value head do not fit a tile", G ? H / G : 0);
    if (splits < 1 || G > 65535 || splits > 65535) return fail(HFB_EINVAL, "attention_fast: bad split or group count");
    if (splits > 1 && (!scratch || scratch_bytes < hfb_attention_fast_scratch(T, H, d, splits)))
        return fail(HFB_EINVAL, "attention_fast: scratch of %zu bytes is too small for %d splits", scratch_bytes, splits);
    AttnParams p;
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.block_table = block_table; p.positions = positions;
    p.tile_seq = tile_seq; p.tile_t0 = tile_t0; p.tile_nt = tile_nt;
    p.part_o = (float *)scratch; p.part_ml = splits > 1 ? (float *)scratch + (size_t)T * H * splits * d : nullptr;
    p.max_blocks = max_blocks; p.block_size = block_size; p.window = window; p.H = H; p.G = G; p.splits = splits;
    p.num_pages = num_pages; p.scale_log2 = scale * 1.4426950408889634f;
    p.counters = nullptr;
    cudaStream_t st = (cudaStream_t)s;
    int rc;
    const bool deep = stages >= 4;              // a deeper pipeline for CTAs that have an SM to themselves (decode)
    if (d == 128) rc = warps == 8 ? launch_attention<128, 8, 2>(p, n_tiles, st)
                     : warps == 4 ? (deep ? launch_attention<128, 4, 4>(p, n_tiles, st) : launch_attention<128, 4, 2>(p, n_tiles, st))
                                  : launch_attention<128, 1, 2>(p, n_tiles, st);
    else rc = warps == 8 ? launch_attention<64, 8, 2>(p, n_tiles, st)
            : warps == 4 ? (deep ? launch_attention<64, 4, 4>(p, n_tiles, st) : launch_attention<64, 4, 2>(p, n_tiles, st))
                         : launch_attention<64, 1, 2>(p, n_tiles, st);
    if (rc != HFB_OK || splits == 1) return rc;
    return launch_attention_combine(p, T, d, st);
}
