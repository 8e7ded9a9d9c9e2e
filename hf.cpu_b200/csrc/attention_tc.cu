// Attention over the paged cache for prompt portions, on the 5th-generation tensor cores (head_dim 128, bf16).
//
// Same arithmetic as the other attention kernels (src/model.c:499-528): scores = q.k * scale, causal and window
// masks by absolute position, float32 softmax, weighted values.  One CTA owns 128 rows = the query heads of one
// key/value head for up to 128 / (H/G) consecutive tokens, and walks the keys in tiles of 128:
//   S = Q K^T   tcgen05.mma, M = 128, N = 128 keys, K = head_dim; Q and K from shared memory (K-major, 128-byte
//               swizzle), S (float32) in TMEM;
//   softmax     eight warps, two threads per row (64 keys and 64 output columns each): the scores come from TMEM
//               with tcgen05.ld and stay in registers; the two halves of a row exchange their maxima through
//               shared memory; P (bf16) goes to shared memory as the next A operand;
//   PV = P V    tcgen05.mma, M = 128, N = head_dim, K = 128 keys; V is the B operand in MN-major form, which is
//               how the cache holds it (a key's values are two 128-byte rows, one sub-tile apart); the result lands in
//               TMEM and is added into the row's running output, which lives in the thread's registers.
// K and V tiles are gathered page by page with TMA (one box of block_size keys x 64 values per page and half of
// head_dim), double buffered; pages that are not mapped or lie beyond the last key are requested out of
// range and arrive as zeros.  While the softmax warps fold PV of tile j into their output, the MMA warp already
// computes S of tile j+1.  Every barrier wait is bounded (HFB_ERR_WAIT, TMEM freed, see tc_ptx.cuh).
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();
int tensor_map(const void *ptr, int rows, int cols, int box_rows, CUtensorMap *out);

constexpr int TQ = 128, TKEYS = 128, TD = 128;
constexpr uint32_t SUB = 128 * 64 * 2;              // one swizzled sub-tile: 128 rows of 64 bf16
constexpr uint32_t KV_STAGE = 2 * SUB;              // K (or V) tile: two sub-tiles (the halves of head_dim)
constexpr int ATC_THREADS = 320;                   // TMA warp, MMA warp, eight softmax warps
constexpr int ATC_TMEM_COLS = 256;                  // S: columns 0..127, PV: columns 128..255

struct AttnTcParams {
    const __nv_bfloat16 *q;
    __nv_bfloat16 *out;
    const int32_t *block_table, *positions, *tile_seq, *tile_t0, *tile_nt;
    int max_blocks, block_size, window, H, G;
    int num_slots;                                   // pages * block_size: a row coordinate beyond it reads zeros
    float scale_log2;
};

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Byte offset of the 16-byte chunk `c16` (0..15, eight bf16 each) of row `row` in a [128 x 128] operand held as two
// swizzled sub-tiles.
__device__ __forceinline__ uint32_t sw_off(int row, int c16)
{
    return (uint32_t)(c16 >> 3) * SUB + (uint32_t)row * 128u + (uint32_t)(((c16 & 7) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(ATC_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnTcParams p, int *err)
{
    HFB_TRACE_ENTRY(13);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sQ = base, sP = base + 2 * SUB, sK = base + 4 * SUB, sV = sK + 2 * KV_STAGE;
    const uint32_t bars = sV + 2 * KV_STAGE;
    const uint32_t q_ready = bars, s_full = bars + 8, p_ready = bars + 16, pv_full = bars + 24;
    const uint32_t kv_full0 = bars + 32, kv_empty0 = bars + 48, x_ready = bars + 64;
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(gen + 4 * SUB + 4 * KV_STAGE + 96);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    float *xchg = (float *)(gen + 4 * SUB + 4 * KV_STAGE + 128);       // [2][2][128]: maxima of the row halves, double buffered

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(q_ready, 8); mbar_init(s_full, 1); mbar_init(p_ready, 8); mbar_init(pv_full, 1); mbar_init(x_ready, 8);
        for (int s = 0; s < 2; s++) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"(ATC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_sync();                                      // queries and cache come from the kernels in front

    // tiles late in a prompt see the most keys: they go first
    const int tile = gridDim.x - 1 - blockIdx.x, g = blockIdx.y;
    const int r = p.H / p.G;
    const int seq = p.tile_seq[tile], t0 = p.tile_t0[tile], nt = p.tile_nt[tile];
    const int pos_first = p.positions[t0], pos_last = p.positions[t0 + nt - 1];
    const int lo_all = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int kt_lo = lo_all / TKEYS, n_kt = pos_last / TKEYS + 1 - kt_lo;

    if (warp == 0) {
        // ---- producer: K and V tiles, page by page ----------------------------------------------------
        // The lanes read 32 entries of the block table at a time (one coalesced read for several tiles); lane 0 then
        // asks for tile after tile without a round trip to L2 per page.
        const int32_t *table = p.block_table + (size_t)seq * p.max_blocks;
        const int bs = p.block_size, pages = TKEYS / bs, tiles_per_round = 32 / pages;
        bool ok = true;
        for (int j0 = 0; j0 < n_kt && ok; j0 += tiles_per_round) {
            const int key0 = (kt_lo + j0) * TKEYS + lane * bs, blk = key0 / bs;
            const bool mapped = lane < tiles_per_round * pages && j0 + lane / pages < n_kt && key0 <= pos_last && blk < p.max_blocks;
            const int page = mapped ? table[blk] : -1;
            const int my_row = page >= 0 ? page * bs : p.num_slots;                  // out of range: zeros
            for (int t = 0; t < tiles_per_round && j0 + t < n_kt && ok; t++) {
                const int j = j0 + t, s = j & 1;
                if (lane == 0) {
                    ok = mbar_wait(kv_empty0 + 8 * s, ((j >> 1) & 1) ^ 1, abort_flag, err);
                    if (ok) mbar_arrive_expect_tx(kv_full0 + 8 * s, 2 * KV_STAGE);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                // one copy per page and half of the head for K and for V, each pair issued by a lane of its own
                const int pg = lane >> 1, half = lane & 1;
                const int row = __shfl_sync(0xffffffffu, my_row, t * pages + min(pg, pages - 1));
                if (ok && pg < pages) {
                    const uint32_t off = (uint32_t)s * KV_STAGE + (uint32_t)pg * bs * 128u + half * SUB;
                    tma_load_2d(sK + off, &map_k, g * TD + half * 64, row, kv_full0 + 8 * s);
                    tma_load_2d(sV + off, &map_v, g * TD + half * 64, row, kv_full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = bf16_idesc(TQ, TKEYS, false), idesc_pv = bf16_idesc(TQ, TD, true);
            const uint32_t tS = tmem_base, tPV = tmem_base + 128;
            auto issue_s = [&](int stage) {
#pragma unroll
                for (int kk = 0; kk < TD / 16; kk++) {
                    const uint32_t o = (uint32_t)(kk >> 2) * SUB + (uint32_t)(kk & 3) * 32u;
                    tc_mma_bf16(tS, sw128_desc(sQ + o), sw128_desc(sK + stage * KV_STAGE + o), idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(s_full);
            };
            bool ok = mbar_wait(q_ready, 0, abort_flag, err);
            if (ok && n_kt > 0) {
                ok = mbar_wait(kv_full0, 0, abort_flag, err);
                if (ok) { tc_fence_after(); issue_s(0); }
            }
            for (int j = 0; j < n_kt && ok; j++) {
                const int s = j & 1;
                if (!mbar_wait(p_ready, j & 1, abort_flag, err)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < TKEYS / 16; kk++) {
                    const uint32_t a = sP + (uint32_t)(kk >> 2) * SUB + (uint32_t)(kk & 3) * 32u;
                    const uint32_t b = sV + s * KV_STAGE + (uint32_t)kk * 2048u;                 // 16 keys further
                    // one product for both halves of the head: the second 64 values lie one sub-tile further
                    tc_mma_bf16(tPV, sw128_desc(a), sw128_desc_mn(b, SUB), idesc_pv, kk > 0 ? 1u : 0u);
                }
                tc_commit(pv_full);
                tc_commit(kv_empty0 + 8 * s);
                if (j + 1 < n_kt) {
                    const int s2 = (j + 1) & 1;
                    if (!mbar_wait(kv_full0 + 8 * s2, ((j + 1) >> 1) & 1, abort_flag, err)) { ok = false; break; }
                    tc_fence_after();
                    issue_s(s2);
                }
            }
            // the last commits have landed once the softmax warps saw pv_full; wait for the stage release too
            if (ok && n_kt > 0) mbar_wait(kv_empty0 + 8 * ((n_kt - 1) & 1), ((n_kt - 1) >> 1) & 1, abort_flag, err);
        }
    } else {
        // ---- softmax and output: two threads per row, 64 keys / 64 output columns each ---------------------
        const int q4 = warp & 3, half = (warp - 2) >> 2, row = q4 * 32 + lane;
        const int tl = row / r, hl = row % r;
        const bool valid = tl < nt;
        const size_t th = ((size_t)(t0 + (valid ? tl : 0)) * p.H + g * r + hl) * TD;
        {
            const uint4 *src = (const uint4 *)(p.q + th) + half * 8;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sQ + sw_off(row, half * 8 + c)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        const int pos = valid ? p.positions[t0 + tl] : -1;
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const uint32_t tS = tmem_base + ((uint32_t)(q4 * 32) << 16) + half * 64, tPV = tmem_base + ((uint32_t)(q4 * 32) << 16) + 128 + half * 64;
        float o[64];
#pragma unroll
        for (int i = 0; i < 64; i++) o[i] = 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_kt && ok; j++) {
            const int key0 = (kt_lo + j) * TKEYS + half * 64;         // first key of this thread's half
            if (!mbar_wait(s_full, j & 1, abort_flag, err)) { ok = false; break; }
            tc_fence_after();
            // rows beyond the tile's tokens (zero queries, nothing of them is written) go with the rows that see
            // every key, so that their warp is not split over both branches
            const bool all_visible = !valid || (key0 + 63 <= pos && key0 >= lo);
            uint32_t sv[64];
            tmem_ld16(tS, sv); tmem_ld16(tS + 16, sv + 16); tmem_ld16(tS + 32, sv + 32); tmem_ld16(tS + 48, sv + 48);
            tmem_wait_ld();
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // (four chains: see attention_tc2.cu)
            if (all_visible) {
#pragma unroll
                for (int i = 0; i < 64; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 64; i++) {
                    const int key = key0 + i;
                    const bool see = valid && key >= lo && key <= pos;
                    if (!see) sv[i] = 0xff800000u;                  // -inf: contributes neither to the maximum nor to the sum
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
                }
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            float *xm = xchg + (j & 1) * 256;
            xm[half * 128 + row] = mx;
            __syncwarp();
            if (lane == 0) mbar_arrive(x_ready);                   // the eight softmax warps meet here (a bounded wait)
            if (!mbar_wait(x_ready, j & 1, abort_flag, err)) { ok = false; break; }
            mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]) * p.scale_log2;   // scale > 0 commutes with the maximum
            const float m_new = fmaxf(m, mx);
            const float bs = m_new == -INFINITY ? 0.f : m_new;
            const float corr = ex2(m - bs);                        // 2^-inf = 0 for the first tile
            m = m_new;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                float a = ex2(__uint_as_float(sv[i]) * p.scale_log2 - bs), b = ex2(__uint_as_float(sv[i + 1]) * p.scale_log2 - bs);
                __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                const uint32_t hb = *(uint32_t *)&h;                // the sum runs over the rounded values the product uses:
                sum4[(i >> 1) & 3] += __uint_as_float(hb << 16) + __uint_as_float(hb & 0xffff0000u);   // widened by bit moves, not conversions
                pk[i >> 1] = hb;
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
#pragma unroll
            for (int q = 0; q < 8; q++)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sP + sw_off(row, half * 8 + q)), "r"(pk[4 * q]),
                             "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3]) : "memory");
            l = l * corr + sum;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            if (corr != 1.f) {
#pragma unroll
                for (int i = 0; i < 64; i++) o[i] *= corr;
            }
            if (!mbar_wait(pv_full, j & 1, abort_flag, err)) { ok = false; break; }
            tc_fence_after();
            uint32_t pv[64];
            tmem_ld16(tPV, pv); tmem_ld16(tPV + 16, pv + 16); tmem_ld16(tPV + 32, pv + 32); tmem_ld16(tPV + 48, pv + 48);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 64; i++) o[i] += __uint_as_float(pv[i]);
            tc_fence_before();
        }
        // the two halves of a row saw different keys with the same maxima: their sums add up
        float *xl = xchg + 512;
        xl[half * 128 + row] = l;
        __syncwarp();
        if (lane == 0) mbar_arrive(x_ready);
        ok = ok && mbar_wait(x_ready, n_kt & 1, abort_flag, err);
        l += xl[(half ^ 1) * 128 + row];
        if (ok && valid) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            uint4 *dst = (uint4 *)(p.out + th) + half * 8;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                __nv_bfloat162 h[4];
#pragma unroll
                for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
                dst[c] = *(uint4 *)&h[0];
            }
        }
    }

    // ---- teardown ---------------------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);          // let loads still in flight land
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ATC_TMEM_COLS) : "memory");
    }
}

}  // namespace hfb

using namespace hfb;

// Attention of prompt portions on tcgen05: bfloat16, head_dim 128, block sizes 8..128 that divide 128, at most
// 128 query heads per key/value head.  Tiles (tile_seq, tile_t0, tile_nt) hold at most 128 / (H/G) tokens each.
extern "C" int hfb_attention_tc(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                                int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                                const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window,
                                float scale, void *out, int T, int H, int G, int d, hfb_stream s)
{
    if (n_tiles <= 0) return HFB_OK;
    if (d != TD) return fail(HFB_ENOTSUP, "attention_tc: head_dim %d (128 only)", d);
    if (G <= 0 || H % G || H / G > TQ) return fail(HFB_ENOTSUP, "attention_tc: %d heads over %d key/value heads", H, G);
    if (block_size < 8 || block_size > TKEYS || TKEYS % block_size) return fail(HFB_ENOTSUP, "attention_tc: block size %d (8..128, dividing 128)", block_size);
    if (num_pages * block_size >= (1ll << 31) - TKEYS) return fail(HFB_ENOTSUP, "attention_tc: cache too large for 32-bit coordinates");
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return fail(HFB_ENOTSUP, "attention_tc: operands must be 16-byte aligned");
    if (G > 65535) return fail(HFB_ENOTSUP, "attention_tc: too many key/value heads");
    (void)T;
    CUtensorMap mk, mv;
    int rc;
    const int slots = (int)(num_pages * block_size);
    if ((rc = tensor_map(k_cache, slots, G * d, block_size, &mk)) != HFB_OK) return rc;
    if ((rc = tensor_map(v_cache, slots, G * d, block_size, &mv)) != HFB_OK) return rc;
    AttnTcParams p;
    p.q = (const __nv_bfloat16 *)q; p.out = (__nv_bfloat16 *)out;
    p.block_table = block_table; p.positions = positions; p.tile_seq = tile_seq; p.tile_t0 = tile_t0; p.tile_nt = tile_nt;
    p.max_blocks = max_blocks; p.block_size = block_size; p.window = window; p.H = H; p.G = G; p.num_slots = slots;
    p.scale_log2 = scale * 1.4426950408889634f;
    constexpr uint32_t smem = 1024 + 4 * SUB + 4 * KV_STAGE + 128 + 768 * 4;
    static bool configured[64] = {false};                 // (the opt-in is a property of the function on one device)
    if (!configured[current_device()]) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "attention_tc: cannot opt in to %u bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[current_device()] = true;
    }
    g_launch_err = launch_pdl(attention_tc_kernel, dim3(n_tiles, G), dim3(ATC_THREADS), smem, (cudaStream_t)s, mk, mv, p, error_word());
    return check_pdl_launch(g_launch_err, "attention_tc");
}
