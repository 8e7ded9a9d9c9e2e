// Attention over the paged cache for long prompt portions on tcgen05, two query tiles per CTA (head_dim 64 or 128, bf16).
//
// The arithmetic is that of attention_tc.cu (src/model.c:499-528 of the reference: scores = q.k * scale, causal
// and window masks by absolute position, float32 softmax, weighted values).  What differs is how the softmax and
// the tensor core share the time:
//   * one CTA owns two tiles of 128 rows (the query heads of one key/value head for 2 x 128/(H/G) consecutive
//     tokens).  Both use the same K and V tiles, which are fetched once; while the softmax warps of one tile work
//     on their scores, the tensor core computes the other tile's products, and the other way round;
//   * a row belongs to one thread (128 scores in registers), so its maximum needs no exchange;
//   * the running output O lives in TMEM and P V is accumulated into it by the tensor core; nothing of it is
//     read back per tile.  The exponentials use a reference maximum that is only raised when a row's maximum grew
//     by more than 2^8 since it was set (weights stay below 2^8, well inside bfloat16's and float32's range; sum
//     and output carry the same factor, which cancels in the end); only then is O rescaled in TMEM
//     (tcgen05.ld, multiply, tcgen05.st), by the row's own thread, between two products into it.
// TMEM: S0, S1 (128 columns each), O0, O1 (head_dim columns each).  Shared memory: Q0, Q1, P0, P1 (32 KB each), one K tile
// and two V tiles (128 keys of head_dim elements: 16 or 32 KB):
// K is free again once both S products of a step are done, early in the step, and is refilled while the softmax
// runs; V is in use until the step's last product, so the next one is fetched into the other buffer meanwhile.
// Every barrier wait is bounded (HFB_ERR_WAIT, TMEM freed; tc_ptx.cuh).
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();
int tensor_map(const void *ptr, int rows, int cols, int box_rows, CUtensorMap *out);

constexpr int U_ROWS = 128, U_KEYS = 128;
constexpr uint32_t U_SUB = 128 * 64 * 2;            // one swizzled sub-tile: 128 rows of 64 bf16
constexpr uint32_t U_TILE = 2 * U_SUB;              // a [128 x 128] bf16 operand (P; Q, K, V at head_dim 128): two sub-tiles
constexpr int U_THREADS = 320;                     // TMA warp, MMA warp, four softmax warps per query tile
constexpr int U_TMEM_COLS = 512;
constexpr float U_TAU = 8.0f;                       // log2 of how far a row's maximum may outgrow its reference

struct AttnTc2Params {
    const __nv_bfloat16 *q;
    __nv_bfloat16 *out;
    const int32_t *block_table, *positions, *tile_seq, *tile_t0, *tile_nt;
    int max_blocks, block_size, window, H, G;
    int per;                                         // tokens per query tile: 128 / (H / G)
    int n_tiles;                                     // double tiles in all
    int num_slots;                                   // pages * block_size: a row coordinate beyond it reads zeros
    float scale_log2;
};

__device__ __forceinline__ float u_ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t u_sw_off(int row, int c16)
{
    return (uint32_t)(c16 >> 3) * U_SUB + (uint32_t)row * 128u + (uint32_t)(((c16 & 7) ^ (row & 7)) << 4);
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *v)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(U_THREADS, 1)
attention_tc2_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnTc2Params p, int *err)
{
    HFB_TRACE_ENTRY(13);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    constexpr uint32_t HT = (D / 64) * U_SUB;        // a [128 x D] bf16 operand: Q, K or V
    constexpr uint32_t U_BARS = 2 * U_TILE + 5 * HT; // bytes of the tiles in front of the barriers
    const uint32_t sQ = base, sK = base + 2 * HT, sV = base + 3 * HT, sP = base + 5 * HT;
    const uint32_t bars = base + U_BARS;             // V has two stages: sV, sV + HT
    // per query tile i: q_ready + 8i, s_full + 8i, p_ready + 8i, pv_done + 8i; per V stage s: v_full + 8s, v_empty + 8s
    const uint32_t q_ready = bars, s_full = bars + 16, p_ready = bars + 32, pv_done = bars + 48;
    const uint32_t k_full = bars + 64, k_empty = bars + 72, v_full = bars + 80, v_empty = bars + 96;
    const uint32_t s_free = bars + 112;              // + 8i: tile i's scores have been read out of TMEM
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(gen + U_BARS + 128);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; i++) {
            mbar_init(q_ready + 8 * i, 4); mbar_init(s_full + 8 * i, 1); mbar_init(p_ready + 8 * i, 4); mbar_init(pv_done + 8 * i, 1);
            mbar_init(s_free + 8 * i, 4);
        }
        mbar_init(k_full, 1); mbar_init(k_empty, 1);
        for (int st = 0; st < 2; st++) { mbar_init(v_full + 8 * st, 1); mbar_init(v_empty + 8 * st, 1); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"(U_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_sync();                                      // queries and cache come from the kernels in front

    // Work items are (double tile, key/value head), heaviest first (tiles late in a prompt see the most keys).  A CTA
    // takes one item per round, the rounds running over the CTAs forwards and backwards in turn, so that every CTA
    // gets long and short items; barriers, TMEM and shared memory are set up once.  Each role walks the same items
    // and keeps count of how often every barrier has been used.
    const int r = p.H / p.G;
    const int n_items = p.n_tiles * p.G, n_ctas = gridDim.x;
    struct Item { int g, seq, t0, nt0, nt1, pos_last, kt_lo, n_kt0, n_kt1, n_kt; };
    auto item_of = [&](int round, Item &it) -> bool {
        const int idx = round * n_ctas + ((round & 1) ? n_ctas - 1 - (int)blockIdx.x : (int)blockIdx.x);
        if (idx >= n_items) return false;
        const int tile = p.n_tiles - 1 - idx / p.G;
        it.g = idx % p.G;
        it.seq = p.tile_seq[tile]; it.t0 = p.tile_t0[tile];
        const int nt = p.tile_nt[tile];
        it.nt0 = min(nt, p.per); it.nt1 = nt - it.nt0;                  // tokens of the two query tiles
        const int pos_first = p.positions[it.t0], pos_last0 = p.positions[it.t0 + it.nt0 - 1];
        it.pos_last = p.positions[it.t0 + nt - 1];
        const int lo_all = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
        it.kt_lo = lo_all / U_KEYS;
        it.n_kt0 = pos_last0 / U_KEYS + 1 - it.kt_lo;
        it.n_kt1 = it.nt1 > 0 ? it.pos_last / U_KEYS + 1 - it.kt_lo : 0;
        it.n_kt = max(it.n_kt0, it.n_kt1);
        return true;
    };
    const int n_rounds = (n_items + n_ctas - 1) / n_ctas;

    if (warp == 0) {
        // ---- producer: one K tile and (in two buffers) one V tile per step, page by page ----------------------
        // The lanes read 32 entries of the block table at a time (the pages of several steps, one coalesced read);
        // the copies of a step, one per page and half of the head, are issued by as many lanes.
        const int bs = p.block_size, pages = U_KEYS / bs, steps_per_round = 32 / pages;
        bool ok = true;
        uint32_t gs = 0;                                  // steps so far: K's use count, V's use count
        for (int round = 0; round < n_rounds && ok; round++) {
            Item it;
            if (!item_of(round, it)) continue;
            const int32_t *table = p.block_table + (size_t)it.seq * p.max_blocks;
            for (int j0 = 0; j0 < it.n_kt && ok; j0 += steps_per_round) {
                const int key0 = (it.kt_lo + j0) * U_KEYS + lane * bs, blk = key0 / bs;
                const bool mapped = lane < steps_per_round * pages && j0 + lane / pages < it.n_kt && key0 <= it.pos_last && blk < p.max_blocks;
                const int page = mapped ? table[blk] : -1;
                const int my_row = page >= 0 ? page * bs : p.num_slots;              // out of range: zeros
                for (int t = 0; t < steps_per_round && j0 + t < it.n_kt && ok; t++, gs++) {
#pragma unroll 1
                    for (int kv = 0; kv < 2 && ok; kv++) {
                        const uint32_t st = gs & 1;                                   // V's stage
                        const uint32_t full = kv ? v_full + 8 * st : k_full, empty = kv ? v_empty + 8 * st : k_empty;
                        const uint32_t dst = kv ? sV + st * HT : sK;
                        if (lane == 0) {
                            ok = mbar_wait(empty, kv ? (((gs >> 1) & 1) ^ 1) : ((gs & 1) ^ 1), abort_flag, err);
                            if (ok) mbar_arrive_expect_tx(full, HT);
                        }
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        const int pg = D == 128 ? lane >> 1 : lane, half = D == 128 ? lane & 1 : 0;
                        const int row = __shfl_sync(0xffffffffu, my_row, t * pages + min(pg, pages - 1));
                        if (ok && pg < pages)
                            tma_load_2d(dst + (uint32_t)pg * bs * 128u + half * U_SUB, kv ? &map_v : &map_k, it.g * D + half * 64, row, full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = bf16_idesc(U_ROWS, U_KEYS, false), idesc_pv = bf16_idesc(U_ROWS, D, true);
            // Every operand sits at a fixed place, so all descriptors are made once: a single thread issues 32
            // products per step, and what it computes between two of them is time the tensor core waits.
            uint64_t dq[2][D / 16], dk[D / 16], dp[2][U_KEYS / 16], dv[U_KEYS / 16];
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                const uint32_t o = (uint32_t)(kk >> 2) * U_SUB + (uint32_t)(kk & 3) * 32u;
#pragma unroll
                for (int i = 0; i < 2; i++) dp[i][kk] = sw128_desc(sP + i * U_TILE + o);
                if (kk < D / 16) {
                    dk[kk] = sw128_desc(sK + o);
#pragma unroll
                    for (int i = 0; i < 2; i++) dq[i][kk] = sw128_desc(sQ + i * HT + o);
                }
                dv[kk] = sw128_desc_mn(sV + (uint32_t)kk * 2048u, U_SUB);                // 16 keys further; every 64-wide piece of the head
            }
            const uint32_t tS0 = tmem_base, tO0 = tmem_base + 256;
            auto issue_s = [&](int i) {
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++)
                    tc_mma_bf16(tS0 + i * 128, i ? dq[1][kk] : dq[0][kk], dk[kk], idesc_s, kk > 0 ? 1u : 0u);
                tc_commit(s_full + 8 * i);
            };
            auto issue_pv = [&](int i, bool accumulate, uint64_t v_stage) {      // v_stage: 0 or the second V buffer
#pragma unroll
                for (int kk = 0; kk < U_KEYS / 16; kk++)
                    tc_mma_bf16(tO0 + i * D, i ? dp[1][kk] : dp[0][kk], dv[kk] + v_stage, idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
                tc_commit(pv_done + 8 * i);
            };
            bool ok = true;
            uint32_t gs = 0, g_tile[2] = {0, 0}, q_uses[2] = {0, 0};      // steps so far, per tile, and items per tile
            for (int round = 0; round < n_rounds && ok; round++) {
                Item it;
                if (!item_of(round, it)) continue;
                const int n_of[2] = {it.n_kt0, it.n_kt1};
                for (int i = 0; i < 2 && ok; i++)
                    if (n_of[i] > 0) ok = mbar_wait(q_ready + 8 * i, q_uses[i]++ & 1, abort_flag, err);
                if (ok && it.n_kt > 0) {
                    ok = mbar_wait(k_full, gs & 1, abort_flag, err);
                    if (ok) {
                        tc_fence_after();
                        if (it.n_kt0 > 0) issue_s(0);
                        if (it.n_kt1 > 0) issue_s(1);
                        tc_commit(k_empty);
                    }
                }
                for (int j = 0; j < it.n_kt && ok; j++, gs++) {
                    const uint32_t st = gs & 1;
                    const uint64_t v_stage = st ? (uint64_t)(HT >> 4) : 0;          // added to a descriptor's address field
                    // The scores of step j + 1 are queued as soon as those of step j have left TMEM for the softmax
                    // threads' registers, long before their exponentials are done: a tile's softmax warps then go
                    // from one step to the next without waiting for the tensor core.
                    if (j + 1 < it.n_kt) {
                        if (!mbar_wait(k_full, (gs + 1) & 1, abort_flag, err)) { ok = false; break; }
                        for (int i = 0; i < 2 && ok; i++) {
                            if (j + 1 < n_of[i]) {
                                ok = mbar_wait(s_free + 8 * i, (g_tile[i] + j) & 1, abort_flag, err);
                                if (ok) { tc_fence_after(); issue_s(i); }
                            }
                        }
                        if (!ok) break;
                        tc_commit(k_empty);                          // both tiles' products with K of step j + 1 are queued
                    }
                    if (!mbar_wait(v_full + 8 * st, (gs >> 1) & 1, abort_flag, err)) { ok = false; break; }
                    for (int i = 0; i < 2 && ok; i++) {
                        if (j < n_of[i]) {
                            ok = mbar_wait(p_ready + 8 * i, (g_tile[i] + j) & 1, abort_flag, err);
                            if (ok) { tc_fence_after(); issue_pv(i, j > 0, v_stage); }
                        }
                    }
                    if (!ok) break;
                    tc_commit(v_empty + 8 * st);
                }
                g_tile[0] += it.n_kt0; g_tile[1] += it.n_kt1;
            }
            // nothing of this CTA's is in flight once the last release of V has landed
            if (ok && gs > 0) mbar_wait(v_empty + 8 * ((gs - 1) & 1), ((gs - 1) >> 1) & 1, abort_flag, err);
        }
    } else {
        // ---- softmax and output: one thread per row --------------------------------------------------------
        const int i = (warp - 2) >> 2;                                   // query tile
        const int row = (warp & 3) * 32 + lane;                          // TMEM lane = row; a warp reads its own quarter
        const int tl = row / r, hl = row % r;
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t tS = lane_base + i * 128, tO = lane_base + 256 + i * D;
        uint32_t g_mine = 0;                                             // this tile's steps so far
        bool ok = true;
        for (int round = 0; round < n_rounds && ok; round++) {
            Item it;
            if (!item_of(round, it)) continue;
            const int n_mine = i ? it.n_kt1 : it.n_kt0, nt_mine = i ? it.nt1 : it.nt0, t_first = it.t0 + i * p.per;
            if (n_mine <= 0) continue;
            const bool valid = tl < nt_mine;
            const size_t th = ((size_t)(t_first + (valid ? tl : 0)) * p.H + it.g * r + hl) * D;
            {
                // the tile's products of the item before are done (their scores have all been waited for)
                const uint4 *src = (const uint4 *)(p.q + th);
#pragma unroll
                for (int c = 0; c < D / 8; c++) {
                    uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sQ + i * HT + u_sw_off(row, c)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(q_ready + 8 * i);
            }
            const int pos = valid ? p.positions[t_first + tl] : -1;
            const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            float m_ref = -INFINITY, l = 0.f;        // the maximum the exponentials refer to, and the sum in its scale
            for (int j = 0; j < n_mine && ok; j++) {
                const uint32_t ph = (g_mine + j) & 1;
                const int key0 = (it.kt_lo + j) * U_KEYS;
                if (!mbar_wait(s_full + 8 * i, ph, abort_flag, err)) { ok = false; break; }
                tc_fence_after();
                uint32_t sv[128];
#pragma unroll
                for (int c = 0; c < 8; c++) tmem_ld16(tS + 16 * c, sv + 16 * c);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free + 8 * i);         // the tensor core may write the next scores
                // (the maximum and the sum each run in four independent chains: with two warps per scheduler a chain of
                // 128 dependent operations is not hidden by the other warp)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                // rows beyond the tile's tokens (their queries are zeros, nothing of them is written) go with the
                // rows that see every key, so that their warp is not split over both branches
                const bool all_visible = !valid || (key0 + U_KEYS - 1 <= pos && key0 >= lo);
                if (all_visible) {
#pragma unroll
                    for (int c = 0; c < 128; c++) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
                } else {
#pragma unroll
                    for (int c = 0; c < 128; c++) {
                        const int key = key0 + c;
                        const bool see = valid && key >= lo && key <= pos;
                        if (!see) sv[c] = 0xff800000u;              // -inf: contributes neither to the maximum nor to the sum
                        mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
                    }
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                mx *= p.scale_log2;                                  // scale > 0 commutes with the maximum
                // raise the reference only when the row's maximum has outgrown it by 2^TAU (or there was none yet)
                float corr = 1.f;
                if (mx > m_ref + U_TAU || (m_ref == -INFINITY && mx > -INFINITY)) {
                    corr = m_ref == -INFINITY ? 0.f : u_ex2(m_ref - mx);
                    m_ref = mx;
                }
                const float bs = m_ref == -INFINITY ? 0.f : m_ref;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[64];
#pragma unroll
                for (int c = 0; c < 128; c += 2) {
                    const float a = u_ex2(__uint_as_float(sv[c]) * p.scale_log2 - bs), b = u_ex2(__uint_as_float(sv[c + 1]) * p.scale_log2 - bs);
                    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    const uint32_t hb = *(uint32_t *)&h;            // the sum runs over the rounded values the product uses:
                    sum4[(c >> 1) & 3] += __uint_as_float(hb << 16) + __uint_as_float(hb & 0xffff0000u);   // widened by bit moves, not conversions
                    pk[c >> 1] = hb;
                }
                const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                l = l * corr + sum;
                if (j > 0) {
                    // P of the step before has been used, and O holds everything up to it
                    if (!mbar_wait(pv_done + 8 * i, ph ^ 1, abort_flag, err)) { ok = false; break; }
                    tc_fence_after();
                    if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
                        for (int c = 0; c < D / 16; c++) {
                            uint32_t ov[16];
                            tmem_ld16(tO + 16 * c, ov);
                            tmem_wait_ld();
#pragma unroll
                            for (int e = 0; e < 16; e++) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * corr);
                            tmem_st16(tO + 16 * c, ov);
                        }
                        tmem_wait_st();
                    }
                }
#pragma unroll
                for (int q = 0; q < 16; q++)
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sP + i * U_TILE + u_sw_off(row, q)), "r"(pk[4 * q]),
                                 "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3]) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready + 8 * i);
            }
            g_mine += n_mine;
            if (ok) ok = mbar_wait(pv_done + 8 * i, (g_mine - 1) & 1, abort_flag, err);
            if (ok) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                uint4 *dst = (uint4 *)(p.out + th);
#pragma unroll 1
                for (int c = 0; c < D / 16; c += 4) {                 // four reads of 16 columns under way together
                    uint32_t ov[64];
#pragma unroll
                    for (int u = 0; u < 4; u++) tmem_ld16(tO + 16 * (c + u), ov + 16 * u);   // all lanes take part, valid row or not
                    tmem_wait_ld();
                    if (valid) {
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            __nv_bfloat162 h[8];
#pragma unroll
                            for (int e = 0; e < 8; e++)
                                h[e] = __floats2bfloat162_rn(__uint_as_float(ov[16 * u + 2 * e]) * inv, __uint_as_float(ov[16 * u + 2 * e + 1]) * inv);
                            dst[2 * (c + u)] = *(uint4 *)&h[0];
                            dst[2 * (c + u) + 1] = *(uint4 *)&h[4];
                        }
                    }
                }
                tc_fence_before();
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(U_TMEM_COLS) : "memory");
    }
}

template <int D>
static int launch_tc2(const CUtensorMap &mk, const CUtensorMap &mv, const AttnTc2Params &p, int grid, cudaStream_t st)
{
    constexpr uint32_t smem = 1024 + 2 * U_TILE + 5 * (D / 64) * U_SUB + 160;
    static_assert(smem <= 227 * 1024, "the tiles do not fit");
    static bool configured[64] = {false};                 // (the opt-in is a property of the function on one device)
    if (!configured[current_device()]) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "attention_tc2: cannot opt in to %u bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[current_device()] = true;
    }
    g_launch_err = launch_pdl(attention_tc2_kernel<D>, dim3(grid), dim3(U_THREADS), smem, st, mk, mv, p, error_word());
    return check_pdl_launch(g_launch_err, "attention_tc2");
}

}  // namespace hfb

using namespace hfb;

// Attention of long prompt portions with two query tiles per CTA: bfloat16, head_dim 64 or 128, block sizes 8..128 that
// divide 128, at most 128 query heads per key/value head.  Tiles (tile_seq, tile_t0, tile_nt) hold at most
// 2 * (128 / (H/G)) consecutive tokens of one request each.
extern "C" int hfb_attention_tc2(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                                 int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                                 const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window,
                                 float scale, void *out, int T, int H, int G, int d, hfb_stream s)
{
    if (n_tiles <= 0) return HFB_OK;
    if (d != 64 && d != 128) return fail(HFB_ENOTSUP, "attention_tc2: head_dim %d (64 and 128 only)", d);
    if (G <= 0 || H % G || H / G > U_ROWS) return fail(HFB_ENOTSUP, "attention_tc2: %d heads over %d key/value heads", H, G);
    if (block_size < 8 || block_size > U_KEYS || U_KEYS % block_size) return fail(HFB_ENOTSUP, "attention_tc2: block size %d (8..128, dividing 128)", block_size);
    if (num_pages * block_size >= (1ll << 31) - U_KEYS) return fail(HFB_ENOTSUP, "attention_tc2: cache too large for 32-bit coordinates");
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return fail(HFB_ENOTSUP, "attention_tc2: operands must be 16-byte aligned");
    if (G > 65535) return fail(HFB_ENOTSUP, "attention_tc2: too many key/value heads");
    (void)T;
    CUtensorMap mk, mv;
    int rc;
    const int slots = (int)(num_pages * block_size);
    if ((rc = tensor_map(k_cache, slots, G * d, block_size, &mk)) != HFB_OK) return rc;
    if ((rc = tensor_map(v_cache, slots, G * d, block_size, &mv)) != HFB_OK) return rc;
    AttnTc2Params p;
    p.q = (const __nv_bfloat16 *)q; p.out = (__nv_bfloat16 *)out;
    p.block_table = block_table; p.positions = positions; p.tile_seq = tile_seq; p.tile_t0 = tile_t0; p.tile_nt = tile_nt;
    p.max_blocks = max_blocks; p.block_size = block_size; p.window = window; p.H = H; p.G = G; p.num_slots = slots;
    p.per = U_ROWS / (H / G);
    p.n_tiles = n_tiles;
    p.scale_log2 = scale * 1.4426950408889634f;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long items = (long long)n_tiles * G;
    const int grid = (int)(items < sms ? items : (sms > 0 ? sms : 1));      // one CTA per SM walks its share of the items
    return d == 128 ? launch_tc2<128>(mk, mv, p, grid, (cudaStream_t)s) : launch_tc2<64>(mk, mv, p, grid, (cudaStream_t)s);
}
