// Decode attention over the paged cache for bfloat16: the keys and values arrive by TMA, page by page.
//
// With one new token per request the work is a pure read of the request's keys and values, and what costs
// is every instruction spent on moving them.  A fifth warp owns the copies: for each tile of 64 keys it looks
// up the tile's pages and asks the TMA unit for them, one request per page that brings the page's keys and values of
// one head at once (a box [keys|values][128-byte piece of the head][block_size keys][64 elements] through a map of
// rank 4, 128-byte swizzle; two requests where keys and values are not one array; a page the table does not map is
// read from beyond the cache and arrives as zeros): a request costs the issuing thread a few hundred cycles whatever
// its size, and at one per page and piece of keys or values that was what bounded this kernel.  The copies run
// several tiles ahead of the four warps that compute.  Those share each tile as the cp.async
// form does (attention_fast.cu): 16 keys per warp, the query heads of one key/value head on the 16 rows of
// mma.sync m16n8k16, a running maximum and sum per warp, merged in warp order at the end.  Full and empty
// mbarriers pair the two sides, so the loop has no CTA-wide barrier.  Tiles that lie wholly inside every row's
// range skip the masks, and the accumulator is rescaled only when a maximum grew.
// Rows of a mapped page beyond the request's length hold old (finite) values or the zeros the cache starts
// with; their scores are masked to -inf, so their weights are exactly zero.
// Same arithmetic as src/model.c:499-528 of the reference, in flash-attention form.
#include <cuda.h>

#include "attention_common.cuh"
#include "tc_ptx.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();
int tensor_map_kv(const void *k, const void *v, int slots, int row_elems, int box_keys, int halves, CUtensorMap *maps, bool *single);

constexpr int ADT_THREADS = 160;        // four computing warps and the copying warp

// A stage holds a tile of 64 keys page by page: [page][keys | values][128-byte piece of the head][key of the page][64
// elements], as the page copies arrive.  Byte offset, from the page's keys (or values), of 16-byte chunk `c` of the
// page's key `kr`, written by the TMA unit with the 128-byte swizzle (every piece of a page starts on a multiple of
// 1024 bytes: pages hold 8 keys or more).
__device__ __forceinline__ uint32_t page_off(int kr, int c, int bs)
{
    return (uint32_t)(c >> 3) * (uint32_t)bs * 128u + (uint32_t)kr * 128u + (uint32_t)(((c & 7) ^ (kr & 7)) << 4);
}

template <int D, int STAGES, bool ONE_MAP>
__global__ void __launch_bounds__(ADT_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, AttnParams p,
                            int num_slots, int *err)
{
    HFB_TRACE_ENTRY(3);
    constexpr int CH = D / 8, HALVES = D / 64;
    constexpr uint32_t TILE = HALVES * ABN * 128;        // bytes of the keys (or the values) of one tile
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t st0 = base, sq = base + 2 * STAGES * TILE;   // stage s: keys and values of a tile, page by page
    const uint32_t page_bytes = (uint32_t)p.block_size * HALVES * 128u;   // a page's keys (or values) of one head
    const uint32_t full0 = sq + 16 * D * 2, empty0 = full0 + 8 * STAGES;
    volatile int *abort_flag = (volatile int *)(gen + 2 * STAGES * TILE + 16 * D * 2 + 16 * STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // The tiling, the positions and the block table are inputs of the step, and the keys of earlier steps are in
    // the cache already: none of that waits for the kernel in front.  Only the queries and the tiles that hold
    // this step's tokens do.
    const int tile = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int r = p.H / p.G;
    const int seq = p.tile_seq[tile], t0 = p.tile_t0[tile], nt = p.tile_nt[tile];
    const int pos_first = p.positions[t0], pos_last = p.positions[t0 + nt - 1];
    const int lo_first = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int lo_last = p.window > 0 ? max(0, pos_last - p.window + 1) : 0;
    int kt_lo = lo_first / ABN, kt_hi = pos_last / ABN + 1;
    if (p.splits > 1) {
        int per = (kt_hi - kt_lo + p.splits - 1) / p.splits;
        kt_lo = kt_lo + split * per;
        kt_hi = min(kt_hi, kt_lo + per);
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int row0 = lane >> 2, row1 = row0 + 8;

    if (warp == 4) {
        // ---- the copying warp ------------------------------------------------------------------------
        // The lanes look up 32 pages at a time (the pages of several tiles, one coalesced read of the block
        // table); lane 0 then asks for tile after tile without waiting for another table entry.
        const int32_t *table = p.block_table + (size_t)seq * p.max_blocks;
        const int bs = p.block_size, pages = ABN / bs, tiles_per_round = 32 / pages;
        bool waited = false;
        for (int kt0 = kt_lo; kt0 < kt_hi; kt0 += tiles_per_round) {
            const int key0 = kt0 * ABN + lane * bs, blk = key0 / bs;
            const bool mapped = lane < tiles_per_round * pages && kt0 + lane / pages < kt_hi && key0 <= pos_last && blk < p.max_blocks;
            const long long page = mapped ? table[blk] : -1;
            const int my_row = (page >= 0 && page < p.num_pages) ? (int)(page * bs) : num_slots;     // beyond the cache: zeros
            bool ok = true;
            for (int t = 0; t < tiles_per_round && kt0 + t < kt_hi; t++) {
                const int j = kt0 + t - kt_lo, s = j % STAGES;
                if (!waited && (kt0 + t) * ABN + ABN - 1 >= pos_first) {
                    pdl_wait();                           // this tile holds keys the kernel in front writes
                    waited = true;
                }
                if (lane == 0) {
                    ok = mbar_wait(empty0 + 8 * s, ((j / STAGES) & 1) ^ 1, abort_flag, err);
                    if (ok) mbar_arrive_expect_tx(full0 + 8 * s, 2 * TILE);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                for (int pg = 0; pg < pages; pg++) {
                    const int row = __shfl_sync(0xffffffffu, my_row, t * pages + pg);
                    if (lane == 0) {
                        const uint32_t dst = st0 + (uint32_t)s * 2 * TILE + (uint32_t)pg * 2 * page_bytes;
                        if (ONE_MAP) {
                            tma_load_4d(dst, &map_k, 0, row, g * HALVES, 0, full0 + 8 * s);
                        } else {
                            tma_load_3d(dst, &map_k, 0, row, g * HALVES, full0 + 8 * s);
                            tma_load_3d(dst + page_bytes, &map_v, 0, row, g * HALVES, full0 + 8 * s);
                        }
                    }
                }
            }
            if (!ok) break;
        }
    } else {
        // ---- the computing warps: 16 keys of every tile each --------------------------------------------
        pdl_sync();                                       // the queries come from the kernel in front
        for (int i = threadIdx.x; i < 16 * CH; i += 128) {
            int row = i / CH, c = i % CH;
            int tl = row / r, hl = row % r;
            bool valid = tl < nt;
            const __nv_bfloat16 *src = p.q + ((size_t)(t0 + (valid ? tl : 0)) * p.H + g * r + hl) * D + c * 8;
            cp_async16(sq + swz<D>(row, c), src, valid);
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        HFB_TRACE_MARK(5);
        uint32_t qf[D / 16][4];
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++)
            ldsm_x4(sq + swz<D>(lane & 15, kk * 2 + (lane >> 4)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);

        const int tl0 = row0 / r, tl1 = row1 / r;
        const bool v0 = tl0 < nt, v1 = tl1 < nt;
        const int pos0 = v0 ? p.positions[t0 + tl0] : -1, pos1 = v1 ? p.positions[t0 + tl1] : -1;
        const int lo0 = p.window > 0 ? max(0, pos0 - p.window + 1) : 0, lo1 = p.window > 0 ? max(0, pos1 - p.window + 1) : 0;
        const int kbase = warp * 16, mi = lane >> 3;
        // the 8 keys whose rows this lane names to ldmatrix lie in one page (pages hold 8 keys or more)
        const int bs = p.block_size;
        const int krow = kbase + (mi >> 1) * 8 + (lane & 7), vrow = kbase + (mi & 1) * 8 + (lane & 7);
        const uint32_t k_page = (uint32_t)(krow / bs) * 2 * page_bytes, v_page = (uint32_t)(vrow / bs) * 2 * page_bytes + page_bytes;
        const int k_kr = krow % bs, v_kr = vrow % bs;

        for (int kt = kt_lo; kt < kt_hi; kt++) {
            const int j = kt - kt_lo, s = j % STAGES;
            if (!mbar_wait(full0 + 8 * s, (j / STAGES) & 1, abort_flag, err)) break;
            const uint32_t ks = st0 + s * 2 * TILE + k_page, vs = st0 + s * 2 * TILE + v_page;
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(ks + page_off(k_kr, kk * 2 + (mi & 1), bs), b0, b1, b2, b3);
                mma_bf16(sc[0], qf[kk], b0, b1);
                mma_bf16(sc[1], qf[kk], b2, b3);
            }
            // a tile wholly inside every row's range needs no mask
            const bool edge = kt * ABN + ABN - 1 > pos_first || kt * ABN < lo_last;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 2; i++) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    float a = sc[i][e] * p.scale_log2, b = sc[i][2 + e] * p.scale_log2;
                    if (edge) {
                        const int key = kt * ABN + kbase + i * 8 + (lane & 3) * 2 + e;
                        a = (v0 && key >= lo0 && key <= pos0) ? a : -INFINITY;
                        b = (v1 && key >= lo1 && key <= pos1) ? b : -INFINITY;
                    }
                    sc[i][e] = a; sc[i][2 + e] = b;
                    mx0 = fmaxf(mx0, a); mx1 = fmaxf(mx1, b);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            if (__any_sync(0xffffffffu, mn0 > m0 || mn1 > m1)) {
                // a maximum grew somewhere in the warp: rescale what has been summed so far
                const float c0 = fast_exp2(m0 - (mn0 == -INFINITY ? 0.f : mn0)), c1 = fast_exp2(m1 - (mn1 == -INFINITY ? 0.f : mn1));
                l0 *= c0; l1 *= c1;
#pragma unroll
                for (int i = 0; i < D / 8; i++) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
                m0 = mn0; m1 = mn1;
            }
            const float base0 = m0 == -INFINITY ? 0.f : m0, base1 = m1 == -INFINITY ? 0.f : m1;
            uint32_t pf[4];
            const float p00 = fast_exp2(sc[0][0] - base0), p01 = fast_exp2(sc[0][1] - base0), p10 = fast_exp2(sc[0][2] - base1), p11 = fast_exp2(sc[0][3] - base1);
            const float q00 = fast_exp2(sc[1][0] - base0), q01 = fast_exp2(sc[1][1] - base0), q10 = fast_exp2(sc[1][2] - base1), q11 = fast_exp2(sc[1][3] - base1);
            pf[0] = pack_bf16(p00, p01); pf[1] = pack_bf16(p10, p11); pf[2] = pack_bf16(q00, q01); pf[3] = pack_bf16(q10, q11);
            l0 += p00 + p01 + q00 + q01;
            l1 += p10 + p11 + q10 + q11;
#pragma unroll
            for (int dn = 0; dn < D / 16; dn++) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(vs + page_off(v_kr, dn * 2 + (mi >> 1), bs), b0, b1, b2, b3);
                mma_bf16(o[2 * dn], pf, b0, b1);
                mma_bf16(o[2 * dn + 1], pf, b2, b3);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }

    // ---- merge the four warps (they saw disjoint keys) in warp order -------------------------------------
    __syncthreads();                                      // every tile has been used: its buffers are free
    HFB_TRACE_MARK(6);
    const bool dead = *abort_flag != 0;
    if (dead) {
        // a wait ran out: give copies that are still in flight time to land before the shared memory goes away
        if (threadIdx.x == 0)
            for (int i = 0; i < 2000; i++) __nanosleep(1000);
        __syncthreads();
        return;
    }
    float *mo = (float *)gen;                             // [4][16][D]
    float *mml = mo + 4 * 16 * D;                         // [4][16][2]
    if (warp < 4) {
#pragma unroll
        for (int i = 0; i < D / 8; i++) {
            int col = i * 8 + (lane & 3) * 2;
            *(float2 *)(mo + ((size_t)warp * 16 + row0) * D + col) = make_float2(o[i][0], o[i][1]);
            *(float2 *)(mo + ((size_t)warp * 16 + row1) * D + col) = make_float2(o[i][2], o[i][3]);
        }
        if ((lane & 3) == 0) {
            *(float2 *)(mml + (warp * 16 + row0) * 2) = make_float2(m0, l0);
            *(float2 *)(mml + (warp * 16 + row1) * 2) = make_float2(m1, l1);
        }
    }
    __syncthreads();
    const int rows = nt * r;
    // Every thread works out the four warps' weights of its row itself (four exponentials) instead of waiting at a
    // barrier for sixteen threads to do it: a piece of four columns per thread and turn.
    for (int idx = threadIdx.x; idx < rows * (D / 4); idx += ADT_THREADS) {
        const int row = idx / (D / 4), c4 = idx % (D / 4);
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) m = fmaxf(m, mml[(w * 16 + row) * 2]);
        float denom = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 4; w++) {                     // in warp order
            const float mw = mml[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - m);
            denom += mml[(w * 16 + row) * 2 + 1] * f;
            const float4 v = *(const float4 *)(mo + ((size_t)w * 16 + row) * D + 4 * c4);
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        const int tok = t0 + row / r, head = g * r + row % r;
        const size_t th = (size_t)tok * p.H + head;
        if (p.splits > 1) {
            *(float4 *)(p.part_o + (th * p.splits + split) * D + 4 * c4) = acc;
            if (c4 == 0) *(float2 *)(p.part_ml + (th * p.splits + split) * 2) = make_float2(m, denom);
        } else {
            const float inv = denom > 0.f ? 1.0f / denom : 0.f;       // (as the merge of key splits normalises)
            const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
            *(uint2 *)(p.out + th * D + 4 * c4) = make_uint2(*(const uint32_t *)&lo, *(const uint32_t *)&hi);
        }
    }
    if (p.splits > 1 && p.counters) {
        // This split is in global memory.  Count it; the CTA that brings the count of its (tile, key/value head) to
        // the number of splits merges them, in split order whichever CTA it is, with the arithmetic of
        // attention_combine_kernel: out = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s.
        volatile int *last_flag = abort_flag + 1;
        __syncthreads();
        HFB_TRACE_MARK(7);
        if (threadIdx.x == 0) {
            __threadfence();                              // (after the barrier: it covers every thread's stores)
            int *cnt = p.counters + (size_t)tile * p.G + g;
            const int last = atomicAdd(cnt, 1) == p.splits - 1;
            if (last) *cnt = 0;
            *last_flag = last;
        }
        __syncthreads();
        if (!*last_flag) return;
        if (tile == 0 && g == 0) HFB_TRACE_ANY(8);
        __threadfence();
        // What this costs is the latency of reads from the L2 cache, so they are issued many at a time.  First, per
        // row, the weight of every split: f_s = 2^(m_s - m) / sum_s' l_s' 2^(m_s' - m).
        constexpr int MAXS = 64;                          // (the host asks for no more splits than this)
        float *fs = (float *)gen;                         // [16][MAXS]; the tile buffers are free
        const int n_elems = rows * (D / 4);               // float4 pieces of the merged rows
        if (p.splits <= 16) {
            // Up to sixteen splits: every thread reads the splits' maxima and sums of its row itself, beside its piece
            // of their outputs, all at once: one trip to L2 instead of two with a barrier between them (batch 8: 1.2 %
            // of the step, batch 1: 2 %).  The same arithmetic in the same order as below.
            for (int e = threadIdx.x; e < n_elems; e += ADT_THREADS) {
                const int row = e / (D / 4), c4 = e % (D / 4);
                const size_t th = (size_t)(t0 + row / r) * p.H + g * r + row % r;
                const float2 *ml = (const float2 *)(p.part_ml + th * p.splits * 2);
                const float4 *src = (const float4 *)(p.part_o + th * p.splits * D) + c4;
                float2 w[16];
                float4 v[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    w[i] = i < p.splits ? __ldcg(ml + i) : make_float2(-INFINITY, 0.f);
                    v[i] = i < p.splits ? __ldcg(src + (size_t)i * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float m = -INFINITY;
#pragma unroll
                for (int i = 0; i < 16; i++) m = fmaxf(m, w[i].x);
                float denom = 0.f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 16; i++) {                 // in split order
                    const float f = (i >= p.splits || w[i].x == -INFINITY) ? 0.f : exp2f(w[i].x - m);
                    if (i < p.splits) denom += w[i].y * f;
                    acc.x += v[i].x * f; acc.y += v[i].y * f; acc.z += v[i].z * f; acc.w += v[i].w * f;
                }
                const float inv = denom > 0.f ? 1.0f / denom : 0.f;
                const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                *(uint2 *)(p.out + th * D + 4 * c4) = make_uint2(*(const uint32_t *)&lo, *(const uint32_t *)&hi);
            }
            if (tile == 0 && g == 0) HFB_TRACE_ANY(9);
            return;
        }
        if (threadIdx.x < rows) {
            const int row = threadIdx.x;
            const size_t th = (size_t)(t0 + row / r) * p.H + g * r + row % r;
            const float2 *ml = (const float2 *)(p.part_ml + th * p.splits * 2);
            float m = -INFINITY;
            for (int c = 0; c < p.splits; c += 16) {
                float2 v[16];
#pragma unroll
                for (int i = 0; i < 16; i++) v[i] = c + i < p.splits ? __ldcg(ml + c + i) : make_float2(-INFINITY, 0.f);
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    m = fmaxf(m, v[i].x);
                    if (c + i < p.splits) { fs[row * MAXS + c + i] = v[i].x; fs[(16 + row) * MAXS + c + i] = v[i].y; }
                }
            }
            float denom = 0.f;
            for (int s = 0; s < p.splits; s++) {
                const float ms = fs[row * MAXS + s];
                const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
                denom += fs[(16 + row) * MAXS + s] * f;
                fs[row * MAXS + s] = f;
            }
            const float inv = denom > 0.f ? 1.0f / denom : 0.f;
            fs[(16 + row) * MAXS] = inv;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < n_elems; e += ADT_THREADS) {
            const int row = e / (D / 4), c4 = e % (D / 4);
            const size_t th = (size_t)(t0 + row / r) * p.H + g * r + row % r;
            const float4 *src = (const float4 *)(p.part_o + th * p.splits * D) + c4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = 0; c < p.splits; c += 16) {
                float4 v[16];
#pragma unroll
                for (int i = 0; i < 16; i++)
                    v[i] = c + i < p.splits ? __ldcg(src + (size_t)(c + i) * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 16; i++) {                 // in split order
                    const float f = c + i < p.splits ? fs[row * MAXS + c + i] : 0.f;
                    acc.x += v[i].x * f; acc.y += v[i].y * f; acc.z += v[i].z * f; acc.w += v[i].w * f;
                }
            }
            const float inv = fs[(16 + row) * MAXS];
            const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
            *(uint2 *)(p.out + th * D + 4 * c4) = make_uint2(*(const uint32_t *)&lo, *(const uint32_t *)&hi);
        }
        if (tile == 0 && g == 0) HFB_TRACE_ANY(9);
    }
}

template <int D, int STAGES, bool ONE_MAP>
static int launch_decode_tma(const CUtensorMap &mk, const CUtensorMap &mv, const AttnParams &p, int num_slots, int n_tiles, cudaStream_t st)
{
    constexpr uint32_t TILE = (D / 64) * ABN * 128;
    constexpr int smem = 1024 + 2 * STAGES * TILE + 16 * D * 2 + 16 * STAGES + 16;
    static_assert(2 * STAGES * TILE >= (4 * 16 * (D + 2) + 96) * 4 && 2 * STAGES * TILE >= 32 * 64 * 4, "the merge reuses the tile buffers");
    static bool configured[64] = {false};                 // (the opt-in is a property of the function on one device)
    if (!configured[current_device()]) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<D, STAGES, ONE_MAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "attention_decode: cannot opt in to %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[current_device()] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, p.G, p.splits);
    cfg.blockDim = dim3(ADT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    g_launch_err = cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<D, STAGES, ONE_MAP>, mk, mv, p, num_slots, error_word());
    return check_pdl_launch(g_launch_err, "attention_decode");
}

template <int D, bool ONE_MAP>
static int launch_decode_stages(int stages, const CUtensorMap &mk, const CUtensorMap &mv, const AttnParams &p, int num_slots, int n_tiles, cudaStream_t st)
{
    return stages >= 4 ? launch_decode_tma<D, 4, ONE_MAP>(mk, mv, p, num_slots, n_tiles, st)
         : stages == 3 ? launch_decode_tma<D, 3, ONE_MAP>(mk, mv, p, num_slots, n_tiles, st)
                       : launch_decode_tma<D, 2, ONE_MAP>(mk, mv, p, num_slots, n_tiles, st);
}

}  // namespace hfb

using namespace hfb;

// Decode attention (tiles of one or two tokens of one request each, as hfb_attention_fast's 16-row form makes
// them): bfloat16, head_dim 64 or 128, block sizes 8..64 that divide 64, at most 16 query rows per tile.
// `stages` tiles of 64 keys are in flight per CTA (2..4); `splits` > 1 cuts each request's keys over that many
// CTAs and needs hfb_attention_fast_scratch(T, H, d, splits) bytes of float32 scratch.  The splits are merged in
// split order: by the CTA that stores a tile's last split, when `counters` (n_tiles * G ints, zero before the first
// launch; every launch leaves them zero) is given, else by a second kernel.
extern "C" int hfb_attention_decode(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                                    int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                                    const int32_t *tile_nt, int n_tiles, int stages, int splits, int block_size,
                                    int64_t num_pages, int window, float scale, void *out, void *scratch, size_t scratch_bytes,
                                    int T, int H, int G, int d, int *counters, int counters_len, hfb_stream s)
{
    if (n_tiles <= 0) return HFB_OK;
    if (d != 64 && d != 128) return fail(HFB_ENOTSUP, "attention_decode: head_dim %d (64 and 128 only)", d);
    if (G <= 0 || H % G || H / G > 16) return fail(HFB_ENOTSUP, "attention_decode: %d heads over %d key/value heads do not fit 16 rows", H, G);
    if (block_size < 8 || block_size > ABN || ABN % block_size) return fail(HFB_ENOTSUP, "attention_decode: block size %d (8..64, dividing 64)", block_size);
    if (num_pages * block_size >= (1ll << 31) - ABN) return fail(HFB_ENOTSUP, "attention_decode: cache too large for 32-bit coordinates");
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return fail(HFB_ENOTSUP, "attention_decode: operands must be 16-byte aligned");
    if (splits < 1 || G > 65535 || splits > 65535) return fail(HFB_EINVAL, "attention_decode: bad split or group count");
    if (splits > 1 && (!scratch || scratch_bytes < (size_t)T * H * splits * (d + 2) * sizeof(float)))
        return fail(HFB_EINVAL, "attention_decode: scratch of %zu bytes is too small for %d splits", scratch_bytes, splits);
    CUtensorMap maps[2];
    bool one_map = false;
    int rc;
    const int slots = (int)(num_pages * block_size);
    if ((rc = tensor_map_kv(k_cache, v_cache, slots, G * d, block_size, d / 64, maps, &one_map)) != HFB_OK) return rc;
    const CUtensorMap &mk = maps[0], &mv = maps[one_map ? 0 : 1];
    AttnParams p;
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.block_table = block_table; p.positions = positions;
    p.tile_seq = tile_seq; p.tile_t0 = tile_t0; p.tile_nt = tile_nt;
    p.part_o = (float *)scratch; p.part_ml = splits > 1 ? (float *)scratch + (size_t)T * H * splits * d : nullptr;
    p.max_blocks = max_blocks; p.block_size = block_size; p.window = window; p.H = H; p.G = G; p.splits = splits;
    p.num_pages = num_pages; p.scale_log2 = scale * 1.4426950408889634f;
    p.counters = (splits > 1 && splits <= 64 && counters && counters_len >= n_tiles * G) ? counters : nullptr;
    cudaStream_t st = (cudaStream_t)s;
    if (one_map) rc = d == 128 ? launch_decode_stages<128, true>(stages, mk, mv, p, slots, n_tiles, st)
                               : launch_decode_stages<64, true>(stages, mk, mv, p, slots, n_tiles, st);
    else rc = d == 128 ? launch_decode_stages<128, false>(stages, mk, mv, p, slots, n_tiles, st)
                       : launch_decode_stages<64, false>(stages, mk, mv, p, slots, n_tiles, st);
    if (rc != HFB_OK || splits == 1 || p.counters) return rc;
    return launch_attention_combine(p, T, d, st);
}
