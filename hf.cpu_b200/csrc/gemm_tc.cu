// out[M,N] (=|+=) a[M,K] . w[N,K]^T (+ bias) for bfloat16 operands on the 5th-generation tensor cores.
//
// Both operands are K-major (rows of K contiguous elements), which is what tcgen05.mma wants of
// shared-memory operands, so one kernel serves prefill and decode by choosing which operand
// supplies the 128 accumulator rows ("X", rows -> TMEM lanes) and which the columns ("Y", rows ->
// TMEM columns, 16..256 of them):
//   * many tokens: X = activations, Y = weights (tile 128 tokens x BN features);
//   * few tokens (decode): X = weights, Y = activations (tile 128 features x BN tokens, "swapped"),
//     so that the tensor core's 128 rows are filled by the weight matrix that has to be streamed
//     from HBM anyway, with split-K when there are fewer weight tiles than SMs.
// Above 128 tokens the inner dimension is split as well when the output has few tiles and K is long (mid_splits).
// Pipeline per CTA (persistent over work items): warp 0 issues TMA loads of 128-byte-swizzled K
// blocks into a ring of shared-memory stages (the weights of the first round before the kernel in front has finished,
// warp 10 the activations of that round as soon as it has); warp 1 issues tcgen05.mma from shared memory into one
// of two TMEM accumulators and commits to the stage's "empty" barrier; warps 2..9 read a finished
// accumulator with tcgen05.ld (two warps per quarter of its lanes, half of the columns each), apply the epilogue and
// store, while the next tile's products run.
// Every barrier wait has a time limit: on expiry the kernel raises HFB_ERR_WAIT in the device error
// word, lets its copies land, frees its TMEM and returns.
//
// The reference computes the same products with one dot per (row, token) after widening the weight
// row to float (src/model.c:369-440, src/kern_avx2.c:79-95); accumulation here is float32 too.
#include <cuda.h>

#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tc_ptx.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

constexpr int BK = 64;                 // bf16 elements per K block: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int TILE_X = 128;            // accumulator rows (TMEM lanes)
constexpr uint32_t X_BYTES = TILE_X * BK * 2;
constexpr int GEMM_THREADS = 352;            // weight-tile warp, MMA warp, eight epilogue warps, activation-tile warp
constexpr int HELPER_WARP = 10;
constexpr int PAIR_THREADS = 224;            // pair kernel: weight-tile warp, MMA warp, four epilogue warps, activation-tile warp
constexpr int PAIR_ACT_WARP = 6;

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_PARTIAL = 2, EPI_SWIGLU = 3, EPI_ROPE_KV = 4 };

struct GemmParams {
    int M, N, K;                       // logical sizes: tokens, output features, inner
    int swapped;                       // X = weights, Y = activations
    int pair;                          // tiles of 256 tokens on pairs of CTAs (gemm_tc_pair_kernel)
    int tiles_x, tiles_y, splits, kb_total, kb_per_split;
    void *out; int out_dt;             // [M, N]
    const void *bias; int bias_dt;     // [N] or null
    int mode;
    float *partial;                    // [splits, M, N] when mode == EPI_PARTIAL
    // mode == EPI_ROPE_KV (pair kernel, tiles of whole heads): the output is the q|k|v row of a token; bias, rounding
    // to bfloat16, rotation of the query and key heads by the token's position, queries to q_out, keys and values to
    // the token's cache slot
    const float *cos_sin;              // [n_positions, d / 2, 2]
    const int32_t *positions, *slots;  // per token; slots may be null (nothing is cached)
    __nv_bfloat16 *q_out, *k_cache, *v_cache;
    long long cache_slots;
    int n_positions, H, G, d;
};

// Shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_X >> 4) << 24);
}

template <int BN> constexpr int tmem_cols()
{
    int need = 2 * BN, c = 32;
    while (c < need) c <<= 1;
    return c;
}

template <int BN, int STAGES> constexpr uint32_t gemm_smem_bytes()
{
    return 1024 + STAGES * (X_BYTES + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16;
}

// One chunk of 16 accumulator columns of one row: v[i] is element (xr, y0 + i) of X . Y^T.
// `live` false: the same instructions, nothing stored (the few-token form runs its epilogue once this way while the
// first weights are on their way, so that its code is in the instruction cache when the first tile is done: fetched
// at that moment it waits behind the weight stream, several microseconds for a 64-token tile).
__device__ __forceinline__ void epilogue_chunk(const GemmParams &p, const uint32_t *v, int xr, int y0, int split, int lane,
                                               bool live = true)
{
    if (!live && !p.swapped) return;
    if (p.swapped && p.mode == EPI_SWIGLU) {
        // rows alternate gate, up: even lanes hold gate_i, the next lane holds up_i; out is [M, N/2].  The two lanes
        // of a pair exchange their values and share the work: of every two tokens the even lane finishes the first,
        // the odd lane the second.
        const int odd = lane & 1;
        const int in_chunk = min(16, p.M - y0);                                  // the same for the whole warp
        const int n_tok = (live && (xr | 1) < p.N) ? in_chunk : 0;
        const size_t half_n = (size_t)(p.N >> 1), at = (size_t)y0 * half_n + (size_t)(xr >> 1);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (2 * j >= in_chunk) break;
            const float first = __uint_as_float(v[2 * j]), second = __uint_as_float(v[2 * j + 1]);
            const float their_first = __shfl_xor_sync(0xffffffffu, first, 1);
            const float their_second = __shfl_xor_sync(0xffffffffu, second, 1);
            const float g = odd ? their_second : first, u = odd ? second : their_first;
            const float h = (g / (1.0f + expf(-g))) * u;
            const int i = 2 * j + odd;
            if (i < n_tok) {
                if (p.out_dt == HFB_BF16) ((__nv_bfloat16 *)p.out)[at + (size_t)i * half_n] = __float2bfloat16_rn(h);
                else ((float *)p.out)[at + (size_t)i * half_n] = h;
            }
        }
    } else if (p.swapped) {
        // xr = output feature, y = token.  One warp per scheduler runs this, so the work per token is kept to a
        // handful of instructions: the mode is decided outside the loops, the address is a base plus i rows.
        if (xr < p.N) {
            const int n_tok = live ? min(16, p.M - y0) : 0;
            const size_t at = (size_t)y0 * p.N + xr;
            if (p.mode == EPI_PARTIAL) {
                float *dst = p.partial + (size_t)split * p.M * p.N + at;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    if (i >= n_tok) break;               // (the same for the whole warp: with one token, one turn)
                    dst[(size_t)i * p.N] = __uint_as_float(v[i]);
                }
            } else {
                const float b = p.bias ? load_any(p.bias, p.bias_dt, xr) : 0.f;
                if (p.mode == EPI_ADD) {
                    float *dst = (float *)p.out + at;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        if (i >= n_tok) break;
                        dst[(size_t)i * p.N] += __uint_as_float(v[i]) + b;
                    }
                } else if (p.out_dt == HFB_BF16) {
                    __nv_bfloat16 *dst = (__nv_bfloat16 *)p.out + at;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        if (i >= n_tok) break;
                        dst[(size_t)i * p.N] = __float2bfloat16_rn(__uint_as_float(v[i]) + b);
                    }
                } else {
                    float *dst = (float *)p.out + at;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        if (i >= n_tok) break;
                        dst[(size_t)i * p.N] = __uint_as_float(v[i]) + b;
                    }
                }
            }
        }
    } else if (p.mode == EPI_SWIGLU) {
        // columns alternate gate, up: 8 pairs -> 8 outputs of row xr, out is [M, N/2]
        if (xr < p.M && y0 < p.N) {
            float h[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float g = __uint_as_float(v[2 * i]), u = __uint_as_float(v[2 * i + 1]);
                h[i] = (g / (1.0f + expf(-g))) * u;
            }
            size_t o = (size_t)xr * (p.N >> 1) + (y0 >> 1);
            if (y0 + 16 <= p.N && (p.N & 15) == 0 && p.out_dt == HFB_BF16) {
                __nv_bfloat162 hh[4];
#pragma unroll
                for (int i = 0; i < 4; i++) hh[i] = __floats2bfloat162_rn(h[2 * i], h[2 * i + 1]);
                *(uint4 *)((__nv_bfloat16 *)p.out + o) = *(uint4 *)&hh[0];
            } else {
                for (int i = 0; i < 8 && y0 + 2 * i + 1 < p.N; i++) store_any(p.out, p.out_dt, o + i, h[i]);
            }
        }
    } else if (xr < p.M && y0 < p.N) {
        // xr = token, y = output feature: 16 consecutive features of one row
        size_t o = (size_t)xr * p.N + y0;
        bool full = y0 + 16 <= p.N && (p.N & 7) == 0;
        float f[16];
#pragma unroll
        for (int i = 0; i < 16; i++) f[i] = __uint_as_float(v[i]);
        if (p.bias && p.mode != EPI_PARTIAL) {
            if (full && p.bias_dt == HFB_BF16) {
                // 16 consecutive bias values in two 16-byte loads (N is a multiple of 8 here, so they are aligned)
                const uint4 *bp = (const uint4 *)((const __nv_bfloat16 *)p.bias + y0);
                uint4 b0 = bp[0], b1 = bp[1];
                const __nv_bfloat162 *h0 = (const __nv_bfloat162 *)&b0, *h1 = (const __nv_bfloat162 *)&b1;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float2 x = __bfloat1622float2(h0[i]), y = __bfloat1622float2(h1[i]);
                    f[2 * i] += x.x; f[2 * i + 1] += x.y; f[8 + 2 * i] += y.x; f[8 + 2 * i + 1] += y.y;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (full || y0 + i < p.N) f[i] += load_any(p.bias, p.bias_dt, y0 + i);
            }
        }
        if (p.mode == EPI_PARTIAL) {
            float *dst = p.partial + (size_t)split * p.M * p.N + o;
            if (full) {
#pragma unroll
                for (int i = 0; i < 16; i += 4) *(float4 *)(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
            } else {
                for (int i = 0; i < 16 && y0 + i < p.N; i++) dst[i] = f[i];
            }
        } else if (p.mode == EPI_ADD) {
            float *dst = (float *)p.out + o;
            if (full) {
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    float4 r = *(float4 *)(dst + i);
                    *(float4 *)(dst + i) = make_float4(r.x + f[i], r.y + f[i + 1], r.z + f[i + 2], r.w + f[i + 3]);
                }
            } else {
                for (int i = 0; i < 16 && y0 + i < p.N; i++) dst[i] += f[i];
            }
        } else if (p.out_dt == HFB_BF16 && full) {
            __nv_bfloat162 h[8];
#pragma unroll
            for (int i = 0; i < 8; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            uint4 *dst = (uint4 *)((__nv_bfloat16 *)p.out + o);
            dst[0] = *(uint4 *)&h[0];
            dst[1] = *(uint4 *)&h[4];
        } else if (p.out_dt == HFB_F32 && full) {
            float *dst = (float *)p.out + o;
#pragma unroll
            for (int i = 0; i < 16; i += 4) *(float4 *)(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
        } else {
            for (int i = 0; i < 16 && y0 + i < p.N; i++) store_any(p.out, p.out_dt, o + i, f[i]);
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, GemmParams p, int *err)
{
    HFB_TRACE_ENTRY(1);
    constexpr uint32_t Y_BYTES = BN * BK * 2;
    constexpr int TCOLS = tmem_cols<BN>();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sx = base, sy = base + STAGES * X_BYTES;
    const uint32_t bars = sy + STAGES * Y_BYTES;
    const uint32_t full0 = bars, empty0 = bars + STAGES * 8, tfull0 = bars + 2 * STAGES * 8, tempty0 = tfull0 + 16;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(gen_base + STAGES * (X_BYTES + Y_BYTES) + (2 * STAGES + 4) * 8);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 8); }       // eight epilogue warps
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"(TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    HFB_TRACE_MARK(2);

    const int total_items = p.tiles_x * p.tiles_y * p.splits;
    const int per_split = p.tiles_x * p.tiles_y;

    if (warp == 0 || warp == HELPER_WARP) {
        // ---- two requesting threads, one per operand -------------------------------------------------------------
        // The weights do not depend on the kernel before this one, the activations do.  Lane 0 of warp 0 arms each
        // stage's "full" barrier and asks for its weight tile, without ever waiting for that kernel: the first STAGES
        // tiles are under way long before it has finished.  Lane 0 of the last warp waits for it and asks for the
        // activation tiles (both copies count on the stage's barrier, whose phase ends when the armed bytes have
        // arrived, in whichever order).  The other lanes of both warps do nothing: a lane in griddepcontrol.wait
        // would hold up its whole warp.
        const bool weights = warp == 0;
        if (lane == 0) {
            if (!weights) { pdl_sync(); HFB_TRACE_READY_HERE(); }
            uint32_t it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                int split = item / per_split, t = item % per_split;
                int tx = t % p.tiles_x, ty = t / p.tiles_x;
                int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    int s = it % STAGES;
                    uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, err)) { ok = false; break; }
                    if (weights) mbar_arrive_expect_tx(full0 + 8 * s, X_BYTES + Y_BYTES);
                    if (weights == (p.swapped != 0)) tma_load_2d(sx + s * X_BYTES, &map_x, kb * BK, tx * TILE_X, full0 + 8 * s);
                    else tma_load_2d(sy + s * Y_BYTES, &map_y, kb * BK, ty * BN, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ------------------------------------------------------------------
        pdl_sync();
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            int last_s = -1;
            uint32_t last_ph = 0;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, tile_it++) {
                int split = item / per_split;
                int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                int a = tile_it & 1;
                uint32_t aph = (tile_it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * a, aph ^ 1, abort_flag, err)) { ok = false; break; }
                tc_fence_after();
                uint32_t d = tmem_base + a * BN;
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    int s = it % STAGES;
                    uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, err)) { ok = false; break; }
                    tc_fence_after();
                    uint64_t dx = smem_desc(sx + s * X_BYTES), dy = smem_desc(sy + s * Y_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        tc_mma_bf16(d, dx + 2 * k, dy + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * s);
                    last_s = s;
                    last_ph = ph;
                }
                if (ok) tc_commit(tfull0 + 8 * a);
            }
            // all commits have landed once the last one has: nothing of this CTA's is in flight afterwards
            if (ok && last_s >= 0) mbar_wait(empty0 + 8 * last_s, last_ph, abort_flag, err);
        }
    } else {
        // ---- epilogue: TMEM -> registers -> global ------------------------------------------------
        // Warps 2..5 and 6..9: two warps for each quarter of the TMEM lanes (a warp may read the quarter its index
        // names), each with half of the accumulator's columns, so that a tile's last, exposed epilogue takes half the time.
        const int q = warp & 3;                       // the TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        constexpr int C_STEP = BN >= 32 ? 32 : 16;
        constexpr int C_SPLIT = BN >= 64 ? ((BN / 32 + 1) / 2) * 32 : BN;
        const int c_lo = warp >= 6 ? C_SPLIT : 0, c_hi = warp >= 6 ? BN : C_SPLIT;
        uint32_t tile_it = 0;
        bool ok = true;
        // With few tokens the first turn of this loop is a rehearsal: it reads whatever the accumulator holds and
        // stores nothing, before the kernel in front is known to have finished (see epilogue_chunk).
        bool rehearsal = p.swapped != 0;
        if (!rehearsal) pdl_sync();                   // nothing is written before the kernel in front has finished
        for (int item = blockIdx.x; item < total_items && ok;) {
            int split = item / per_split, t = item % per_split;
            int tx = t % p.tiles_x, ty = t / p.tiles_x;
            int a = tile_it & 1;
            uint32_t aph = (tile_it >> 1) & 1;
            if (!rehearsal) {
                if (!mbar_wait(tfull0 + 8 * a, aph, abort_flag, err)) { ok = false; break; }
                tc_fence_after();
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * BN;
            const int xr = tx * TILE_X + row;         // row of X this thread holds
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += C_STEP) {
                uint32_t v[C_STEP];
                const bool two = BN >= 32 && c0 + 16 < c_hi;     // widths such as 208 end on a single chunk
                tmem_ld16(taddr + c0, v);
                if (two) tmem_ld16(taddr + c0 + 16, v + (BN >= 32 ? 16 : 0));
                tmem_wait_ld();
                epilogue_chunk(p, v, xr, ty * BN + c0, split, lane, !rehearsal);
                if (two) epilogue_chunk(p, v + (BN >= 32 ? 16 : 0), xr, ty * BN + c0 + 16, split, lane, !rehearsal);
            }
            if (rehearsal) {
                rehearsal = false;
                pdl_sync();
                continue;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * a);
            item += gridDim.x;
            tile_it++;
        }
        if (rehearsal) pdl_sync();                    // (no work item at all)
    }

    // ---- teardown --------------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // a wait ran out: give loads that are still in flight time to land before the shared memory goes away
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TCOLS) : "memory");
    }
}


// ---- the same product on pairs of SMs (cta_group::2), for many tokens ---------------------------------------
// Two CTAs of a thread-block cluster share a tile of 256 tokens x BN features.  Each loads its 128 rows of the
// activations and its half of the weight tile (BN/2 rows); the tensor cores of both SMs read both halves, so a k
// block costs each SM 32 KB of shared-memory traffic for 128 x 256 x 64 products instead of 48 KB, which is what
// bounds the single-CTA kernel.  The even CTA of the pair issues every product (tcgen05.mma.cta_group::2, M = 256)
// and releases stages and accumulators in both CTAs with one multicast commit; the copies of both CTAs complete on
// the even CTA's "full" barrier (the loads themselves are plain, not multicast); each CTA drains its own 128 rows
// of the accumulator from its own TMEM.  Waits are bounded as everywhere; the cluster barriers at both ends are
// reached on every path.
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_barrier()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// a plain (not multicast) tiled copy whose bytes are counted on a barrier that may lie in the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar_cluster_addr)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the products issued so far are done, on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}

// The q|k|v epilogue of one head of one token (see GemmParams): `lo` and `hi` are 32 accumulator columns each, of the
// head's first half from j0 on and of its second half from j0 on; the rotation pairs column i with column i + d/2.
__device__ __forceinline__ void rope_kv_piece(const GemmParams &p, const uint32_t *lo, const uint32_t *hi, int col, int j0,
                                              const float *cs, bool rotate, __nv_bfloat16 *dst)
{
    const int half = p.d >> 1;
    float bl[32], bh[32];
    if (p.bias) {
        const uint4 *b0 = (const uint4 *)((const __nv_bfloat16 *)p.bias + col + j0), *b1 = (const uint4 *)((const __nv_bfloat16 *)p.bias + col + half + j0);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint4 x = b0[q], y = b1[q];
            const __nv_bfloat162 *hx = (const __nv_bfloat162 *)&x, *hy = (const __nv_bfloat162 *)&y;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 fx = __bfloat1622float2(hx[e]), fy = __bfloat1622float2(hy[e]);
                bl[8 * q + 2 * e] = fx.x; bl[8 * q + 2 * e + 1] = fx.y; bh[8 * q + 2 * e] = fy.x; bh[8 * q + 2 * e + 1] = fy.y;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; i++) bl[i] = bh[i] = 0.f;
    }
    __align__(16) __nv_bfloat16 ol[32], oh[32];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        // the separate kernels round q|k|v to bfloat16 before they rotate; the same values here
        const float a0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[i]) + bl[i]));
        const float a1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[i + 1]) + bl[i + 1]));
        const float b0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[i]) + bh[i]));
        const float b1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[i + 1]) + bh[i + 1]));
        if (rotate) {
            const float4 c = *(const float4 *)(cs + 2 * (j0 + i));           // cos, sin of pair j0 + i and of the next
            float l0, h0, l1, h1;
            rope_pair(a0, b0, c.x, c.y, l0, h0);
            rope_pair(a1, b1, c.z, c.w, l1, h1);
            ol[i] = __float2bfloat16_rn(l0); oh[i] = __float2bfloat16_rn(h0);
            ol[i + 1] = __float2bfloat16_rn(l1); oh[i + 1] = __float2bfloat16_rn(h1);
        } else {
            ol[i] = __float2bfloat16_rn(a0); oh[i] = __float2bfloat16_rn(b0);
            ol[i + 1] = __float2bfloat16_rn(a1); oh[i + 1] = __float2bfloat16_rn(b1);
        }
    }
#pragma unroll
    for (int q = 0; q < 4; q++) {
        *(uint4 *)(dst + j0 + 8 * q) = *(const uint4 *)(ol + 8 * q);
        *(uint4 *)(dst + half + j0 + 8 * q) = *(const uint4 *)(oh + 8 * q);
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, GemmParams p, int *err)
{
    HFB_TRACE_ENTRY(1);
    constexpr uint32_t Y_BYTES = (BN / 2) * BK * 2;          // this CTA's half of the weight tile
    constexpr int TCOLS = tmem_cols<BN>();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sx = base, sy = base + STAGES * X_BYTES;
    const uint32_t bars = sy + STAGES * Y_BYTES;
    const uint32_t full0 = bars, empty0 = bars + STAGES * 8, tfull0 = bars + 2 * STAGES * 8, tempty0 = tfull0 + 16;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot = (volatile uint32_t *)(gen_base + STAGES * (X_BYTES + Y_BYTES) + (2 * STAGES + 4) * 8);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                    // 0: issues the products; 1: its peer
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 8); }   // 4 warps of 2 CTAs
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"(TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier();                                       // both CTAs' barriers exist before either is signalled
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    const int per_split = p.tiles_x * p.tiles_y;             // tiles_x counts tiles of 256 tokens here
    const int total_items = per_split * p.splits;

    if (warp == 0 || warp == PAIR_ACT_WARP) {
        // Two requesting threads, one per operand.  Lane 0 of warp 0 asks for this CTA's half of the weight tile and
        // arms the stage's barrier; it never waits for the kernel in front, on which the weights do not depend, so the
        // first STAGES tiles are under way long before that kernel ends.  Lane 0 of the last warp waits for it and
        // then asks for the activation tiles.  Both copies count on the leader's "full" barrier, whose phase ends
        // when the armed bytes have arrived, in whichever order.  (The other lanes of these warps do nothing: a lane
        // in griddepcontrol.wait would hold up its whole warp.)
        const bool weights = warp == 0;
        if (lane == 0) {
            if (!weights) { pdl_sync(); HFB_TRACE_READY_HERE(); }
            uint32_t it = 0;
            bool ok = true;
            for (int item = pair; item < total_items && ok; item += pairs) {
                const int split = item / per_split, t = item % per_split;
                const int tx = t % p.tiles_x, ty = t / p.tiles_x;
                const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, err)) { ok = false; break; }
                    const uint32_t full_leader = map_to_rank(full0 + 8 * s, 0);
                    if (weights) {
                        if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * (X_BYTES + Y_BYTES));
                        tma_load_2d_pair(sy + s * Y_BYTES, &map_y, kb * BK, ty * BN + (int)rank * (BN / 2), full_leader);
                    } else {
                        tma_load_2d_pair(sx + s * X_BYTES, &map_x, kb * BK, tx * 256 + (int)rank * TILE_X, full_leader);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            int last_s = -1;
            uint32_t last_ph = 0;
            for (int item = pair; item < total_items && ok; item += pairs, tile_it++) {
                const int a = tile_it & 1;
                const uint32_t aph = (tile_it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * a, aph ^ 1, abort_flag, err)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + a * BN;
                const int split = item / per_split;
                const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, err)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t dx = smem_desc(sx + s * X_BYTES), dy = smem_desc(sy + s * Y_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        tc_mma_bf16_pair(d, dx + 2 * k, dy + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty0 + 8 * s);
                    last_s = s;
                    last_ph = ph;
                }
                if (ok) tc_commit_pair(tfull0 + 8 * a);
            }
            if (ok && last_s >= 0) mbar_wait(empty0 + 8 * last_s, last_ph, abort_flag, err);
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        uint32_t tile_it = 0;
        bool ok = true;
        pdl_sync();                                          // nothing is written before the kernel in front has finished
        for (int item = pair; item < total_items && ok; item += pairs, tile_it++) {
            const int split = item / per_split, t = item % per_split;
            const int tx = t % p.tiles_x, ty = t / p.tiles_x;
            const int a = tile_it & 1;
            const uint32_t aph = (tile_it >> 1) & 1;
            if (!mbar_wait_long(tfull0 + 8 * a, aph, abort_flag, err)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * BN;
            const int xr = tx * 256 + (int)rank * TILE_X + row;
            if ((BN == 256 || BN == 128) && p.mode == EPI_ROPE_KV) {
                // the tile holds whole heads of the q|k|v rows of 128 tokens per CTA; a thread has one token
                const bool row_ok = xr < p.M;
                const int half = p.d >> 1;
                int pos = row_ok ? p.positions[xr] : 0;
                if (pos < 0 || pos >= p.n_positions) { atomicOr(err, HFB_ERR_POSITION); pos = 0; }
                long long slot = (row_ok && p.slots) ? p.slots[xr] : -1;
                if (slot >= p.cache_slots) { atomicOr(err, HFB_ERR_SLOT); slot = -1; }
                const float *cs = p.cos_sin + (size_t)pos * half * 2;
#pragma unroll 1
                for (int h0 = 0; h0 < BN; h0 += p.d) {
                    const int col = ty * BN + h0, head = col / p.d;
                    if (col >= p.N) break;                   // (the same for every thread)
                    __nv_bfloat16 *dst = nullptr;
                    if (row_ok) {
                        if (head < p.H) dst = p.q_out + ((size_t)xr * p.H + head) * p.d;
                        else if (slot >= 0) dst = (head < p.H + p.G ? p.k_cache + ((size_t)slot * p.G + (head - p.H)) * p.d
                                                                      : p.v_cache + ((size_t)slot * p.G + (head - p.H - p.G)) * p.d);
                    }
#pragma unroll 1
                    for (int j0 = 0; j0 < half; j0 += 32) {
                        uint32_t lo[32], hi[32];
                        tmem_ld16(taddr + h0 + j0, lo); tmem_ld16(taddr + h0 + j0 + 16, lo + 16);
                        tmem_ld16(taddr + h0 + half + j0, hi); tmem_ld16(taddr + h0 + half + j0 + 16, hi + 16);
                        tmem_wait_ld();
                        if (dst) rope_kv_piece(p, lo, hi, col, j0, cs, head < p.H + p.G, dst);
                    }
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                const bool two = c0 + 16 < BN;
                tmem_ld16(taddr + c0, v);
                if (two) tmem_ld16(taddr + c0 + 16, v + 16);
                tmem_wait_ld();
                epilogue_chunk(p, v, xr, ty * BN + c0, split, lane);
                if (two) epilogue_chunk(p, v + 16, xr, ty * BN + c0 + 16, split, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(tempty0 + 8 * a);
                else mbar_arrive_remote(map_to_rank(tempty0 + 8 * a, 0));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
    }
    __syncthreads();
    cluster_barrier();                                       // neither CTA leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TCOLS) : "memory");
    }
}

// Sums split-K partials in split order and applies the epilogue.
__global__ void splitk_reduce_kernel(const float *partial, int splits, size_t MN, int N, const void *bias, int bias_dt,
                                     void *out, int out_dt, int mode)
{
    HFB_TRACE_ENTRY(8);
    pdl_sync();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MN) return;
    float v = 0.f;
    for (int s = 0; s < splits; s++) v += partial[(size_t)s * MN + i];
    if (bias) v += load_any(bias, bias_dt, i % N);
    if (mode == EPI_ADD) ((float *)out)[i] += v;
    else store_any(out, out_dt, i, v);
}

// ---- host side --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

struct MapKey {
    const void *ptr; int rows, cols, box_rows;
    bool operator==(const MapKey &o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const
    {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        return h * 1000003u ^ (size_t)k.box_rows;
    }
};

// A 2-D map over a row-major bf16 matrix [rows, cols] with boxes of [box_rows, 64] and 128-byte swizzle.
int tensor_map(const void *ptr, int rows, int cols, int box_rows, CUtensorMap *out)
{
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return HFB_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(HFB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HFB_ECUDA, "cuTensorMapEncodeTiled failed with %d (rows=%d cols=%d box=%d)", (int)r, rows, cols, box_rows);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return HFB_OK;
}

// Index of the current device (0 where it cannot be told), for what is remembered per device.
// Maps over a paged key/value cache [slots, row_elems] of bfloat16 for copies of whole pages: a box holds `box_keys`
// consecutive slots of the `halves` 128-byte pieces of one head ([piece][key][64 elements] in shared memory, 128-byte
// swizzle).  Where the values lie a multiple of 16 bytes above the keys, ONE map of rank 4 covers both (box
// [keys|values][piece][key][64], *single = true, written to maps[0]); else maps[0] covers the keys and maps[1] the values
// (rank 3).  Coordinates: (0, slot, head * halves [, 0]).
int tensor_map_kv(const void *k, const void *v, int slots, int row_elems, int box_keys, int halves, CUtensorMap *maps, bool *single)
{
    struct Key {
        const void *k, *v; int slots, row_elems, box_keys, halves;
        bool operator==(const Key &o) const { return k == o.k && v == o.v && slots == o.slots && row_elems == o.row_elems && box_keys == o.box_keys && halves == o.halves; }
    };
    struct Val { CUtensorMap m[2]; bool single; };
    struct Hash { size_t operator()(const Key &x) const { return ((size_t)x.k * 1000003u ^ (size_t)x.v) * 1000003u ^ (size_t)x.slots * 31u ^ (size_t)x.box_keys; } };
    static std::unordered_map<Key, Val, Hash> cache;
    static std::mutex mu;
    Key key{k, v, slots, row_elems, box_keys, halves};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { maps[0] = it->second.m[0]; maps[1] = it->second.m[1]; *single = it->second.single; return HFB_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(HFB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const long long gap = (const char *)v - (const char *)k;
    Val val{};
    val.single = gap > 0 && (gap & 15) == 0 && gap < (1ll << 40);
    cuuint64_t dims[4] = {64, (cuuint64_t)slots, (cuuint64_t)(row_elems / 64), 2};
    cuuint64_t strides[3] = {(cuuint64_t)row_elems * 2, 128, (cuuint64_t)(val.single ? gap : 0)};
    cuuint32_t box[4] = {64, (cuuint32_t)box_keys, (cuuint32_t)halves, 2};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const int rank = val.single ? 4 : 3;
    for (int i = 0; i < (val.single ? 1 : 2); i++) {
        CUresult r = fn(&val.m[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(i ? v : k), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(HFB_ECUDA, "cuTensorMapEncodeTiled (key/value pages) failed with %d", (int)r);
    }
    if (cache.size() > 4096) cache.clear();
    cache[key] = val;
    maps[0] = val.m[0]; maps[1] = val.m[1]; *single = val.single;
    return HFB_OK;
}

static int sm_count()
{
    static int n[64] = {0};
    const int dev = current_device();
    if (!n[dev]) {
        cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
        if (n[dev] <= 0) n[dev] = 1;
    }
    return n[dev];
}

static int env_int(const char *name, int dflt)
{
    const char *v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

template <int BN, int STAGES>
static int launch(const CUtensorMap &mx, const CUtensorMap &my, const GemmParams &p, cudaStream_t st)
{
    constexpr uint32_t smem = gemm_smem_bytes<BN, STAGES>();
    // CTAs that can share an SM by shared memory must also all find their TMEM columns (512 per SM)
    static_assert((227 * 1024 / smem) * tmem_cols<BN>() <= 512, "co-resident CTAs would wait for TMEM columns");
    static bool configured[64] = {false};                 // the opt-in is a property of the function on one device
    const int dev = current_device();
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "gemm_tc: cannot opt in to %u bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[dev] = true;
    }
    int items = p.tiles_x * p.tiles_y * p.splits;
    int cap = sm_count();                          // one CTA per SM: the stages take most of its shared memory
    int grid = items < cap ? items : cap;
    g_launch_err = launch_pdl(gemm_tc_kernel<BN, STAGES>, dim3(grid), dim3(GEMM_THREADS), smem, st, mx, my, p, error_word());
    return check_pdl_launch(g_launch_err, "gemm_tc");
}


template <int BN, int STAGES>
static int launch_pair(const CUtensorMap &mx, const CUtensorMap &my, const GemmParams &p, cudaStream_t st)
{
    constexpr uint32_t smem = 1024 + STAGES * (X_BYTES + (BN / 2) * BK * 2) + (2 * STAGES + 4) * 8 + 16;
    static_assert(smem <= 227 * 1024, "the stages do not fit");
    static bool configured[64] = {false};
    const int dev = current_device();
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "gemm_tc: cannot opt in to %u bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[dev] = true;
    }
    const int items = p.tiles_x * p.tiles_y * p.splits, pairs_cap = sm_count() / 2;
    const int pairs = items < pairs_cap ? items : pairs_cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    n_attr++;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    g_launch_err = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN, STAGES>, mx, my, p, error_word());
    return check_pdl_launch(g_launch_err, "gemm_tc_pair");
}

}  // namespace hfb

using namespace hfb;

static int pair_min_tokens() { static const int v = hfb::env_int("HFB_GEMM_PAIR", 256); return v; }     // 0: never
static bool takes_pairs(int M) { return pair_min_tokens() > 0 && M >= pair_min_tokens() && hfb::sm_count() >= 2; }

// More than 128 tokens with so few output tiles that most SMs would stand idle or wait for a few (a product with
// few output features and a long inner dimension, at a few hundred tokens): how many ways to split the inner
// dimension.  The cost of a choice is counted in K blocks: the rounds the busiest SM (or pair) makes over its work
// items of 128 (or 256) tokens x 256 features, times the blocks of a slice, plus the pass over the partial sums.
// 1: no split.
static int mid_splits(int M, int N, int K)
{
    using namespace hfb;
    static const int on = env_int("HFB_GEMM_MID_SPLIT", 1);
    if (!on || M <= 128) return 1;
    const bool pair = takes_pairs(M);
    const int rows = pair ? 2 * TILE_X : TILE_X, units = pair ? sm_count() / 2 : sm_count();
    const long items = (long)((M + rows - 1) / rows) * ((N + 255) / 256);
    const int kb = (K + BK - 1) / BK;
    const int per_item = 6;                             // filling the pipeline and draining the accumulator
    long best = (items + units - 1) / units * (kb + per_item);
    int best_s = 1;
    for (int s = 2; s <= 8 && kb / s >= 32; s++) {     // shorter slices do not pay for the pass over the partial sums (measured)
        const long slice = (kb + s - 1) / s;
        const long cost = (items * s + units - 1) / units * (slice + per_item) + 4 + (long)s * M * N / 100000;
        if (cost < best) { best = cost; best_s = s; }
    }
    return best_s;
}

// Common set-up of the product's tiling: fills p (sizes, tiles, maps) for `bn`.  `splits` > 1 (more than 128 tokens
// only; see mid_splits) asks for that many slices of the inner dimension; the caller then sets the partial-sum mode.
static int plan_and_maps(const void *a, const void *w, int M, int N, int K, hfb::GemmParams &p, int &bn, CUtensorMap &mx, CUtensorMap &my,
                         int splits = 1, int force_bn = 0)
{
    using namespace hfb;
    p.M = M; p.N = N; p.K = K;
    p.kb_total = (K + BK - 1) / BK;
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    p.partial = nullptr;
    p.swapped = M <= 128;
    int rc;
    if (p.swapped) {
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        p.tiles_x = (N + TILE_X - 1) / TILE_X;
        p.tiles_y = 1;
        if ((rc = tensor_map(w, N, K, TILE_X, &mx)) != HFB_OK) return rc;
        if ((rc = tensor_map(a, M, K, bn, &my)) != HFB_OK) return rc;
    } else {
        // the tile width that needs the fewest column-rounds over the SMs (every CTA walks its tiles in turn);
        // from 256 tokens on, tiles of 256 tokens on pairs of SMs
        p.pair = takes_pairs(M);
        const int rows = p.pair ? 2 * TILE_X : TILE_X, units = p.pair ? sm_count() / 2 : sm_count();
        p.tiles_x = (M + rows - 1) / rows;
        bn = 256;
        if (splits > 1) {
            p.kb_per_split = (p.kb_total + splits - 1) / splits;
            p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
        } else if (force_bn) {
            bn = force_bn;
        } else {
            const int widths[6] = {256, 240, 224, 208, 192, 128};
            long best = -1;
            for (int i = 0; i < 6; i++) {
                long tiles = (long)p.tiles_x * ((N + widths[i] - 1) / widths[i]);
                // a k block of a pair's tile takes about 265 ns + 0.6 ns per column (measured at 128..256 columns: a
                // narrow tile is hardly cheaper than a wide one); on one CTA its time goes with the width
                long cost = (tiles + units - 1) / units * (p.pair ? 424 + widths[i] : widths[i]);
                if (best < 0 || cost < best) { best = cost; bn = widths[i]; }
            }
        }
        p.tiles_y = (N + bn - 1) / bn;
        if ((rc = tensor_map(a, M, K, TILE_X, &mx)) != HFB_OK) return rc;
        if ((rc = tensor_map(w, N, K, p.pair ? bn / 2 : bn, &my)) != HFB_OK) return rc;
    }
    return HFB_OK;
}

static int launch_bn(int bn, const CUtensorMap &mx, const CUtensorMap &my, const hfb::GemmParams &p, cudaStream_t st)
{
    using namespace hfb;
    if (p.pair) {
        switch (bn) {
        case 128: return launch_pair<128, 7>(mx, my, p, st);
        case 192: return launch_pair<192, 7>(mx, my, p, st);
        case 208: return launch_pair<208, 7>(mx, my, p, st);
        case 224: return launch_pair<224, 7>(mx, my, p, st);
        case 240: return launch_pair<240, 7>(mx, my, p, st);
        default: return launch_pair<256, 7>(mx, my, p, st);
        }
    }
    switch (bn) {
    case 16: return launch<16, 10>(mx, my, p, st);
    case 32: return launch<32, 9>(mx, my, p, st);
    case 64: return launch<64, 8>(mx, my, p, st);
    case 128: return launch<128, 6>(mx, my, p, st);
    case 192: return launch<192, 5>(mx, my, p, st);
    case 208: return launch<208, 5>(mx, my, p, st);
    case 224: return launch<224, 5>(mx, my, p, st);
    case 240: return launch<240, 4>(mx, my, p, st);
    default: return launch<256, 4>(mx, my, p, st);
    }
}

static int check_tc_args(const char *who, const void *a, const void *w, const void *out, int M, int N, int K,
                         const void *bias = nullptr)
{
    if (K <= 0 || (K & 7)) return fail(HFB_ENOTSUP, "%s: K = %d must be a positive multiple of 8", who, K);
    // (the many-token epilogue reads the bias sixteen bytes at a time)
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || ((uintptr_t)bias & 15))
        return fail(HFB_ENOTSUP, "%s: operands (and the bias) must be 16-byte aligned", who);
    (void)M; (void)N;
    return HFB_OK;
}

// Split-K partial sums of the few-token form (weights on the accumulator rows): bytes, 0 when there is no split.
static size_t swapped_split_bytes(int M, int N, int K)
{
    using namespace hfb;
    int tiles = (N + TILE_X - 1) / TILE_X, kb = (K + BK - 1) / BK;
    int cap = sm_count();
    int splits = tiles >= cap ? 1 : cap / tiles;                    // at most one work item per CTA slot
    if (splits > kb / 4) splits = kb / 4 > 0 ? kb / 4 : 1;
    if (splits > 16) splits = 16;
    return splits > 1 ? (size_t)splits * M * N * sizeof(float) : 0;
}

// Bytes of float32 workspace hfb_linear_tc may use for split-K partials with these sizes (0: none needed).
extern "C" size_t hfb_linear_tc_workspace(int M, int N, int K)
{
    if (M <= 128) return swapped_split_bytes(M, N, K);
    const int splits = mid_splits(M, N, K);
    return splits > 1 ? (size_t)splits * M * N * sizeof(float) : 0;
}

extern "C" int hfb_linear_tc(const void *a, const void *w, const void *bias, int bias_dt, void *out, int out_dt,
                             int accumulate, int M, int N, int K, void *workspace, size_t workspace_bytes, hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    int rc = check_tc_args("linear_tc", a, w, out, M, N, K, bias);
    if (rc != HFB_OK) return rc;
    if (!valid_dt(out_dt) || (bias && !valid_dt(bias_dt))) return fail(HFB_EINVAL, "linear_tc: bad element types");
    if (accumulate && out_dt != HFB_F32) return fail(HFB_EINVAL, "linear_tc: accumulation needs a float32 output");
    cudaStream_t st = (cudaStream_t)s;
    GemmParams p{};
    CUtensorMap mx, my;
    int bn;
    const size_t need = hfb_linear_tc_workspace(M, N, K);
    const bool split_ok = need && workspace && workspace_bytes >= need;
    if ((rc = plan_and_maps(a, w, M, N, K, p, bn, mx, my, (M > 128 && split_ok) ? mid_splits(M, N, K) : 1)) != HFB_OK) return rc;
    p.out = out; p.out_dt = out_dt; p.bias = bias; p.bias_dt = bias_dt;
    p.mode = accumulate ? EPI_ADD : EPI_STORE;
    if (!p.swapped && p.splits > 1) { p.partial = (float *)workspace; p.mode = EPI_PARTIAL; }
    if (p.swapped) {
        if (split_ok) {
            int splits = (int)(need / ((size_t)M * N * sizeof(float)));
            p.kb_per_split = (p.kb_total + splits - 1) / splits;
            p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
            if (p.splits > 1) { p.partial = (float *)workspace; p.mode = EPI_PARTIAL; }
            else p.kb_per_split = p.kb_total;
        }
    }
    if ((rc = launch_bn(bn, mx, my, p, st)) != HFB_OK) return rc;
    if (p.mode == EPI_PARTIAL) {
        size_t MN = (size_t)M * N;
        g_launch_err = launch_pdl(splitk_reduce_kernel, dim3((unsigned)((MN + 255) / 256)), dim3(256), 0, st, p.partial, p.splits, MN, N, bias, bias_dt, out, out_dt,
                                                                          accumulate ? EPI_ADD : EPI_STORE);
        return check_pdl_launch(g_launch_err, "splitk_reduce");
    }
    return HFB_OK;
}

// h[M, N/2] = silu(g) * u where row 2i of w holds gate feature i and row 2i+1 up feature i: the activation runs in
// the product's epilogue, from the float32 accumulators.
extern "C" int hfb_linear_tc_swiglu(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    int rc = check_tc_args("linear_tc_swiglu", a, w, out, M, N, K);
    if (rc != HFB_OK) return rc;
    if ((N & 1) || !valid_dt(out_dt)) return fail(HFB_EINVAL, "linear_tc_swiglu: N must be even (gate and up rows alternate)");
    GemmParams p{};
    CUtensorMap mx, my;
    int bn;
    if ((rc = plan_and_maps(a, w, M, N, K, p, bn, mx, my)) != HFB_OK) return rc;
    p.out = out; p.out_dt = out_dt; p.bias = nullptr; p.mode = EPI_SWIGLU;
    return launch_bn(bn, mx, my, p, (cudaStream_t)s);
}

// q|k|v of many tokens (256 and more: the pair kernel) with the rest of the step in the product's epilogue: bias,
// rounding to bfloat16, rotation of the query and key heads by cos_sin [n_positions, d / 2, 2] at the tokens'
// positions, queries to q_out [M, H d], keys and values to cache slot slots[t] (null: nothing is cached).  bfloat16
// bias and outputs, head sizes 64 and 128, the whole head rotated.  HFB_ENOTSUP, with nothing launched, where the
// sizes are not these: the caller then runs the product and hfb_rope_kv_write.
extern "C" int hfb_linear_tc_rope_kv(const void *a, const void *w, const void *bias, const float *cos_sin, int n_positions,
                                     const int32_t *positions, const int32_t *slots, void *q_out, void *k_cache, void *v_cache,
                                     int64_t cache_slots, int M, int K, int H, int G, int d, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (!takes_pairs(M) || (d != 64 && d != 128) || H <= 0 || G <= 0 || !cos_sin || !positions || n_positions <= 0)
        return fail(HFB_ENOTSUP, "linear_tc_rope_kv: takes 256 tokens and more, head sizes 64 and 128, a rotation table");
    const int N = (H + 2 * G) * d;
    int rc = check_tc_args("linear_tc_rope_kv", a, w, q_out, M, N, K, bias);
    if (rc != HFB_OK) return rc;
    if (((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)cos_sin & 15))
        return fail(HFB_ENOTSUP, "linear_tc_rope_kv: cache and table must be 16-byte aligned");
    GemmParams p{};
    CUtensorMap mx, my;
    int bn;
    // tiles of whole heads: 256 columns, or 128 where that leaves fewer rounds over the pairs
    const int units = sm_count() / 2, tiles_x = (M + 255) / 256;
    const long r256 = ((long)tiles_x * ((N + 255) / 256) + units - 1) / units * (424 + 256);
    const long r128 = ((long)tiles_x * ((N + 127) / 128) + units - 1) / units * (424 + 128);
    if ((rc = plan_and_maps(a, w, M, N, K, p, bn, mx, my, 1, r128 < r256 ? 128 : 256)) != HFB_OK) return rc;
    p.out = q_out; p.out_dt = HFB_BF16; p.bias = bias; p.bias_dt = HFB_BF16; p.mode = EPI_ROPE_KV;
    p.cos_sin = cos_sin; p.positions = positions; p.slots = slots; p.n_positions = n_positions;
    p.q_out = (__nv_bfloat16 *)q_out; p.k_cache = (__nv_bfloat16 *)k_cache; p.v_cache = (__nv_bfloat16 *)v_cache;
    p.cache_slots = cache_slots; p.H = H; p.G = G; p.d = d;
    return launch_bn(bn, mx, my, p, (cudaStream_t)s);
}

// Only the split-K partial sums: partial[s, M, N] float32 for s < *splits, in `workspace`
// (hfb_linear_tc_partials_workspace bytes; above 128 rows that is 0 for a product that is not split, which this
// entry then refuses).  A fused reduction kernel finishes the product.
extern "C" size_t hfb_linear_tc_partials_workspace(int M, int N, int K)
{
    size_t need = hfb_linear_tc_workspace(M, N, K);
    if (M > 128) return need;                        // 0: this product is not split, there are no partial sums to be had
    return need ? need : (size_t)M * N * sizeof(float);
}

extern "C" int hfb_linear_tc_partials(const void *a, const void *w, int M, int N, int K, void *workspace,
                                      size_t workspace_bytes, int *splits, hfb_stream s)
{
    if (M <= 0 || N <= 0) { *splits = 0; return HFB_OK; }
    if (M > 128 && mid_splits(M, N, K) < 2) return fail(HFB_ENOTSUP, "linear_tc_partials: M=%d N=%d K=%d is not split (its workspace size is 0)", M, N, K);
    int rc = check_tc_args("linear_tc_partials", a, w, workspace, M, N, K);
    if (rc != HFB_OK) return rc;
    size_t need = hfb_linear_tc_partials_workspace(M, N, K);
    if (!workspace || workspace_bytes < need) return fail(HFB_EINVAL, "linear_tc_partials: workspace of %zu bytes, %zu needed", workspace_bytes, need);
    GemmParams p{};
    CUtensorMap mx, my;
    int bn;
    if ((rc = plan_and_maps(a, w, M, N, K, p, bn, mx, my, mid_splits(M, N, K))) != HFB_OK) return rc;
    if (p.swapped) {
        int want = (int)(need / ((size_t)M * N * sizeof(float)));
        p.kb_per_split = (p.kb_total + want - 1) / want;
        p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    }
    p.partial = (float *)workspace;
    p.mode = EPI_PARTIAL;
    *splits = p.splits;
    return launch_bn(bn, mx, my, p, (cudaStream_t)s);
}

// ---- the entry point that allocates nothing (see hfb200_noalloc.h) ----------------------------------------
#include "hfb200_noalloc.h"

namespace hfb {

// Split-K partial sums of hfb_linear_tc_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress; the kernels get the device address that call returns.
static __device__ __align__(256) float g_noalloc_scratch[HFB_NOALLOC_SCRATCH_BYTES / sizeof(float)];

// Device address of the array on the current device, looked up at the first call on that device.
static int noalloc_scratch(float **out)
{
    static float *ptr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(HFB_ECUDA, "linear_tc_noalloc: no current device");
    if (!ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return fail(HFB_ECUDA, "linear_tc_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        ptr[dev] = (float *)p;
    }
    *out = ptr[dev];
    return HFB_OK;
}

// The same map as tensor_map() builds, written into the caller's storage without touching the cache.
static int tensor_map_uncached(const void *ptr, int rows, int cols, int box_rows, CUtensorMap *out)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(HFB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HFB_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return HFB_OK;
}

}  // namespace hfb

extern "C" int hfb_linear_tc_noalloc(const void *a, const void *w, const void *bias, int bias_dt, void *out, int out_dt,
                                     int accumulate, int M, int N, int K, hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    if (K <= 0 || (K & 7)) return fail(HFB_ENOTSUP, "linear_tc_noalloc: K = %d must be a positive multiple of 8", K);
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || ((uintptr_t)bias & 15))
        return fail(HFB_ENOTSUP, "linear_tc_noalloc: operands (and the bias) must be 16-byte aligned");
    if (!valid_dt(out_dt) || (bias && !valid_dt(bias_dt))) return fail(HFB_EINVAL, "linear_tc_noalloc: bad element types");
    if (accumulate && out_dt != HFB_F32) return fail(HFB_EINVAL, "linear_tc_noalloc: accumulation needs a float32 output");
    size_t need = M <= 128 ? swapped_split_bytes(M, N, K) : 0;
    if (need > HFB_NOALLOC_SCRATCH_BYTES)
        return fail(HFB_ERANGE, "linear_tc_noalloc: split-K partial sums for M=%d N=%d K=%d take %zu bytes, the built-in "
                                "array holds %u; use hfb_linear_tc with a workspace of your own", M, N, K, need,
                    (unsigned)HFB_NOALLOC_SCRATCH_BYTES);
    float *scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc != HFB_OK) return rc;
    cudaStream_t st = (cudaStream_t)s;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K;
    p.out = out; p.out_dt = out_dt; p.bias = bias; p.bias_dt = bias_dt;
    p.mode = accumulate ? EPI_ADD : EPI_STORE;
    p.kb_total = (K + BK - 1) / BK;
    p.splits = 1;
    p.kb_per_split = p.kb_total;
    p.swapped = M <= 128;
    int bn = 256;
    if (p.swapped) {
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        p.tiles_x = (N + TILE_X - 1) / TILE_X;
        p.tiles_y = 1;
        if (need) {
            int splits = (int)(need / ((size_t)M * N * sizeof(float)));
            p.kb_per_split = (p.kb_total + splits - 1) / splits;
            p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
            if (p.splits > 1) { p.partial = scratch; p.mode = EPI_PARTIAL; }
            else p.kb_per_split = p.kb_total;
        }
    } else {
        p.tiles_x = (M + TILE_X - 1) / TILE_X;
        p.tiles_y = (N + bn - 1) / bn;
    }
    CUtensorMap mx, my;
    if (p.swapped) {
        if ((rc = tensor_map_uncached(w, N, K, TILE_X, &mx)) != HFB_OK) return rc;
        if ((rc = tensor_map_uncached(a, M, K, bn, &my)) != HFB_OK) return rc;
    } else {
        if ((rc = tensor_map_uncached(a, M, K, TILE_X, &mx)) != HFB_OK) return rc;
        if ((rc = tensor_map_uncached(w, N, K, bn, &my)) != HFB_OK) return rc;
    }
    switch (bn) {
    case 16: rc = launch<16, 10>(mx, my, p, st); break;
    case 32: rc = launch<32, 9>(mx, my, p, st); break;
    case 64: rc = launch<64, 8>(mx, my, p, st); break;
    case 128: rc = launch<128, 6>(mx, my, p, st); break;
    default: rc = launch<256, 4>(mx, my, p, st); break;
    }
    if (rc != HFB_OK) return rc;
    if (p.mode == EPI_PARTIAL) {
        size_t MN = (size_t)M * N;
        g_launch_err = launch_pdl(splitk_reduce_kernel, dim3((unsigned)((MN + 255) / 256)), dim3(256), 0, st, p.partial, p.splits, MN, N, bias, bias_dt, out, out_dt,
                                                                          accumulate ? EPI_ADD : EPI_STORE);
        return check_pdl_launch(g_launch_err, "splitk_reduce");
    }
    return HFB_OK;
}
