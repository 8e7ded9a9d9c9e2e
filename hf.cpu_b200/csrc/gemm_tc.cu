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
// warp 6 the activations of that round as soon as it has); warp 1 issues tcgen05.mma from shared memory into one
// of two TMEM accumulators and commits to the stage's "empty" barrier; warps 2..5 read a finished
// accumulator with tcgen05.ld, apply the epilogue and store, while the next tile's products run.
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
constexpr int GEMM_THREADS = 224;            // TMA warp, MMA warp, four epilogue warps, the warp for the first activation tiles
constexpr int PAIR_THREADS = 192;            // (the pair kernel has no such warp)

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_PARTIAL = 2, EPI_SWIGLU = 3 };

enum { FIN_NONE = 0, FIN_RESIDUAL = 1, FIN_ROPE_KV = 2 };

// What the CTA that stores the last split of a weight tile does with the tile's sum (few-token form only): the
// reduction of the split-K partial sums and the memory-bound step that follows it, without another kernel.
//   FIN_RESIDUAL: residual[t, n] += sum (+ bias); y[t, n] = residual * norm_w[n] (the next RMSNorm without its row
//     factor) and, per row and quarter of the tile, the sum of squares of the new residual in sumsq[tile * 4 + q, t]:
//     whoever consumes y multiplies by rsqrt(sum of the parts / N + eps) per row.
//   FIN_ROPE_KV: the tile holds whole heads of the q|k|v row (128 % d == 0): + bias, rotary encoding, q to q_out,
//     k and v into the paged cache, as reduce_rope_kv_kernel does.
struct FinishParams {
    int kind;
    int *counters;                     // one per weight tile; zero before the launch, zero again after it
    float *residual; const void *norm_w; int norm_w_dt; void *y; int y_dt; float *sumsq;
    const float *cos_sin; int n_rot, n_positions; const int32_t *positions, *slots;
    void *q_out, *k_cache, *v_cache; long long cache_slots; int H, G, d;
};

// The activations are the rows of an RMSNorm still to be multiplied by their row factor: sumsq[parts, M] holds
// partial sums of squares per row, summed in order here; the factor rsqrt(sum / width + eps) is applied to the
// accumulators (a product is linear in its rows).  sumsq == null: the activations are complete.
struct RowScale { const float *sumsq; int parts; float eps; int width; };

struct GemmParams {
    int M, N, K;                       // logical sizes: tokens, output features, inner
    int swapped;                       // X = weights, Y = activations
    int pair;                          // tiles of 256 tokens on pairs of CTAs (gemm_tc_pair_kernel)
    int tiles_x, tiles_y, splits, kb_total, kb_per_split;
    void *out; int out_dt;             // [M, N]
    const void *bias; int bias_dt;     // [N] or null
    int mode;
    float *partial;                    // [splits, M, N] when mode == EPI_PARTIAL
    FinishParams fin;                  // few-token form with partial sums only
    RowScale scale;                    // few-token form only
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

constexpr uint32_t FIN_SMEM_BYTES = 128 * 4;                 // row factors of up to 128 tokens

template <int BN> constexpr int tmem_cols()
{
    int need = 2 * BN, c = 32;
    while (c < need) c <<= 1;
    return c;
}

template <int BN, int STAGES> constexpr uint32_t gemm_smem_bytes()
{
    return 1024 + STAGES * (X_BYTES + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16 + FIN_SMEM_BYTES;
}

// One chunk of 16 accumulator columns of one row: v[i] is element (xr, y0 + i) of X . Y^T.
// `live` false: the same instructions, nothing stored (the few-token form runs its epilogue once this way while the
// first weights are on their way, so that its code is in the instruction cache when the first tile is done: fetched
// at that moment it waits behind the weight stream, several microseconds for a 64-token tile).
__device__ __forceinline__ void epilogue_chunk(const GemmParams &p, uint32_t *v, int xr, int y0, int split, int lane,
                                               bool live = true, const float *rstd = nullptr)
{
    if (!live && !p.swapped) return;
    if (rstd && p.mode != EPI_PARTIAL) {
        // the tokens' row factors (all lanes read the same words of shared memory); partial sums are scaled when
        // they are summed
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * rstd[(y0 + i) & 127]);
    }
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

// ---- finishing a weight tile in the CTA that stored its last split ----------------------------------------
// The four epilogue warps (128 threads) meet on a named barrier of their own.
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// The finishing work is a read of splits x tokens x 128 floats from the L2 cache by one CTA: what it costs is
// latency, so every thread keeps many 16-byte loads in flight.  A warp takes every fourth token, a lane four
// consecutive features of the tile; TB tokens are summed at a time, their loads of up to SMAX splits issued together
// (TB * SMAX = 32 loads of 16 bytes per thread).  Loads go past the L1 cache (__ldcg), which may hold lines of an
// earlier launch's partial sums at the same addresses.
constexpr int FIN_MAX_SPLITS = 16;

//
// `dry`: the same instructions with every load and store switched off.  The few-token form runs its finishing step
// once this way before it waits for the kernel in front (as it does with its epilogue), so that the code is in the
// instruction cache when a tile's last split arrives: fetched at that moment it would wait, line after line, behind
// the weight streams of the CTAs that are still running.
template <int TB, int SMAX>
__device__ __forceinline__ void sum_splits4(const GemmParams &p, int t0, int n0, float4 (&acc)[TB], bool dry)
{
    const size_t MN = (size_t)p.M * p.N;
    float4 v[TB][SMAX];
#pragma unroll
    for (int j = 0; j < TB; j++) {
        const int t = t0 + 4 * j;
#pragma unroll
        for (int s = 0; s < SMAX; s++)
            v[j][s] = (t < p.M && s < p.splits && !dry) ? __ldcg((const float4 *)(p.partial + (size_t)s * MN + (size_t)t * p.N + n0))
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < TB; j++) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < SMAX; s++) { a.x += v[j][s].x; a.y += v[j][s].y; a.z += v[j][s].z; a.w += v[j][s].w; }   // split order
        acc[j] = a;
    }
}

__device__ __forceinline__ float4 load4_any(const void *p, int dt, size_t i)
{
    if (dt == HFB_F32) return *(const float4 *)((const float *)p + i);
    const uint2 raw = *(const uint2 *)((const __nv_bfloat16 *)p + i);
    const float2 lo = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.x), hi = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.y);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <typename T> __device__ __forceinline__ void store4(T *dst, float4 v);
template <> __device__ __forceinline__ void store4<float>(float *dst, float4 v) { *(float4 *)dst = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *dst, float4 v)
{
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *(uint2 *)dst = make_uint2(*(const uint32_t *)&lo, *(const uint32_t *)&hi);
}

// q = this warp among the four: it takes tokens q, q + 4, ...; the lane takes features 4 * lane .. 4 * lane + 3.
template <int TB, int SMAX>
__device__ __forceinline__ void finish_residual(const GemmParams &p, int tx, int q, int lane, bool dry)
{
    const FinishParams &fp = p.fin;
    const int n0 = tx * TILE_X + 4 * lane;
    const bool live = n0 < p.N && !dry;                   // (N is a multiple of 4: a lane's four features are in or out)
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 b = (live && p.bias) ? load4_any(p.bias, p.bias_dt, n0) : zero;
    const float4 w = (live && fp.y) ? load4_any(fp.norm_w, fp.norm_w_dt, n0) : zero;
    for (int t0 = q; t0 < p.M; t0 += 4 * TB) {
        float4 acc[TB], res[TB];
#pragma unroll
        for (int j = 0; j < TB; j++) {
            const int t = t0 + 4 * j;
            res[j] = (live && t < p.M) ? __ldcg((const float4 *)(fp.residual + (size_t)t * p.N + n0)) : zero;
        }
        sum_splits4<TB, SMAX>(p, t0, n0, acc, !live);
#pragma unroll
        for (int j = 0; j < TB; j++) {
            const int t = t0 + 4 * j;
            if (t >= p.M) break;
            float4 v = zero;
            if (live) {
                v = make_float4((acc[j].x + b.x) + res[j].x, (acc[j].y + b.y) + res[j].y, (acc[j].z + b.z) + res[j].z,
                                (acc[j].w + b.w) + res[j].w);
                *(float4 *)(fp.residual + (size_t)t * p.N + n0) = v;
                if (fp.y) {
                    const float4 yv = make_float4(v.x * w.x, v.y * w.y, v.z * w.z, v.w * w.w);
                    if (fp.y_dt == HFB_BF16) store4((__nv_bfloat16 *)fp.y + (size_t)t * p.N + n0, yv);
                    else store4((float *)fp.y + (size_t)t * p.N + n0, yv);
                }
            }
            if (fp.sumsq) {
                const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
                if (lane == 0 && !dry) fp.sumsq[(size_t)tx * p.M + t] = ss;
            }
        }
    }
}

// The tile holds whole heads (128 % d == 0) and a lane's four features lie in one half of a rotation pair (n_rot is a
// multiple of 8): the partner values are four lanes' worth away, fetched with a shuffle.
template <typename T, int TB, int SMAX>
__device__ __forceinline__ void finish_rope_kv(const GemmParams &p, int tx, int q, int lane, const float *rstd, int *err, bool dry)
{
    const FinishParams &fp = p.fin;
    const int n0 = tx * TILE_X + 4 * lane, d = fp.d, half = fp.n_rot >> 1;
    const bool live = n0 < p.N && !dry;
    const int head = n0 / d, i0 = n0 - head * d;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 b = (live && p.bias) ? load4_any(p.bias, p.bias_dt, n0) : zero;
    const bool rotate = live && head < fp.H + fp.G && i0 < fp.n_rot;
    const bool low = i0 < half;                           // this lane holds the first elements of its pairs
    const int partner = low ? lane + (half >> 2) : lane - (half >> 2);
    for (int t0 = q; t0 < p.M; t0 += 4 * TB) {
        float4 acc[TB];
        sum_splits4<TB, SMAX>(p, t0, n0, acc, !live);
#pragma unroll
        for (int j = 0; j < TB; j++) {
            const int t = t0 + 4 * j;
            if (t >= p.M) break;                          // (the same for the whole warp)
            float4 v = acc[j];
            if (rstd) { const float r = rstd[t & 127]; v.x *= r; v.y *= r; v.z *= r; v.w *= r; }
            // the separate kernels round q|k|v to the run type before rotating; keep the same values
            v = make_float4(to_f32(from_f32<T>(v.x + b.x)), to_f32(from_f32<T>(v.y + b.y)), to_f32(from_f32<T>(v.z + b.z)),
                            to_f32(from_f32<T>(v.w + b.w)));
            float4 o;
            o.x = __shfl_sync(0xffffffffu, v.x, partner & 31); o.y = __shfl_sync(0xffffffffu, v.y, partner & 31);
            o.z = __shfl_sync(0xffffffffu, v.z, partner & 31); o.w = __shfl_sync(0xffffffffu, v.w, partner & 31);
            float4 out = v;
            if (rotate || dry) {
                int pos = live ? fp.positions[t] : 0;
                if (pos < 0 || pos >= fp.n_positions) { atomicOr(err, HFB_ERR_POSITION); pos = 0; }
                const int k = low ? i0 : i0 - half;
                const float4 *cs = (const float4 *)(fp.cos_sin + ((size_t)pos * half + k) * 2);   // (cos, sin) of 4 pairs
                const float4 c01 = live ? cs[0] : zero, c23 = live ? cs[1] : zero;
                if (low) out = make_float4(v.x * c01.x - o.x * c01.y, v.y * c01.z - o.y * c01.w, v.z * c23.x - o.z * c23.y, v.w * c23.z - o.w * c23.w);
                else out = make_float4(o.x * c01.y + v.x * c01.x, o.y * c01.w + v.y * c01.z, o.z * c23.y + v.z * c23.x, o.w * c23.w + v.w * c23.z);
            }
            if (head < fp.H) {
                if (live) store4((T *)fp.q_out + ((size_t)t * fp.H + head) * d + i0, out);
            } else {
                long long slot = (fp.slots && live) ? fp.slots[t] : -1;
                if (slot >= fp.cache_slots) { atomicOr(err, HFB_ERR_SLOT); slot = -1; }
                if (slot >= 0) {
                    if (head < fp.H + fp.G) store4((T *)fp.k_cache + ((size_t)slot * fp.G + (head - fp.H)) * d + i0, out);
                    else store4((T *)fp.v_cache + ((size_t)slot * fp.G + (head - fp.H - fp.G)) * d + i0, out);
                }
            }
        }
    }
}

// Picks the number of tokens a warp sums at a time by the number of splits, so that about 32 loads are in flight.
template <typename T>
__device__ __forceinline__ void finish_tile(const GemmParams &p, int tx, int q, int lane, const float *rstd, int *err, bool dry)
{
    if (p.fin.kind == FIN_RESIDUAL) {
        if (p.splits <= 4) finish_residual<8, 4>(p, tx, q, lane, dry);
        else if (p.splits <= 8) finish_residual<4, 8>(p, tx, q, lane, dry);
        else finish_residual<2, 16>(p, tx, q, lane, dry);
    } else {
        if (p.splits <= 4) finish_rope_kv<T, 8, 4>(p, tx, q, lane, rstd, err, dry);
        else if (p.splits <= 8) finish_rope_kv<T, 4, 8>(p, tx, q, lane, rstd, err, dry);
        else finish_rope_kv<T, 2, 16>(p, tx, q, lane, rstd, err, dry);
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
    volatile int *last_flag = (volatile int *)(tmem_slot + 2);       // this CTA stored a tile's last split
    float *rstd_smem = (float *)(tmem_slot + 4);                     // [128] row factors

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
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

    if (warp == 0) {
        // ---- producer: TMA loads --------------------------------------------------------------
        // The weights do not depend on the kernel before this one, the activations do.  One lane requests the weight
        // tiles of the first STAGES k blocks at once, long before that kernel has finished; the activation tiles of
        // those blocks are requested by the seventh warp the moment it has (both count on the stage's "full" barrier,
        // whose phase ends when the armed byte count has arrived, in whichever order).  From the second round on the
        // producer has waited too and requests both.  The other lanes of this warp do nothing: a lane that sat in
        // griddepcontrol.wait would hold up its whole warp, the requesting lane with it.
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true, dep_ready = false;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                int split = item / per_split, t = item % per_split;
                int tx = t % p.tiles_x, ty = t / p.tiles_x;
                int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    int s = it % STAGES;
                    uint32_t ph = (it / STAGES) & 1;
                    if (!dep_ready && it >= STAGES) { pdl_sync(); dep_ready = true; }
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, err)) { ok = false; break; }
                    mbar_arrive_expect_tx(full0 + 8 * s, X_BYTES + Y_BYTES);
                    if (p.swapped) tma_load_2d(sx + s * X_BYTES, &map_x, kb * BK, tx * TILE_X, full0 + 8 * s);
                    else tma_load_2d(sy + s * Y_BYTES, &map_y, kb * BK, ty * BN, full0 + 8 * s);
                    if (dep_ready) {
                        if (p.swapped) tma_load_2d(sy + s * Y_BYTES, &map_y, kb * BK, ty * BN, full0 + 8 * s);
                        else tma_load_2d(sx + s * X_BYTES, &map_x, kb * BK, tx * TILE_X, full0 + 8 * s);
                    }
                }
            }
            if (!dep_ready) pdl_sync();
        }
    } else if (warp == 6) {
        // ---- the activation tiles of the first STAGES k blocks, as soon as the kernel in front has finished ----
        pdl_sync();
        if (lane == 0) {
            uint32_t it = 0;
            for (int item = blockIdx.x; item < total_items && it < (uint32_t)STAGES; item += gridDim.x) {
                int split = item / per_split, t = item % per_split;
                int tx = t % p.tiles_x, ty = t / p.tiles_x;
                int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.kb_total);
                for (int kb = kb0; kb < kb1 && it < (uint32_t)STAGES; kb++, it++) {
                    if (p.swapped) tma_load_2d(sy + it * Y_BYTES, &map_y, kb * BK, ty * BN, full0 + 8 * it);
                    else tma_load_2d(sx + it * X_BYTES, &map_x, kb * BK, tx * TILE_X, full0 + 8 * it);
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
        const int q = warp & 3;                       // the TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        uint32_t tile_it = 0;
        bool ok = true;
        const float *rstd = (p.swapped && p.scale.sumsq) ? rstd_smem : nullptr;
        // With few tokens the first turn of this loop is a rehearsal: it reads whatever the accumulator holds and
        // stores nothing, before the kernel in front is known to have finished (see epilogue_chunk).
        bool rehearsal = p.swapped != 0;
        auto after_wait = [&]() {
            // what comes from the kernel in front: the rows' sums of squares.  Thread t sums the parts of token t in
            // order and keeps the row factor where the four warps find it.
            if (rstd) {
                if (row < p.M) {
                    float ss = 0.f;
                    for (int i = 0; i < p.scale.parts; i++) ss += __ldcg(p.scale.sumsq + (size_t)i * p.M + row);
                    rstd_smem[row] = 1.0f / sqrtf(ss / (float)p.scale.width + p.scale.eps);
                }
                epi_bar();
            }
        };
        if (!rehearsal) { pdl_sync(); after_wait(); } // nothing is written before the kernel in front has finished
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
            for (int c0 = 0; c0 < BN; c0 += (BN >= 32 ? 32 : 16)) {
                uint32_t v[BN >= 32 ? 32 : 16];
                const bool two = BN >= 32 && c0 + 16 < BN;       // widths such as 208 end on a single chunk
                tmem_ld16(taddr + c0, v);
                if (two) tmem_ld16(taddr + c0 + 16, v + (BN >= 32 ? 16 : 0));
                tmem_wait_ld();
                epilogue_chunk(p, v, xr, ty * BN + c0, split, lane, !rehearsal, rstd);
                if (two) epilogue_chunk(p, v + (BN >= 32 ? 16 : 0), xr, ty * BN + c0 + 16, split, lane, !rehearsal, rstd);
            }
            if (rehearsal) {
                if (BN <= 128 && p.fin.kind != FIN_NONE) {
                    if (p.out_dt == HFB_BF16) finish_tile<__nv_bfloat16>(p, tx, warp - 2, lane, rstd, err, true);
                    else finish_tile<float>(p, tx, warp - 2, lane, rstd, err, true);
                }
                rehearsal = false;
                pdl_sync();
                after_wait();
                continue;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * a);
            if (BN <= 128 && p.swapped && p.fin.kind != FIN_NONE) {      // (the few-token form has at most 128 columns)
                // The split is in global memory.  Count it; the CTA that brings a tile's count to the number of
                // splits sums the tile in split order, whichever CTA that is, and does the step that follows.
                epi_bar();
                if (row == 0) {
                    __threadfence();                             // (after the barrier: it covers the four warps' stores)
                    const int before = atomicAdd(&p.fin.counters[tx], 1);
                    const int last = before == p.splits - 1;
                    if (last) p.fin.counters[tx] = 0;            // every split has counted: ready for the next launch
                    *last_flag = last;
                }
                epi_bar();
                if (*last_flag) {
                    __threadfence();
                    const int fq = warp - 2;                     // the finishing step's own numbering of the four warps
                    if (p.out_dt == HFB_BF16) finish_tile<__nv_bfloat16>(p, tx, fq, lane, rstd, err, false);
                    else finish_tile<float>(p, tx, fq, lane, rstd, err, false);
                }
                epi_bar();                                       // the flag may be rewritten for the next item
            }
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
    pdl_sync();

    const int pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    const int per_split = p.tiles_x * p.tiles_y;             // tiles_x counts tiles of 256 tokens here
    const int total_items = per_split * p.splits;

    if (warp == 0) {
        if (lane == 0) {
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
                    if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * (X_BYTES + Y_BYTES));
                    const uint32_t full_leader = map_to_rank(full0 + 8 * s, 0);
                    tma_load_2d_pair(sx + s * X_BYTES, &map_x, kb * BK, tx * 256 + (int)rank * TILE_X, full_leader);
                    tma_load_2d_pair(sy + s * Y_BYTES, &map_y, kb * BK, ty * BN + (int)rank * (BN / 2), full_leader);
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
        for (int item = pair; item < total_items && ok; item += pairs, tile_it++) {
            const int split = item / per_split, t = item % per_split;
            const int tx = t % p.tiles_x, ty = t / p.tiles_x;
            const int a = tile_it & 1;
            const uint32_t aph = (tile_it >> 1) & 1;
            if (!mbar_wait(tfull0 + 8 * a, aph, abort_flag, err)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * BN;
            const int xr = tx * 256 + (int)rank * TILE_X + row;
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
static int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    return dev;
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
                         int splits = 1)
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
        } else {
            const int widths[6] = {256, 240, 224, 208, 192, 128};
            long best = -1;
            for (int i = 0; i < 6; i++) {
                long tiles = (long)p.tiles_x * ((N + widths[i] - 1) / widths[i]);
                long cost = (tiles + units - 1) / units * widths[i];
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
static int linear_tc_swiglu(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, const hfb::RowScale &scale,
                            hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    int rc = check_tc_args("linear_tc_swiglu", a, w, out, M, N, K);
    if (rc != HFB_OK) return rc;
    if ((N & 1) || !valid_dt(out_dt)) return fail(HFB_EINVAL, "linear_tc_swiglu: N must be even (gate and up rows alternate)");
    if (scale.sumsq && M > 128) return fail(HFB_ENOTSUP, "linear_tc_swiglu: row factors are applied with at most 128 rows (got %d)", M);
    GemmParams p{};
    CUtensorMap mx, my;
    int bn;
    if ((rc = plan_and_maps(a, w, M, N, K, p, bn, mx, my)) != HFB_OK) return rc;
    p.out = out; p.out_dt = out_dt; p.bias = nullptr; p.mode = EPI_SWIGLU;
    p.scale = scale;
    return launch_bn(bn, mx, my, p, (cudaStream_t)s);
}

extern "C" int hfb_linear_tc_swiglu(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, hfb_stream s)
{
    return linear_tc_swiglu(a, w, out, out_dt, M, N, K, hfb::RowScale{}, s);
}

// The same where the rows of `a` still lack their RMSNorm row factor (see hfb_linear_tc_residual_y): M <= 128.
extern "C" int hfb_linear_tc_swiglu_scaled(const void *a, const void *w, void *out, int out_dt, int M, int N, int K,
                                           const float *sumsq, int parts, float eps, hfb_stream s)
{
    if (!sumsq || parts < 1) return fail(HFB_EINVAL, "linear_tc_swiglu_scaled: no sums of squares");
    return linear_tc_swiglu(a, w, out, out_dt, M, N, K, hfb::RowScale{sumsq, parts, eps, K}, s);
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

// ---- few tokens: the product, its split-K reduction and the step after it in one kernel ---------------------
// Sets up the few-token product with partial sums in `workspace` (hfb_linear_tc_partials_workspace bytes) and checks
// the tile counters.
static int plan_fused(const char *who, const void *a, const void *w, int M, int N, int K, void *workspace, size_t workspace_bytes,
                      int *counters, int counters_len, hfb::GemmParams &p, int &bn, CUtensorMap &mx, CUtensorMap &my)
{
    using namespace hfb;
    if (M > 128) return fail(HFB_ENOTSUP, "%s: at most 128 rows (got %d)", who, M);
    int rc = check_tc_args(who, a, w, workspace, M, N, K);
    if (rc != HFB_OK) return rc;
    const size_t need = hfb_linear_tc_partials_workspace(M, N, K);
    if (!workspace || workspace_bytes < need) return fail(HFB_EINVAL, "%s: workspace of %zu bytes, %zu needed", who, workspace_bytes, need);
    if ((rc = plan_and_maps(a, w, M, N, K, p, bn, mx, my)) != HFB_OK) return rc;
    if (!counters || counters_len < p.tiles_x) return fail(HFB_EINVAL, "%s: %d tile counters needed, %d given", who, p.tiles_x, counters_len);
    if (N & 3) return fail(HFB_ENOTSUP, "%s: N = %d must be a multiple of 4", who, N);
    const int want = (int)(need / ((size_t)M * N * sizeof(float)));
    p.kb_per_split = (p.kb_total + want - 1) / want;
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    if (p.splits > FIN_MAX_SPLITS) return fail(HFB_ENOTSUP, "%s: %d splits exceed %d", who, p.splits, FIN_MAX_SPLITS);
    p.partial = (float *)workspace;
    p.mode = EPI_PARTIAL;
    p.fin.counters = counters;
    return HFB_OK;
}

// Row-factor parts hfb_linear_tc_residual_y writes per row for N output features.
extern "C" int hfb_linear_tc_sumsq_parts(int N) { return (N + hfb::TILE_X - 1) / hfb::TILE_X; }

// residual[M, N] += a . w^T (+ bias), M <= 128, in one kernel: the CTA that stores the last split of a weight tile
// sums the splits in split order and adds them into the float32 residual.  With `y`: y = residual * norm_w (the
// next RMSNorm without its row factor) and sumsq[hfb_linear_tc_sumsq_parts(N), M] = partial sums of squares of the
// new residual rows; the row factor is rsqrt(sum over the parts / N + eps), which hfb_linear_tc_swiglu_scaled and
// hfb_linear_tc_rope_kv apply.  `counters`: at least ceil(N / 128) ints, zero before the first launch (every launch
// leaves them zero).
extern "C" int hfb_linear_tc_residual_y(const void *a, const void *w, const void *bias, int bias_dt, float *residual,
                                        const void *norm_w, int norm_w_dt, void *y, int y_dt, float *sumsq, int M, int N, int K,
                                        void *workspace, size_t workspace_bytes, int *counters, int counters_len, hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    if ((bias && !valid_dt(bias_dt)) || (y && (!valid_dt(y_dt) || !valid_dt(norm_w_dt) || !norm_w || !sumsq)))
        return fail(HFB_EINVAL, "linear_tc_residual_y: bad arguments");
    GemmParams p{};
    CUtensorMap mx, my;
    int bn, rc;
    if ((rc = plan_fused("linear_tc_residual_y", a, w, M, N, K, workspace, workspace_bytes, counters, counters_len, p, bn, mx, my)) != HFB_OK) return rc;
    p.bias = bias; p.bias_dt = bias_dt; p.out_dt = HFB_F32;
    p.fin.kind = FIN_RESIDUAL;
    p.fin.residual = residual; p.fin.norm_w = norm_w; p.fin.norm_w_dt = norm_w_dt; p.fin.y = y; p.fin.y_dt = y_dt;
    p.fin.sumsq = y ? sumsq : nullptr;
    return launch_bn(bn, mx, my, p, (cudaStream_t)s);
}

// q|k|v = a . w^T (scaled by the rows' factors when `in_sumsq` is given) + bias, rotary encoding of q and k, q to q_out
// [M, H*d], k and v into the paged cache at `slots` (null: q only), M <= 128, in one kernel; head sizes that divide
// 128.  Element type `dt` of q_out and the cache.  Same arithmetic as hfb_reduce_rope_kv.
extern "C" int hfb_linear_tc_rope_kv(const void *a, const void *w, const void *bias, int bias_dt, const float *in_sumsq, int in_parts,
                                     float in_eps, const float *cos_sin, int n_rot, int n_positions, const int32_t *positions,
                                     const int32_t *slots, void *q_out, void *k_cache, void *v_cache, int64_t cache_slots, int dt,
                                     int M, int H, int G, int d, int K, void *workspace, size_t workspace_bytes, int *counters,
                                     int counters_len, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (!valid_dt(dt) || H <= 0 || G <= 0 || d <= 0 || n_rot < 0 || n_rot > d || (n_rot & 1) || (bias && !valid_dt(bias_dt)))
        return fail(HFB_EINVAL, "linear_tc_rope_kv: bad arguments");
    if (TILE_X % d || (d & 3)) return fail(HFB_ENOTSUP, "linear_tc_rope_kv: head size %d does not divide %d", d, TILE_X);
    if (n_rot & 7) return fail(HFB_ENOTSUP, "linear_tc_rope_kv: a rotary width of %d is not a multiple of 8", n_rot);
    if (((uintptr_t)q_out & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)cos_sin & 15))
        return fail(HFB_ENOTSUP, "linear_tc_rope_kv: outputs and the rotary table must be 16-byte aligned");
    if (n_rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "linear_tc_rope_kv: rotation needs a table and positions");
    const int N = (H + 2 * G) * d;
    GemmParams p{};
    CUtensorMap mx, my;
    int bn, rc;
    if ((rc = plan_fused("linear_tc_rope_kv", a, w, M, N, K, workspace, workspace_bytes, counters, counters_len, p, bn, mx, my)) != HFB_OK) return rc;
    p.bias = bias; p.bias_dt = bias_dt; p.out_dt = dt;
    if (in_sumsq) p.scale = RowScale{in_sumsq, in_parts, in_eps, K};
    p.fin.kind = FIN_ROPE_KV;
    p.fin.cos_sin = cos_sin; p.fin.n_rot = n_rot; p.fin.n_positions = n_positions; p.fin.positions = positions; p.fin.slots = slots;
    p.fin.q_out = q_out; p.fin.k_cache = k_cache; p.fin.v_cache = v_cache; p.fin.cache_slots = cache_slots;
    p.fin.H = H; p.fin.G = G; p.fin.d = d;
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
