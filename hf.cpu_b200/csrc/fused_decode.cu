// Kernels that finish a split-K product and do the next memory-bound step in the same pass (decode path).
//
// With few tokens the tensor-core product leaves float32 partial sums [splits, M, N].  Summing them (in split
// order), adding bias and residual, and normalising the row for the next product are one pass over a row here
// instead of three kernels; likewise the sum, bias, rotary encoding and cache write of the q|k|v product.
// Arithmetic as in the separate kernels: src/model.c:606-611 (residual, then RMSNorm, src/mathx.c:65-75) and
// src/model.c:581-601 (bias after the dot, rotation, cache write).
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

// residual[m, :] += sum_s partial[s, m, :] (+ bias);  xn[m, :] = residual[m, :] * rsqrt(mean(residual^2) + eps) * w
__global__ void reduce_residual_norm_kernel(const float *partial, int splits, int M, int N, const void *bias, int bias_dt,
                                            float *residual, const void *w, int w_dt, float eps, void *xn, int xn_dt)
{
    HFB_TRACE_ENTRY(11);
    pdl_entry();
    pdl_sync_small();
    const int m = blockIdx.x;
    const size_t MN = (size_t)M * N;
    float *res = residual + (size_t)m * N;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < splits; s++) v += partial[(size_t)s * MN + (size_t)m * N + i];
        if (bias) v += load_any(bias, bias_dt, i);
        v += res[i];
        res[i] = v;
        ss += v * v;
    }
    __shared__ float part[32];
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? part[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) part[0] = t;
    }
    __syncthreads();
    if (!xn) return;
    const float r = 1.0f / sqrtf(part[0] / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x)       // each thread re-reads what it wrote itself
        store_any(xn, xn_dt, (size_t)m * N + i, (res[i] * r) * load_any(w, w_dt, i));
}

// The same with 16-byte accesses and the row's sums kept in registers between the two passes: one CTA of up to
// 1024 threads per row, each thread owning up to RRN_VEC float4 columns.
constexpr int RRN_VEC = 4;

template <typename TW, typename TO>
__global__ void __launch_bounds__(1024)
reduce_residual_norm_vec_kernel(const float *partial, int splits, int M, int N, const void *bias, int bias_dt,
                                float *residual, const TW *w, float eps, TO *xn)
{
    HFB_TRACE_ENTRY(5);
    pdl_entry();
    const int m = blockIdx.x, N4 = N >> 2;
    // the norm's weights and the bias do not come from the kernel in front: fetch them while it finishes
    float4 wv[RRN_VEC], bv[RRN_VEC];
#pragma unroll
    for (int j = 0; j < RRN_VEC; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        wv[j] = bv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < N4) {
            if (xn) wv[j] = make_float4(to_f32(w[4 * i]), to_f32(w[4 * i + 1]), to_f32(w[4 * i + 2]), to_f32(w[4 * i + 3]));
            if (bias) bv[j] = make_float4(load_any(bias, bias_dt, 4 * i), load_any(bias, bias_dt, 4 * i + 1),
                                          load_any(bias, bias_dt, 4 * i + 2), load_any(bias, bias_dt, 4 * i + 3));
        }
    }
    pdl_sync_small();
    const size_t MN4 = ((size_t)M * N) >> 2;
    const float4 *part = (const float4 *)partial + (size_t)m * N4;
    float4 *res = (float4 *)(residual + (size_t)m * N);
    float4 vals[RRN_VEC];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < RRN_VEC; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        float4 v = bv[j];
        if (i < N4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s0 = 0; s0 < splits; s0 += 8) {          // eight reads in flight: their latency is what this costs
                float4 q[8];
#pragma unroll
                for (int k = 0; k < 8; k++) q[k] = s0 + k < splits ? part[(size_t)(s0 + k) * MN4 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int k = 0; k < 8; k++) { acc.x += q[k].x; acc.y += q[k].y; acc.z += q[k].z; acc.w += q[k].w; }
            }
            v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;       // (sum of the splits) + bias, as before
            float4 r = res[i];
            v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            res[i] = v;
        }
        vals[j] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (!xn) return;
    __shared__ float part_ss[32];
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) part_ss[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? part_ss[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) part_ss[0] = t;
    }
    __syncthreads();
    const float r = 1.0f / sqrtf(part_ss[0] / (float)N + eps);
#pragma unroll
    for (int j = 0; j < RRN_VEC; j++) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i >= N4) continue;
        const float4 v = vals[j];
        float y0 = (v.x * r) * wv[j].x, y1 = (v.y * r) * wv[j].y;
        float y2 = (v.z * r) * wv[j].z, y3 = (v.w * r) * wv[j].w;
        TO *o = xn + (size_t)m * N + 4 * i;
        if (sizeof(TO) == 4) *(float4 *)o = make_float4(y0, y1, y2, y3);
        else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            *(uint2 *)o = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
        }
    }
    HFB_TRACE_MARK(4);
}

// q|k|v row = sum_s partial[s, t, :] + bias; rotate q and k; q -> q_out, k and v -> the paged cache.
template <typename T>
__global__ void reduce_rope_kv_kernel(const float *partial, int splits, int Tn, const void *bias, int bias_dt,
                                      const float *cos_sin, int n_rot, int n_positions, const int32_t *positions,
                                      const int32_t *slots, T *q_out, T *k_cache, T *v_cache, long long cache_slots,
                                      int H, int G, int d, int *err)
{
    HFB_TRACE_ENTRY(2);
    pdl_entry();
    // The slot, the position, the rotation's cosines and sines and the bias are inputs of the step or constants:
    // they are fetched before the wait for the product in front, whose partial sums are read after it.
    const int t = blockIdx.x, head = blockIdx.y;
    const int N = (H + 2 * G) * d;
    const size_t TN = (size_t)Tn * N, row = (size_t)t * N + (size_t)head * d;
    T *dst = nullptr;
    bool rotate, live = true;
    if (head < H) {
        dst = q_out + (size_t)t * H * d + (size_t)head * d;
        rotate = true;
    } else {
        long long slot = slots ? slots[t] : -1;
        if (slot >= cache_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); slot = -1; }
        live = slot >= 0;
        if (!live) slot = 0;
        if (head < H + G) { dst = k_cache + ((size_t)slot * G + (head - H)) * d; rotate = true; }
        else { dst = v_cache + ((size_t)slot * G + (head - H - G)) * d; rotate = false; }
    }
    const int half = n_rot / 2;
    const float *cs = cos_sin;
    float c0 = 1.f, s0 = 0.f;                             // of this thread's first pair
    if (live && rotate && half > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= n_positions) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
        cs = cos_sin + (size_t)pos * half * 2;
        if ((int)threadIdx.x < half) { c0 = cs[2 * threadIdx.x]; s0 = cs[2 * threadIdx.x + 1]; }
    }
    const float b0 = (bias && (int)threadIdx.x < d) ? load_any(bias, bias_dt, (size_t)head * d + threadIdx.x) : 0.f;
    const float b1 = (bias && (int)threadIdx.x + half < d) ? load_any(bias, bias_dt, (size_t)head * d + threadIdx.x + half) : 0.f;
    pdl_sync_small();
    if (!live) return;
    auto value = [&](int i) {
        float v = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float q[8];
#pragma unroll
            for (int k = 0; k < 8; k++) q[k] = s0 + k < splits ? partial[(size_t)(s0 + k) * TN + row + i] : 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) v += q[k];
        }
        if (bias) v += (i == (int)threadIdx.x) ? b0 : (i == (int)threadIdx.x + half) ? b1 : load_any(bias, bias_dt, (size_t)head * d + i);
        return v;
    };
    if (rotate && half > 0) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const bool first = i == (int)threadIdx.x;
            float c = first ? c0 : cs[2 * i], s = first ? s0 : cs[2 * i + 1];
            float a = value(i), b = value(i + half);
            // the separate kernels round q|k|v to the run type before rotating; keep the same values
            a = to_f32(from_f32<T>(a)); b = to_f32(from_f32<T>(b));
            float lo, hi;
            rope_pair(a, b, c, s, lo, hi);
            dst[i] = from_f32<T>(lo);
            dst[i + half] = from_f32<T>(hi);
        }
        for (int i = n_rot + threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<T>(value(i));
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_f32<T>(value(i));
    }
}

// arg-max in two passes so that many blocks share a row: (value, index) per chunk, then the best chunk.
// (value, index) pairs: the larger value wins, the smaller index among equals; an index below 0 is "none yet"
__device__ __forceinline__ void argmax_take(float &best, int &bi, float v, int i)
{
    if (i >= 0 && (bi < 0 || v > best || (v == best && i < bi))) { best = v; bi = i; }
}

// A chunk of 4,096 logits per block of 256 threads: where the rows allow 16-byte reads a thread's four reads are under
// way together (what this kernel costs is latency, not bytes); warps reduce by shuffles, the eight warps through
// shared memory once.
__global__ void __launch_bounds__(256) argmax_chunks_kernel(const float *logits, int V, int chunk, float *best_v, int32_t *best_i)
{
    HFB_TRACE_ENTRY(9);
    pdl_entry();
    pdl_sync_small();
    const int row = blockIdx.y, c = blockIdx.x;
    const float *p = logits + (size_t)row * V;
    const int lo = c * chunk, hi = min(V, lo + chunk);
    float best = 0.f;
    int bi = -1;
    if ((V & 3) == 0 && (chunk & 3) == 0 && (((uintptr_t)logits) & 15) == 0 && chunk == 4096) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = lo + 4 * ((int)threadIdx.x + 256 * j);
            v[j] = i < hi ? *(const float4 *)(p + i) : make_float4(0.f, 0.f, 0.f, 0.f);      // (hi is a multiple of 4 too)
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = lo + 4 * ((int)threadIdx.x + 256 * j);
            if (i < hi) {
                argmax_take(best, bi, v[j].x, i); argmax_take(best, bi, v[j].y, i + 1);
                argmax_take(best, bi, v[j].z, i + 2); argmax_take(best, bi, v[j].w, i + 3);
            }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_take(best, bi, p[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(best, bi, v2, i2);
    }
    __shared__ float sv[8];
    __shared__ int si[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) argmax_take(best, bi, sv[w], si[w]);
        best_v[(size_t)row * gridDim.x + c] = best; best_i[(size_t)row * gridDim.x + c] = bi;
    }
}

__global__ void argmax_final_kernel(const float *best_v, const int32_t *best_i, int chunks, int32_t *out)
{
    HFB_TRACE_ENTRY(10);
    pdl_entry();
    pdl_sync_small();
    const int row = blockIdx.x;
    float best = 0.f;
    int bi = -1;
    for (int c = threadIdx.x; c < chunks; c += 32) {
        float v = best_v[(size_t)row * chunks + c];
        int i = best_i[(size_t)row * chunks + c];
        if (i >= 0 && (bi < 0 || v > best || (v == best && i < bi))) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float v2 = __shfl_xor_sync(0xffffffffu, best, o);
        int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
        if (i2 >= 0 && (bi < 0 || v2 > best || (v2 == best && i2 < bi))) { best = v2; bi = i2; }
    }
    if (threadIdx.x == 0) out[row] = bi < 0 ? 0 : bi;
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_reduce_residual_norm(const float *partial, int splits, int M, int N, const void *bias, int bias_dt,
                                        float *residual, const void *w, int w_dt, float eps, void *xn, int xn_dt,
                                        hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (splits < 1 || N <= 0 || (bias && !valid_dt(bias_dt)) || (xn && (!valid_dt(w_dt) || !valid_dt(xn_dt))))
        return fail(HFB_EINVAL, "reduce_residual_norm: bad arguments");
    if ((N & 3) == 0 && N <= 4 * RRN_VEC * 1024 && ((uintptr_t)partial & 15) == 0 && ((uintptr_t)residual & 15) == 0 &&
        (!xn || (((uintptr_t)xn & 15) == 0 && ((uintptr_t)w & 15) == 0))) {
        int threads = (N / 4 + 31) / 32 * 32;          // one float4 per thread where the row allows, four at most
        if (threads > 1024) threads = 1024;
        cudaStream_t st = (cudaStream_t)s;
        dim3 grid(M), block(threads);
#define RRN(TW, TO) g_launch_err = launch_pdl(reduce_residual_norm_vec_kernel<TW, TO>, grid, block, 0, st, partial, splits, M, N, bias, bias_dt, residual, (const TW *)w, eps, (TO *)xn)
        if (w_dt == HFB_F32 && xn_dt == HFB_F32) RRN(float, float);
        else if (w_dt == HFB_F32) RRN(float, __nv_bfloat16);
        else if (xn_dt == HFB_F32) RRN(__nv_bfloat16, float);
        else RRN(__nv_bfloat16, __nv_bfloat16);
#undef RRN
        return check_pdl_launch(g_launch_err, "reduce_residual_norm");
    }
    int threads = N >= 2048 ? 512 : (N >= 512 ? 256 : 128);
    g_launch_err = launch_pdl(reduce_residual_norm_kernel, dim3(M), dim3(threads), 0, (cudaStream_t)s, partial, splits, M, N, bias, bias_dt, residual, w, w_dt, eps, xn, xn_dt);
    return check_pdl_launch(g_launch_err, "reduce_residual_norm");
}

extern "C" int hfb_reduce_rope_kv(const float *partial, int splits, int dt, const void *bias, int bias_dt,
                                  const float *cos_sin, int n_rot, int n_positions, const int32_t *positions,
                                  const int32_t *slots, void *q_out, void *k_cache, void *v_cache, int64_t cache_slots,
                                  int T, int H, int G, int d, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(dt) || splits < 1 || H <= 0 || G <= 0 || d <= 0 || n_rot < 0 || n_rot > d || (n_rot & 1) || (bias && !valid_dt(bias_dt)))
        return fail(HFB_EINVAL, "reduce_rope_kv: bad arguments");
    if (n_rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "reduce_rope_kv: rotation needs a table and positions");
    if (H + 2 * G > 65535) return fail(HFB_ENOTSUP, "reduce_rope_kv: %d heads exceed the grid limit", H + 2 * G);
    dim3 grid(T, H + 2 * G);
    int threads = d >= 128 ? 64 : 32;
    cudaStream_t st = (cudaStream_t)s;
    if (dt == HFB_F32)
        g_launch_err = launch_pdl(reduce_rope_kv_kernel<float>, dim3(grid), dim3(threads), 0, st, partial, splits, T, bias, bias_dt, cos_sin, n_rot, n_positions, positions,
            slots, (float *)q_out, (float *)k_cache, (float *)v_cache, cache_slots, H, G, d, error_word());
    else
        g_launch_err = launch_pdl(reduce_rope_kv_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, st, partial, splits, T, bias, bias_dt, cos_sin, n_rot, n_positions,
            positions, slots, (__nv_bfloat16 *)q_out, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, cache_slots, H, G, d, error_word());
    return check_pdl_launch(g_launch_err, "reduce_rope_kv");
}

// Floats + ints of scratch hfb_argmax2 needs for M rows of V logits.
extern "C" size_t hfb_argmax2_scratch(int M, int V)
{
    int chunks = (V + 4095) / 4096;
    return (size_t)M * chunks * 8;
}

extern "C" int hfb_argmax2(const float *logits, int32_t *out, int M, int V, void *scratch, size_t scratch_bytes, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (V <= 0) return fail(HFB_EINVAL, "argmax: empty vocabulary");
    int chunks = (V + 4095) / 4096;
    if (!scratch || scratch_bytes < hfb_argmax2_scratch(M, V)) return fail(HFB_EINVAL, "argmax: scratch too small");
    if (M > 65535) return fail(HFB_ENOTSUP, "argmax: %d rows exceed the grid limit", M);
    float *bv = (float *)scratch;
    int32_t *bi = (int32_t *)(bv + (size_t)M * chunks);
    g_launch_err = launch_pdl(argmax_chunks_kernel, dim3(chunks, M), dim3(256), 0, (cudaStream_t)s, logits, V, 4096, bv, bi);
    g_launch_err = launch_pdl(argmax_final_kernel, dim3(M), dim3(32), 0, (cudaStream_t)s, bv, bi, chunks, out);
    return check_pdl_launch(g_launch_err, "argmax2");
}
