// Embedding gather, RMSNorm, rotary + cache write, SwiGLU, arg-max: the memory-bound steps.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

// ---- embedding (src/model.c:566-571) ---------------------------------------------------------
__global__ void embed_kernel(const int32_t *ids, const void *table, int dt, float *out, int V, int E, int *err)
{
    HFB_TRACE_ENTRY(7);
    pdl_entry();
    pdl_sync_small();
    int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(err, HFB_ERR_TOKEN_ID);
        for (int i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)t * E + i] = 0.f;
        return;
    }
    size_t base = (size_t)id * E;
    if (dt == HFB_BF16 && (E & 7) == 0 && ((uintptr_t)table & 15) == 0) {
        // eight values per 16-byte read
        const uint4 *src = (const uint4 *)((const __nv_bfloat16 *)table + base);
        float4 *dst = (float4 *)(out + (size_t)t * E);
        for (int i = threadIdx.x; i < (E >> 3); i += blockDim.x) {
            const uint4 v = src[i];
            const __nv_bfloat162 *h = (const __nv_bfloat162 *)&v;
            const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), e = __bfloat1622float2(h[3]);
            dst[2 * i] = make_float4(a.x, a.y, b.x, b.y);
            dst[2 * i + 1] = make_float4(c.x, c.y, e.x, e.y);
        }
        return;
    }
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)t * E + i] = load_any(table, dt, base + i);
}

// ---- RMSNorm (src/mathx.c:65-75): products and sum in float32 ---------------------------------
__global__ void rmsnorm_kernel(const float *x, const void *w, int w_dt, float eps, void *out, int out_dt,
                               const int32_t *rows, int E)
{
    HFB_TRACE_ENTRY(15);
    pdl_entry();
    pdl_sync_small();
    int m = blockIdx.x;
    const float *xr = x + (size_t)(rows ? rows[m] : m) * E;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    __shared__ float part[32];
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < nw ? part[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) part[0] = v;
    }
    __syncthreads();
    float r = 1.0f / sqrtf(part[0] / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x)
        store_any(out, out_dt, (size_t)m * E + i, (xr[i] * r) * load_any(w, w_dt, i));
}

// The same with 16-byte accesses, for widths that are a multiple of 4.
template <typename TW, typename TO>
__global__ void rmsnorm_vec_kernel(const float *x, const TW *w, float eps, TO *out, const int32_t *rows, int E)
{
    HFB_TRACE_ENTRY(6);
    pdl_entry();
    pdl_sync_small();
    int m = blockIdx.x;
    const float4 *xr = (const float4 *)(x + (size_t)(rows ? rows[m] : m) * E);
    const int E4 = E >> 2;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E4; i += blockDim.x) { float4 v = xr[i]; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    __shared__ float part[32];
    ss = warp_sum(ss);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float v = lane < nw ? part[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) part[0] = v;
    }
    __syncthreads();
    float r = 1.0f / sqrtf(part[0] / (float)E + eps);
    for (int i = threadIdx.x; i < E4; i += blockDim.x) {
        float4 v = xr[i];
        float w0 = to_f32(w[4 * i]), w1 = to_f32(w[4 * i + 1]), w2 = to_f32(w[4 * i + 2]), w3 = to_f32(w[4 * i + 3]);
        float y0 = (v.x * r) * w0, y1 = (v.y * r) * w1, y2 = (v.z * r) * w2, y3 = (v.w * r) * w3;
        TO *o = out + (size_t)m * E + 4 * i;
        if (sizeof(TO) == 4) *(float4 *)o = make_float4(y0, y1, y2, y3);
        else {
            __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
            *(uint2 *)o = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
        }
    }
}

// The same for rows of up to 256 * 4 * PER values: a thread keeps its part of the row in registers between the sum of
// squares and the scaling, so the row is read once and all of a thread's reads are under way together.
template <typename TW, typename TO, int PER>
__global__ void __launch_bounds__(256) rmsnorm_reg_kernel(const float *x, const TW *w, float eps, TO *out, const int32_t *rows, int E)
{
    HFB_TRACE_ENTRY(6);
    pdl_entry();
    pdl_sync_small();
    const int m = blockIdx.x;
    const float4 *xr = (const float4 *)(x + (size_t)(rows ? rows[m] : m) * E);
    const int E4 = E >> 2;
    float4 v[PER];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < E4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < PER; j++) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    __shared__ float part[8];
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += part[i];              // (every thread adds the eight sums in the same order)
    const float r = 1.0f / sqrtf(total / (float)E + eps);
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < E4) {
            const float w0 = to_f32(w[4 * i]), w1 = to_f32(w[4 * i + 1]), w2 = to_f32(w[4 * i + 2]), w3 = to_f32(w[4 * i + 3]);
            const float y0 = (v[j].x * r) * w0, y1 = (v[j].y * r) * w1, y2 = (v[j].z * r) * w2, y3 = (v[j].w * r) * w3;
            TO *o = out + (size_t)m * E + 4 * i;
            if (sizeof(TO) == 4) *(float4 *)o = make_float4(y0, y1, y2, y3);
            else {
                __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
                *(uint2 *)o = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
            }
        }
    }
}

// ---- rotary + cache write (src/model.c:587-601, :468-493) -------------------------------------
// One block per (token, head of the fused q|k|v row).  Pairs (i, i + n_rot/2) rotate; the rest copies.
template <typename T>
__global__ void rope_kv_write_kernel(const T *qkv, const float *cos_sin, int n_rot, int n_positions,
                                     const int32_t *positions, const int32_t *slots, T *q_out, T *k_cache,
                                     T *v_cache, long long cache_slots, int H, int G, int d, int *err)
{
    HFB_TRACE_ENTRY(16);
    pdl_entry();
    pdl_sync_small();
    int t = blockIdx.x, head = blockIdx.y;
    const T *src = qkv + (size_t)t * (H + 2 * G) * d + (size_t)head * d;
    T *dst;
    bool rotate;
    if (head < H) {
        dst = q_out + (size_t)t * H * d + (size_t)head * d;
        rotate = true;
    } else {
        if (!slots) return;
        long long slot = slots[t];
        if (slot < 0) return;
        if (slot >= cache_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); return; }
        if (head < H + G) { dst = k_cache + ((size_t)slot * G + (head - H)) * d; rotate = true; }
        else { dst = v_cache + ((size_t)slot * G + (head - H - G)) * d; rotate = false; }
    }
    int half = n_rot / 2;
    if (rotate && half > 0) {
        int pos = positions[t];
        if (pos < 0 || pos >= n_positions) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
        const float *cs = cos_sin + (size_t)pos * half * 2;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float c = cs[2 * i], s = cs[2 * i + 1];
            float a = to_f32(src[i]), b = to_f32(src[i + half]);
            float lo, hi;
            rope_pair(a, b, c, s, lo, hi);
            dst[i] = from_f32<T>(lo);
            dst[i + half] = from_f32<T>(hi);
        }
        for (int i = n_rot + threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
    }
}

// The same with 16-byte accesses: one block per token walks all heads; VEC elements per access.
template <typename T>
__global__ void rope_kv_write_vec_kernel(const T *qkv, const float *cos_sin, int n_rot, int n_positions,
                                         const int32_t *positions, const int32_t *slots, T *q_out, T *k_cache,
                                         T *v_cache, long long cache_slots, int H, int G, int d, int *err)
{
    HFB_TRACE_ENTRY(16);
    pdl_entry();
    pdl_sync_small();
    constexpr int VEC = 16 / sizeof(T);
    struct alignas(16) Pack { T e[VEC]; };
    const int t = blockIdx.x;
    const int half = n_rot / 2, per_head = d / VEC;
    long long slot = slots ? slots[t] : -1;
    if (slot >= cache_slots) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_SLOT); slot = -1; }
    int pos = positions ? positions[t] : 0;
    if (half > 0 && (pos < 0 || pos >= n_positions)) { if (threadIdx.x == 0) atomicOr(err, HFB_ERR_POSITION); pos = 0; }
    const float *cs = half > 0 ? cos_sin + (size_t)pos * half * 2 : nullptr;
    const T *row = qkv + (size_t)t * (H + 2 * G) * d;
    for (int item = threadIdx.x; item < (H + 2 * G) * per_head; item += blockDim.x) {
        const int head = item / per_head, e0 = (item % per_head) * VEC;
        T *dst;
        bool rotate = head < H + G;
        if (head < H) dst = q_out + (size_t)t * H * d + (size_t)head * d;
        else if (slot < 0) continue;
        else if (head < H + G) dst = k_cache + ((size_t)slot * G + (head - H)) * d;
        else dst = v_cache + ((size_t)slot * G + (head - H - G)) * d;
        const T *src = row + (size_t)head * d;
        if (rotate && e0 < half) {
            Pack a = *(const Pack *)(src + e0), b = *(const Pack *)(src + e0 + half), ra, rb;
            // the VEC (cos, sin) pairs of these elements: 16-byte reads (VEC is even, the table's rows are 8-byte pairs)
            float csv[2 * VEC];
#pragma unroll
            for (int i = 0; i < VEC / 2; i++) *(float4 *)(csv + 4 * i) = *(const float4 *)(cs + 2 * e0 + 4 * i);
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                float c = csv[2 * i], sn = csv[2 * i + 1];
                float x = to_f32(a.e[i]), y = to_f32(b.e[i]);
                float lo, hi;
                rope_pair(x, y, c, sn, lo, hi);
                ra.e[i] = from_f32<T>(lo);
                rb.e[i] = from_f32<T>(hi);
            }
            *(Pack *)(dst + e0) = ra;
            *(Pack *)(dst + e0 + half) = rb;
        } else if (!rotate || e0 >= n_rot) {
            *(Pack *)(dst + e0) = *(const Pack *)(src + e0);
        }
    }
}

// ---- SwiGLU (src/model.c:532-538, src/mathx.c:34) ----------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T *gu, T *out, int F, size_t total, int interleaved)
{
    HFB_TRACE_ENTRY(14);
    pdl_entry();
    pdl_sync_small();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t t = i / F;
    int f = (int)(i % F);
    // gate and up either fill the two halves of a row or alternate along it
    float g = to_f32(gu[t * 2 * F + (interleaved ? 2 * f : f)]), u = to_f32(gu[t * 2 * F + (interleaved ? 2 * f + 1 : F + f)]);
    out[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
}

// ---- arg-max, the lowest index wins ties (src/sample.c:72-77) ---------------------------------
__global__ void argmax_kernel(const float *logits, int32_t *out, int V)
{
    pdl_sync_small();
    const float *row = logits + (size_t)blockIdx.x * V;
    float best = 0.f;
    int bi = -1;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float v = row[i];
        if (bi < 0 || v > best) { best = v; bi = i; }
    }
    __shared__ float sv[1024];
    __shared__ int si[1024];
    sv[threadIdx.x] = best; si[threadIdx.x] = bi;
    __syncthreads();
    for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            float v2 = sv[threadIdx.x + o], v1 = sv[threadIdx.x];
            int i2 = si[threadIdx.x + o], i1 = si[threadIdx.x];
            if (i2 >= 0 && (i1 < 0 || v2 > v1 || (v2 == v1 && i2 < i1))) { sv[threadIdx.x] = v2; si[threadIdx.x] = i2; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = si[0] < 0 ? 0 : si[0];
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_embed(const int32_t *ids, const void *table, int table_dt, float *out, int T, int V, int E, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(table_dt) || V <= 0 || E <= 0) return fail(HFB_EINVAL, "embed: bad arguments");
    g_launch_err = launch_pdl(embed_kernel, dim3(T), dim3(256), 0, (cudaStream_t)s, ids, table, table_dt, out, V, E, error_word());
    return check_pdl_launch(g_launch_err, "embed");
}

extern "C" int hfb_rmsnorm(const float *x, const void *w, int w_dt, float eps, void *out, int out_dt,
                           const int32_t *rows, int M, int E, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (!valid_dt(w_dt) || !valid_dt(out_dt) || E <= 0) return fail(HFB_EINVAL, "rmsnorm: bad arguments");
    int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : 128);
    cudaStream_t st = (cudaStream_t)s;
    const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)w & 15) == 0;
    if ((E & 3) == 0 && aligned && w_dt == HFB_BF16 && out_dt == HFB_BF16 && E <= 8192 && M >= 64) {
        // many rows of the serving types: the row stays in registers
        const __nv_bfloat16 *wb = (const __nv_bfloat16 *)w;
        __nv_bfloat16 *ob = (__nv_bfloat16 *)out;
        if (E <= 2048) g_launch_err = launch_pdl(rmsnorm_reg_kernel<__nv_bfloat16, __nv_bfloat16, 2>, dim3(M), dim3(256), 0, st, x, wb, eps, ob, rows, E);
        else if (E <= 4096) g_launch_err = launch_pdl(rmsnorm_reg_kernel<__nv_bfloat16, __nv_bfloat16, 4>, dim3(M), dim3(256), 0, st, x, wb, eps, ob, rows, E);
        else g_launch_err = launch_pdl(rmsnorm_reg_kernel<__nv_bfloat16, __nv_bfloat16, 8>, dim3(M), dim3(256), 0, st, x, wb, eps, ob, rows, E);
    } else if ((E & 3) == 0 && aligned) {
        if (w_dt == HFB_F32 && out_dt == HFB_F32) g_launch_err = launch_pdl(rmsnorm_vec_kernel<float, float>, dim3(M), dim3(threads), 0, st, x, (const float *)w, eps, (float *)out, rows, E);
        else if (w_dt == HFB_F32) g_launch_err = launch_pdl(rmsnorm_vec_kernel<float, __nv_bfloat16>, dim3(M), dim3(threads), 0, st, x, (const float *)w, eps, (__nv_bfloat16 *)out, rows, E);
        else if (out_dt == HFB_F32) g_launch_err = launch_pdl(rmsnorm_vec_kernel<__nv_bfloat16, float>, dim3(M), dim3(threads), 0, st, x, (const __nv_bfloat16 *)w, eps, (float *)out, rows, E);
        else g_launch_err = launch_pdl(rmsnorm_vec_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(M), dim3(threads), 0, st, x, (const __nv_bfloat16 *)w, eps, (__nv_bfloat16 *)out, rows, E);
    } else {
        g_launch_err = launch_pdl(rmsnorm_kernel, dim3(M), dim3(threads), 0, st, x, w, w_dt, eps, out, out_dt, rows, E);
    }
    return check_pdl_launch(g_launch_err, "rmsnorm");
}

extern "C" int hfb_rope_kv_write(const void *qkv, int dt, const float *cos_sin, int n_rot, int n_positions,
                                 const int32_t *positions, const int32_t *slots, void *q_out, void *k_cache,
                                 void *v_cache, int64_t cache_slots, int T, int H, int G, int d, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(dt) || H <= 0 || G <= 0 || d <= 0 || n_rot < 0 || n_rot > d || (n_rot & 1))
        return fail(HFB_EINVAL, "rope_kv_write: bad arguments (H=%d G=%d d=%d n_rot=%d)", H, G, d, n_rot);
    if (n_rot > 0 && (!cos_sin || !positions)) return fail(HFB_EINVAL, "rope_kv_write: rotation needs a table and positions");
    if (H + 2 * G > 65535) return fail(HFB_ENOTSUP, "rope_kv_write: %d heads exceed the grid limit", H + 2 * G);
    const int vec = dt == HFB_F32 ? 4 : 8;
    if (d % vec == 0 && (n_rot / 2) % vec == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)cos_sin & 15) == 0 &&
        ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0) {
        int items = (H + 2 * G) * (d / vec);
        int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
        if (dt == HFB_F32)
            g_launch_err = launch_pdl(rope_kv_write_vec_kernel<float>, dim3(T), dim3(threads), 0, (cudaStream_t)s, (const float *)qkv, cos_sin, n_rot, n_positions,
                positions, slots, (float *)q_out, (float *)k_cache, (float *)v_cache, cache_slots, H, G, d, error_word());
        else
            g_launch_err = launch_pdl(rope_kv_write_vec_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, (cudaStream_t)s, (const __nv_bfloat16 *)qkv, cos_sin, n_rot,
                n_positions, positions, slots, (__nv_bfloat16 *)q_out, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache,
                cache_slots, H, G, d, error_word());
        return check_pdl_launch(g_launch_err, "rope_kv_write");
    }
    dim3 grid(T, H + 2 * G);
    int threads = d >= 128 ? 64 : 32;
    if (dt == HFB_F32)
        g_launch_err = launch_pdl(rope_kv_write_kernel<float>, dim3(grid), dim3(threads), 0, (cudaStream_t)s, (const float *)qkv, cos_sin, n_rot, n_positions,
            positions, slots, (float *)q_out, (float *)k_cache, (float *)v_cache, cache_slots, H, G, d, error_word());
    else
        g_launch_err = launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, (cudaStream_t)s, (const __nv_bfloat16 *)qkv, cos_sin, n_rot,
            n_positions, positions, slots, (__nv_bfloat16 *)q_out, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache,
            cache_slots, H, G, d, error_word());
    return check_pdl_launch(g_launch_err, "rope_kv_write");
}

extern "C" int hfb_swiglu(const void *gu, void *out, int dt, int T, int F, int interleaved, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(dt) || F <= 0) return fail(HFB_EINVAL, "swiglu: bad arguments");
    size_t total = (size_t)T * F;
    unsigned blocks = (unsigned)((total + 255) / 256);
    if (dt == HFB_F32) g_launch_err = launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const float *)gu, (float *)out, F, total, interleaved);
    else g_launch_err = launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, (cudaStream_t)s, (const __nv_bfloat16 *)gu, (__nv_bfloat16 *)out, F, total, interleaved);
    return check_pdl_launch(g_launch_err, "swiglu");
}

extern "C" int hfb_argmax(const float *logits, int32_t *out, int M, int V, hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (V <= 0) return fail(HFB_EINVAL, "argmax: empty vocabulary");
    g_launch_err = launch_pdl(argmax_kernel, dim3(M), dim3(1024), 0, (cudaStream_t)s, logits, out, V);
    return check_pdl_launch(g_launch_err, "argmax");
}
