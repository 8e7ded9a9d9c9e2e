// Attention over the paged cache, plain kernel: one block per (token, head).
//
// For token t at position pos of its request, head h reads key/value head h / (H/G) over keys
// lo..pos; score = dot(q, k) * scale (scale after the dot), softmax in float32, out = sum p_j v_j
// (src/model.c:499-528, src/mathx.c:77-86).  Each warp takes every fourth key with a running
// maximum and sum; the four partial results are merged in a fixed order, so the result depends
// only on (lo, pos) and the values, never on what else is in the batch.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {
int *error_word();

constexpr int ATT_WARPS = 4;
constexpr int MAX_D_PER_LANE = 8;      // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_plain_kernel(const T *q, const T *k_cache, const T *v_cache, const int32_t *block_table, int max_blocks,
                       const int32_t *token_seq, const int32_t *positions, int block_size, long long num_pages,
                       int window, float scale, T *out, int H, int G, int d, int *err)
{
    pdl_sync();
    int t = blockIdx.x, h = blockIdx.y;
    int g = h / (H / G);
    int seq = token_seq[t], pos = positions[t];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int32_t *table = block_table + (size_t)seq * max_blocks;

    __shared__ float sq[256];
    __shared__ float s_m[ATT_WARPS], s_l[ATT_WARPS];
    __shared__ float s_acc[ATT_WARPS][256];
    const T *qr = q + ((size_t)t * H + h) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) sq[i] = to_f32(qr[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.f, acc[MAX_D_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_D_PER_LANE; i++) acc[i] = 0.f;

    for (int j = lo + warp; j <= pos; j += ATT_WARPS) {
        int blk = j / block_size;
        long long page = blk < max_blocks ? table[blk] : -1;
        if (page < 0 || page >= num_pages) { if (lane == 0) atomicOr(err, HFB_ERR_PAGE); continue; }
        size_t base = (((size_t)page * block_size + (j % block_size)) * G + g) * d;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_D_PER_LANE; i++) {
            int c = lane + 32 * i;
            if (c < d) dot = fmaf(sq[c], to_f32(k_cache[base + c]), dot);
        }
        dot = warp_sum(dot) * scale;
        float m_new = fmaxf(m, dot);
        float corr = expf(m - m_new);            // exp(-inf) = 0 on the first key
        float p = expf(dot - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_D_PER_LANE; i++) {
            int c = lane + 32 * i;
            if (c < d) acc[i] = acc[i] * corr + p * to_f32(v_cache[base + c]);
        }
        m = m_new;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < MAX_D_PER_LANE; i++) {
        int c = lane + 32 * i;
        if (c < d) s_acc[warp][c] = acc[i];
    }
    __syncthreads();
    float mm = -INFINITY;
    for (int w = 0; w < ATT_WARPS; w++) mm = fmaxf(mm, s_m[w]);
    float ll = 0.f;
    float f[ATT_WARPS];
    for (int w = 0; w < ATT_WARPS; w++) {
        f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - mm);
        ll += s_l[w] * f[w];
    }
    float inv = ll > 0.f ? 1.0f / ll : 0.f;
    T *o = out + ((size_t)t * H + h) * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < ATT_WARPS; w++) v += s_acc[w][c] * f[w];
        o[c] = from_f32<T>(v * inv);
    }
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_attention_plain(const void *q, const void *k_cache, const void *v_cache, int dt,
                                   const int32_t *block_table, int max_blocks, const int32_t *token_seq,
                                   const int32_t *positions, int block_size, int64_t num_pages, int window,
                                   float scale, void *out, int T, int H, int G, int d, hfb_stream s)
{
    if (T <= 0) return HFB_OK;
    if (!valid_dt(dt) || H <= 0 || G <= 0 || H % G || block_size <= 0 || max_blocks <= 0 || window < 0)
        return fail(HFB_EINVAL, "attention: bad arguments (H=%d G=%d block=%d)", H, G, block_size);
    if (d <= 0 || d > 32 * MAX_D_PER_LANE)
        return fail(HFB_ENOTSUP, "attention: head_dim %d is not supported (1..%d)", d, 32 * MAX_D_PER_LANE);
    if (H > 65535) return fail(HFB_ENOTSUP, "attention: %d heads exceed the grid limit", H);
    dim3 grid(T, H);
    if (dt == HFB_F32)
        g_launch_err = launch_pdl(attention_plain_kernel<float>, dim3(grid), dim3(ATT_WARPS * 32), 0, (cudaStream_t)s, (const float *)q, (const float *)k_cache,
            (const float *)v_cache, block_table, max_blocks, token_seq, positions, block_size, num_pages, window, scale,
            (float *)out, H, G, d, error_word());
    else
        g_launch_err = launch_pdl(attention_plain_kernel<__nv_bfloat16>, dim3(grid), dim3(ATT_WARPS * 32), 0, (cudaStream_t)s, (const __nv_bfloat16 *)q,
            (const __nv_bfloat16 *)k_cache, (const __nv_bfloat16 *)v_cache, block_table, max_blocks, token_seq, positions,
            block_size, num_pages, window, scale, (__nv_bfloat16 *)out, H, G, d, error_word());
    return check_pdl_launch(g_launch_err, "attention_plain");
}
