// out[M,N] (=|+=) a[M,K] . w[N,K]^T for very few rows (M <= 16, decode): a weight-streaming kernel.
//
// With a handful of tokens the product is a pure read of the weight matrix, and what counts is that every SM
// pulls weights from HBM from its first cycle to its last with nothing staged in between.  Each CTA owns 16
// consecutive weight rows; its 8 warps split K between them; each lane loads 16 bytes of two rows straight
// from global memory into registers and feeds them to mma.sync m16n8k16 as the A operand (weights on the 16
// rows, 8 tokens on the columns), with the token activations as the B operand read in the same k order.  The
// warps' partial sums meet in shared memory and are added in warp order, so there are no partial sums in
// global memory, no second kernel, and the epilogue (bias, residual, SwiGLU of adjacent gate/up rows) runs in
// place.  The first batch of weight loads is issued before the kernel waits for its predecessor.
// (The tcgen05 kernel in gemm_tc.cu takes over from 17 rows on, where the tensor-core work starts to matter.)
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

constexpr int GV_WARPS = 8, GV_ROWS = 16, GV_UNROLL = 6;
enum { GV_STORE = 0, GV_ADD = 1, GV_SWIGLU = 2 };

__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float *c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_mma_kernel(const __nv_bfloat16 *a, const __nv_bfloat16 *w, const void *bias, int bias_dt, void *out, int out_dt,
                int mode, int M, int N, int K)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * GV_ROWS;
    const bool va = row0 + g < N, vb = row0 + g + 8 < N;
    const __nv_bfloat16 *wa = w + (size_t)(va ? row0 + g : 0) * K, *wb = w + (size_t)(vb ? row0 + g + 8 : 0) * K;
    // K in units of 32 elements (one 16-byte load per lane of a quad); the warps take consecutive ranges of units
    const int units = (K + 31) / 32;
    const int u0 = (int)((long long)units * warp / GV_WARPS), u1 = (int)((long long)units * (warp + 1) / GV_WARPS);
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    bool first = true;

    for (int u = u0; u < u1 || first; u += GV_UNROLL) {
        uint4 ra[GV_UNROLL], rb[GV_UNROLL];
#pragma unroll
        for (int i = 0; i < GV_UNROLL; i++) {
            const int k = (u + i) * 32 + t * 8;
            const bool in = u + i < u1 && k < K;
            ra[i] = in && va ? ldg_stream(wa + k) : zero;
            rb[i] = in && vb ? ldg_stream(wb + k) : zero;
        }
        if (first) { pdl_sync(); first = false; }        // the weights are on their way; now the activations may be read
#pragma unroll
        for (int i = 0; i < GV_UNROLL; i++) {
            const int k = (u + i) * 32 + t * 8;
            const bool in = u + i < u1 && k < K;
#pragma unroll
            for (int n = 0; n < NT; n++) {
                const int tok = n * 8 + g;
                uint4 x = in && tok < M ? *(const uint4 *)(a + (size_t)tok * K + k) : zero;
                mma16816(acc[n], ra[i].x, rb[i].x, ra[i].y, rb[i].y, x.x, x.y);
                mma16816(acc[n], ra[i].z, rb[i].z, ra[i].w, rb[i].w, x.z, x.w);
            }
        }
    }

    // ---- the warps' partial sums meet in shared memory, summed in warp order ---------------------------
    __shared__ float red[GV_WARPS][GV_ROWS][8 * NT + 1];
#pragma unroll
    for (int n = 0; n < NT; n++) {
        red[warp][g][n * 8 + 2 * t] = acc[n][0];
        red[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
        red[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
        red[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
    }
    __syncthreads();
    const int per_row = 8 * NT;
    if (mode == GV_SWIGLU) {
        // rows alternate gate, up: one thread per (pair of rows, token); out is [M, N/2]
        for (int i = threadIdx.x; i < (GV_ROWS / 2) * per_row; i += blockDim.x) {
            const int pr = i / per_row, tok = i % per_row, row = row0 + 2 * pr;
            if (row + 1 >= N || tok >= M) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int wv = 0; wv < GV_WARPS; wv++) { gate += red[wv][2 * pr][tok]; up += red[wv][2 * pr + 1][tok]; }
            store_any(out, out_dt, (size_t)tok * (N >> 1) + (row >> 1), (gate / (1.0f + expf(-gate))) * up);
        }
        return;
    }
    for (int i = threadIdx.x; i < GV_ROWS * per_row; i += blockDim.x) {
        const int r = i % GV_ROWS, tok = i / GV_ROWS, row = row0 + r;      // consecutive threads -> consecutive features
        if (row >= N || tok >= M) continue;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < GV_WARPS; wv++) v += red[wv][r][tok];
        if (bias) v += load_any(bias, bias_dt, row);
        const size_t o = (size_t)tok * N + row;
        if (mode == GV_ADD) ((float *)out)[o] += v;
        else store_any(out, out_dt, o, v);
    }
}

}  // namespace hfb

using namespace hfb;

// mode: 0 store (+bias), 1 accumulate into a float32 out (+bias), 2 SwiGLU of alternating gate/up rows (out [M, N/2]).
extern "C" int hfb_linear_mma(const void *a, const void *w, const void *bias, int bias_dt, void *out, int out_dt,
                              int mode, int M, int N, int K, hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    if (M > 16) return fail(HFB_ENOTSUP, "linear_mma: at most 16 rows (got %d)", M);
    if (K <= 0 || (K & 7)) return fail(HFB_ENOTSUP, "linear_mma: K = %d must be a positive multiple of 8", K);
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return fail(HFB_ENOTSUP, "linear_mma: operands must be 16-byte aligned");
    if (!valid_dt(out_dt) || (bias && !valid_dt(bias_dt)) || mode < 0 || mode > 2) return fail(HFB_EINVAL, "linear_mma: bad arguments");
    if (mode == GV_ADD && out_dt != HFB_F32) return fail(HFB_EINVAL, "linear_mma: accumulation needs a float32 output");
    if (mode == GV_SWIGLU && (N & 1)) return fail(HFB_EINVAL, "linear_mma: N must be even for SwiGLU");
    dim3 grid((N + GV_ROWS - 1) / GV_ROWS);
    cudaStream_t st = (cudaStream_t)s;
    const __nv_bfloat16 *pa = (const __nv_bfloat16 *)a, *pw = (const __nv_bfloat16 *)w;
    if (M <= 8) g_launch_err = launch_pdl(gemv_mma_kernel<1>, grid, dim3(GV_WARPS * 32), 0, st, pa, pw, bias, bias_dt, out, out_dt, mode, M, N, K);
    else g_launch_err = launch_pdl(gemv_mma_kernel<2>, grid, dim3(GV_WARPS * 32), 0, st, pa, pw, bias, bias_dt, out, out_dt, mode, M, N, K);
    return check_pdl_launch(g_launch_err, "linear_mma");
}
