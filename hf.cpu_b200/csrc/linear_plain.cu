// out[M,N] (=|+=) a[M,K] . w[N,K]^T (+ bias): the plain matrix product.
//
// Float32 multiply-adds only, one fixed summation order over k for every output element, any sizes,
// any mix of float32 / bfloat16 operands.  It is the whole float32 path's product and the comparison
// for the tensor-core kernels, in the way the reference keeps portable kernels beside its vector ones
// (src/kern_generic.c:84-91 beside src/kern_avx2.c:79-95; call shape src/model.c:419-425).
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
linear_plain_kernel(const TA *__restrict__ a, const TW *__restrict__ w, const void *bias, int bias_dt,
                    void *out, int out_dt, int accumulate, int M, int N, int K)
{
    pdl_sync();
    __shared__ float sa[TK][TM + 1];
    __shared__ float sw[TK][TN + 1];
    int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int e = threadIdx.x; e < TM * TK; e += 256) {
            int r = e / TK, c = e % TK;
            int gm = m0 + r, gk = k0 + c;
            sa[c][r] = (gm < M && gk < K) ? to_f32(a[(size_t)gm * K + gk]) : 0.f;
        }
        for (int e = threadIdx.x; e < TN * TK; e += 256) {
            int r = e / TK, c = e % TK;
            int gn = n0 + r, gk = k0 + c;
            sw[c][r] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk++) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_any(bias, bias_dt, gn);
            size_t o = (size_t)gm * N + gn;
            if (accumulate) ((float *)out)[o] += v;
            else store_any(out, out_dt, o, v);
        }
    }
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_linear_plain(const void *a, int a_dt, const void *w, int w_dt, const void *bias, int bias_dt,
                                void *out, int out_dt, int accumulate, int M, int N, int K, hfb_stream s)
{
    if (M <= 0 || N <= 0) return HFB_OK;
    if (!valid_dt(a_dt) || !valid_dt(w_dt) || !valid_dt(out_dt) || (bias && !valid_dt(bias_dt)) || K <= 0)
        return fail(HFB_EINVAL, "linear: bad arguments (M=%d N=%d K=%d)", M, N, K);
    if (accumulate && out_dt != HFB_F32) return fail(HFB_EINVAL, "linear: accumulation needs a float32 output");
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return fail(HFB_ENOTSUP, "linear: %d rows exceed the plain kernel's grid", M);
    cudaStream_t st = (cudaStream_t)s;
#define LAUNCH(TA, TW) g_launch_err = launch_pdl(linear_plain_kernel<TA, TW>, dim3(grid), dim3(256), 0, st, (const TA *)a, (const TW *)w, bias, bias_dt, out, out_dt, accumulate, M, N, K)
    if (a_dt == HFB_F32 && w_dt == HFB_F32) LAUNCH(float, float);
    else if (a_dt == HFB_F32) LAUNCH(float, __nv_bfloat16);
    else if (w_dt == HFB_F32) LAUNCH(__nv_bfloat16, float);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
    return check_pdl_launch(g_launch_err, "linear_plain");
}
