// Temperature sampling with top-k, min-p and top-p on the device, one block per row of logits.
//
// Order of operations as the reference's sampler (src/sample.c:66-116): candidates in the order
// (logit descending, id ascending); cut to top-k; p = exp((l - max)/temp) / sum; min-p keeps
// p >= min_p * p_max; top-p keeps the smallest prefix whose cumulative p reaches top_p; the draw
// takes the first candidate whose cumulative p exceeds r = u * sum(kept), else the last kept.
//
// The order is never materialised for the whole vocabulary.  Each candidate has a 64-bit rank key
// (orderable logit bits, then inverted id), descending key = the reference's order, and a cut in
// that order is found by a radix descent over the key's bytes: a histogram of counts (top-k) or of
// probability mass (top-p, the draw) per byte value, walked from the top.  When top-k leaves at
// most 1024 candidates they are sorted in shared memory and the rest runs sequentially on them,
// summing in the reference's order.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SMALL_K = 1024;

__device__ __forceinline__ unsigned long long rank_key(float l, int id)
{
    unsigned u = __float_as_uint(l);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned)(0xFFFFFFFFu - (unsigned)id);
}

struct Row {
    const float *l;
    int V;
    float lmax, temp, sum;
    __device__ float e(int i) const { return expf((l[i] - lmax) / temp); }
};

__device__ float block_sum(float v, float *red)
{
    v = warp_sum(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    float r = red[0];
    __syncthreads();
    return r;
}

enum { BY_COUNT = 0, BY_MASS_GE = 1, BY_MASS_GT = 2 };

// Finds the first candidate, in descending key order among those with key >= cut, at which the running
// count reaches `target` (BY_COUNT) or the running mass p reaches / exceeds it.  Returns its key, or 0 when
// the whole set stays below the target.  Shared: hist[256] floats, *result.
template <int MODE>
__device__ unsigned long long descend(const Row &r, unsigned long long cut, float target, float *hist,
                                      unsigned long long *result)
{
    unsigned long long prefix = 0;          // the bytes fixed so far, in place
    float before = 0.f;                     // count or mass of candidates that rank above the current prefix
    bool found = true;
    for (int b = 7; b >= 0; b--) {
        if (b == 3) { prefix |= 0xFFull << 24; continue; }        // ids stay below 2^24: this byte is constant
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.f;
        __syncthreads();
        int cur = -1;
        float run = 0.f;
        unsigned long long hi_mask = b == 7 ? 0ull : (~0ull << (8 * (b + 1)));
        for (int i = threadIdx.x; i < r.V; i += blockDim.x) {
            unsigned long long k = rank_key(r.l[i], i);
            if (k < cut || (k & hi_mask) != (prefix & hi_mask)) continue;
            int bin = (int)((k >> (8 * b)) & 0xFF);
            float w = MODE == BY_COUNT ? 1.f : r.e(i) / r.sum;
            if (bin != cur) {
                if (cur >= 0) atomicAdd(&hist[cur], run);
                cur = bin;
                run = 0.f;
            }
            run += w;
        }
        if (cur >= 0) atomicAdd(&hist[cur], run);
        __syncthreads();
        if (threadIdx.x == 0) {
            float acc = before;
            int pick = -1, lowest = -1;
            for (int bin = 255; bin >= 0; bin--) {
                float h = hist[bin];
                if (h == 0.f) continue;
                bool hit = MODE == BY_MASS_GT ? (acc + h > target) : (acc + h >= target);
                if (hit) { pick = bin; break; }
                acc += h;
                lowest = bin;
            }
            // Below the first byte the target is known to lie inside the chosen bucket; if re-summing its
            // mass in finer bins falls short by rounding, the bucket's last candidate is the one.
            if (pick < 0 && b < 7 && lowest >= 0) { pick = lowest; acc -= hist[lowest]; }
            result[0] = pick < 0 ? ~0ull : (unsigned long long)pick;
            ((float *)(result + 1))[0] = acc;
        }
        __syncthreads();
        unsigned long long pick = result[0];
        before = ((float *)(result + 1))[0];
        __syncthreads();
        if (pick == ~0ull) { found = false; break; }
        prefix |= pick << (8 * b);
    }
    return found ? prefix : 0ull;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float *logits, int V, const float *temps, const int32_t *top_ks, const float *top_ps,
              const float *min_ps, const float *uniforms, int32_t *out)
{
    pdl_sync();
    __shared__ float red[32];
    __shared__ float hist[256];
    __shared__ unsigned long long result[2];
    __shared__ unsigned long long cand[SMALL_K];
    __shared__ int n_cand;

    int row = blockIdx.x;
    Row r;
    r.l = logits + (size_t)row * V;
    r.V = V;
    r.temp = temps[row];
    r.sum = 1.f;
    int K = top_ks[row];
    float top_p = top_ps[row], min_p = min_ps[row], u = uniforms[row];

    // the maximum and, for greedy rows, its first index
    unsigned long long best = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) best = max(best, rank_key(r.l[i], i));
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) ((unsigned long long *)hist)[threadIdx.x >> 5] = best;    // 32 x 8 bytes = hist[0..63]
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long b = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) b = max(b, ((unsigned long long *)hist)[w]);
        result[0] = b;
    }
    __syncthreads();
    best = result[0];
    __syncthreads();
    int best_id = (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFu));
    if (r.temp <= 0.f) {
        if (threadIdx.x == 0) out[row] = best_id;
        return;
    }
    r.lmax = r.l[best_id];

    // top-k: the cut is the key of the K-th candidate
    unsigned long long cut = 0;
    bool limited = K > 0 && K < V;
    if (limited) cut = descend<BY_COUNT>(r, 0, (float)K, hist, result);

    if (limited && K <= SMALL_K) {
        // few candidates: sort them and run the reference's sequence on the sorted list
        if (threadIdx.x == 0) n_cand = 0;
        for (int i = threadIdx.x; i < SMALL_K; i += blockDim.x) cand[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            unsigned long long k = rank_key(r.l[i], i);
            if (k >= cut) { int at = atomicAdd(&n_cand, 1); if (at < SMALL_K) cand[at] = k; }
        }
        __syncthreads();
        for (int size = 2; size <= SMALL_K; size <<= 1)
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                for (int i = threadIdx.x; i < SMALL_K; i += blockDim.x) {
                    int j = i ^ stride;
                    if (j > i) {
                        bool desc = (i & size) == 0;
                        unsigned long long a = cand[i], b = cand[j];
                        if (desc ? a < b : a > b) { cand[i] = b; cand[j] = a; }
                    }
                }
                __syncthreads();
            }
        if (threadIdx.x == 0) {
            int m = min(n_cand, K);
            float sum = 0.f;
            for (int i = 0; i < m; i++) sum += r.e((int)(0xFFFFFFFFu - (unsigned)(cand[i] & 0xFFFFFFFFu)));
            auto prob = [&](int i) { return r.e((int)(0xFFFFFFFFu - (unsigned)(cand[i] & 0xFFFFFFFFu))) / sum; };
            float pmax = prob(0);
            int kept = m;
            if (min_p > 0.f) { kept = 0; while (kept < m && prob(kept) >= min_p * pmax) kept++; if (kept == 0) kept = 1; }
            if (top_p > 0.f && top_p < 1.f) {
                float cum = 0.f;
                for (int i = 0; i < kept; i++) { cum += prob(i); if (cum >= top_p) { kept = i + 1; break; } }
            }
            float s2 = 0.f;
            for (int i = 0; i < kept; i++) s2 += prob(i);
            float rr = u * s2, cum = 0.f;
            int pick = kept - 1;
            for (int i = 0; i < kept; i++) { cum += prob(i); if (rr < cum) { pick = i; break; } }
            out[row] = (int)(0xFFFFFFFFu - (unsigned)(cand[pick] & 0xFFFFFFFFu));
        }
        return;
    }

    // many candidates: cuts by radix descent over probability mass
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
        if (rank_key(r.l[i], i) >= cut) s += r.e(i);
    float sum1 = block_sum(s, red);
    r.sum = sum1;
    if (min_p > 0.f) {
        // p is monotone in the order, so the kept prefix is the set of candidates that pass the test
        float pmax = 1.0f / sum1;
        unsigned long long lowest = ~0ull;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            unsigned long long k = rank_key(r.l[i], i);
            if (k >= cut && r.e(i) / sum1 >= min_p * pmax) lowest = min(lowest, k);
        }
        for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) ((unsigned long long *)hist)[threadIdx.x >> 5] = lowest;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long b = ~0ull;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) b = min(b, ((unsigned long long *)hist)[w]);
            result[0] = b == ~0ull ? best : b;
        }
        __syncthreads();
        cut = max(cut, result[0]);
        __syncthreads();
    }
    if (top_p > 0.f && top_p < 1.f) {
        unsigned long long c = descend<BY_MASS_GE>(r, cut, top_p, hist, result);
        if (c) cut = c;
    }
    s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
        if (rank_key(r.l[i], i) >= cut) s += r.e(i) / r.sum;
    float kept_sum = block_sum(s, red);
    unsigned long long pick = descend<BY_MASS_GT>(r, cut, u * kept_sum, hist, result);
    if (!pick) {
        // rounding left r at or above the total: the last kept candidate (src/sample.c:113)
        unsigned long long lowest = ~0ull;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            unsigned long long k = rank_key(r.l[i], i);
            if (k >= cut) lowest = min(lowest, k);
        }
        for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) ((unsigned long long *)hist)[threadIdx.x >> 5] = lowest;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long b = ~0ull;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) b = min(b, ((unsigned long long *)hist)[w]);
            result[0] = b;
        }
        __syncthreads();
        pick = result[0];
    }
    if (threadIdx.x == 0) out[row] = (int)(0xFFFFFFFFu - (unsigned)(pick & 0xFFFFFFFFu));
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_sample(const float *logits, int M, int V, const float *temps, const int32_t *top_ks,
                          const float *top_ps, const float *min_ps, const float *uniforms, int32_t *out,
                          hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (V <= 0 || V >= (1 << 24)) return fail(HFB_ENOTSUP, "sample: vocabulary of %d is not supported (1..2^24-1)", V);
    g_launch_err = launch_pdl(sample_kernel, dim3(M), dim3(SAMPLE_THREADS), 0, (cudaStream_t)s, logits, V, temps, top_ks, top_ps, min_ps, uniforms, out);
    return check_pdl_launch(g_launch_err, "sample");
}
