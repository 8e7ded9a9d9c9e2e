// Temperature sampling with top-k, min-p and top-p on the device: a thread-block cluster of eight CTAs per row of logits.
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
//
// A row is the work of a thread-block cluster of SAMPLE_CLUSTER CTAs: each walks its slice of the vocabulary, and
// what a walk finds (a maximum, a sum, a histogram, candidates) is combined over the cluster through distributed
// shared memory in rank order, every CTA arriving at the same value, so that all take the same decisions.
#include "common.cuh"

static thread_local cudaError_t g_launch_err = cudaSuccess;      // what the last launch_pdl returned

namespace hfb {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SMALL_K = 1024;
constexpr int SAMPLE_CLUSTER = 8;       // CTAs per row

__device__ __forceinline__ unsigned long long rank_key(float l, int id)
{
    unsigned u = __float_as_uint(l);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned)(0xFFFFFFFFu - (unsigned)id);
}

__device__ __forceinline__ float key_logit(unsigned long long k)
{
    const unsigned u = (unsigned)(k >> 32);
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
}

struct Row {
    const float *l;
    int V;
    int lo, hi;                         // this CTA's slice of the vocabulary (lo is a multiple of 4)
    float lmax, temp, sum;
    __device__ float e(int i) const { return expf((l[i] - lmax) / temp); }
    __device__ float e_of(float logit) const { return expf((logit - lmax) / temp); }
};

// Calls f(index, logit) for every logit of this CTA's slice of the row, each thread of the block taking its share.  A thread has
// sixteen logits on their way (four 16-byte reads) before it looks at the first: one block walks the whole
// vocabulary several times, and with one read in flight per thread each walk cost a round trip to L2 per logit.
template <typename F>
__device__ __forceinline__ void scan_row(const Row &r, F f)
{
    if (r.lo >= r.hi) return;
    const bool vec = (((uintptr_t)r.l) & 15) == 0;
    const int first4 = r.lo >> 2, V4 = vec ? (first4 + ((r.hi - r.lo) >> 2)) : first4, n = blockDim.x;
    const float4 *l4 = (const float4 *)r.l;
    int i = first4 + threadIdx.x;
    for (; i + 3 * n < V4; i += 4 * n) {
        const float4 a = l4[i], b = l4[i + n], c = l4[i + 2 * n], d = l4[i + 3 * n];
        f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
        f(4 * (i + n), b.x); f(4 * (i + n) + 1, b.y); f(4 * (i + n) + 2, b.z); f(4 * (i + n) + 3, b.w);
        f(4 * (i + 2 * n), c.x); f(4 * (i + 2 * n) + 1, c.y); f(4 * (i + 2 * n) + 2, c.z); f(4 * (i + 2 * n) + 3, c.w);
        f(4 * (i + 3 * n), d.x); f(4 * (i + 3 * n) + 1, d.y); f(4 * (i + 3 * n) + 2, d.z); f(4 * (i + 3 * n) + 3, d.w);
    }
    for (; i < V4; i += n) {
        const float4 a = l4[i];
        f(4 * i, a.x); f(4 * i + 1, a.y); f(4 * i + 2, a.z); f(4 * i + 3, a.w);
    }
    for (int j = 4 * V4 + threadIdx.x; j < r.hi; j += n) f(j, r.l[j]);
}

// ---- the cluster ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t rank_addr(const void *p, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_rank_f32(uint32_t a)
{
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ int ld_rank_s32(uint32_t a)
{
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_rank_u64(uint32_t a)
{
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared memory of a CTA.  `x_*` is what the CTAs of the cluster show one another, in two copies used in turn:
// a CTA writes the copy of exchange n + 2 only after the barrier of exchange n + 1, which every CTA enters after
// it has read exchange n, so one barrier per exchange is enough.  `turn` counts the exchanges, alike in all threads.
struct Shared {
    float x_hist[2][256];
    unsigned long long x_word[2];
    float x_value[2];
    float hist[256];                                    // a histogram summed over the cluster
    float whist[(SAMPLE_THREADS / 32) * 256];           // a histogram per warp; the CTA's candidates when they are few
    unsigned long long cand[SMALL_K];
    unsigned long long keys[32];
    unsigned long long result[2];
    float red[32];
    int n_cand;
    int n_listed;
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

// the sum over the cluster, the CTAs' sums added in rank order
__device__ float cluster_sum(float v, Shared *sh, unsigned &turn)
{
    const float mine = block_sum(v, sh->red);
    const unsigned t = turn++ & 1;
    if (threadIdx.x == 0) sh->x_value[t] = mine;
    cluster_sync_all();
    float acc = 0.f;
    for (int rk = 0; rk < SAMPLE_CLUSTER; rk++) acc += ld_rank_f32(rank_addr(&sh->x_value[t], rk));
    return acc;
}

// the largest (or smallest) key over the cluster
template <bool LARGEST>
__device__ unsigned long long cluster_key(unsigned long long v, Shared *sh, unsigned &turn)
{
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long w = __shfl_xor_sync(0xffffffffu, v, o);
        v = LARGEST ? max(v, w) : min(v, w);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh->keys[threadIdx.x >> 5] = v;
    __syncthreads();
    const unsigned t = turn++ & 1;
    if (threadIdx.x == 0) {
        unsigned long long b = LARGEST ? 0ull : ~0ull;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) b = LARGEST ? max(b, sh->keys[w]) : min(b, sh->keys[w]);
        sh->x_word[t] = b;
    }
    cluster_sync_all();
    unsigned long long acc = LARGEST ? 0ull : ~0ull;
    for (int rk = 0; rk < SAMPLE_CLUSTER; rk++) {
        const unsigned long long w = ld_rank_u64(rank_addr(&sh->x_word[t], rk));
        acc = LARGEST ? max(acc, w) : min(acc, w);
    }
    return acc;
}

enum { BY_COUNT = 0, BY_MASS_GE = 1, BY_MASS_GT = 2 };

// Finds the first candidate, in descending key order among those with key >= cut, at which the running
// count reaches `target` (BY_COUNT) or the running mass p reaches / exceeds it.  Returns its key, or 0 when
// the whole set stays below the target.
//
// Once a byte is fixed, the candidates that still match are usually few: while a CTA walks its slice for the next
// byte it also lists the keys that match (in sh->cand, as long as they fit), and the bytes after that are read off
// the list instead of the vocabulary.
template <int MODE>
__device__ unsigned long long descend(const Row &r, unsigned long long cut, float target, Shared *sh, unsigned &turn)
{
    unsigned long long prefix = 0;          // the bytes fixed so far, in place
    float before = 0.f;                     // count or mass of candidates that rank above the current prefix
    bool found = true;
    bool listed = false;                    // this CTA's candidates that match the prefix are in sh->cand[0 .. n_list)
    int n_list = 0;
    for (int b = 7; b >= 0; b--) {
        if (b == 3) { prefix |= 0xFFull << 24; continue; }        // ids stay below 2^24: this byte is constant
        // Every warp has a histogram of its own (no two warps add to the same word) and every thread keeps the
        // four bins it met last in registers: the top bytes of the keys take few values, which all threads
        // would otherwise be adding to at once.  The warps' histograms are summed in warp order, the CTAs' in
        // rank order.
        float *mine = sh->whist + (threadIdx.x >> 5) * 256;
        for (int i = threadIdx.x; i < 256 * (int)(blockDim.x >> 5); i += blockDim.x) sh->whist[i] = 0.f;
        if (threadIdx.x == 0) sh->n_listed = 0;
        __syncthreads();
        int c_bin[4] = {-1, -1, -1, -1};
        float c_run[4] = {0.f, 0.f, 0.f, 0.f};
        int victim = 0;
        const unsigned long long hi_mask = b == 7 ? 0ull : (~0ull << (8 * (b + 1)));
        auto count_in = [&](unsigned long long k, float logit) {
            const int bin = (int)((k >> (8 * b)) & 0xFF);
            const float w = MODE == BY_COUNT ? 1.f : r.e_of(logit) / r.sum;
            if (bin == c_bin[0]) c_run[0] += w;
            else if (bin == c_bin[1]) c_run[1] += w;
            else if (bin == c_bin[2]) c_run[2] += w;
            else if (bin == c_bin[3]) c_run[3] += w;
            else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (j == victim) {
                        if (c_bin[j] >= 0) atomicAdd(&mine[c_bin[j]], c_run[j]);
                        c_bin[j] = bin;
                        c_run[j] = w;
                    }
                victim = (victim + 1) & 3;
            }
        };
        if (listed) {
            for (int i = threadIdx.x; i < n_list; i += blockDim.x) {
                const unsigned long long k = sh->cand[i];
                if ((k & hi_mask) == (prefix & hi_mask)) count_in(k, key_logit(k));
            }
        } else {
            const bool list_them = b < 7;
            scan_row(r, [&](int i, float logit) {
                const unsigned long long k = rank_key(logit, i);
                if (k < cut || (k & hi_mask) != (prefix & hi_mask)) return;
                if (list_them && *(volatile int *)&sh->n_listed <= SMALL_K) {       // (no more additions once it is full)
                    const int at = atomicAdd(&sh->n_listed, 1);
                    if (at < SMALL_K) sh->cand[at] = k;
                }
                count_in(k, logit);
            });
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (c_bin[j] >= 0) atomicAdd(&mine[c_bin[j]], c_run[j]);
        __syncthreads();
        if (!listed && b < 7 && sh->n_listed <= SMALL_K) { listed = true; n_list = sh->n_listed; }
        const unsigned t = turn++ & 1;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            float s = 0.f;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) s += sh->whist[w * 256 + i];
            sh->x_hist[t][i] = s;
        }
        cluster_sync_all();
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            float s = 0.f;
            for (int rk = 0; rk < SAMPLE_CLUSTER; rk++) s += ld_rank_f32(rank_addr(&sh->x_hist[t][i], rk));
            sh->hist[i] = s;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // The first warp walks the bins from the top: a lane has eight of them, the sums of the lanes before
            // it come from a scan, and the first lane that meets the target has the bin.
            const int lane = threadIdx.x;
            float h[8], tot = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) { h[j] = sh->hist[255 - 8 * lane - j]; tot += h[j]; }
            float inc = tot;
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            const float above = __shfl_up_sync(0xffffffffu, inc, 1);
            float acc = before + (lane ? above : 0.f), acc_at = 0.f;
            int pick = -1, lowest = -1;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (h[j] == 0.f) continue;
                lowest = 255 - 8 * lane - j;
                if (pick >= 0) continue;
                const bool hit = MODE == BY_MASS_GT ? (acc + h[j] > target) : (acc + h[j] >= target);
                if (hit) { pick = lowest; acc_at = acc; }
                else acc += h[j];
            }
            const unsigned hits = __ballot_sync(0xffffffffu, pick >= 0), filled = __ballot_sync(0xffffffffu, lowest >= 0);
            const float total = before + __shfl_sync(0xffffffffu, inc, 31);
            if (hits) {
                const int src = __ffs(hits) - 1;
                pick = __shfl_sync(0xffffffffu, pick, src);
                acc_at = __shfl_sync(0xffffffffu, acc_at, src);
            } else if (b < 7 && filled) {
                // Below the first byte the target is known to lie inside the chosen bucket; if re-summing its
                // mass in finer bins falls short by rounding, the bucket's last candidate is the one.
                pick = __shfl_sync(0xffffffffu, lowest, 31 - __clz(filled));
                acc_at = total - sh->hist[pick];
            }
            if (lane == 0) {
                sh->result[0] = pick < 0 ? ~0ull : (unsigned long long)pick;
                ((float *)(sh->result + 1))[0] = acc_at;
            }
        }
        __syncthreads();
        unsigned long long pick = sh->result[0];
        before = ((float *)(sh->result + 1))[0];
        __syncthreads();
        if (pick == ~0ull) { found = false; break; }
        prefix |= pick << (8 * b);
    }
    return found ? prefix : 0ull;
}

__device__ __forceinline__ int key_id(unsigned long long k) { return (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFu)); }

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float *logits, int V, const float *temps, const int32_t *top_ks, const float *top_ps,
              const float *min_ps, const float *uniforms, int32_t *out)
{
    pdl_sync();
    __shared__ Shared shared;
    Shared *sh = &shared;
    unsigned turn = 0;
    // Nobody leaves while another CTA may still be reading its shared memory.
    auto leave = [&]() { cluster_sync_all(); };

    const int row = blockIdx.x / SAMPLE_CLUSTER, rank = (int)cluster_rank();
    const int share = ((V + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER + 3) & ~3;
    Row r;
    r.l = logits + (size_t)row * V;
    r.V = V;
    r.lo = min(V, rank * share);
    r.hi = min(V, r.lo + share);
    r.temp = temps[row];
    r.sum = 1.f;
    int K = top_ks[row];
    float top_p = top_ps[row], min_p = min_ps[row], u = uniforms[row];

    // the maximum and, for greedy rows, its first index
    unsigned long long best = 0;
    scan_row(r, [&](int i, float logit) { best = max(best, rank_key(logit, i)); });
    best = cluster_key<true>(best, sh, turn);
    int best_id = key_id(best);
    if (r.temp <= 0.f) {
        if (threadIdx.x == 0 && rank == 0) out[row] = best_id;
        return leave();
    }
    r.lmax = r.l[best_id];

    // top-k: the cut is the key of the K-th candidate
    unsigned long long cut = 0;
    bool limited = K > 0 && K < V;
    if (limited) cut = descend<BY_COUNT>(r, 0, (float)K, sh, turn);

    if (limited && K <= SMALL_K) {
        // few candidates: the first CTA collects and sorts them and runs the reference's sequence on the sorted list
        unsigned long long *found = (unsigned long long *)sh->whist;
        if (threadIdx.x == 0) sh->n_cand = 0;
        __syncthreads();
        scan_row(r, [&](int i, float logit) {
            unsigned long long k = rank_key(logit, i);
            if (k >= cut) { int at = atomicAdd(&sh->n_cand, 1); if (at < SMALL_K) found[at] = k; }
        });
        cluster_sync_all();
        if (rank != 0) return leave();
        for (int i = threadIdx.x; i < SMALL_K; i += blockDim.x) sh->cand[i] = 0;
        __syncthreads();
        int at = 0;
        for (int rk = 0; rk < SAMPLE_CLUSTER; rk++) {
            const int n = min(ld_rank_s32(rank_addr(&sh->n_cand, rk)), SMALL_K);
            for (int i = threadIdx.x; i < n && at + i < SMALL_K; i += blockDim.x)
                sh->cand[at + i] = ld_rank_u64(rank_addr(&found[i], rk));
            at = min(at + n, SMALL_K);
        }
        __syncthreads();
        unsigned long long *cand = sh->cand;
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
        // exp of every candidate at once; the sums then run over them in the reference's order
        const int m = min(at, K);
        float *e = sh->whist;               // this CTA's own candidates have been copied out of it
        for (int i = threadIdx.x; i < m; i += blockDim.x) e[i] = r.e(key_id(cand[i]));
        __syncthreads();
        if (threadIdx.x == 0) {
            float sum = 0.f;
            for (int i = 0; i < m; i++) sum += e[i];
            sh->red[0] = sum;
        }
        __syncthreads();
        const float sum = sh->red[0];
        for (int i = threadIdx.x; i < m; i += blockDim.x) e[i] = e[i] / sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            auto prob = [&](int i) { return e[i]; };
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
            out[row] = key_id(cand[pick]);
        }
        return leave();
    }

    // many candidates: cuts by radix descent over probability mass
    float s = 0.f;
    scan_row(r, [&](int i, float logit) { if (rank_key(logit, i) >= cut) s += r.e_of(logit); });
    float sum1 = cluster_sum(s, sh, turn);
    r.sum = sum1;
    if (min_p > 0.f) {
        // p is monotone in the order, so the kept prefix is the set of candidates that pass the test
        float pmax = 1.0f / sum1;
        unsigned long long lowest = ~0ull;
        scan_row(r, [&](int i, float logit) {
            unsigned long long k = rank_key(logit, i);
            if (k >= cut && r.e_of(logit) / sum1 >= min_p * pmax) lowest = min(lowest, k);
        });
        lowest = cluster_key<false>(lowest, sh, turn);
        cut = max(cut, lowest == ~0ull ? best : lowest);
    }
    if (top_p > 0.f && top_p < 1.f) {
        unsigned long long c = descend<BY_MASS_GE>(r, cut, top_p, sh, turn);
        if (c) cut = c;
    }
    s = 0.f;
    scan_row(r, [&](int i, float logit) { if (rank_key(logit, i) >= cut) s += r.e_of(logit) / r.sum; });
    float kept_sum = cluster_sum(s, sh, turn);
    unsigned long long pick = descend<BY_MASS_GT>(r, cut, u * kept_sum, sh, turn);
    if (!pick) {
        // rounding left r at or above the total: the last kept candidate (src/sample.c:113)
        unsigned long long lowest = ~0ull;
        scan_row(r, [&](int i, float logit) {
            unsigned long long k = rank_key(logit, i);
            if (k >= cut) lowest = min(lowest, k);
        });
        pick = cluster_key<false>(lowest, sh, turn);
    }
    if (threadIdx.x == 0 && rank == 0) out[row] = key_id(pick);
    leave();
}

}  // namespace hfb

using namespace hfb;

extern "C" int hfb_sample(const float *logits, int M, int V, const float *temps, const int32_t *top_ks,
                          const float *top_ps, const float *min_ps, const float *uniforms, int32_t *out,
                          hfb_stream s)
{
    if (M <= 0) return HFB_OK;
    if (V <= 0 || V >= (1 << 24)) return fail(HFB_ENOTSUP, "sample: vocabulary of %d is not supported (1..2^24-1)", V);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M * SAMPLE_CLUSTER);
    cfg.blockDim = dim3(SAMPLE_THREADS);
    cfg.stream = (cudaStream_t)s;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = SAMPLE_CLUSTER;
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
    g_launch_err = cudaLaunchKernelEx(&cfg, sample_kernel, logits, V, temps, top_ks, top_ps, min_ps, uniforms, out);
    return check_pdl_launch(g_launch_err, "sample");
}
