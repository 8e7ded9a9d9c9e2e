// Pieces the mma.sync attention kernels share: the tile width, cp.async, ldmatrix and mma wrappers, the parameter
// block and the shared-memory swizzle of the cp.async tiles.
#pragma once
#include "common.cuh"

namespace hfb {

constexpr int ABN = 64;                 // keys per tile

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid)
{
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float *c, const uint32_t *a, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (relative error about 2^-22, far below bfloat16's own rounding)
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t *)&h;
}

struct AttnParams {
    const __nv_bfloat16 *q, *k_cache, *v_cache;
    __nv_bfloat16 *out;
    const int32_t *block_table, *positions, *tile_seq, *tile_t0, *tile_nt;
    float *part_o, *part_ml;            // split mode: [T*H, splits, D] and [T*H, splits, 2]
    int *counters;                      // decode kernel, split mode: one per (tile, key/value head), zero between
                                        // launches; the CTA that brings one to `splits` merges that tile (null: a
                                        // second kernel merges)
    int max_blocks, block_size, window, H, G, splits;
    long long num_pages;
    float scale_log2;                   // scale * log2(e)
};

// Byte offset of 16-byte chunk `c` of row `row` in a tile whose rows hold D bf16 (D = 64 or 128).
template <int D> __device__ __forceinline__ uint32_t swz(int row, int c)
{
    return (uint32_t)(row * (D * 2) + ((c ^ (row & 7)) << 4));
}

// Merges the key splits of every (token, head) in split order and writes the bfloat16 result (splits > 1 only).
int launch_attention_combine(const AttnParams &p, int T, int d, cudaStream_t st);

}  // namespace hfb
