/* hfb200.h - C entry points of the CUDA library (sm_100a).
 *
 * Every function takes device pointers, sizes and the CUDA stream to launch on, returns HFB_OK or
 * an error code, and allocates nothing unless its comment says so.  `hfb_last_error()` gives the
 * message of the last failure on the calling thread.  Element types are passed as HFB_F32 /
 * HFB_BF16 codes.  Matrices are row-major with the inner dimension contiguous: activations
 * [rows, features], weights [out, in] (the reference's layout, src/model.h:14-21).
 */
#ifndef HFB200_H
#define HFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { HFB_F32 = 0, HFB_BF16 = 1 };

/* status codes, named after the reference's (src/hfc.h:12-22) */
enum { HFB_OK = 0, HFB_EINVAL = 1, HFB_ENOTSUP = 2, HFB_ECUDA = 3, HFB_ERANGE = 4, HFB_EIO = 5 };

typedef void *hfb_stream;     /* a cudaStream_t */

const char *hfb_last_error(void);
int hfb_version(void);

/* x[t, :] = table[ids[t], :] as float32.  ids outside [0, V) raise the device error word. */
int hfb_embed(const int32_t *ids, const void *table, int table_dt, float *out, int T, int V, int E, hfb_stream s);

/* out[m, :] = x[rows ? rows[m] : m, :] * rsqrt(mean(x^2) + eps) * w, sums in float32. */
int hfb_rmsnorm(const float *x, const void *w, int w_dt, float eps, void *out, int out_dt,
                const int32_t *rows, int M, int E, hfb_stream s);

/* out[M,N] (=|+=) a[M,K] . w[N,K]^T (+ bias[N]); plain float32-accumulating kernel for any sizes and
 * any mix of element types.  accumulate != 0 requires a float32 `out`. */
int hfb_linear_plain(const void *a, int a_dt, const void *w, int w_dt, const void *bias, int bias_dt,
                     void *out, int out_dt, int accumulate, int M, int N, int K, hfb_stream s);

/* The same product for bfloat16 a and w on the tensor cores (tcgen05, TMA, TMEM).  K must be a multiple of 8
 * and the operands 16-byte aligned, else HFB_ENOTSUP.  Where there are fewer output tiles than SMs (few rows; or a
 * few hundred rows, few output features and a long K) the kernel may split K over more CTAs and sum float32
 * partials kept in `workspace`; hfb_linear_tc_workspace gives the bytes that takes (0 = none); with a smaller or
 * null workspace it runs unsplit.  The kernels are launched so that they may start while the kernel in front of them
 * on the stream still runs (programmatic dependent launch), and they read `w`, the weights, before they wait for
 * that kernel: `w` must be complete before the kernel in front is launched (weights are; an operand that the
 * kernel in front computes belongs in `a`).  HFB_PDL=0 in the environment turns the early start off. */
size_t hfb_linear_tc_workspace(int M, int N, int K);
int hfb_linear_tc(const void *a, const void *w, const void *bias, int bias_dt, void *out, int out_dt,
                  int accumulate, int M, int N, int K, void *workspace, size_t workspace_bytes, hfb_stream s);

/* The product with a SwiGLU epilogue: w holds gate row i at 2i and up row i at 2i+1; out[M, N/2]. */
int hfb_linear_tc_swiglu(const void *a, const void *w, void *out, int out_dt, int M, int N, int K, hfb_stream s);

/* q|k|v of 256 tokens and more with the rest of the step in the product's epilogue: bias, rounding to bfloat16,
 * rotation of the query and key heads by cos_sin [n_positions, d / 2, 2] at the tokens' positions, queries to q_out
 * [M, H d], keys and values to cache slot slots[t] (null: nothing is cached).  bfloat16 throughout, head sizes 64 and
 * 128, the whole head rotated.  HFB_ENOTSUP, with nothing launched, for other sizes. */
int hfb_linear_tc_rope_kv(const void *a, const void *w, const void *bias, const float *cos_sin, int n_positions,
                          const int32_t *positions, const int32_t *slots, void *q_out, void *k_cache, void *v_cache,
                          int64_t cache_slots, int M, int K, int H, int G, int d, hfb_stream s);

/* Only the split-K partial sums partial[*splits, M, N] (float32) of a product, for a fused reduction to finish;
 * `workspace` must hold hfb_linear_tc_partials_workspace bytes.  Above 128 rows that size is 0 for a product that
 * would not be split, and this entry refuses it (HFB_ENOTSUP). */
size_t hfb_linear_tc_partials_workspace(int M, int N, int K);
int hfb_linear_tc_partials(const void *a, const void *w, int M, int N, int K, void *workspace, size_t workspace_bytes,
                           int *splits, hfb_stream s);

/* residual[M,N] += sum_s partial[s] (+ bias); if xn: xn = rmsnorm(residual) * w (the next product's input). */
int hfb_reduce_residual_norm(const float *partial, int splits, int M, int N, const void *bias, int bias_dt,
                             float *residual, const void *w, int w_dt, float eps, void *xn, int xn_dt, hfb_stream s);

/* hfb_rope_kv_write reading sum_s partial[s] + bias instead of a finished q|k|v row. */
int hfb_reduce_rope_kv(const float *partial, int splits, int dt, const void *bias, int bias_dt, const float *cos_sin,
                       int n_rot, int n_positions, const int32_t *positions, const int32_t *slots, void *q_out,
                       void *k_cache, void *v_cache, int64_t cache_slots, int T, int H, int G, int d, hfb_stream s);

/* arg-max with many blocks per row (two passes; scratch of hfb_argmax2_scratch bytes). */
size_t hfb_argmax2_scratch(int M, int V);
int hfb_argmax2(const float *logits, int32_t *out, int M, int V, void *scratch, size_t scratch_bytes, hfb_stream s);

/* Splits qkv[T, (H+2G)*d] into rotated queries q_out[T, H*d], rotated keys and plain values written
 * to the paged cache at slots[t] (page * block_size + offset; < 0 or slots == NULL: not written).
 * cos_sin is float32 [positions, n_rot/2, 2]; n_rot == 0 means no rotation. */
int hfb_rope_kv_write(const void *qkv, int dt, const float *cos_sin, int n_rot, int n_positions,
                      const int32_t *positions, const int32_t *slots, void *q_out, void *k_cache, void *v_cache,
                      int64_t cache_slots, int T, int H, int G, int d, hfb_stream s);

/* Attention of every token over its request's cached keys lo..pos (lo = max(0, pos - window + 1) when
 * window > 0, else 0), plain kernel: one block per (token, head), float32 softmax. */
int hfb_attention_plain(const void *q, const void *k_cache, const void *v_cache, int dt,
                        const int32_t *block_table, int max_blocks, const int32_t *token_seq,
                        const int32_t *positions, int block_size, int64_t num_pages, int window, float scale,
                        void *out, int T, int H, int G, int d, hfb_stream s);

/* The same for bfloat16 with head_dim 64 or 128 and a block size that divides 64, tiled, on tensor cores.
 * Tiles (tile_seq, tile_t0 = first token index, tile_nt = tokens) cover the step's tokens; a tile holds at
 * most hfb_attention_fast_tile_tokens(H, G, warps) tokens of one request.  warps = 4 for prompt portions and
 * mixed batches (splits must be 1), warps = 1 for decode, where `splits` > 1 cuts each request's keys into
 * that many ranges whose partial results are merged in order; they live in `scratch`
 * (stages = 4 with warps = 4 selects a deeper load pipeline for CTAs that have an SM to themselves)
 * (hfb_attention_fast_scratch bytes). */
int hfb_attention_fast_tile_tokens(int H, int G, int warps);
size_t hfb_attention_fast_scratch(int T, int H, int d, int splits);
int hfb_attention_fast(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                       int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                       const int32_t *tile_nt, int n_tiles, int warps, int stages, int splits, int block_size,
                       int64_t num_pages, int window, float scale, void *out, void *scratch, size_t scratch_bytes,
                       int T, int H, int G, int d, hfb_stream s);

/* Decode attention with the keys and values fetched by TMA: tiles as hfb_attention_fast's 16-row form takes them
 * (one or two tokens of one request), bfloat16, head_dim 64 or 128, block sizes 8..64 dividing 64.  `stages` (2..4)
 * tiles of 64 keys are in flight per CTA; `splits` > 1 needs hfb_attention_fast_scratch bytes of scratch, and is
 * merged by the CTA that stores a tile's last split when `counters` (n_tiles * G ints, zero before the first launch
 * and after every launch) is given, else by a second kernel. */
int hfb_attention_decode(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                         int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                         const int32_t *tile_nt, int n_tiles, int stages, int splits, int block_size, int64_t num_pages,
                         int window, float scale, void *out, void *scratch, size_t scratch_bytes, int T, int H, int G,
                         int d, int *counters, int counters_len, hfb_stream s);

/* Attention of prompt portions on tcgen05 (S and PV accumulators in TMEM, K and V gathered page by page with
 * TMA): bfloat16, head_dim 128, block sizes 8..128 that divide 128.  Tiles hold at most 128 / (H/G) tokens. */
int hfb_attention_tc(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                     int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                     const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window,
                     float scale, void *out, int T, int H, int G, int d, hfb_stream s);

/* The same with two 128-row tiles per CTA (tiles hold at most 2 * (128 / (H/G)) tokens): the softmax of one tile
 * runs while the tensor core works on the other; the running output stays in TMEM.  head_dim 64 or 128. */
int hfb_attention_tc2(const void *q, const void *k_cache, const void *v_cache, const int32_t *block_table,
                      int max_blocks, const int32_t *positions, const int32_t *tile_seq, const int32_t *tile_t0,
                      const int32_t *tile_nt, int n_tiles, int block_size, int64_t num_pages, int window, float scale,
                      void *out, int T, int H, int G, int d, hfb_stream s);

/* out[t, f] = silu(g) * u with g = gu[t, f], u = gu[t, F + f], or, interleaved, g = gu[t, 2f], u = gu[t, 2f + 1] */
int hfb_swiglu(const void *gu, void *out, int dt, int T, int F, int interleaved, hfb_stream s);

/* out[m] = index of the first maximum of logits[m, :] */
int hfb_argmax(const float *logits, int32_t *out, int M, int V, hfb_stream s);

/* One token per row: greedy where temps[m] <= 0, else temperature sampling with top-k (0 = off), min-p
 * (0 = off) and top-p (1 = off) in the reference's order of operations (src/sample.c:66-116);
 * uniforms[m] in [0, 1) is the row's draw. */
int hfb_sample(const float *logits, int M, int V, const float *temps, const int32_t *top_ks,
               const float *top_ps, const float *min_ps, const float *uniforms, int32_t *out, hfb_stream s);

/* Device error word: kernels set bits instead of touching memory out of range.  Reading syncs the stream. */
enum { HFB_ERR_TOKEN_ID = 1, HFB_ERR_PAGE = 2, HFB_ERR_SLOT = 4, HFB_ERR_WAIT = 8, HFB_ERR_POSITION = 16 };
int hfb_error_word_take(int32_t *word, hfb_stream s);
/* Queues a copy of the word into pinned host memory and returns; read it after your own wait on the stream. */
int hfb_error_word_peek_async(int32_t *host_word, hfb_stream s);

#ifdef __cplusplus
}
#endif
#endif
