/*
 * CPU oracle for yaxus's paged attention path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain C++ restatement of the reference CPU backend's attention
 * (crates/yaxus-backend-cpu/src/lib.rs) and of the page-slot arithmetic of
 * crates/yaxus-model/src/kv.rs.  It exists to check the CUDA library and to give a
 * CPU timing; the shipped library never links, loads or calls it.
 *
 * Pinning: the reference holds no stored numeric vectors for attention.  The oracle is
 * pinned by restating the reference's own known-answer test
 * `paged_attention_matches_dense_attention` (crates/yaxus-backend-cpu/src/lib.rs:676-714)
 * with the same PRNG, shapes, page tables and tolerance (yxref_selftest), and by the
 * committed fixtures under tests/golden/.  The reference's Rust code cannot be compiled
 * where this was written (no rustc), so beyond that known-answer test parity is unpinned
 * by reference-produced data.
 *
 * Arithmetic rules kept from the reference: 16-lane partial sums in the dot product,
 * sequential f32 sums everywhere else, two passes over the keys in the softmax, one page
 * table lookup per key, no fused multiply-add (build with -ffp-contract=off).
 */
#ifndef YX_REF_H
#define YX_REF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Tokens per KV page (crates/yaxus-model/src/kv.rs:17). */
#define YXREF_PAGE 128

/* Arena slot of position `pos` under page table `pages` (kv.rs:20-22). */
uint64_t yxref_slot(const uint32_t *pages, uint64_t pos);

/* 16-lane dot product (crates/yaxus-backend-cpu/src/lib.rs:280-294). */
float yxref_dot(const float *a, const float *b, size_t n);

/* out = (offset + w) * (x * rsqrt(mean(x^2) + eps))  (cpu lib.rs:296-302). */
void yxref_rmsnorm_row(const float *x, const float *w, float offset, float eps, float *out, size_t n);

/* Half-split rotation in place (cpu lib.rs:304-311). */
void yxref_rope_inplace(float *x, const float *cos_, const float *sin_, size_t n);

/* cos/sin of one position, dim/2 long each, scaled by `concentration`
 * (crates/yaxus-model/src/config.rs:213-219): f32 angle, f64 cos/sin, f32 result. */
void yxref_cos_sin(const float *inv_freq, size_t half, float concentration, uint64_t pos,
                   float *cos_, float *sin_);

/* RoPE inverse frequencies without scaling (config.rs:185-188): 1 / theta^(i/dim), f32. */
void yxref_rope_default(size_t dim, double theta, float *inv_freq);

/* Round-to-nearest-even storage conversions.  bf16 as crates/yaxus-model/src/weights.rs:100-111. */
uint16_t yxref_f32_to_bf16(float x);
float yxref_bf16_to_f32(uint16_t x);
uint16_t yxref_f32_to_f16(float x);
float yxref_f16_to_f32(uint16_t x);
/* dtype: 0 = f32 (copy), 1 = f16, 2 = bf16.  Rounds to the storage type and widens back. */
void yxref_round_through(const float *x, float *out, size_t n, int dtype);

/*
 * write_rows (cpu lib.rs:359-385): normalise + rotate q and k of every row, write k and v
 * to the row's slot of the arenas K,V `[slots][hkv*d]`, return q `[T][hq*d]`.
 * qkv is `[T][(hq+2hkv)*d]`.  `store_dtype` != 0 additionally rounds the stored k and v
 * through that storage type (the extension used for f16/bf16 caches).
 */
void yxref_write_rows(const float *qkv, size_t T, const uint32_t *pos, const uint32_t *kv_slot,
                      const float *q_norm, const float *k_norm, size_t hq, size_t hkv, size_t d,
                      float eps, const float *inv_freq, float concentration, int store_dtype,
                      float *K, float *V, float *q_out);

/* Plain append: k_rows,v_rows `[T][hkv*d]` copied to the rows' slots (the tail of write_rows). */
void yxref_append_rows(const float *k_rows, const float *v_rows, size_t T, const uint32_t *kv_slot,
                       size_t kvd, float *K, float *V);

/*
 * attend (cpu lib.rs:389-427).  q `[T][hq*d]`, out `[T][hq*d]`.  window < 0 means none.
 * Parallel over (row, head) like the reference's par_chunks_mut(d); threads <= 0 uses
 * the OpenMP default.
 */
void yxref_attend(const float *q, size_t T, const uint32_t *pos, const uint32_t *pt_off,
                  const uint32_t *pages, size_t hq, size_t hkv, size_t d, int64_t window,
                  const float *K, const float *V, float *out, int threads);

/*
 * The same attention restricted to keys in [key_lo, key_hi): the (m, l, o) triple of
 * split-key attention (crates/yaxus-backend-gpu/src/shaders.rs:1466-1579).  o is NOT
 * normalised; a (row, head) with no live key gets (m, l) = (-1e30, 0) and o untouched.
 * m,l `[T][hq]`, o `[T][hq][d]`.
 */
void yxref_attend_partial(const float *q, size_t T, const uint32_t *pos, const uint32_t *pt_off,
                          const uint32_t *pages, size_t hq, size_t hkv, size_t d, int64_t window,
                          uint64_t key_lo, uint64_t key_hi, const float *K, const float *V,
                          float *m, float *l, float *o, int threads);

/*
 * Merge of `n_parts` partial triples per (row, head) (shaders.rs:1581-1637): running
 * maximum, parts with l <= 0 dropped by value.  m,l `[n_parts][n]`, o `[n_parts][n][d]`,
 * out `[n][d]`, n = T*hq.
 */
void yxref_combine(const float *m, const float *l, const float *o, size_t n_parts, size_t n,
                   size_t d, float *out);

/* copy_page for one layer's K and V (cpu lib.rs:472-479). */
void yxref_copy_page(float *K, float *V, size_t kvd, uint32_t src, uint32_t dst);

/* ---- the other Backend operators (the model's path either side of attention) ---- */

/* dot_bf16 (cpu lib.rs:234-249): bf16 weights times f32 activations, 16 lanes, then the tail. */
float yxref_dot_bf16(const uint16_t *w, const float *x, size_t n);

/* matmul (cpu lib.rs:314-357): out [T][N] = x [T][K] . w[N][K]^T.  Below four rows the reference
 * takes dot_bf16 per output, from four rows on it widens the weight row to f32 and takes `dot`:
 * the same products summed in the same order, so one routine restates both. */
void yxref_matmul_bf16(const float *x, const uint16_t *w, size_t T, size_t N, size_t K, float *out, int threads);

/* swiglu (cpu lib.rs:532-542): [T][2I] -> [T][I], g / (1 + exp(-g)) * u. */
void yxref_swiglu(const float *x, size_t T, size_t inner, float *out);

/* embed (cpu lib.rs:485-497): out[r] = f32(table[ids[r]]), table bf16 [V][H]. */
void yxref_embed(const uint16_t *table, size_t h, const uint32_t *ids, size_t T, float *out);

/* rmsnorm over rows (cpu lib.rs:499-507). */
void yxref_rmsnorm(const float *x, const float *w, size_t T, size_t cols, float offset, float eps, float *out);

/* add_norm (crates/yaxus-model/src/lib.rs:149-162): x += rmsnorm(delta, post); out = rmsnorm(x, pre). */
void yxref_add_norm(float *x, const float *delta, const float *post_w, float post_offset, const float *pre_w,
                    float pre_offset, float eps, size_t T, size_t cols, float *out);

/* argmax (cpu lib.rs:430-441): first maximum, NaNs skipped, 0 when the row holds no number. */
uint32_t yxref_argmax(const float *row, size_t n);

/* The reference test's value generator (cpu lib.rs:572-582): xorshift64 in [-1, 1). */
void yxref_values(float *out, size_t n, uint64_t seed);

/*
 * The reference's known-answer test restated (cpu lib.rs:676-714).  Returns the largest
 * |paged - dense| over both window settings, or a negative number on a set-up error.
 * The reference accepts < 1e-5.
 */
double yxref_selftest(void);

int yxref_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
