// CPU oracle for yaxus's paged attention path.  TEST INFRASTRUCTURE ONLY: see yx_ref.h.
// Build: g++ -O2 -ffp-contract=off -fopenmp -shared -fPIC (no -ffast-math), so that every
// multiply and add rounds separately, as the reference's Rust code does.
#include "yx_ref.h"

#include <math.h>
#include <string.h>

#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {
constexpr size_t PAGE = YXREF_PAGE;

// PassMeta::slot (crates/yaxus-model/src/lib.rs:79-89): the row's page table starts at
// pt_off[row] inside the concatenated `pages`.
inline size_t row_slot(const uint32_t *pages, const uint32_t *pt_off, size_t row, size_t pos) {
    return (size_t)yxref_slot(pages + pt_off[row], pos);
}

inline size_t window_lo(size_t p, int64_t window) {
    // cpu lib.rs:402-405: (p + 1).saturating_sub(w)
    if (window < 0) return 0;
    size_t w = (size_t)window;
    return p + 1 > w ? p + 1 - w : 0;
}
}  // namespace

extern "C" {

uint64_t yxref_slot(const uint32_t *pages, uint64_t pos) {
    return (uint64_t)pages[pos / PAGE] * PAGE + pos % PAGE;
}

float yxref_dot(const float *a, const float *b, size_t n) {
    float acc[16];
    for (int i = 0; i < 16; i++) acc[i] = 0.0f;
    size_t full = n / 16 * 16;
    for (size_t c = 0; c < full; c += 16)
        for (int i = 0; i < 16; i++) acc[i] += a[c + i] * b[c + i];
    float s = 0.0f;
    for (int i = 0; i < 16; i++) s += acc[i];
    for (size_t i = full; i < n; i++) s += a[i] * b[i];
    return s;
}

void yxref_rmsnorm_row(const float *x, const float *w, float offset, float eps, float *out, size_t n) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) ss += x[i] * x[i];
    float ms = ss / (float)n;
    float r = 1.0f / sqrtf(ms + eps);
    for (size_t i = 0; i < n; i++) out[i] = (offset + w[i]) * (x[i] * r);
}

void yxref_rope_inplace(float *x, const float *cos_, const float *sin_, size_t n) {
    size_t half = n / 2;
    for (size_t j = 0; j < half; j++) {
        float a = x[j], b = x[j + half];
        x[j] = a * cos_[j] - b * sin_[j];
        x[j + half] = b * cos_[j] + a * sin_[j];
    }
}

void yxref_cos_sin(const float *inv_freq, size_t half, float concentration, uint64_t pos,
                   float *cos_, float *sin_) {
    for (size_t j = 0; j < half; j++) {
        float a = (float)pos * inv_freq[j];
        cos_[j] = (float)cos((double)a) * concentration;
        sin_[j] = (float)sin((double)a) * concentration;
    }
}

void yxref_rope_default(size_t dim, double theta, float *inv_freq) {
    size_t j = 0;
    for (size_t i = 0; i < dim; i += 2, j++) {
        float f = powf((float)theta, (float)i / (float)dim);
        inv_freq[j] = 1.0f / f;
    }
}

uint16_t yxref_f32_to_bf16(float x) {
    uint32_t b;
    memcpy(&b, &x, 4);
    if (x != x) return (uint16_t)((b >> 16) | 0x40);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}

float yxref_bf16_to_f32(uint16_t x) {
    uint32_t b = (uint32_t)x << 16;
    float f;
    memcpy(&f, &b, 4);
    return f;
}

// IEEE binary16, round to nearest even, overflow to infinity, subnormals kept.
uint16_t yxref_f32_to_f16(float x) {
    uint32_t b;
    memcpy(&b, &x, 4);
    uint32_t sign = (b >> 16) & 0x8000u;
    uint32_t mag = b & 0x7fffffffu;
    if (mag >= 0x7f800000u) {  // inf or NaN
        return (uint16_t)(sign | 0x7c00u | (mag > 0x7f800000u ? 0x0200u | ((mag >> 13) & 0x3ffu) : 0u));
    }
    if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to >= 65520 -> inf
    if (mag < 0x33000001u) return (uint16_t)sign;               // below half the smallest subnormal
    int32_t e = (int32_t)(mag >> 23) - 127;
    uint32_t man = (mag & 0x7fffffu) | 0x800000u;
    uint32_t shift, half_exp;
    if (e < -14) {  // subnormal half: value = man * 2^(e-23), unit 2^-24
        shift = (uint32_t)(13 + (-14 - e));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    // For normals q carries the implicit bit (0x400): adding it to (exp-1)<<10 lets a
    // mantissa carry ripple into the exponent.
    uint32_t out = half_exp ? ((half_exp - 1) << 10) + q : q;
    return (uint16_t)(sign | out);
}

float yxref_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t b;
    if (e == 0) {
        if (man == 0) {
            b = sign;
        } else {
            int sh = 0;
            while (!(man & 0x400u)) {
                man <<= 1;
                sh++;
            }
            man &= 0x3ffu;
            b = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | (man << 13);
        }
    } else if (e == 31) {
        b = sign | 0x7f800000u | (man << 13);
    } else {
        b = sign | ((e + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &b, 4);
    return f;
}

void yxref_round_through(const float *x, float *out, size_t n, int dtype) {
    for (size_t i = 0; i < n; i++) {
        if (dtype == 1)
            out[i] = yxref_f16_to_f32(yxref_f32_to_f16(x[i]));
        else if (dtype == 2)
            out[i] = yxref_bf16_to_f32(yxref_f32_to_bf16(x[i]));
        else
            out[i] = x[i];
    }
}

void yxref_write_rows(const float *qkv, size_t T, const uint32_t *pos, const uint32_t *kv_slot,
                      const float *q_norm, const float *k_norm, size_t hq, size_t hkv, size_t d,
                      float eps, const float *inv_freq, float concentration, int store_dtype,
                      float *K, float *V, float *q_out) {
    size_t qd = hq * d, kvd = hkv * d, cols = qd + 2 * kvd;
    std::vector<float> cs(d / 2), sn(d / 2);
    for (size_t i = 0; i < T; i++) {
        const float *row = qkv + i * cols;
        yxref_cos_sin(inv_freq, d / 2, concentration, pos[i], cs.data(), sn.data());
        for (size_t h = 0; h < hq; h++) {
            float *dst = q_out + i * qd + h * d;
            yxref_rmsnorm_row(row + h * d, q_norm, 1.0f, eps, dst, d);
            yxref_rope_inplace(dst, cs.data(), sn.data(), d);
        }
        size_t slot = kv_slot[i];
        for (size_t h = 0; h < hkv; h++) {
            float *kd = K + slot * kvd + h * d;
            yxref_rmsnorm_row(row + qd + h * d, k_norm, 1.0f, eps, kd, d);
            yxref_rope_inplace(kd, cs.data(), sn.data(), d);
            float *vd = V + slot * kvd + h * d;
            memcpy(vd, row + qd + kvd + h * d, d * sizeof(float));
            if (store_dtype) {
                yxref_round_through(kd, kd, d, store_dtype);
                yxref_round_through(vd, vd, d, store_dtype);
            }
        }
    }
}

void yxref_append_rows(const float *k_rows, const float *v_rows, size_t T, const uint32_t *kv_slot,
                       size_t kvd, float *K, float *V) {
    for (size_t i = 0; i < T; i++) {
        memcpy(K + (size_t)kv_slot[i] * kvd, k_rows + i * kvd, kvd * sizeof(float));
        memcpy(V + (size_t)kv_slot[i] * kvd, v_rows + i * kvd, kvd * sizeof(float));
    }
}

void yxref_attend(const float *q, size_t T, const uint32_t *pos, const uint32_t *pt_off,
                  const uint32_t *pages, size_t hq, size_t hkv, size_t d, int64_t window,
                  const float *K, const float *V, float *out, int threads) {
    size_t qd = hq * d, kvd = hkv * d, group = hq / hkv;
    float scale = 1.0f / sqrtf((float)d);
    long n_tasks = (long)(T * hq);
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
#endif
    for (long idx = 0; idx < n_tasks; idx++) {
        size_t i = (size_t)idx / hq, h = (size_t)idx % hq, kh = h / group;
        size_t p = pos[i];
        size_t lo = window_lo(p, window);
        const float *qv = q + i * qd + h * d;
        float *o = out + i * qd + h * d;
        for (size_t j = 0; j < d; j++) o[j] = 0.0f;
        std::vector<float> scores(p - lo + 1);
        for (size_t s = lo; s <= p; s++) {
            size_t off = row_slot(pages, pt_off, i, s) * kvd + kh * d;
            scores[s - lo] = yxref_dot(qv, K + off, d) * scale;
        }
        float m = -INFINITY;
        for (float sc : scores) m = fmaxf(m, sc);
        float denom = 0.0f;
        for (size_t s = lo; s <= p; s++) {
            float e = expf(scores[s - lo] - m);
            denom += e;
            const float *vv = V + row_slot(pages, pt_off, i, s) * kvd + kh * d;
            for (size_t j = 0; j < d; j++) o[j] += e * vv[j];
        }
        for (size_t j = 0; j < d; j++) o[j] /= denom;
    }
    (void)threads;
}

void yxref_attend_partial(const float *q, size_t T, const uint32_t *pos, const uint32_t *pt_off,
                          const uint32_t *pages, size_t hq, size_t hkv, size_t d, int64_t window,
                          uint64_t key_lo, uint64_t key_hi, const float *K, const float *V,
                          float *m_out, float *l_out, float *o_out, int threads) {
    size_t qd = hq * d, kvd = hkv * d, group = hq / hkv;
    float scale = 1.0f / sqrtf((float)d);
    long n_tasks = (long)(T * hq);
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt)
#endif
    for (long idx = 0; idx < n_tasks; idx++) {
        size_t i = (size_t)idx / hq, h = (size_t)idx % hq, kh = h / group;
        size_t p = pos[i];
        size_t lo = window_lo(p, window);
        size_t a = lo > key_lo ? lo : (size_t)key_lo;
        size_t b = p + 1 < key_hi ? p + 1 : (size_t)key_hi;  // exclusive
        if (a >= b) {
            m_out[idx] = -1e30f;
            l_out[idx] = 0.0f;
            continue;
        }
        const float *qv = q + i * qd + h * d;
        float *o = o_out + (size_t)idx * d;
        for (size_t j = 0; j < d; j++) o[j] = 0.0f;
        std::vector<float> scores(b - a);
        for (size_t s = a; s < b; s++) {
            size_t off = row_slot(pages, pt_off, i, s) * kvd + kh * d;
            scores[s - a] = yxref_dot(qv, K + off, d) * scale;
        }
        float m = -INFINITY;
        for (float sc : scores) m = fmaxf(m, sc);
        float denom = 0.0f;
        for (size_t s = a; s < b; s++) {
            float e = expf(scores[s - a] - m);
            denom += e;
            const float *vv = V + row_slot(pages, pt_off, i, s) * kvd + kh * d;
            for (size_t j = 0; j < d; j++) o[j] += e * vv[j];
        }
        m_out[idx] = m;
        l_out[idx] = denom;
    }
    (void)threads;
}

void yxref_combine(const float *m, const float *l, const float *o, size_t n_parts, size_t n,
                   size_t d, float *out) {
    for (size_t i = 0; i < n; i++) {
        float mx = -1e30f, ls = 0.0f;
        std::vector<float> acc(d, 0.0f);
        for (size_t c = 0; c < n_parts; c++) {
            float em = m[c * n + i], el = l[c * n + i];
            float nm = fmaxf(mx, em);
            float r = expf(mx - nm);
            bool live = el > 0.0f;
            float w = live ? expf(em - nm) : 0.0f;
            ls = ls * r + el * w;
            const float *po = o + (c * n + i) * d;
            for (size_t j = 0; j < d; j++) acc[j] = acc[j] * r + (live ? po[j] * w : 0.0f);
            mx = nm;
        }
        for (size_t j = 0; j < d; j++) out[i * d + j] = acc[j] / ls;
    }
}

void yxref_copy_page(float *K, float *V, size_t kvd, uint32_t src, uint32_t dst) {
    size_t n = PAGE * kvd;
    memmove(K + (size_t)dst * n, K + (size_t)src * n, n * sizeof(float));
    memmove(V + (size_t)dst * n, V + (size_t)src * n, n * sizeof(float));
}

float yxref_dot_bf16(const uint16_t *w, const float *x, size_t n) {
    float acc[16];
    for (int i = 0; i < 16; i++) acc[i] = 0.0f;
    size_t full = n / 16 * 16;
    for (size_t c = 0; c < full; c += 16)
        for (int i = 0; i < 16; i++) acc[i] += yxref_bf16_to_f32(w[c + i]) * x[c + i];
    float s = 0.0f;
    for (int i = 0; i < 16; i++) s += acc[i];
    for (size_t i = full; i < n; i++) s += yxref_bf16_to_f32(w[i]) * x[i];
    return s;
}

void yxref_matmul_bf16(const float *x, const uint16_t *w, size_t T, size_t N, size_t K, float *out, int threads) {
    // One task per weight row, as the reference's par_chunks_mut over the transposed result.
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#pragma omp parallel for schedule(static) num_threads(nt)
#endif
    for (long j = 0; j < (long)N; j++)
        for (size_t i = 0; i < T; i++) out[i * N + (size_t)j] = yxref_dot_bf16(w + (size_t)j * K, x + i * K, K);
    (void)threads;
}

void yxref_swiglu(const float *x, size_t T, size_t inner, float *out) {
    for (size_t r = 0; r < T; r++)
        for (size_t j = 0; j < inner; j++) {
            float g = x[r * 2 * inner + j];
            out[r * inner + j] = g / (1.0f + expf(-g)) * x[r * 2 * inner + inner + j];
        }
}

void yxref_embed(const uint16_t *table, size_t h, const uint32_t *ids, size_t T, float *out) {
    for (size_t r = 0; r < T; r++)
        for (size_t c = 0; c < h; c++) out[r * h + c] = yxref_bf16_to_f32(table[(size_t)ids[r] * h + c]);
}

void yxref_rmsnorm(const float *x, const float *w, size_t T, size_t cols, float offset, float eps, float *out) {
    for (size_t r = 0; r < T; r++) yxref_rmsnorm_row(x + r * cols, w, offset, eps, out + r * cols, cols);
}

void yxref_add_norm(float *x, const float *delta, const float *post_w, float post_offset, const float *pre_w,
                    float pre_offset, float eps, size_t T, size_t cols, float *out) {
    std::vector<float> d(cols);
    for (size_t r = 0; r < T; r++) {
        yxref_rmsnorm_row(delta + r * cols, post_w, post_offset, eps, d.data(), cols);
        for (size_t c = 0; c < cols; c++) x[r * cols + c] += d[c];
        yxref_rmsnorm_row(x + r * cols, pre_w, pre_offset, eps, out + r * cols, cols);
    }
}

uint32_t yxref_argmax(const float *row, size_t n) {
    size_t best = 0;
    float best_v = -INFINITY;
    for (size_t i = 0; i < n; i++)
        if (row[i] > best_v) {
            best = i;
            best_v = row[i];
        }
    return (uint32_t)best;
}

void yxref_values(float *out, size_t n, uint64_t seed) {
    uint64_t s = (seed * 0x9e3779b97f4a7c15ull) | 1ull;
    for (size_t i = 0; i < n; i++) {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        out[i] = (float)(s >> 40) / (float)(1ull << 23) - 1.0f;
    }
}

int yxref_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// The reference's known-answer test, restated (cpu lib.rs:596-714).
// ---------------------------------------------------------------------------------------
namespace {

// Dense attention of one sequence's rows at positions 0..n (the test's `naive`, :596-641).
std::vector<std::vector<float>> dense(const std::vector<std::vector<float>> &qkv, size_t hq, size_t hkv,
                                      size_t d, float eps, int64_t window, const float *inv_freq,
                                      float conc) {
    size_t qd = hq * d, kvd = hkv * d;
    std::vector<float> zero_w(d, 0.0f), cs(d / 2), sn(d / 2);
    std::vector<std::vector<float>> qs, ks, vs;
    for (size_t p = 0; p < qkv.size(); p++) {
        const std::vector<float> &row = qkv[p];
        yxref_cos_sin(inv_freq, d / 2, conc, p, cs.data(), sn.data());
        std::vector<float> q(qd), k(kvd);
        for (size_t h = 0; h < hq; h++) {
            yxref_rmsnorm_row(&row[h * d], zero_w.data(), 1.0f, eps, &q[h * d], d);
            yxref_rope_inplace(&q[h * d], cs.data(), sn.data(), d);
        }
        for (size_t h = 0; h < hkv; h++) {
            yxref_rmsnorm_row(&row[qd + h * d], zero_w.data(), 1.0f, eps, &k[h * d], d);
            yxref_rope_inplace(&k[h * d], cs.data(), sn.data(), d);
        }
        qs.push_back(q);
        ks.push_back(k);
        vs.emplace_back(row.begin() + qd + kvd, row.end());
    }
    float scale = 1.0f / sqrtf((float)d);
    std::vector<std::vector<float>> outs;
    for (size_t p = 0; p < qkv.size(); p++) {
        size_t lo = window_lo(p, window);
        std::vector<float> out(qd, 0.0f);
        for (size_t h = 0; h < hq; h++) {
            size_t kh = h / (hq / hkv);
            std::vector<float> sc;
            for (size_t s = lo; s <= p; s++) sc.push_back(yxref_dot(&qs[p][h * d], &ks[s][kh * d], d) * scale);
            float m = -INFINITY;
            for (float x : sc) m = fmaxf(m, x);
            std::vector<float> w;
            for (float x : sc) w.push_back(expf(x - m));
            float z = 0.0f;
            for (float x : w) z += x;
            for (size_t s = lo; s <= p; s++)
                for (size_t j = 0; j < d; j++) out[h * d + j] += w[s - lo] / z * vs[s][kh * d + j];
        }
        outs.push_back(out);
    }
    return outs;
}

}  // namespace

extern "C" double yxref_selftest(void) {
    const size_t hq = 4, hkv = 2, d = 8, cols = (hq + 2 * hkv) * d, kvd = hkv * d, qd = hq * d;
    const float eps = 1e-6f;
    const float inv_freq[4] = {1.0f, 0.3f, 0.05f, 0.01f};
    const float conc = 1.1f;
    const std::vector<std::vector<uint32_t>> pages = {{3, 1}, {0}};
    const size_t lens[2] = {140, 9};
    double worst = 0.0;
    const int64_t windows[2] = {-1, 16};
    for (int64_t window : windows) {
        std::vector<float> K(4 * PAGE * kvd, 0.0f), V(4 * PAGE * kvd, 0.0f);
        std::vector<std::vector<std::vector<float>>> qkv(2), want(2), got(2);
        for (size_t s = 0; s < 2; s++) {
            for (size_t p = 0; p < lens[s]; p++) {
                std::vector<float> row(cols);
                yxref_values(row.data(), cols, (uint64_t)(s * 1000 + p));
                qkv[s].push_back(row);
            }
            want[s] = dense(qkv[s], hq, hkv, d, eps, window, inv_freq, conc);
            got[s].assign(lens[s], std::vector<float>());
        }
        // Two passes: 100 rows of sequence 0 and 4 of sequence 1, then the rest.
        std::vector<std::vector<std::pair<size_t, size_t>>> passes(2);
        for (size_t p = 0; p < 100; p++) passes[0].push_back({0, p});
        for (size_t p = 0; p < 4; p++) passes[0].push_back({1, p});
        for (size_t p = 100; p < 140; p++) passes[1].push_back({0, p});
        for (size_t p = 4; p < 9; p++) passes[1].push_back({1, p});
        std::vector<float> zero_w(d, 0.0f);
        for (const auto &rows : passes) {
            std::vector<uint32_t> pos, slot, pt_off, pt;
            std::vector<int64_t> off(2, -1);
            std::vector<float> x;
            for (auto [sq, p] : rows) {
                if (off[sq] < 0) {
                    off[sq] = (int64_t)pt.size();
                    pt.insert(pt.end(), pages[sq].begin(), pages[sq].end());
                }
                pos.push_back((uint32_t)p);
                slot.push_back((uint32_t)yxref_slot(pages[sq].data(), p));
                pt_off.push_back((uint32_t)off[sq]);
                x.insert(x.end(), qkv[sq][p].begin(), qkv[sq][p].end());
            }
            size_t T = rows.size();
            std::vector<float> q(T * qd), out(T * qd);
            yxref_write_rows(x.data(), T, pos.data(), slot.data(), zero_w.data(), zero_w.data(), hq, hkv, d,
                             eps, inv_freq, conc, 0, K.data(), V.data(), q.data());
            yxref_attend(q.data(), T, pos.data(), pt_off.data(), pt.data(), hq, hkv, d, window, K.data(),
                         V.data(), out.data(), 1);
            for (size_t r = 0; r < T; r++)
                got[rows[r].first][rows[r].second].assign(out.begin() + r * qd, out.begin() + (r + 1) * qd);
        }
        for (size_t s = 0; s < 2; s++)
            for (size_t p = 0; p < lens[s]; p++) {
                if (got[s][p].size() != qd) return -1.0;
                for (size_t j = 0; j < qd; j++) {
                    double e = fabs((double)got[s][p][j] - (double)want[s][p][j]);
                    if (!(e <= worst)) worst = e;
                }
            }
    }
    return worst;
}
