/*
 * rq_oracle.c -- CPU restatement of ruquant's W4A4 / W4A4H MUL_MAT arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with (tests, the smoke check and
 * the CPU-baseline leg of the benchmark).  It is never linked into, loaded by or called from the product library.
 *
 * Every function names the reference code it restates, as file:line of the reference project, where
 * "patch" = patches/llama.cpp-ruquant.patch.  Parity of this restatement is pinned two ways: against
 * libruquant_ref.so (the reference's own lines compiled by oracle/build_ref.py, when the reference is present) and
 * against the golden vectors under tests/golden/ that were generated from that library.
 *
 * Build: gcc -O3 -std=gnu11 -ffp-contract=off -fopenmp -fPIC -shared rq_oracle.c -o librq_oracle.so -lm
 * No -march flag and no fast-math: fp32 operations must round one at a time, in the order written.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define RQO_API __attribute__((visibility("default")))
#define RQO_QK 256          /* codes per block                      patch:38 */
#define RQO_SHIFT 4         /* per-group term shift                 patch:39 */
#define RQO_MMAX 255        /* largest activation group multiplier  patch:2487 */

/* 144-byte block: patch:44-50 */
typedef struct {
    float    d;
    int32_t  sum;
    int32_t  pad[2];
    uint32_t qs[RQO_QK / 8];
} rqo_block;

/* signed value of nibble j of a word: element 8w+j sits in bits [4j+3:4j], two's complement   patch:28, 2503-2505 */
static inline int32_t rqo_nib(uint32_t word, int j) {
    const int32_t v = (int32_t) ((word >> (4 * j)) & 0xF);
    return v >= 8 ? v - 16 : v;
}

/* weight multiplier of 64-input group g of a block, from the header word `sum`   patch:40-43 */
static inline int32_t rqo_wmult(int32_t sum, int g) {
    const uint32_t s = (uint32_t) sum;
    if ((s >> 29) == 3u) return (int32_t) ((s >> (4 * g)) & 0xF);
    if ((s >> 30) == 1u) return (int32_t) (s & 0xF);
    return 1;
}

/* -------------------------------------------------------------------------------- Hadamard   patch:2413-2485 */

static int rqo_prime(int q) {
    if (q < 2) return 0;
    for (int d = 2; d * d <= q; ++d) if (q % d == 0) return 0;
    return 1;
}

/* smallest p in {1} + {p <= 128 : p % 4 == 0, p - 1 prime and = 3 mod 4} with n / p a power of two   patch:2419-2430 */
RQO_API int rqo_hadamard_factor(int64_t n, int * p, int * m) {
    for (int c = 1; c <= 128 && c <= n; ++c) {
        if (c > 1 && !(c % 4 == 0 && rqo_prime(c - 1) && (c - 1) % 4 == 3)) continue;
        if (n % c) continue;
        const int64_t rest = n / c;
        if (rest & (rest - 1)) continue;
        *p = c;
        *m = (int) rest;
        return 1;
    }
    return 0;
}

/* Paley I matrix of order p as +1 / -1 bytes, A = I + S   patch:2432-2448 */
RQO_API void rqo_paley(int p, int8_t * A) {
    const int q = p - 1;
    int8_t chi[128];
    memset(chi, -1, sizeof(chi));
    chi[0] = 0;
    for (int i = 1; i < q; ++i) chi[(i * i) % q] = 1;
    for (int i = 0; i < p; ++i) {
        for (int j = 0; j < p; ++j) {
            int s;
            if (i == 0) s = j ? 1 : 0;
            else if (j == 0) s = -1;
            else s = chi[(((j - i) % q) + q) % q];
            A[i * p + j] = (int8_t) (s + (i == j));
        }
    }
}

/* x <- x (H_p kron H_m) / sqrt(n); butterflies h = 1, 2, 4, ..., then each Paley output summed from 0.0f over
 * ascending i, then one multiply by 1/sqrtf(n)   patch:2450-2485 */
RQO_API int rqo_hadamard(float * x, int64_t n, int transpose) {
    int p, m;
    if (!rqo_hadamard_factor(n, &p, &m)) return -1;
    for (int c = 0; c < p; ++c) {
        float * v = x + (int64_t) c * m;
        for (int h = 1; h < m; h *= 2) {
            for (int base = 0; base < m; base += 2 * h) {
                for (int k = base; k < base + h; ++k) {
                    const float a = v[k], b = v[k + h];
                    v[k] = a + b;
                    v[k + h] = a - b;
                }
            }
        }
    }
    if (p > 1) {
        int8_t * A = (int8_t *) malloc((size_t) p * p);
        float col[128];
        rqo_paley(p, A);
        for (int j = 0; j < m; ++j) {
            for (int i = 0; i < p; ++i) col[i] = x[(int64_t) i * m + j];
            for (int a = 0; a < p; ++a) {
                float acc = 0.0f;
                for (int i = 0; i < p; ++i) {
                    const int8_t e = transpose ? A[a * p + i] : A[i * p + a];
                    if (e > 0) acc = acc + col[i]; else acc = acc - col[i];
                }
                x[(int64_t) a * m + j] = acc;
            }
        }
        free(A);
    }
    const float scale = 1.0f / sqrtf((float) n);
    for (int64_t i = 0; i < n; ++i) x[i] = x[i] * scale;
    return 0;
}

/* block-diagonal rotation: each run of n_rot inputs gets its own H   patch:2697-2699 */
RQO_API int rqo_rotate_row(float * x, int64_t K, int64_t n_rot) {
    if (n_rot <= 0 || K % n_rot) return -1;
    for (int64_t o = 0; o < K; o += n_rot) if (rqo_hadamard(x + o, n_rot, 0)) return -1;
    return 0;
}

/* -------------------------------------------------------------------------------- weights   patch:2489-2580 */

/* 13-step clip search: s = amax * (1 - 0.025 r) / 7 with the least squared rounding error (double sum, in index
 * order, first best wins)   patch:2509-2527 */
static float rqo_wscale(const float * x, int64_t n) {
    float amax = 0.0f;
    for (int64_t i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
    if (!(amax > 0.0f)) return 0.0f;
    float best = 0.0f;
    double best_err = INFINITY;
    for (int r = 0; r < 13; ++r) {
        const float s = amax * (1.0f - 0.025f * r) / 7.0f;
        double err = 0.0;
        for (int64_t i = 0; i < n; ++i) {
            const float q = fminf(fmaxf(rintf(x[i] / s), -8.0f), 7.0f);
            const double e = (double) (q * s) - (double) x[i];
            err += e * e;
        }
        if (err < best_err) { best_err = err; best = s; }
    }
    return best;
}

static void rqo_pack_row(rqo_block * y, const int8_t * codes, int64_t K, float d, int32_t sum) {   /* patch:2489-2501 */
    for (int64_t b = 0; b < K / RQO_QK; ++b) {
        y[b].d = d;
        y[b].sum = sum;
        y[b].pad[0] = (int32_t) K;
        y[b].pad[1] = 0;
        for (int w = 0; w < RQO_QK / 8; ++w) {
            uint32_t word = 0;
            for (int j = 0; j < 8; ++j) word |= (uint32_t) (codes[b * RQO_QK + 8 * w + j] & 0xF) << (4 * j);
            y[b].qs[w] = word;
        }
    }
}

static inline int8_t rqo_wcode(float x, float s) {
    return s > 0.0f ? (int8_t) fminf(fmaxf(rintf(x / s), -8.0f), 7.0f) : 0;
}

/* one row: wgroup 0 = one scale per row (header sum = the row's code sum), 256 = a multiplier per block,
 * 64 = a multiplier per 64 inputs   patch:2541-2580 */
static void rqo_quantize_weight_row(const float * x, rqo_block * y, int64_t K, int wgroup) {
    int8_t * codes = (int8_t *) malloc((size_t) K);
    if (wgroup == 0) {
        const float s = rqo_wscale(x, K);
        int32_t sum = 0;
        for (int64_t i = 0; i < K; ++i) { codes[i] = rqo_wcode(x[i], s); sum += codes[i]; }
        rqo_pack_row(y, codes, K, s, sum);
        free(codes);
        return;
    }
    const int gs = wgroup, ng = (int) (K / gs);
    float * sg = (float *) malloc(sizeof(float) * (size_t) ng);
    int32_t * kg = (int32_t *) malloc(sizeof(int32_t) * (size_t) ng);
    float smax = 0.0f;
    for (int g = 0; g < ng; ++g) { sg[g] = rqo_wscale(x + (int64_t) g * gs, gs); smax = fmaxf(smax, sg[g]); }
    const float unit = smax / 15.0f;
    for (int g = 0; g < ng; ++g) {
        kg[g] = unit > 0.0f ? (int32_t) fminf(fmaxf(rintf(sg[g] / unit), 1.0f), 15.0f) : 1;
        const float s = (float) kg[g] * unit;
        for (int i = 0; i < gs; ++i) codes[(int64_t) g * gs + i] = rqo_wcode(x[(int64_t) g * gs + i], s);
    }
    rqo_pack_row(y, codes, K, unit, 0);
    for (int64_t b = 0; b < K / RQO_QK; ++b) {
        y[b].sum = gs == RQO_QK ? (int32_t) (1u << 30 | (uint32_t) kg[b])
                                : (int32_t) (3u << 29 | (uint32_t) kg[4 * b] | (uint32_t) kg[4 * b + 1] << 4 |
                                             (uint32_t) kg[4 * b + 2] << 8 | (uint32_t) kg[4 * b + 3] << 12);
    }
    free(kg);
    free(sg);
    free(codes);
}

/* rows of fp32 -> rows of blocks.  hadamard: rotate each row by blocks of K / rot_blocks first and store that
 * length in pad[0]   patch:2681-2710, 2775-2789 */
RQO_API int rqo_quantize_weights(const float * src, void * dst, int64_t nrows, int64_t K, int hadamard, int wgroup,
                                 int rot_blocks, int n_threads) {
    if (K % RQO_QK) return -1;
    const int64_t n_rot = (rot_blocks > 1 && K % rot_blocks == 0) ? K / rot_blocks : K;
    int p, m;
    if (hadamard && !rqo_hadamard_factor(n_rot, &p, &m)) return -1;
    #pragma omp parallel for schedule(dynamic, 4) num_threads(n_threads > 0 ? n_threads : 1)
    for (int64_t r = 0; r < nrows; ++r) {
        rqo_block * y = (rqo_block *) dst + r * (K / RQO_QK);
        if (!hadamard) {
            rqo_quantize_weight_row(src + r * K, y, K, wgroup);
        } else {
            float * t = (float *) malloc(sizeof(float) * (size_t) K);
            memcpy(t, src + r * K, sizeof(float) * (size_t) K);
            rqo_rotate_row(t, K, n_rot);
            rqo_quantize_weight_row(t, y, K, wgroup);
            for (int64_t b = 0; b < K / RQO_QK; ++b) y[b].pad[0] = (int32_t) n_rot;
            free(t);
        }
    }
    return 0;
}

/* -------------------------------------------------------------------------------- activations   patch:2633-2679 */

/* One token row -> K/256 blocks.  G in {64,128,256}.  Group range [min(x,0), max(x,0)] * clip; R the widest range
 * of the token (2 if 0); u = R / (15 * 255); m_g = clamp(ceil((range_g * 255) / R), 1, 255);
 * inv = 1 / (m_g * u); z_g = clamp(rint(-lo_g * inv), 0, 15); code = clamp(rint(x * inv) + z_g, 0, 15) - 8.
 * n_rot > 0: rotate a copy of the row first and record n_rot in pad[1]   patch:2728-2736 */
RQO_API int rqo_quantize_act(const float * x_in, void * dst, int64_t K, float clip, int G, int64_t n_rot) {
    if (K % RQO_QK || !(G == 64 || G == 128 || G == 256)) return -1;
    float * x = (float *) malloc(sizeof(float) * (size_t) K);
    memcpy(x, x_in, sizeof(float) * (size_t) K);
    if (n_rot > 0 && rqo_rotate_row(x, K, n_rot)) { free(x); return -1; }
    rqo_block * y = (rqo_block *) dst;
    const int lsub = G == 64 ? 2 : G == 128 ? 1 : 0;
    const int64_t ng = K / G;
    float * lo = (float *) malloc(sizeof(float) * 2 * (size_t) ng);
    float * hi = lo + ng;
    float R = 0.0f;
    for (int64_t g = 0; g < ng; ++g) {
        float mn = 0.0f, mx = 0.0f;
        for (int i = 0; i < G; ++i) { mn = fminf(mn, x[g * G + i]); mx = fmaxf(mx, x[g * G + i]); }
        lo[g] = mn * clip;
        hi[g] = mx * clip;
        R = fmaxf(R, hi[g] - lo[g]);
    }
    if (R == 0.0f) R = 2.0f;
    const float u = R / (15.0f * RQO_MMAX);
    for (int64_t b = 0; b < K / RQO_QK; ++b) {
        y[b].d = u;
        y[b].sum = lsub << 16;
        y[b].pad[0] = 0;
        y[b].pad[1] = (int32_t) (n_rot > 0 ? n_rot : K);
    }
    for (int64_t g = 0; g < ng; ++g) {
        const int m = (int) fminf(fmaxf(ceilf(((hi[g] - lo[g]) * (float) RQO_MMAX) / R), 1.0f), (float) RQO_MMAX);
        const float inv = 1.0f / ((float) m * u);
        const float zf = fminf(fmaxf(rintf(-lo[g] * inv), 0.0f), 15.0f);
        rqo_block * yb = &y[g * G / RQO_QK];
        const int sg = (int) (g % (RQO_QK / G));
        yb->sum |= (int32_t) zf << (4 * sg);
        yb->pad[0] = (int32_t) ((uint32_t) yb->pad[0] | (uint32_t) m << (8 * sg));
        for (int w = sg * G / 8; w < (sg + 1) * G / 8; ++w) {
            uint32_t word = 0;
            for (int j = 0; j < 8; ++j) {
                const float q = fminf(fmaxf(rintf(x[(g - sg) * G + 8 * w + j] * inv) + zf, 0.0f), 15.0f);
                word |= (uint32_t) (((int) q - 8) & 0xF) << (4 * j);
            }
            yb->qs[w] = word;
        }
    }
    free(lo);
    free(x);
    return 0;
}

/* -------------------------------------------------------------------------------- dot product   patch:148-177 */

/* one weight row x one activation row, the reference's own form: per activation group acc = sum cx*cy and
 * colsum = sum cx; total += (k * m * (acc + (8 - z) * colsum)) >> 4; y = ((float(total) * 16) * u) * s_w */
RQO_API float rqo_vec_dot(int64_t K, const void * w_row, const void * a_row) {
    const rqo_block * x = (const rqo_block *) w_row;
    const rqo_block * y = (const rqo_block *) a_row;
    int32_t total = 0;
    for (int64_t b = 0; b < K / RQO_QK; ++b) {
        const int lsub = (y[b].sum >> 16) & 3;
        const int gw = (RQO_QK / 8) >> lsub;
        for (int sg = 0; sg < (1 << lsub); ++sg) {
            int32_t acc = 0, colsum = 0;
            for (int w = sg * gw; w < (sg + 1) * gw; ++w) {
                for (int j = 0; j < 8; ++j) {
                    const int32_t cx = rqo_nib(x[b].qs[w], j), cy = rqo_nib(y[b].qs[w], j);
                    acc += cx * cy;
                    colsum += cx;
                }
            }
            const int32_t z = (y[b].sum >> (4 * sg)) & 0xF;
            const int32_t m = (int32_t) (((uint32_t) y[b].pad[0] >> (8 * sg)) & 0xFF);
            const int32_t k = rqo_wmult(x[b].sum, sg << (2 - lsub));
            total += (k * m * (acc + (8 - z) * colsum)) >> RQO_SHIFT;
        }
    }
    return (((float) total * (float) (1 << RQO_SHIFT)) * y[0].d) * x[0].d;
}

/* -------------------------------------------------------------------------------- MUL_MAT   patch:103-122 */

/* clip: the override if > 0, else block 0's pad[1] as a float if > 0, else 1   patch:2590-2606 */
RQO_API float rqo_resolve_clip(const void * w_blocks, float override_clip) {
    float c;
    memcpy(&c, &((const rqo_block *) w_blocks)->pad[1], sizeof(c));
    return override_clip > 0.0f ? override_clip : c > 0.0f ? c : 1.0f;
}

/* Hadamard length of a W4A4H tensor: block 0's pad[0]; must divide K and factor, else -1   patch:2608-2620 */
RQO_API int64_t rqo_resolve_rot(const void * w_blocks, int64_t K) {
    const int32_t n = ((const rqo_block *) w_blocks)->pad[0];
    int p, m;
    if (n <= 0 || K % n || !rqo_hadamard_factor(n, &p, &m)) return -1;
    return n;
}

/* Y[t*ldy + n] for all tokens and rows.  Same numbers as one rqo_vec_dot per output, computed from codes widened
 * to int8 once per row / token: sum c*(q - z) over a group equals acc + (8 - z)*colsum.
 * type 44 = W4A4, 45 = W4A4H.  Returns 0, or -1 on a bad shape / unfactorable rotation length. */
RQO_API int rqo_mul_mat(const void * w, int type, int64_t K, int64_t N, const float * x, int64_t ldx, int64_t M,
                        float * y, int64_t ldy, float clip_override, int G, int n_threads) {
    if (K % RQO_QK || !(type == 44 || type == 45)) return -1;
    const int nt = n_threads > 0 ? n_threads : 1;
    const float clip = rqo_resolve_clip(w, clip_override);
    const int64_t n_rot = type == 45 ? rqo_resolve_rot(w, K) : 0;
    if (n_rot < 0) return -1;
    const int64_t nb = K / RQO_QK, ng = K / G;
    const rqo_block * W = (const rqo_block *) w;
    if ((((uint32_t) W[0].sum) >> 29) == 3u && G != 64) return -1;   /* patch:171 */
    rqo_block * A = (rqo_block *) malloc(sizeof(rqo_block) * (size_t) (M * nb));
    int8_t * a8 = (int8_t *) malloc((size_t) (M * K));           /* q - z */
    int32_t * mg = (int32_t *) malloc(sizeof(int32_t) * (size_t) (M * ng));
    int rc = 0;
    #pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t t = 0; t < M; ++t) {
        rqo_block * yb = A + t * nb;
        if (rqo_quantize_act(x + t * ldx, yb, K, clip, G, n_rot)) { rc = -1; continue; }
        for (int64_t g = 0; g < ng; ++g) {
            const rqo_block * b = &yb[g * G / RQO_QK];
            const int sg = (int) (g % (RQO_QK / G));
            const int z = (b->sum >> (4 * sg)) & 0xF;
            mg[t * ng + g] = (int32_t) (((uint32_t) b->pad[0] >> (8 * sg)) & 0xFF);
            for (int i = 0; i < G; ++i) {
                const int e = (int) ((g * G + i) % RQO_QK);
                a8[t * K + g * G + i] = (int8_t) (rqo_nib(b->qs[e / 8], e % 8) + 8 - z);
            }
        }
    }
    if (rc == 0) {
        #pragma omp parallel num_threads(nt)
        {
            int8_t * c8 = (int8_t *) malloc((size_t) K);
            int32_t * kw = (int32_t *) malloc(sizeof(int32_t) * (size_t) (K / 64));
            #pragma omp for schedule(dynamic, 8)
            for (int64_t n = 0; n < N; ++n) {
                const rqo_block * wr = W + n * nb;
                for (int64_t b = 0; b < nb; ++b) {
                    for (int e = 0; e < RQO_QK; ++e) c8[b * RQO_QK + e] = (int8_t) rqo_nib(wr[b].qs[e / 8], e % 8);
                    for (int s = 0; s < 4; ++s) kw[4 * b + s] = rqo_wmult(wr[b].sum, s);
                }
                for (int64_t t = 0; t < M; ++t) {
                    const int8_t * av = a8 + t * K;
                    int32_t total = 0;
                    for (int64_t g = 0; g < ng; ++g) {
                        int32_t s = 0;
                        for (int i = 0; i < G; ++i) s += (int32_t) c8[g * G + i] * (int32_t) av[g * G + i];
                        total += (kw[g * G / 64] * mg[t * ng + g] * s) >> RQO_SHIFT;
                    }
                    y[t * ldy + n] = (((float) total * (float) (1 << RQO_SHIFT)) * A[t * nb].d) * wr[0].d;
                }
            }
            free(kw);
            free(c8);
        }
    }
    free(mg);
    free(a8);
    free(A);
    return rc;
}
