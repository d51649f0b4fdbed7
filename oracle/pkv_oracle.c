/*
 * CPU oracle for the PhaseKV stage-B hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's
 *   src/phasekv/kernels/packing.py     (pack_low_bits :41-65, unpack_low_bits :67-79,
 *                                       quantize_pack :115-155, unpack_dequantize :158-175)
 *   src/phasekv/kernels/reference.py   (fused_decode_attention_reference :72-96)
 *   src/phasekv/phasekv_cache.py       (_cool_aged_tokens value-norm top-k :322-333)
 * so that the CUDA kernels can be checked on a machine that has no copy of the
 * reference.  It is only ever used as a checker (tests, the smoke check and the
 * CPU-baseline leg of the benchmark); no product code path may call it.
 *
 * Parity of this restatement with the reference is pinned by the fixtures under
 * tests/golden/, which were produced by running the reference's own Python on CPU.
 *
 * Floating point rules that make the integer outputs bit-exact:
 *   - every division is an IEEE-754 round-to-nearest float division (no reciprocal),
 *   - rounding of quotients is round-half-to-even (rintf in the default mode),
 *   - codes are computed with the float32 scale; the stored scale is that value
 *     rounded to float16 afterwards,
 *   - the file must be compiled with -ffp-contract=off and without -ffast-math.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

static inline uint16_t f2h(float f) {
    _Float16 v = (_Float16)f; /* IEEE round-to-nearest-even, as torch .to(float16) */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

int pkvo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void pkvo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* packing.py:41-65 — code i of a byte occupies bits [i*bits, (i+1)*bits); the tail is zero. */
void pkvo_pack_low_bits(const uint8_t* codes, int64_t rows, int64_t len, int bits, uint8_t* out) {
    const int vpb = 8 / bits;
    const int64_t nbytes = (len + vpb - 1) / vpb;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t* c = codes + r * len;
        uint8_t* o = out + r * nbytes;
        for (int64_t b = 0; b < nbytes; ++b) {
            unsigned v = 0;
            for (int i = 0; i < vpb; ++i) {
                int64_t j = b * vpb + i;
                if (j < len) v += (unsigned)c[j] << (i * bits);
            }
            o[b] = (uint8_t)v; /* the reference sums in int32 and casts to uint8 */
        }
    }
}

/* packing.py:67-79 */
void pkvo_unpack_low_bits(const uint8_t* packed, int64_t rows, int64_t len, int bits, uint8_t* out) {
    const int vpb = 8 / bits;
    const int64_t nbytes = (len + vpb - 1) / vpb;
    const unsigned mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint8_t* p = packed + r * nbytes;
        uint8_t* o = out + r * len;
        for (int64_t j = 0; j < len; ++j) o[j] = (uint8_t)((p[j / vpb] >> ((j % vpb) * bits)) & mask);
    }
}

/*
 * packing.py:115-155.  x is float16 viewed as [outer, A, inner]; the quantisation
 * axis is A.  Outputs have the axis moved last:
 *   packed [outer, inner, ceil(A/vpb)]   scale, mins [outer, inner, ceil(A/gs)]
 * gs must already be clamped to [1, A] by the caller (packing.py:130).
 * The reference pads the tail group by repeating the last element, which changes
 * neither min nor max, so the tail group simply reduces over its real elements.
 */
void pkvo_quantize_pack(const uint16_t* x, int64_t outer, int64_t A, int64_t inner, int bits,
                        int64_t gs, uint8_t* packed, uint16_t* scale, uint16_t* mins) {
    const int vpb = 8 / bits;
    const float qmax = (float)((1 << bits) - 1);
    const int64_t nb = (A + vpb - 1) / vpb;
    const int64_t ng = (A + gs - 1) / gs;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t o = 0; o < outer; ++o) {
        for (int64_t j = 0; j < inner; ++j) {
            const uint16_t* xp = x + o * A * inner + j;
            uint8_t* pk = packed + (o * inner + j) * nb;
            memset(pk, 0, (size_t)nb);
            for (int64_t g = 0; g < ng; ++g) {
                const int64_t a0 = g * gs;
                const int64_t a1 = (a0 + gs < A) ? a0 + gs : A;
                float lo = h2f(xp[a0 * inner]), hi = lo;
                for (int64_t a = a0 + 1; a < a1; ++a) {
                    float v = h2f(xp[a * inner]);
                    lo = v < lo ? v : lo;
                    hi = v > hi ? v : hi;
                }
                float range = hi - lo;
                if (range < 1e-8f) range = 1e-8f;   /* clamp_(min=1e-8) */
                const float sc = range / qmax;       /* true division */
                for (int64_t a = a0; a < a1; ++a) {
                    float qv = rintf((h2f(xp[a * inner]) - lo) / sc);
                    if (qv < 0.f) qv = 0.f;
                    if (qv > qmax) qv = qmax;
                    pk[a / vpb] |= (uint8_t)((unsigned)qv << ((a % vpb) * bits));
                }
                scale[(o * inner + j) * ng + g] = f2h(sc);
                mins[(o * inner + j) * ng + g] = f2h(lo);
            }
        }
    }
}

/* packing.py:158-175: float32 code*scale then +mins (two roundings), then float16. */
void pkvo_unpack_dequantize(const uint8_t* packed, const uint16_t* scale, const uint16_t* mins,
                            int64_t outer, int64_t A, int64_t inner, int bits, int64_t gs,
                            uint16_t* out) {
    const int vpb = 8 / bits;
    const unsigned mask = (1u << bits) - 1u;
    const int64_t nb = (A + vpb - 1) / vpb;
    const int64_t ng = (A + gs - 1) / gs;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t o = 0; o < outer; ++o) {
        for (int64_t a = 0; a < A; ++a) {
            for (int64_t j = 0; j < inner; ++j) {
                const uint8_t byte = packed[(o * inner + j) * nb + a / vpb];
                const float c = (float)((byte >> ((a % vpb) * bits)) & mask);
                const float s = h2f(scale[(o * inner + j) * ng + a / gs]);
                const float m = h2f(mins[(o * inner + j) * ng + a / gs]);
                volatile float prod = c * s; /* keep the two roundings separate */
                out[(o * A + a) * inner + j] = f2h(prod + m);
            }
        }
    }
}

/*
 * reference.py:72-96 for one batch element and one query step, on already
 * dequantised float16 K and V ([Hkv, S, hd], the concatenation prompt -> cold -> hot):
 * GQA expansion by head index, scores = (q . k) / sqrt(hd), softmax over all S
 * tokens, out = probs @ V, rounded to float16.  Dot products are accumulated in
 * double so that the checker carries no summation-order noise of its own; the
 * reference accumulates in float32, which differs from this by about 1e-6.
 * m/l/acc (optional, may be NULL) return the un-normalised flash partial
 * (running max, sum of exp, weighted V sum) as attention_triton.py:257-266 defines it.
 */
void pkvo_attention_dense(const uint16_t* q, const uint16_t* K, const uint16_t* V, int Hq, int Hkv,
                          int64_t S, int hd, uint16_t* out, float* out_f32, float* m_out,
                          float* l_out, float* acc_out) {
    const int group = Hq / Hkv;
    const double sm = 1.0 / sqrt((double)hd);
#pragma omp parallel for schedule(static)
    for (int h = 0; h < Hq; ++h) {
        const int kv = h / group;
        const uint16_t* Kh = K + (int64_t)kv * S * hd;
        const uint16_t* Vh = V + (int64_t)kv * S * hd;
        float* qf = (float*)malloc(sizeof(float) * (size_t)hd);
        float* sc = (float*)malloc(sizeof(float) * (size_t)S);
        double* acc = (double*)calloc((size_t)hd, sizeof(double));
        for (int d = 0; d < hd; ++d) qf[d] = h2f(q[h * hd + d]);
        float mx = -INFINITY;
        for (int64_t n = 0; n < S; ++n) {
            double dot = 0.0;
            const uint16_t* kr = Kh + n * hd;
            for (int d = 0; d < hd; ++d) dot += (double)qf[d] * (double)h2f(kr[d]);
            sc[n] = (float)(dot * sm);
            if (sc[n] > mx) mx = sc[n];
        }
        double l = 0.0;
        for (int64_t n = 0; n < S; ++n) {
            const double p = exp((double)sc[n] - (double)mx);
            l += p;
            const uint16_t* vr = Vh + n * hd;
            for (int d = 0; d < hd; ++d) acc[d] += p * (double)h2f(vr[d]);
        }
        for (int d = 0; d < hd; ++d) {
            const float o = (float)(acc[d] / l);
            if (out) out[h * hd + d] = f2h(o);
            if (out_f32) out_f32[h * hd + d] = o;
            if (acc_out) acc_out[h * hd + d] = (float)acc[d];
        }
        if (m_out) m_out[h] = mx;
        if (l_out) l_out[h] = (float)l;
        free(qf);
        free(sc);
        free(acc);
    }
}

/*
 * phasekv_cache.py:328-333: importance = L2 norm of V over head_dim (float32 in the
 * reference), keep the `keep` largest per row, return their indices ascending.
 * V is float16 [rows, aged, hd].  Squared norms are accumulated in double; ties are
 * broken towards the lower index.  min_gap[r] reports the relative gap between the
 * smallest kept and the largest dropped squared norm, so a caller can recognise a
 * near-tie (where float32 summation order in the reference could pick differently)
 * instead of reporting a false mismatch.
 */
void pkvo_value_norm_topk(const uint16_t* V, int64_t rows, int64_t aged, int hd, int64_t keep,
                          int64_t* idx_out, double* min_gap) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double* n2 = (double*)malloc(sizeof(double) * (size_t)aged);
        for (int64_t a = 0; a < aged; ++a) {
            double s = 0.0;
            const uint16_t* v = V + (r * aged + a) * hd;
            for (int d = 0; d < hd; ++d) {
                const double f = (double)h2f(v[d]);
                s += f * f;
            }
            n2[a] = s;
        }
        int64_t k = 0;
        double kept_min = INFINITY, drop_max = -INFINITY;
        for (int64_t a = 0; a < aged; ++a) {
            int64_t rank = 0;
            for (int64_t b = 0; b < aged; ++b)
                if (n2[b] > n2[a] || (n2[b] == n2[a] && b < a)) ++rank;
            if (rank < keep) {
                idx_out[r * keep + k++] = a;
                if (n2[a] < kept_min) kept_min = n2[a];
            } else if (n2[a] > drop_max) {
                drop_max = n2[a];
            }
        }
        if (min_gap)
            min_gap[r] = (drop_max < 0.0 || kept_min <= 0.0) ? INFINITY
                                                             : (kept_min - drop_max) / kept_min;
        free(n2);
    }
}

/*
 * quant.py:34-79 _grouped_affine_quant_dequant ("fake quantisation" of stage A), on float32:
 * x viewed as [outer, A, inner], groups of gs (already clamped to [1, A]) along A.  Unlike the packed
 * path, scale and zero stay float32 and bits may be anything from 1 to 15.  The reference pads the tail
 * group by repeating the last element (no effect on min / max).  out = q * scale + min with the product
 * and the sum rounded separately, as torch evaluates `q * scale + g_min`.  The caller converts to and
 * from the tensor's element type.
 */
void pkvo_fake_quant(const float* x, int64_t outer, int64_t A, int64_t inner, int bits, int64_t gs,
                     float* out) {
    const float qmax = (float)((1 << bits) - 1);
    const int64_t ng = (A + gs - 1) / gs;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t o = 0; o < outer; ++o) {
        for (int64_t j = 0; j < inner; ++j) {
            const float* xp = x + o * A * inner + j;
            float* op = out + o * A * inner + j;
            for (int64_t g = 0; g < ng; ++g) {
                const int64_t a0 = g * gs;
                const int64_t a1 = (a0 + gs < A) ? a0 + gs : A;
                float lo = xp[a0 * inner], hi = lo;
                for (int64_t a = a0 + 1; a < a1; ++a) {
                    const float v = xp[a * inner];
                    lo = v < lo ? v : lo;
                    hi = v > hi ? v : hi;
                }
                float range = hi - lo;
                if (range < 1e-8f) range = 1e-8f;
                const float sc = range / qmax;
                for (int64_t a = a0; a < a1; ++a) {
                    float q = rintf((xp[a * inner] - lo) / sc);
                    if (q < 0.f) q = 0.f;
                    if (q > qmax) q = qmax;
                    const float prod = q * sc;
                    op[a * inner] = prod + lo;
                }
            }
        }
    }
}
