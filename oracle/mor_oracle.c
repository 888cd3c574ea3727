/*
 * CPU oracle for the MoR fake-quantization path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of the reference operators in
 * mor/csrc/cuda/fake_quantize.cu (boryiings/mor), including the order in which
 * the reference adds up its floating-point error sums.  It exists so that the
 * CUDA kernels of this repository can be checked bit for bit on a machine
 * without the reference.  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may call it; the product never does.
 *
 * Build: make -C oracle   (gcc, -O2 -ffp-contract=off, no fast-math: every
 * multiply, divide and add below must be a single IEEE binary32 operation,
 * as the reference is built with nvcc -O3 and no --use_fast_math and contains
 * no a*b+c pattern that nvcc could contract).
 *
 * Pinning: tests/test_oracle_golden.py checks this file against the known-answer
 * matrices of the reference's own tests (test/test_fake_quantize.py:225-374,
 * 787-948), against torch's CPU float8 casts (the reference tests' own oracle),
 * against the NVIDIA conversion headers, and against outputs recorded from the
 * unmodified reference extension running on a B200 (tests/golden/).
 *
 * "ref:" comments give the line range of mor/csrc/cuda/fake_quantize.cu that a
 * function follows.
 */
#include <math.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define MOR_O_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* bit casts                                                                 */
/* ------------------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ref: 38-44.  bf16 bits (low 16 bits of v) widened to binary32. */
MOR_O_API float mor_o_bf16_to_fp32(uint32_t v) { return u2f((v & 0xFFFFu) << 16); }

/* ref: 46-60.  binary32 -> bf16 bits: the 7-bit mantissa is incremented when bit
 * 15 is set (round half AWAY from zero, not to even); a mantissa carry bumps the
 * exponent, and the three fields are OR-ed together, so an exponent that reaches
 * 256 (only a NaN whose top eight mantissa bits are ones) lands on the sign bit:
 * such NaNs come out as 0x8000 whatever their sign. */
MOR_O_API uint32_t mor_o_fp32_to_bf16(float value) {
    uint32_t b = f2u(value);
    uint32_t sign = b >> 31;
    uint32_t expo = (b >> 23) & 0xFFu;
    uint32_t man = (b >> 16) & 0x7Fu;
    if ((b >> 15) & 1u) {
        man += 1;
        if (man == 128) { man = 0; expo += 1; }
    }
    return (sign << 15) | (expo << 7) | man;
}

/* ------------------------------------------------------------------------- */
/* narrow formats                                                            */
/* ------------------------------------------------------------------------- */
enum { FMT_E4M3 = 0, FMT_E5M2 = 1, FMT_E3M2 = 2, FMT_E2M3 = 3 };

typedef struct {
    int ebits, mbits, bias;
    int top;        /* largest exponent field holding finite values ("before_overflow") */
    int saturates;  /* E3M2/E2M3: no NaN encoding, overflow clamps to the maximum        */
} fmt_t;

/* ref: 72-122 (Exponent5/4/3/2, Mantissa3/2 traits) */
static const fmt_t FMTS[4] = {
    {4, 3, 7, 15, 0},  /* E4M3: field 15 is finite except mantissa 111 (NaN) */
    {5, 2, 15, 30, 0}, /* E5M2: field 31 is inf/NaN                          */
    {3, 2, 3, 7, 1},   /* E3M2: max 28                                       */
    {2, 3, 1, 3, 1},   /* E2M3: max 7.5                                      */
};

static const uint32_t NAN_ALL_ONES = 0x7FFFFFFFu;

/* ref: 125-215, quant_dequant_fp32<E,M>: binary32 -> narrow float -> binary32 with
 * round-to-nearest-even, gradual underflow, and
 *   - E3M2/E2M3: clamp to the largest magnitude on overflow (also for inf/NaN input);
 *   - E4M3/E5M2: return the NaN 0x7fffffff on overflow (NOT saturating);
 *   - a result of zero is +0.0 even for a negative input. */
static float narrow_custom(float x, int fmt) {
    const fmt_t *F = &FMTS[fmt];
    const uint32_t b = f2u(x);
    const uint32_t sign = b >> 31;
    const int drop = 23 - F->mbits; /* mantissa bits that do not fit */
    const uint32_t mmask = (1u << F->mbits) - 1u;
    int e = (int)((b >> 23) & 0xFFu) - 127 + F->bias;
    uint32_t man = 0, guard = 0, sticky = 0;

    if (e > 0) {
        man = (b >> drop) & mmask;
        guard = (b >> (drop - 1)) & 1u;
        sticky = (b & ((1u << (drop - 1)) - 1u)) != 0;
    } else {
        const int rs = 1 - e; /* extra right shift into the subnormal range */
        e = 0;
        if (rs <= F->mbits + 1) {
            uint32_t sig = (b & 0x7FFFFFu) | (1u << 23);
            sticky = (sig & ((1u << (rs + drop - 1)) - 1u)) != 0;
            sig >>= rs;
            guard = (sig >> (drop - 1)) & 1u;
            man = (sig >> drop) & mmask;
        }
    }
    if (guard && (sticky || (man & 1u))) {
        man += 1;
        if (man == (1u << F->mbits)) { man = 0; e += 1; }
    }
    if (F->saturates) {
        if (e > F->top) { e = (1 << F->ebits) - 1; man = mmask; }
    } else {
        if (e > F->top) return u2f(NAN_ALL_ONES);
        if (e == F->top && fmt == FMT_E4M3 && man == mmask) return u2f(NAN_ALL_ONES);
    }
    uint32_t out = 0;
    if (e > 0) {
        out = (sign << 31) | ((uint32_t)(e + 127 - F->bias) << 23) | (man << drop);
    } else if (man) {
        int ex = 127 - F->bias + 1;
        while (!(man & (1u << F->mbits))) { man <<= 1; ex -= 1; }
        man &= mmask;
        out = (sign << 31) | ((uint32_t)ex << 23) | (man << drop);
    }
    return u2f(out);
}

/* ref: 222-227, static_cast<__nv_fp8_e4m3 / __nv_fp8_e5m2>(float) and back
 * (NVIDIA cuda_fp8.hpp, CUDA 12.9; __NV_SATFINITE): round-to-nearest-even,
 * overflow and infinities clamp to +-448 / +-57344, NaN gives the fp8 NaN, whose
 * widening is the half NaN 0x7fff -> binary32 0x7fffe000 (sign dropped), and a
 * zero result keeps the sign of the input. */
static float narrow_satfinite(float x, int fmt) {
    const fmt_t *F = &FMTS[fmt];
    const uint32_t b = f2u(x);
    const uint32_t sign = b & 0x80000000u;
    const uint32_t mag = b & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return u2f(0x7FFFE000u);
    const float maxv = (fmt == FMT_E4M3) ? 448.0f : 57344.0f;
    if (u2f(mag) >= maxv) return u2f(sign | f2u(maxv));
    /* finite and below the maximum: round the magnitude onto the format's grid.
     * The grid spacing at magnitude 2^k is 2^(k-mbits), never finer than the
     * subnormal spacing 2^(1-bias-mbits).  Adding and subtracting 2^23 times the
     * spacing rounds to nearest even in one IEEE addition. */
    int k = (int)(mag >> 23) - 127;
    if (k < 1 - F->bias) k = 1 - F->bias;
    const float spacing = ldexpf(1.0f, k - F->mbits);
    const float big = spacing * 8388608.0f * 1.5f;
    float r = (u2f(mag) + big) - big;
    if (r > maxv) r = maxv; /* rounding up past the maximum clamps */
    return u2f(sign | f2u(r));
}

/* ref: 218-245 quant_dequant_common<E,M,use_cuda_cast> */
static float quant_dequant(float x, int fmt, int cuda_cast) {
    if (cuda_cast && (fmt == FMT_E4M3 || fmt == FMT_E5M2)) return narrow_satfinite(x, fmt);
    return narrow_custom(x, fmt);
}

/* flag word collecting the device-side assert()s of the reference that a given
 * input would trip (the reference is built without NDEBUG).  Inputs that set a
 * flag are outside the reference's domain and are never run on its GPU code. */
enum {
    MOR_O_ASSERT_E8_EXPONENT = 1,   /* ref: 286, 302 */
    MOR_O_ASSERT_SCALE_1E30 = 2,    /* ref: 761, 775, 789 */
    MOR_O_ASSERT_NNZ_ZERO = 4,      /* ref: 1047 */
    MOR_O_ASSERT_AMAX_ZERO = 8,     /* ref: 1338, 1343 */
};
static int g_assert_flags = 0;
MOR_O_API int mor_o_assert_flags(void) { return g_assert_flags; }
MOR_O_API void mor_o_clear_assert_flags(void) { g_assert_flags = 0; }
static inline void raise_flag(int f) {
#pragma omp atomic
    g_assert_flags |= f;
}

/* ref: 310-316 */
static float sqdd_fp32_scale(float x, float s, int fmt, int cuda_cast) {
    volatile float scaled = x * s;
    float q = quant_dequant(scaled, fmt, cuda_cast);
    volatile float out = q / s;
    /* a NaN that arithmetic produces on the GPU is the canonical 0x7fffffff (x86 would
     * give 0xffc00000 for 0/0); it matters because fp32_to_bf16 maps the former to 0x8000 */
    if (out != out) return u2f(NAN_ALL_ONES);
    return out;
}

/* ref: 248-306.  Power-of-two scaling done on the exponent FIELD: the scale is
 * 2^(exponent field of s - 127) (round toward zero; the RNE variant may add one),
 * scaling adds it to the value's exponent field and clamps the field at 0, the
 * mantissa is carried along untouched (zeros and subnormals are not special-cased),
 * and descaling subtracts it again with the same clamp. */
static float sqdd_e8_scale(float x, float s, int fmt, int cuda_cast, int rne) {
    const uint32_t sb = f2u(s);
    int e8 = (int)((sb >> 23) & 0xFFu) - 127;
    const uint32_t xb = f2u(x);
    const uint32_t xsign = xb >> 31;
    int xexp = (int)((xb >> 23) & 0xFFu);
    const uint32_t xman = xb & 0x7FFFFFu;
    if (rne) {
        const uint32_t sman = sb & 0x7FFFFFu;
        const uint32_t guard = (sman >> 22) & 1u;
        const uint32_t sticky = (sman & ((1u << 22) - 1u)) != 0;
        /* 6815744 = 0b1101 << 19: the largest mantissa that still rounds down to 1.75 */
        if (guard && xman <= 6815744u && xexp + e8 < 135) {
            if (sticky | ((uint32_t)e8 & 1u)) e8 += 1;
        }
    }
    xexp += e8;
    if (xexp < 0) xexp = 0;
    if (xexp > 254) raise_flag(MOR_O_ASSERT_E8_EXPONENT);
    const float scaled = u2f((xsign << 31) | ((uint32_t)xexp << 23) | xman);
    const float q = quant_dequant(scaled, fmt, cuda_cast);
    const uint32_t qb = f2u(q);
    int qexp = (int)((qb >> 23) & 0xFFu) - e8;
    if (qexp < 0) qexp = 0;
    if (qexp > 254) raise_flag(MOR_O_ASSERT_E8_EXPONENT);
    return u2f((qb & 0x80000000u) | ((uint32_t)qexp << 23) | (qb & 0x7FFFFFu));
}

enum { SF_FP32 = 1, SF_E8 = 2 };

/* ref: 319-379.  Every named wrapper uses E8_RZ; E4M3/E5M2 go through the
 * saturating cast, E2M3 through the custom one. */
static float sqdd(float x, float s, int sf_type, int fmt) {
    const int cuda_cast = (fmt == FMT_E4M3 || fmt == FMT_E5M2);
    return (sf_type == SF_E8) ? sqdd_e8_scale(x, s, fmt, cuda_cast, 0)
                              : sqdd_fp32_scale(x, s, fmt, cuda_cast);
}

/* exported element-level entry points (used by the exhaustive sweeps) */
MOR_O_API float mor_o_quant_dequant_custom(float x, int fmt) { return narrow_custom(x, fmt); }
MOR_O_API float mor_o_quant_dequant_satfinite(float x, int fmt) { return narrow_satfinite(x, fmt); }
MOR_O_API float mor_o_sqdd(float x, float s, int sf_type, int fmt) { return sqdd(x, s, sf_type, fmt); }
MOR_O_API float mor_o_sqdd_e8_custom(float x, float s, int rne) { return sqdd_e8_scale(x, s, FMT_E4M3, 0, rne); }

/* ------------------------------------------------------------------------- */
/* input access: bf16 bits or binary32, one logical "word" = elements (2w, 2w+1) */
/* The reference reads packed uint32 words; it calls the HIGH half (element     */
/* 2w+1) value1 and the LOW half (element 2w) value2 (ref: 423-424).            */
/* ------------------------------------------------------------------------- */
typedef struct {
    const void *in;
    void *out;
    int is_fp32; /* 0: bf16 in, bf16 out.  1: binary32 in, binary32 out (extension) */
} io_t;

static inline float load_elem(const io_t *io, int64_t idx) {
    if (io->is_fp32) return ((const float *)io->in)[idx];
    return u2f((uint32_t)((const uint16_t *)io->in)[idx] << 16);
}
static inline void store_elem(const io_t *io, int64_t idx, float v) {
    if (io->is_fp32) ((float *)io->out)[idx] = v;
    else ((uint16_t *)io->out)[idx] = (uint16_t)mor_o_fp32_to_bf16(v);
}
static inline void copy_elem(const io_t *io, int64_t idx) {
    if (io->is_fp32) ((float *)io->out)[idx] = ((const float *)io->in)[idx];
    else ((uint16_t *)io->out)[idx] = ((const uint16_t *)io->in)[idx];
}

/* ------------------------------------------------------------------------- */
/* CTA-shaped float sums                                                     */
/* ------------------------------------------------------------------------- */
/* ref: 399-405 + 546-575 / 917-948.  v[] holds one partial sum per thread of a
 * CTA in flattened-thread order (n a multiple of 32, at most 1024).  Each warp
 * folds with v[l] += v[l+off], off = 16,8,4,2,1 (what lane 0 of a shfl_down tree
 * sees); lane 0 of warp w parks its sum in slot w; warp 0 reloads the slots
 * (zero beyond the warp count) and folds them the same way. */
static float cta_tree_sum(float *v, int n) {
    float slots[32];
    const int nwarps = n / 32;
    for (int w = 0; w < 32; ++w) slots[w] = 0.0f;
    for (int w = 0; w < nwarps; ++w) {
        float *p = v + 32 * w;
        for (int off = 16; off > 0; off >>= 1)
            for (int l = 0; l < off; ++l) p[l] = p[l] + p[l + off];
        slots[w] = p[0];
    }
    for (int off = 16; off > 0; off >>= 1)
        for (int l = 0; l < off; ++l) slots[l] = slots[l] + slots[l + off];
    return slots[0];
}

/* ref: 1178-1201 (and 1017-1049 for the order-free amax/nnz): one CTA of 1024
 * threads, thread t adds entries t, t+1024, ... in that order, then the tree. */
static float global_sum_1024(const float *a, int64_t n) {
    float part[1024];
    for (int t = 0; t < 1024; ++t) {
        float s = 0.0f;
        for (int64_t i = t; i < n; i += 1024) s += a[i];
        part[t] = s;
    }
    return cta_tree_sum(part, 1024);
}

/* ------------------------------------------------------------------------- */
/* fake_quantize (quantize_kernel)                                           */
/* ------------------------------------------------------------------------- */
enum { QM_MOR = 1, QM_BLOCK_E4M3 = 2, QM_BLOCK_E5M2 = 3, QM_CUR_E4M3 = 4, QM_CUR_E5M2 = 5, QM_BF16 = 7 };
enum { MOR_DYNAMIC_RANGE = 1, MOR_QUANT_ERROR = 2 };
enum { Q_E4M3 = 1, Q_E5M2 = 2, Q_BF16 = 3, Q_E2M3 = 4, Q_E4M3_SMALL = 11, Q_E5M2_SMALL = 12 };

/* CTA shape the reference launches for a block (ref: 1770-1790), in packed words
 * along x.  Blocks of at most 1024 elements get one thread per word. */
static void fq_cta_shape(int brows, int bcols, int *tx, int *ty) {
    if ((int64_t)brows * bcols > 1024) { *tx = 16; *ty = 32; }
    else { *tx = bcols / 2; *ty = brows; }
}

/* ref: 487-584 get_block_error<SF>: per thread, rows then words, add (e_high +
 * e_low) per word, for E4M3 (scale 448/amax) and E5M2 (scale 57344/amax), with
 * e = |q/x - 1| for x != 0. */
static void block_errors(const io_t *io, int64_t rows, int64_t cols, int64_t r0, int64_t c0w,
                         int brows, int bcolsw, int sf_type, float amax,
                         float *err4_out, float *err5_out) {
    int tx, ty;
    fq_cta_shape(brows, bcolsw * 2, &tx, &ty);
    const int nthreads = tx * ty;
    float *e4 = (float *)malloc(sizeof(float) * 2 * (size_t)nthreads);
    float *e5 = e4 + nthreads;
    const int64_t colsw = cols / 2;
    volatile float s4 = 448.0f / amax;
    volatile float s5 = 57344.0f / amax;
    for (int j = 0; j < ty; ++j)
        for (int i = 0; i < tx; ++i) {
            float a4 = 0.0f, a5 = 0.0f;
            for (int64_t r = r0 + j; r < r0 + brows && r < rows; r += ty)
                for (int64_t w = c0w + i; w < c0w + bcolsw && w < colsw; w += tx) {
                    const float hi = load_elem(io, r * cols + 2 * w + 1);
                    const float lo = load_elem(io, r * cols + 2 * w);
                    {
                        const float qh = sqdd(hi, s4, sf_type, FMT_E4M3);
                        const float ql = sqdd(lo, s4, sf_type, FMT_E4M3);
                        float eh = 0.0f, el = 0.0f;
                        if (hi != 0.0f) { volatile float t = qh / hi; eh = fabsf(t - 1.0f); }
                        if (lo != 0.0f) { volatile float t = ql / lo; el = fabsf(t - 1.0f); }
                        volatile float pair = eh + el;
                        a4 += pair;
                    }
                    {
                        const float qh = sqdd(hi, s5, sf_type, FMT_E5M2);
                        const float ql = sqdd(lo, s5, sf_type, FMT_E5M2);
                        float eh = 0.0f, el = 0.0f;
                        if (hi != 0.0f) { volatile float t = qh / hi; eh = fabsf(t - 1.0f); }
                        if (lo != 0.0f) { volatile float t = ql / lo; el = fabsf(t - 1.0f); }
                        volatile float pair = eh + el;
                        a5 += pair;
                    }
                }
            e4[j * tx + i] = a4;
            e5[j * tx + i] = a5;
        }
    *err4_out = cta_tree_sum(e4, nthreads);
    *err5_out = cta_tree_sum(e5, nthreads);
    free(e4);
}

/* ref: 610-682 choose_mor_quant_type */
static int choose_repr(const io_t *io, int64_t rows, int64_t cols, int64_t r0, int64_t c0w,
                       int brows, int bcolsw, int sf_type, float clamp, int mor_mode,
                       float amax, float amin) {
    float range = 0.0f;
    if (amax == 0.0f) { amax = clamp; range = 1.0f; }
    if (range == 0.0f) { volatile float t = amax / amin; range = t; }
    uint32_t e4_range = 28672u;
    if (mor_mode == MOR_QUANT_ERROR) e4_range *= 4u;
    const uint32_t e5_range = 939524096u;
    if (range <= 7.5f) return Q_E2M3;
    if (range <= (float)e4_range) return (amax <= clamp) ? Q_E4M3_SMALL : Q_E4M3;
    if (range <= (float)e5_range) {
        if (mor_mode == MOR_DYNAMIC_RANGE) return (amax <= clamp) ? Q_E5M2_SMALL : Q_E5M2;
        float err4, err5;
        block_errors(io, rows, cols, r0, c0w, brows, bcolsw, sf_type, amax, &err4, &err5);
        if (err4 <= err5) return (amax <= clamp) ? Q_E4M3_SMALL : Q_E4M3;
        return Q_BF16; /* E5M2 is never picked by the error criterion */
    }
    return Q_BF16;
}

/* ref: 684-852 quantize_kernel + 1757-1835 launcher.  meta is [ceil(rows/brows),
 * ceil((cols/2)/(bcols/2))] int32.  Returns 0, or a negative code for arguments
 * the reference rejects or on which its CTA shape is undefined. */
static int fake_quantize_impl(const io_t *io, int32_t *meta, int64_t rows, int64_t cols,
                              int brows, int bcols, double clamp_d, int mode, int sf_type) {
    if (rows <= 0 || cols <= 0 || brows <= 0 || bcols < 2) return -1;
    if (cols % 2 || bcols % 2) return -1;
    if (sf_type != SF_FP32 && sf_type != SF_E8) return -1;
    int qm = mode % 10;
    if (qm != QM_MOR && qm != QM_BLOCK_E4M3 && qm != QM_BLOCK_E5M2 && qm != QM_CUR_E4M3 && qm != QM_CUR_E5M2)
        qm = QM_BF16; /* ref: 1831 */
    const int mor_mode = (mode / 100 > 0) ? MOR_DYNAMIC_RANGE : MOR_QUANT_ERROR;
    if (qm == QM_MOR) {
        int tx, ty;
        if ((int64_t)brows * bcols > 1024 && (brows < 32 || bcols < 32)) return -2; /* ref: 1781-1784 */
        fq_cta_shape(brows, bcols, &tx, &ty);
        if ((tx * ty) % 32 || tx * ty > 1024) return -2; /* partial warps: undefined in the reference */
    }
    const float clamp = (float)clamp_d;
    const int bcolsw = bcols / 2;
    const int64_t colsw = cols / 2;
    const int64_t gx = (colsw - 1) / bcolsw + 1, gy = (rows - 1) / brows + 1;

#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t by = 0; by < gy; ++by)
        for (int64_t bx = 0; bx < gx; ++bx) {
            const int64_t r0 = by * brows, c0w = bx * bcolsw;
            const int64_t r1 = (r0 + brows < rows) ? r0 + brows : rows;
            const int64_t w1 = (c0w + bcolsw < colsw) ? c0w + bcolsw : colsw;
            float amax = 0.0f, amin = 0.0f;
            if (qm != QM_CUR_E4M3 && qm != QM_CUR_E5M2) { /* ref: 407-485 */
                amin = u2f(0x7F7F0000u);
                for (int64_t r = r0; r < r1; ++r)
                    for (int64_t c = 2 * c0w; c < 2 * w1; ++c) {
                        const float a = fabsf(load_elem(io, r * cols + c));
                        amax = fmaxf(amax, a);
                        if (a > 0.0f) amin = fminf(amin, a);
                    }
            }
            int repr = 0, code = 3;
            if (qm == QM_MOR) {
                repr = choose_repr(io, rows, cols, r0, c0w, brows, bcolsw, sf_type, clamp, mor_mode, amax, amin);
                code = repr;
            } else if (qm == QM_BLOCK_E4M3 || qm == QM_CUR_E4M3) code = 1;
            else if (qm == QM_BLOCK_E5M2 || qm == QM_CUR_E5M2) code = 2;
            meta[by * gx + bx] = code;

            int fmt = -1;
            float scale = 1.0f;
            if (qm == QM_MOR) {
                if (repr == Q_E2M3) fmt = FMT_E2M3;
                else if (repr == Q_E4M3 || repr == Q_E4M3_SMALL) fmt = FMT_E4M3;
                else if (repr == Q_E5M2 || repr == Q_E5M2_SMALL) fmt = FMT_E5M2;
            } else if (qm == QM_BLOCK_E4M3 || qm == QM_CUR_E4M3) fmt = FMT_E4M3;
            else if (qm == QM_BLOCK_E5M2 || qm == QM_CUR_E5M2) fmt = FMT_E5M2;
            if (qm == QM_CUR_E4M3 || qm == QM_CUR_E5M2) {
                scale = clamp; /* the scale is handed in through clamp_threshold (ref: 825-842) */
            } else if (fmt >= 0) {
                if (amax > 0.0f) {
                    const float maxv = (fmt == FMT_E2M3) ? 7.5f : (fmt == FMT_E4M3 ? 448.0f : 57344.0f);
                    volatile float t = maxv / amax;
                    scale = t;
                    if (qm == QM_MOR && !(scale < 1e30f)) raise_flag(MOR_O_ASSERT_SCALE_1E30);
                } else fmt = -1; /* all-zero block is copied through (ref: 759, 773, 787, 802, 814) */
            }
            for (int64_t r = r0; r < r1; ++r)
                for (int64_t c = 2 * c0w; c < 2 * w1; ++c) {
                    const int64_t idx = r * cols + c;
                    if (fmt < 0) copy_elem(io, idx);
                    else store_elem(io, idx, sqdd(load_elem(io, idx), scale, sf_type, fmt));
                }
        }
    return 0;
}

MOR_O_API int mor_o_fake_quantize(const uint16_t *in, uint16_t *out, int32_t *meta, int64_t rows, int64_t cols,
                                  int brows, int bcols, double clamp, int mode, int sf_type) {
    io_t io = {in, out, 0};
    return fake_quantize_impl(&io, meta, rows, cols, brows, bcols, clamp, mode, sf_type);
}
MOR_O_API int mor_o_fake_quantize_f32(const float *in, float *out, int32_t *meta, int64_t rows, int64_t cols,
                                      int brows, int bcols, double clamp, int mode, int sf_type) {
    io_t io = {in, out, 1};
    return fake_quantize_impl(&io, meta, rows, cols, brows, bcols, clamp, mode, sf_type);
}

/* ------------------------------------------------------------------------- */
/* block / channel scaling pipeline                                          */
/* ------------------------------------------------------------------------- */
enum { SS_GLOBAL_AMAX = 1, SS_BLOCK_AMAX = 2, SS_E8 = 3, SS_CURRENT = 4 };

/* ref: 1059-1093 get_scaling_factor<SS> */
MOR_O_API float mor_o_scaling_factor(int ss, float global_amax, float block_amax) {
    float sf = 1.0f;
    if (block_amax < 1e-35f) block_amax = 1e-35f;
    if (ss == SS_GLOBAL_AMAX) {
        volatile float ratio = 448.0f / global_amax;
        const uint32_t gman = f2u(ratio) & 0x007FFFFFu;
        volatile float bsf = 448.0f / block_amax;
        const uint32_t bb = f2u(bsf);
        const float adj = u2f((bb & 0xFF800000u) | gman);
        volatile float half = adj / 2.0f;
        sf = (gman <= (bb & 0x007FFFFFu)) ? adj : half;
    } else if (ss == SS_BLOCK_AMAX || ss == SS_E8) {
        volatile float t = 448.0f / block_amax;
        sf = t;
    } else if (ss == SS_CURRENT) {
        if (global_amax > 0.0f) { volatile float t = 448.0f / global_amax; sf = t; }
    }
    return sf;
}

/* The element step of block_e4m3_relative_error[_channel] (ref: 1133-1162,
 * 1712-1740).  `if constexpr (T_SCALING_STRATEGY == SF_E8)` compares a
 * ScalingStrategy with the enumerator SF_E8 == 2, so it is ss_mode 2 that takes the
 * power-of-two path and ss_mode 3 that takes the binary32-scale path. */
static inline float err_step(float x, float sf, int ss, float *deq_out) {
    float deq = 0.0f, err = 0.0f;
    if (x != 0.0f) {
        deq = sqdd(x, sf, (ss == 2) ? SF_E8 : SF_FP32, FMT_E4M3);
        volatile float d = deq - x;
        volatile float q = d / x;
        err = fabsf(q);
    }
    *deq_out = deq; /* zeros are written back as +0 */
    return err;
}

typedef struct {
    int32_t meta;
    float global_amax;
    int64_t global_nnz;
    float global_error;
} scal_out_t;

/* Tensor-level tail shared by the block and channel pipelines: ordered sum of the
 * per-block errors (ref: 1178-1201), the BF16 fallback test (ref: 1203-1241; the
 * average is error / float(nnz)) and, when it fires, the copy of the input over the
 * output.  The reference's copy covers the tensor for 128x128-style blocks and full
 * rows; for 1xk groups with k < 128 and for column blocks its loop bounds miss part
 * of the tensor, which this oracle treats as a defect: the intended result (what the
 * reference's tests assert, test_fake_quantize_channel_scaling.py:384,433) is
 * output == input. */
static void finish_scaling(const io_t *io, int64_t n_elems, const float *block_err, int64_t n_err,
                           float thr, scal_out_t *o) {
    o->global_error = global_sum_1024(block_err, n_err);
    volatile float avg = o->global_error / (float)o->global_nnz;
    if (avg > thr) {
        o->meta = 3;
        for (int64_t i = 0; i < n_elems; ++i) copy_elem(io, i);
    } else o->meta = 1;
}

/* ref: 2013-2102 (+ kernels 951-1241), blocks of brows x bcols with a 32x32-thread
 * CTA: thread (tx,ty) walks rows ty, ty+32, ... and words tx, tx+32, ... of the
 * block, adding the high-half error, then the low-half error, of each word. */
static int block_scaling_impl(const io_t *io, int64_t rows, int64_t cols, int brows, int bcols,
                              double thr_d, int ss, const float *ext_global_amax, scal_out_t *o,
                              float *block_amax_out, float *block_err_out) {
    if (rows <= 0 || cols <= 0 || ss < 1 || ss > 4) return -1;
    if (rows % brows || cols % bcols) return -1;
    if (brows % 32 || bcols % 64) return -2; /* the 32x32 CTA strides the block unguarded */
    const int bcolsw = bcols / 2;
    const int64_t gx = cols / bcols, gy = rows / brows, nb = gx * gy;
    float *bamax = (float *)malloc(sizeof(float) * (size_t)nb * 2);
    float *berr = bamax + nb;
    int64_t nnz = 0;
    float gamax = -FLT_MAX;
#pragma omp parallel for collapse(2) reduction(+ : nnz) reduction(max : gamax)
    for (int64_t by = 0; by < gy; ++by)
        for (int64_t bx = 0; bx < gx; ++bx) {
            float a = -INFINITY;
            for (int64_t r = by * brows; r < (by + 1) * brows; ++r)
                for (int64_t c = bx * bcols; c < (bx + 1) * bcols; ++c) {
                    const float v = fabsf(load_elem(io, r * cols + c));
                    if (v > 0.0f) nnz += 1;
                    a = fmaxf(a, v);
                }
            bamax[by * gx + bx] = a;
            gamax = fmaxf(gamax, a);
        }
    if (ext_global_amax) gamax = *ext_global_amax; /* row-sharded use: amax of the whole tensor */
    if (nnz == 0) raise_flag(MOR_O_ASSERT_NNZ_ZERO);
    o->global_amax = gamax;
    o->global_nnz = nnz;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t by = 0; by < gy; ++by)
        for (int64_t bx = 0; bx < gx; ++bx) {
            const float sf = mor_o_scaling_factor(ss, gamax, bamax[by * gx + bx]);
            float part[1024];
            for (int ty = 0; ty < 32; ++ty)
                for (int tx = 0; tx < 32; ++tx) {
                    float acc = 0.0f;
                    for (int64_t r = by * brows + ty; r < (by + 1) * (int64_t)brows; r += 32)
                        for (int64_t w = bx * bcolsw + tx; w < (bx + 1) * (int64_t)bcolsw; w += 32) {
                            float dh, dl;
                            const int64_t i = r * cols + 2 * w;
                            acc += err_step(load_elem(io, i + 1), sf, ss, &dh);
                            acc += err_step(load_elem(io, i), sf, ss, &dl);
                            store_elem(io, i + 1, dh);
                            store_elem(io, i, dl);
                        }
                    part[ty * 32 + tx] = acc;
                }
            berr[by * gx + bx] = cta_tree_sum(part, 1024);
        }
    if (block_amax_out) memcpy(block_amax_out, bamax, sizeof(float) * (size_t)nb);
    if (block_err_out) memcpy(block_err_out, berr, sizeof(float) * (size_t)nb);
    finish_scaling(io, rows * cols, berr, nb, (float)thr_d, o);
    free(bamax);
    return 0;
}

/* ref: 2431-2526 (+ kernels 1430-1752) with the launch geometry of the e2m3 fork
 * (mor/csrc/cuda/e2m3/fake_quantize_e2m3.cu:2518: grid.y = number of row blocks),
 * which is the one under which every block is visited exactly once.
 *   1 x k row groups, CTA of 64 threads over max(k,128) columns of one row:
 *       thread t owns words t, t+64, ...; separate sums for high and low halves,
 *       added at the end; tree over the 2 warps; the CTA's sum is stored in the
 *       first of its 128/k block slots (k < 128), the others hold 0.
 *   k x 1 column groups, CTA of 32x16 threads over 64 columns x k rows:
 *       thread (tx,ty) owns word tx of rows ty, ty+16, ...; the CTA's sum lands in
 *       the first of its 64 block slots. */
static int channel_scaling_impl(const io_t *io, int64_t rows, int64_t cols, int brows, int bcols,
                                double thr_d, int ss, scal_out_t *o) {
    if (rows <= 0 || cols <= 0 || ss < 1 || ss > 4) return -1;
    if (!(brows == 1 || bcols == 1)) return -1; /* ref: 2501 */
    if (rows % brows || cols % bcols || cols % 2) return -1;
    int64_t n_cta, slots_per_cta;
    if (brows == 1) {
        if (bcols < 128) {
            if (bcols < 2 || 128 % bcols || bcols > 64 || cols % 128) return -2; /* ref: 2407-2414 */
            slots_per_cta = 128 / bcols;
        } else {
            if (bcols % 128) return -2;
            slots_per_cta = 1;
        }
        n_cta = rows * (cols / (bcols < 128 ? 128 : bcols));
    } else {
        if (cols % 64 || brows % 16) return -2;
        slots_per_cta = 64;
        n_cta = (rows / brows) * (cols / 64);
    }
    const int64_t nb = (rows / brows) * (cols / bcols);
    float *bamax = (float *)malloc(sizeof(float) * (size_t)nb * 2);
    float *berr = bamax + nb;
    memset(berr, 0, sizeof(float) * (size_t)nb);
    int64_t nnz = 0;
    float gamax = -FLT_MAX;
    const int64_t gxb = cols / bcols; /* blocks per block-row, natural row-major block index */
#pragma omp parallel for reduction(+ : nnz) reduction(max : gamax)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t r0 = (b / gxb) * brows, c0 = (b % gxb) * bcols;
        float a = 0.0f;
        for (int64_t r = r0; r < r0 + brows; ++r)
            for (int64_t c = c0; c < c0 + bcols; ++c) {
                const float v = fabsf(load_elem(io, r * cols + c));
                if (v > 0.0f) nnz += 1;
                a = fmaxf(a, v);
            }
        bamax[b] = a;
        gamax = fmaxf(gamax, a);
    }
    if (nnz == 0) raise_flag(MOR_O_ASSERT_NNZ_ZERO);
    o->global_amax = gamax;
    o->global_nnz = nnz;

    if (brows == 1) {
        const int64_t span = (bcols < 128) ? 128 : bcols; /* columns per CTA */
        const int64_t ctas_per_row = cols / span;
#pragma omp parallel for schedule(dynamic, 16)
        for (int64_t cta = 0; cta < n_cta; ++cta) {
            const int64_t r = cta / ctas_per_row, c0 = (cta % ctas_per_row) * span;
            float part[64];
            for (int t = 0; t < 64; ++t) {
                float eh = 0.0f, el = 0.0f;
                for (int64_t w = c0 / 2 + t; w < (c0 + span) / 2; w += 64) {
                    const int64_t i = r * cols + 2 * w;
                    const int64_t blk = r * gxb + (2 * w) / bcols;
                    const float sf = mor_o_scaling_factor(ss, gamax, bamax[blk]);
                    float dh, dl;
                    eh += err_step(load_elem(io, i + 1), sf, ss, &dh);
                    el += err_step(load_elem(io, i), sf, ss, &dl);
                    store_elem(io, i + 1, dh);
                    store_elem(io, i, dl);
                }
                part[t] = eh + el;
            }
            berr[cta * slots_per_cta] = cta_tree_sum(part, 64);
        }
    } else {
        const int64_t ctas_per_row = cols / 64;
#pragma omp parallel for schedule(dynamic, 1)
        for (int64_t cta = 0; cta < n_cta; ++cta) {
            const int64_t r0 = (cta / ctas_per_row) * brows, c0 = (cta % ctas_per_row) * 64;
            float part[512];
            for (int ty = 0; ty < 16; ++ty)
                for (int tx = 0; tx < 32; ++tx) {
                    const int64_t ch = c0 + 2 * tx + 1, cl = c0 + 2 * tx;
                    const float sfh = mor_o_scaling_factor(ss, gamax, bamax[(r0 / brows) * gxb + ch]);
                    const float sfl = mor_o_scaling_factor(ss, gamax, bamax[(r0 / brows) * gxb + cl]);
                    float eh = 0.0f, el = 0.0f;
                    for (int64_t r = r0 + ty; r < r0 + brows; r += 16) {
                        float dh, dl;
                        eh += err_step(load_elem(io, r * cols + ch), sfh, ss, &dh);
                        el += err_step(load_elem(io, r * cols + cl), sfl, ss, &dl);
                        store_elem(io, r * cols + ch, dh);
                        store_elem(io, r * cols + cl, dl);
                    }
                    part[ty * 32 + tx] = eh + el;
                }
            berr[cta * slots_per_cta] = cta_tree_sum(part, 512);
        }
    }
    finish_scaling(io, rows * cols, berr, nb, (float)thr_d, o);
    free(bamax);
    return 0;
}

static void unpack_scal(const scal_out_t *o, int32_t *meta, float *gamax, int64_t *gnnz, float *gerr) {
    *meta = o->meta; *gamax = o->global_amax; *gnnz = o->global_nnz; *gerr = o->global_error;
}

MOR_O_API int mor_o_block_scaling(const void *in, void *out, int is_fp32, int64_t rows, int64_t cols, int brows,
                                  int bcols, double thr, int ss, const float *ext_global_amax, int32_t *meta,
                                  float *gamax, int64_t *gnnz, float *gerr, float *block_amax, float *block_err) {
    io_t io = {in, out, is_fp32};
    scal_out_t o;
    int rc = block_scaling_impl(&io, rows, cols, brows, bcols, thr, ss, ext_global_amax, &o, block_amax, block_err);
    if (rc == 0) unpack_scal(&o, meta, gamax, gnnz, gerr);
    return rc;
}
MOR_O_API int mor_o_channel_scaling(const void *in, void *out, int is_fp32, int64_t rows, int64_t cols, int brows,
                                    int bcols, double thr, int ss, int32_t *meta, float *gamax, int64_t *gnnz,
                                    float *gerr) {
    io_t io = {in, out, is_fp32};
    scal_out_t o;
    int rc = channel_scaling_impl(&io, rows, cols, brows, bcols, thr, ss, &o);
    if (rc == 0) unpack_scal(&o, meta, gamax, gnnz, gerr);
    return rc;
}

/* ------------------------------------------------------------------------- */
/* E8Mx                                                                      */
/* ------------------------------------------------------------------------- */
/* ref: 1243-1327 quant_dequant_e8m{1,2,3}: keep the 8-bit exponent, round the
 * 23-bit mantissa to m bits.  The thresholds of the reference are exactly the
 * "<= midpoint rounds down on even, < midpoint on odd" grid of round-to-nearest-even
 * on the top 7 mantissa bits; lower mantissa bits only matter above a threshold. */
static float e8m_round(float v, int m) {
    const uint32_t b = f2u(v);
    const uint32_t sign = b >> 31;
    uint32_t e = (b >> 23) & 0xFFu, man = b & 0x7FFFFFu;
    if (e == 0) man = 0;
    else if (e != 255) {
        const int steps = 1 << m;             /* grid points per binade        */
        const uint32_t step = 0x800000u >> m; /* grid spacing in mantissa units */
        uint32_t k = 0;                       /* chosen grid index, steps = carry */
        /* thresholds: index j is chosen while man <= (j*step + step/2) for even j,
         * and while man <= (j*step + step/2 - 65536) for odd j (ref: 1253-1254,
         * 1280-1283, 1307-1314: 32,95 | 16,47,80,111 | 8,23,40,55,72,87,104,119, all << 16) */
        for (k = 0; k < (uint32_t)steps; ++k) {
            uint32_t lim = k * step + step / 2;
            if (k & 1u) lim -= 65536u;
            if (man <= lim) break;
        }
        if (k < (uint32_t)steps) man = k * step;
        else {
            man = 0; e += 1;
            if (e == 255) { e = 254; man = (uint32_t)(steps - 1) * step; }
        }
    }
    return u2f((sign << 31) | (e << 23) | man);
}
MOR_O_API float mor_o_e8m_round(float v, int m) { return e8m_round(v, m); }

/* ref: 1335-1359 e8mx_scaling_factor<type, SS_GLOBAL_AMAX> (any other strategy: 1.0) */
MOR_O_API float mor_o_e8mx_scale(float gamax, int m, int strategy) {
    if (!(gamax > 0.0f)) raise_flag(MOR_O_ASSERT_AMAX_ZERO);
    if (strategy != SS_GLOBAL_AMAX) return 1.0f;
    uint32_t e = (f2u(gamax) >> 23) + 1;
    if (!(e < 255)) raise_flag(MOR_O_ASSERT_AMAX_ZERO);
    const uint32_t ones = ((1u << m) - 1u) << (23 - m);
    const float fp_max = u2f((e << 23) | ones);
    volatile float s = fp_max / gamax;
    if (s >= 2.0f) { volatile float h = s / 2.0f; return h; }
    return s;
}

/* ref: 2232-2313 + 1361-1428.  block shape only tiles the launch; result is elementwise. */
MOR_O_API int mor_o_e8mx(const uint16_t *in, uint16_t *out, int64_t rows, int64_t cols, int qtype, int strategy,
                         float *gamax_out) {
    if (qtype < 1 || qtype > 3 || rows <= 0 || cols <= 0) return -1;
    const int64_t n = rows * cols;
    float gamax = -FLT_MAX;
    int64_t nnz = 0;
#pragma omp parallel for reduction(max : gamax) reduction(+ : nnz)
    for (int64_t i = 0; i < n; ++i) {
        const float a = fabsf(u2f((uint32_t)in[i] << 16));
        gamax = fmaxf(gamax, a);
        nnz += a > 0.0f;
    }
    if (nnz == 0) raise_flag(MOR_O_ASSERT_NNZ_ZERO);
    if (gamax_out) *gamax_out = gamax;
    const float s = mor_o_e8mx_scale(gamax, qtype, strategy);
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) {
        volatile float v = u2f((uint32_t)in[i] << 16) * s;
        float d = 0.0f;
        if (v != 0.0f) d = e8m_round(v, qtype);
        volatile float r = d / s;
        out[i] = (uint16_t)mor_o_fp32_to_bf16(r);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* test operators                                                            */
/* ------------------------------------------------------------------------- */
/* ref: 854-863, 1909-1964: binary32 in/out, custom cast, no scaling */
MOR_O_API int mor_o_quant_dequant(const float *in, float *out, int64_t n, int fmt) {
    if (fmt < 0 || fmt > 3) return -1;
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) out[i] = narrow_custom(in[i], fmt);
    return 0;
}
/* ref: 865-875, 1966-2011: per-element scale 448/x, power-of-two rounded */
MOR_O_API int mor_o_e4m3_with_e8_scale(const float *in, float *out, int64_t n, int rne) {
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) {
        volatile float s = (float)(448.0 / (double)in[i]); /* 448.0 is a double literal in the reference */
        out[i] = sqdd_e8_scale(in[i], s, FMT_E4M3, 0, rne);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* extension: per-group fake-quantize without the tensor-level pipeline      */
/* ------------------------------------------------------------------------- */
/* MX-style 1 x k groups (and any brows x bcols block): group amax, scale
 * max_normal/amax (power-of-two truncated when sf_type == SF_E8), element cast
 * with the reference's SQDD_{fp32,e8}_{e4m3,e5m2,e2m3} wrappers (ref: 356-379),
 * i.e. quantize_kernel<BLOCK_SCALING_*> semantics (ref: 801-823) extended to E2M3
 * and to block shapes its launcher refuses.  Optionally reports the E8M0 / binary32
 * scale of every group. */
MOR_O_API int mor_o_fake_quantize_group(const void *in, void *out, int is_fp32, float *scales, int64_t rows,
                                        int64_t cols, int brows, int bcols, int fmt, int sf_type) {
    if (rows <= 0 || cols <= 0 || brows <= 0 || bcols <= 0) return -1;
    if (rows % brows || cols % bcols) return -1;
    if (!(fmt == FMT_E4M3 || fmt == FMT_E5M2 || fmt == FMT_E2M3)) return -1;
    if (sf_type != SF_FP32 && sf_type != SF_E8) return -1;
    io_t io = {in, out, is_fp32};
    const int64_t gx = cols / bcols, nb = (rows / brows) * gx;
    const float maxv = (fmt == FMT_E2M3) ? 7.5f : (fmt == FMT_E4M3 ? 448.0f : 57344.0f);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t r0 = (b / gx) * brows, c0 = (b % gx) * bcols;
        float amax = 0.0f;
        for (int64_t r = r0; r < r0 + brows; ++r)
            for (int64_t c = c0; c < c0 + bcols; ++c) amax = fmaxf(amax, fabsf(load_elem(&io, r * cols + c)));
        float scale = 1.0f;
        if (amax > 0.0f) { volatile float t = maxv / amax; scale = t; }
        if (scales) scales[b] = (sf_type == SF_E8 && amax > 0.0f) ? u2f(f2u(scale) & 0x7F800000u) : scale;
        for (int64_t r = r0; r < r0 + brows; ++r)
            for (int64_t c = c0; c < c0 + bcols; ++c) {
                const int64_t i = r * cols + c;
                if (amax > 0.0f) store_elem(&io, i, sqdd(load_elem(&io, i), scale, sf_type, fmt));
                else copy_elem(&io, i);
            }
    }
    return 0;
}

/* Extension (no reference operator): the REAL quantized form of fake_quantize_group with a
 * power-of-two scale -- what the casts inside SQDD_e8_* (ref: 283-305, 356-379) produce before
 * they are widened again.  payload[i] is the narrow-float code of element i (E4M3 / E5M2: the
 * fp8 byte; E2M3: the 6-bit code in a byte), scales[g] the E8M0 byte of group g in the MX
 * convention: element = decode(code) * 2^(scales[g] - 127).  A zero group has scale byte 127.
 * A code of zero decodes to zero; fake quantization returns 2^(-e8-127) there when the
 * scale is below one (an artefact of its exponent-field arithmetic, ref: 296-305), so the
 * two agree on every element except those. */
static uint8_t encode_narrow(float q, int fmt) {
    const fmt_t *F = &FMTS[fmt];
    const uint32_t b = f2u(q);
    const uint32_t sign = (b >> 31) << (F->ebits + F->mbits);
    const uint32_t mag = b & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return 0x7F; /* the fp8 NaN that the saturating cast gives for a NaN input */
    if (mag == 0) return (uint8_t)sign;
    const int e = (int)(mag >> 23) - 127 + F->bias;
    const int drop = 23 - F->mbits;
    if (e > 0) return (uint8_t)(sign | ((uint32_t)e << F->mbits) | ((mag >> drop) & ((1u << F->mbits) - 1u)));
    /* subnormal of the narrow format: value = man * 2^(1 - bias - mbits) */
    const uint32_t sig = (mag & 0x7FFFFFu) | (1u << 23);
    return (uint8_t)(sign | (sig >> (drop + 1 - e)));
}
static float decode_narrow(uint8_t code, int fmt) {
    const fmt_t *F = &FMTS[fmt];
    const uint32_t sign = (code >> (F->ebits + F->mbits)) & 1u;
    const uint32_t e = (code >> F->mbits) & ((1u << F->ebits) - 1u), m = code & ((1u << F->mbits) - 1u);
    float v;
    if (fmt == FMT_E4M3 && e == 15 && m == 7) return u2f(0x7FFFE000u);
    if (fmt == FMT_E5M2 && e == 31) return m ? u2f(0x7FFFE000u) : (sign ? -INFINITY : INFINITY);
    if (e == 0) v = ldexpf((float)m, 1 - F->bias - F->mbits);
    else v = ldexpf((float)((1u << F->mbits) | m), (int)e - F->bias - F->mbits);
    return sign ? -v : v;
}
MOR_O_API int mor_o_quantize_mx(const void *in, uint8_t *payload, uint8_t *scales, int64_t rows, int64_t cols,
                                int bcols, int fmt) {
    if (rows <= 0 || cols <= 0 || bcols <= 0 || cols % bcols) return -1;
    if (!(fmt == FMT_E4M3 || fmt == FMT_E5M2 || fmt == FMT_E2M3)) return -1;
    io_t io = {in, NULL, 0};
    const int cuda_cast = (fmt == FMT_E4M3 || fmt == FMT_E5M2);
    const int64_t gx = cols / bcols, nb = rows * gx;
    const float maxv = (fmt == FMT_E2M3) ? 7.5f : (fmt == FMT_E4M3 ? 448.0f : 57344.0f);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t i0 = (b / gx) * cols + (b % gx) * bcols;
        float amax = 0.0f;
        for (int64_t c = 0; c < bcols; ++c) amax = fmaxf(amax, fabsf(load_elem(&io, i0 + c)));
        int e8 = 0;
        if (amax > 0.0f) { volatile float t = maxv / amax; e8 = (int)((f2u(t) >> 23) & 0xFFu) - 127; }
        scales[b] = (uint8_t)(127 - e8 < 0 ? 0 : (127 - e8 > 254 ? 254 : 127 - e8));
        for (int64_t c = 0; c < bcols; ++c) {
            const uint32_t xb = f2u(load_elem(&io, i0 + c));
            int xexp = (int)((xb >> 23) & 0xFFu) + e8;   /* ref: 283-290: the scale is added to the exponent field */
            if (xexp < 0) xexp = 0;
            if (xexp > 254) { raise_flag(MOR_O_ASSERT_E8_EXPONENT); xexp = 254; }
            const float scaled = u2f((xb & 0x80000000u) | ((uint32_t)xexp << 23) | (xb & 0x7FFFFFu));
            payload[i0 + c] = encode_narrow(quant_dequant(scaled, fmt, cuda_cast), fmt);
        }
    }
    return 0;
}
/* decode(code) * 2^(scale - 127) as bf16 bits (exact: at most four significant bits) */
MOR_O_API int mor_o_dequantize_mx(const uint8_t *payload, const uint8_t *scales, uint16_t *out, int64_t rows,
                                  int64_t cols, int bcols, int fmt) {
    if (rows <= 0 || cols <= 0 || bcols <= 0 || cols % bcols) return -1;
    const int64_t gx = cols / bcols, n = rows * cols;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const int64_t g = (i / cols) * gx + (i % cols) / bcols;
        const float v = ldexpf(decode_narrow(payload[i], fmt), (int)scales[g] - 127);
        out[i] = (uint16_t)(f2u(v) >> 16);
    }
    return 0;
}

/* Extension (no reference operator): the REAL quantized form of fake_quantize_block_scaling /
 * _channel_scaling under a binary32 scale (strategies 1, 3 and 4; ref: get_scaling_factor 1059-1093, the
 * cast inside SQDD_fp32_scale 310-316): payload[i] is the E4M3 byte of RN_e4m3(x * scale), scales[b] the
 * binary32 scale of block b (blocks of brows x bcols in row-major block order; brows x 1 blocks give one
 * scale per column of every row block), and element = decode(code) / scale -- the division the reference
 * applies -- is the fake-quantized value.  A zero element gets code 0 (the reference writes zeros back as
 * +0).  ext_global_amax: amax of the whole tensor when `in` is a slab of it, else NULL. */
MOR_O_API int mor_o_quantize_scaled(const void *in, int is_fp32, uint8_t *payload, float *scales, int64_t rows,
                                    int64_t cols, int brows, int bcols, int ss, const float *ext_global_amax,
                                    float *global_amax_out) {
    if (rows <= 0 || cols <= 0 || brows <= 0 || bcols <= 0 || rows % brows || cols % bcols) return -1;
    if (!(ss == 1 || ss == 3 || ss == 4)) return -1;
    io_t io = {in, NULL, is_fp32};
    const int64_t gx = cols / bcols, gy = rows / brows, nb = gx * gy;
    float *bamax = (float *)malloc(sizeof(float) * (size_t)nb);
    float gamax = -FLT_MAX;
#pragma omp parallel for reduction(max : gamax)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t r0 = (b / gx) * brows, c0 = (b % gx) * bcols;
        float a = -INFINITY;
        for (int64_t r = r0; r < r0 + brows; ++r)
            for (int64_t c = c0; c < c0 + bcols; ++c) a = fmaxf(a, fabsf(load_elem(&io, r * cols + c)));
        bamax[b] = a;
        gamax = fmaxf(gamax, a);
    }
    if (ext_global_amax) gamax = *ext_global_amax;
    if (global_amax_out) *global_amax_out = gamax;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t r0 = (b / gx) * brows, c0 = (b % gx) * bcols;
        const float sf = mor_o_scaling_factor(ss, gamax, bamax[b]);
        scales[b] = sf;
        for (int64_t r = r0; r < r0 + brows; ++r)
            for (int64_t c = c0; c < c0 + bcols; ++c) {
                const float x = load_elem(&io, r * cols + c);
                volatile float xs = x * sf;
                payload[r * cols + c] = (x == 0.0f) ? 0 : encode_narrow(quant_dequant(xs, FMT_E4M3, 1), FMT_E4M3);
            }
    }
    free(bamax);
    return 0;
}
/* decode(code) / scale, rounded to the output type as the fake-quantize operators round it */
MOR_O_API int mor_o_dequantize_scaled(const uint8_t *payload, const float *scales, void *out, int out_is_fp32,
                                      int64_t rows, int64_t cols, int brows, int bcols) {
    if (rows <= 0 || cols <= 0 || brows <= 0 || bcols <= 0 || rows % brows || cols % bcols) return -1;
    io_t io = {NULL, out, out_is_fp32};
    const int64_t gx = cols / bcols, n = rows * cols;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const int64_t b = ((i / cols) / brows) * gx + (i % cols) / bcols;
        volatile float v = decode_narrow(payload[i], FMT_E4M3) / scales[b];
        store_elem(&io, i, v);
    }
    return 0;
}

/* amax + non-zero count of a row slab (phase 1 of the row-sharded pipeline) */
MOR_O_API int mor_o_amax_nnz(const void *in, int is_fp32, int64_t n, float *amax_out, int64_t *nnz_out) {
    io_t io = {in, NULL, is_fp32};
    float gamax = -FLT_MAX;
    int64_t nnz = 0;
#pragma omp parallel for reduction(max : gamax) reduction(+ : nnz)
    for (int64_t i = 0; i < n; ++i) {
        const float a = fabsf(load_elem(&io, i));
        gamax = fmaxf(gamax, a);
        nnz += a > 0.0f;
    }
    *amax_out = gamax;
    *nnz_out = nnz;
    return 0;
}

/* ref: 1178-1241 on an error array gathered from several row slabs: entry i sits at
 * slot i * stride of the reference's array.  Returns the ordered sum; *meta_out gets 3
 * when sum / nnz exceeds the threshold, else 1. */
MOR_O_API float mor_o_finalize(const float *block_err, int64_t n_err, int stride, int64_t nnz, double thr,
                               int32_t *meta_out) {
    float part[1024];
    for (int t = 0; t < 1024; ++t) {
        float acc = 0.0f;
        if (t % stride == 0)
            for (int64_t e = t / stride; e < n_err; e += 1024 / stride) acc += block_err[e];
        part[t] = acc;
    }
    const float total = cta_tree_sum(part, 1024);
    volatile float avg = total / (float)nnz;
    if (meta_out) *meta_out = (avg > (float)thr) ? 3 : 1;
    return total;
}

MOR_O_API int mor_o_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
MOR_O_API void mor_o_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
