/*
 * CPU oracle for the EXL3 decode-step ops.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CUDA ops so that the GPU kernels of this
 * repository can be checked against an independent implementation.  It is never linked into, loaded by, or called
 * from the product library; only the tests, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * Parity status: the reference ships no golden vectors or known-answer tests for these ops.  The restatement is
 * pinned (a) against fixtures produced by running the reference's own CUDA ops (tests/golden), and (b) side by side
 * against those ops wherever the compiled reference library is present.
 *
 * Every function cites the reference source it follows (paths relative to the reference checkout).
 * fp16 arithmetic is emulated exactly: operands are widened to double, the operation is done in double (exact for
 * the sums/products that occur here) and the result is rounded once, to nearest-even, to binary16.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------------------ fp16 helpers */

static inline float h2f(uint16_t h)
{
    uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, m = h & 1023, u;
    if (e == 0) {
        if (m == 0) u = s;
        else { int sh = 0; while (!(m & 0x400)) { m <<= 1; sh++; } m &= 1023; u = s | ((uint32_t)(113 - sh) << 23) | (m << 13); }
    } else if (e == 31) u = s | 0x7f800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}

/* double -> binary16, round to nearest even, single rounding */
static inline uint16_t d2h(double d)
{
    uint64_t u; memcpy(&u, &d, 8);
    uint16_t sign = (uint16_t)((u >> 48) & 0x8000);
    int64_t e = (int64_t)((u >> 52) & 0x7ff);
    uint64_t m = u & 0xFFFFFFFFFFFFFULL;
    if (e == 0x7ff) return (uint16_t)(sign | (m ? 0x7e00 : 0x7c00));
    if (e == 0) return sign;
    int64_t he = e - 1023 + 15;
    m |= 1ULL << 52;
    if (he >= 31) return (uint16_t)(sign | 0x7c00);
    int shift = 42;
    if (he <= 0) { shift = 42 + (int)(1 - he); if (shift > 62) return sign; }
    uint64_t q = m >> shift, rem = m & ((1ULL << shift) - 1), half = 1ULL << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    if (he <= 0) return (uint16_t)(sign | (uint16_t)q);
    uint32_t r = ((uint32_t)(he - 1) << 10) + (uint32_t)q;
    if (r >= 0x7c00) r = 0x7c00;
    return (uint16_t)(sign | r);
}
static inline uint16_t f2h(float f) { return d2h((double)f); }
static inline uint16_t hmul(uint16_t a, uint16_t b) { return d2h((double)h2f(a) * (double)h2f(b)); }
static inline uint16_t hadd(uint16_t a, uint16_t b) { return d2h((double)h2f(a) + (double)h2f(b)); }

uint16_t orc_f2h(float f) { return f2h(f); }
float    orc_h2f(uint16_t h) { return h2f(h); }

/* ------------------------------------------------------------------------------------------ EXL3 tile decoding */

/* 16-bit trellis state -> fp16 weight.  kernels/quant/codebook.cuh:56-90 (decode_3inst<cb>).
 * cb 0 "3INST", cb 1 "MCG": multiply(-add), lop3 0x6a == (x & 0x8fff8fff) ^ 0x3b603b60, then one fp16 add of the two
 * 16-bit halves.  cb 2 "MUL1": multiply, byte sum + 0x6400 read as fp16 (= 1024 + sum), one fp16 fma. */
uint16_t orc_decode_state(int cb, uint32_t x)
{
    x &= 0xffffu;
    if (cb == 0 || cb == 1) {
        if (cb == 0) x = x * 89226354u + 64248484u; else x = x * 0xCBAC1FEDu;
        x = (x & 0x8fff8fffu) ^ 0x3b603b60u;
        return hadd((uint16_t)(x & 0xffff), (uint16_t)(x >> 16));
    }
    x *= 0x83DCD12Du;
    uint32_t s = 0x6400u + (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + (x >> 24);
    return d2h((double)h2f((uint16_t)s) * (double)h2f(0x1eee) + (double)h2f(0xc931));
}

/* State of ring position t (0..255) of one 16x16 tile of 8K uint32 words read MSB first.
 * kernels/quant/exl3_dq.cuh:16-31 (dq<bits,cb>), identical to kernels/cpu/moe_mul1.cpp:163-173. */
static inline uint32_t tile_state(const uint32_t* w, int K, int t)
{
    int nw = 8 * K;
    int b0 = t * K + K - 16 + 256 * K, b1 = b0 + 16;
    int i0 = b0 / 32, i1 = (b1 - 1) / 32, s0 = (i1 + 1) * 32 - b1;
    uint64_t merged = ((uint64_t)w[i0 % nw] << 32) | (uint64_t)w[i1 % nw];
    return (uint32_t)(merged >> s0) & 0xffffu;
}
uint32_t orc_tile_state(const uint32_t* w, int K, int t) { return tile_state(w, K, t); }

/* ring position -> (row, col) inside the tile: the mma.m16n8k16 B-fragment order.
 * kernels/cpu/moe_mul1.cpp:98-112, kernels/quant/reconstruct.cu:46-75. */
static inline void tile_pos(int t, int* row, int* col)
{
    static const int ro[4] = {0, 1, 8, 9};
    int l = t >> 3, j = t & 7;
    *row = 2 * (l & 3) + ro[j & 3];
    *col = (l >> 2) + 8 * (j >> 2);
}

static void decode_tile(const uint16_t* tile16, int K, int cb, const uint16_t* lut, uint16_t out[16][16])
{
    /* the tensor is int16 in memory; the kernels read it as little-endian uint32 words */
    uint32_t w[64];
    for (int i = 0; i < 8 * K; ++i) w[i] = (uint32_t)tile16[2 * i] | ((uint32_t)tile16[2 * i + 1] << 16);
    for (int t = 0; t < 256; ++t) {
        int r, c; tile_pos(t, &r, &c);
        uint32_t st = tile_state(w, K, t);
        out[r][c] = lut ? lut[st] : orc_decode_state(cb, st);
    }
}

static uint16_t* build_lut(int cb)
{
    uint16_t* lut = (uint16_t*)malloc(65536 * 2);
    for (uint32_t s = 0; s < 65536; ++s) lut[s] = orc_decode_state(cb, s);
    return lut;
}

/* Dense fp16 W[k,n] from trellis[k/16][n/16][16K] int16.  kernels/quant/reconstruct.cu:11-84,375-386. */
void orc_reconstruct(uint16_t* out, const uint16_t* trellis, int k, int n, int K, int cb)
{
    uint16_t* lut = build_lut(cb);
    int tk = k / 16, tn = n / 16;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int kt = 0; kt < tk; ++kt)
        for (int nt = 0; nt < tn; ++nt) {
            uint16_t tile[16][16];
            decode_tile(trellis + ((size_t)kt * tn + nt) * 16 * K, K, cb, lut, tile);
            for (int r = 0; r < 16; ++r)
                memcpy(out + (size_t)(kt * 16 + r) * n + nt * 16, tile[r], 32);
        }
    free(lut);
}

/* ------------------------------------------------------------------------------------------------- Hadamard 128 */

/* In-place unnormalised Sylvester FWHT in fp32, butterflies over index bits 0,1,...  Same operation order as the
 * in-register H4 + shfl_xor rounds of kernels/quant/hadamard_inner.cuh:19-44,120-135. */
static void fwht(float* v, int n)
{
    for (int h = 1; h < n; h <<= 1)
        for (int i = 0; i < n; i += 2 * h)
            for (int j = i; j < i + h; ++j) { float a = v[j], b = v[j + h]; v[j] = a + b; v[j + h] = a - b; }
}

/* had_r_128: y = (x.view(-1,128) @ H128) * r_scale with optional per-column pre or post scale.
 * kernels/quant/hadamard.cu:88-173; fp16 path hadamard_inner.cuh:93-147 (pre/post scale are fp16 multiplies),
 * fp32 path :151-212 (scales multiply in fp32).  in_fp32/out_fp32 select the element types. */
void orc_had_r_128(const void* x, void* y, const uint16_t* pre, const uint16_t* post, float r_scale,
                   int64_t rows, int64_t cols, int in_fp32, int out_fp32)
{
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c0 = 0; c0 < cols; c0 += 128) {
            float v[128];
            for (int i = 0; i < 128; ++i) {
                if (in_fp32) {
                    float f = ((const float*)x)[r * cols + c0 + i];
                    v[i] = pre ? f * h2f(pre[c0 + i]) : f;
                } else {
                    uint16_t h = ((const uint16_t*)x)[r * cols + c0 + i];
                    v[i] = h2f(pre ? hmul(h, pre[c0 + i]) : h);
                }
            }
            fwht(v, 128);
            for (int i = 0; i < 128; ++i) {
                float f = v[i] * r_scale;
                if (out_fp32) ((float*)y)[r * cols + c0 + i] = post ? f * h2f(post[c0 + i]) : f;
                else if (in_fp32 || 1) {
                    uint16_t h = f2h(f);
                    ((uint16_t*)y)[r * cols + c0 + i] = post ? hmul(h, post[c0 + i]) : h;
                }
            }
        }
}

/* ---------------------------------------------------------------------------------------------------- EXL3 GEMM */

/* C = H128( (H128(A o suh)/sqrt128 -> fp16) . W ) / sqrt128 o svh
 * kernels/quant/exl3_gemm_kernel.cuh:14-50 (input transform to fp16 A_had, then per-slab MMA with fp32 accumulate),
 * kernels/quant/exl3_gemm_inner.cuh:456-480 (output transform from the fp32 accumulators: fp16 C rounds to fp16 and
 * multiplies by svh in fp16, fp32 C multiplies by float(svh)).  The accumulation here is in double: the reference's
 * own summation order is not defined (stream-K slices), and every fp32 order lies within ~1e-6 relative of this.
 * suh == NULL skips the input transform, svh == NULL the output transform (exl3_gemm.cu:138-152). */
static void exl3_gemm_impl(const uint16_t* A, const uint16_t* trellis, void* C, int c_fp32, const uint16_t* suh,
                           const uint16_t* svh, int m, int k, int n, int K, int cb, float out_scale)
{
    const float rs = 0.088388347648f;
    float* Ah = (float*)malloc((size_t)m * k * sizeof(float));
    if (suh) {
        #pragma omp parallel for schedule(static)
        for (int r = 0; r < m; ++r)
            for (int c0 = 0; c0 < k; c0 += 128) {
                float v[128];
                for (int i = 0; i < 128; ++i) v[i] = h2f(hmul(A[(size_t)r * k + c0 + i], suh[c0 + i]));
                fwht(v, 128);
                for (int i = 0; i < 128; ++i) Ah[(size_t)r * k + c0 + i] = h2f(f2h(v[i] * rs));
            }
    } else {
        for (size_t i = 0; i < (size_t)m * k; ++i) Ah[i] = h2f(A[i]);
    }
    /* A_had transposed [k][m] so the inner loop over rows is contiguous */
    float* At = (float*)malloc((size_t)m * k * sizeof(float));
    for (int r = 0; r < m; ++r) for (int c = 0; c < k; ++c) At[(size_t)c * m + r] = Ah[(size_t)r * k + c];
    free(Ah);

    uint16_t* lut = build_lut(cb);
    float* lutf = (float*)malloc(65536 * sizeof(float));
    for (int i = 0; i < 65536; ++i) lutf[i] = h2f(lut[i]);
    int tk = k / 16, tn = n / 16;
    float* acc = (float*)malloc((size_t)m * n * sizeof(float));
    #pragma omp parallel
    {
        double* cacc = (double*)malloc((size_t)m * 16 * sizeof(double));
        #pragma omp for schedule(dynamic, 4)
        for (int nt = 0; nt < tn; ++nt) {
            memset(cacc, 0, (size_t)m * 16 * sizeof(double));
            for (int kt = 0; kt < tk; ++kt) {
                const uint16_t* t16 = trellis + ((size_t)kt * tn + nt) * 16 * K;
                uint32_t w[64];
                for (int i = 0; i < 8 * K; ++i) w[i] = (uint32_t)t16[2 * i] | ((uint32_t)t16[2 * i + 1] << 16);
                float tile[16][16];
                for (int t = 0; t < 256; ++t) { int r, c; tile_pos(t, &r, &c); tile[r][c] = lutf[tile_state(w, K, t)]; }
                for (int r = 0; r < 16; ++r) {
                    const float* a = At + (size_t)(kt * 16 + r) * m;
                    for (int c = 0; c < 16; ++c) {
                        double wv = tile[r][c];
                        double* dst = cacc + c;
                        for (int mm = 0; mm < m; ++mm) dst[(size_t)mm * 16] += (double)a[mm] * wv;
                    }
                }
            }
            for (int mm = 0; mm < m; ++mm) for (int c = 0; c < 16; ++c)
                acc[(size_t)mm * n + nt * 16 + c] = (float)cacc[(size_t)mm * 16 + c];
        }
        free(cacc);
    }
    free(lut); free(lutf); free(At);

    #pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r)
        for (int c0 = 0; c0 < n; c0 += 128) {
            float v[128];
            for (int i = 0; i < 128; ++i) v[i] = acc[(size_t)r * n + c0 + i];
            const float os = rs * out_scale;      /* the expert weight of exl3_mgemm folds into the transform's scale */
            if (svh) { fwht(v, 128); for (int i = 0; i < 128; ++i) v[i] *= os; }
            for (int i = 0; i < 128; ++i) {
                if (c_fp32) ((float*)C)[(size_t)r * n + c0 + i] = svh ? v[i] * h2f(svh[c0 + i]) : v[i];
                else { uint16_t h = f2h(v[i]); ((uint16_t*)C)[(size_t)r * n + c0 + i] = svh ? hmul(h, svh[c0 + i]) : h; }
            }
        }
    free(acc);
}

void orc_exl3_gemm(const uint16_t* A, const uint16_t* trellis, void* C, int c_fp32, const uint16_t* suh,
                   const uint16_t* svh, int m, int k, int n, int K, int cb)
{
    exl3_gemm_impl(A, trellis, C, c_fp32, suh, svh, m, k, n, K, cb, 1.0f);
}

/* One slot of exl3_mgemm (kernels/quant/exl3_gemm_kernel.cuh:146-247): the same product with the output transform's scale
 * multiplied by the slot's weight (scale = 0.0884 * float(weight), :236-237). */
void orc_exl3_gemm_scaled(const uint16_t* A, const uint16_t* trellis, void* C, int c_fp32, const uint16_t* suh,
                          const uint16_t* svh, int m, int k, int n, int K, int cb, float out_scale)
{
    exl3_gemm_impl(A, trellis, C, c_fp32, suh, svh, m, k, n, K, cb, out_scale);
}

/* Dense fp16 GEMM with fp32-class accumulation, C fp16 or fp32.  kernels/hgemm.cu:19-78 (cublasGemmEx,
 * CUBLAS_COMPUTE_32F).  A [m,k], B [k,n] row-major. */
void orc_hgemm(const uint16_t* A, const uint16_t* B, void* C, int c_fp32, int m, int k, int n)
{
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r) {
        double* acc = (double*)calloc(n, sizeof(double));
        for (int kk = 0; kk < k; ++kk) {
            double a = h2f(A[(size_t)r * k + kk]);
            const uint16_t* b = B + (size_t)kk * n;
            for (int c = 0; c < n; ++c) acc[c] += a * (double)h2f(b[c]);
        }
        for (int c = 0; c < n; ++c) {
            if (c_fp32) ((float*)C)[(size_t)r * n + c] = (float)acc[c];
            else ((uint16_t*)C)[(size_t)r * n + c] = d2h(acc[c]);
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------------------------------------------ RMSNorm */

/* y = x * (w + cbias) * rsqrt(mean(x^2) + eps) * cscale.  kernels/norm.cu:160-304.
 * res != NULL: RES_IN mode, r += x first (r fp32, stored), then the norm of r.  x fp16 or fp32, y fp16 or fp32. */
void orc_rms_norm(const void* x, int x_fp32, const uint16_t* w, void* y, int y_fp32, float* res, float eps,
                  float cbias, float cscale, int rows, int dim)
{
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float* v = (float*)malloc(dim * sizeof(float));
        double ss = 0;
        for (int i = 0; i < dim; ++i) {
            float f = x_fp32 ? ((const float*)x)[(size_t)r * dim + i] : h2f(((const uint16_t*)x)[(size_t)r * dim + i]);
            if (res) { f += res[(size_t)r * dim + i]; res[(size_t)r * dim + i] = f; }
            v[i] = f; ss += (double)f * f;
        }
        float rmf = (float)(1.0 / sqrt(ss / dim + (double)eps)) * cscale;
        for (int i = 0; i < dim; ++i) {
            float o = w ? v[i] * (h2f(w[i]) + cbias) * rmf : v[i] * rmf;
            if (y_fp32) ((float*)y)[(size_t)r * dim + i] = o; else ((uint16_t*)y)[(size_t)r * dim + i] = f2h(o);
        }
        free(v);
    }
}

/* --------------------------------------------------------------------------------------------------------- RoPE */

/* Per-head optional RMSNorm (fp16 weight: v -> fp16, w+bias in fp16, fp16 multiply) then NEOX (mode 2) or GPT-J (mode 1; kernels/rope.cuh:6-8)
 * rotation of the first 2*n_freq dims; pos = token index in the sequence + positions[b] (or + position).
 * kernels/rope.cu:16-255.  q [bsz,seq,nq,hd], k [bsz,seq,nk,hd], in place. */
void orc_rope(uint16_t* q, uint16_t* k, const float* inv_freq, int n_freq, uint32_t position, const int32_t* positions,
              const uint16_t* q_norm, const uint16_t* k_norm, float norm_eps, float norm_cbias, int rope_mode,
              float attn_factor, int bsz, int seq, int nq, int nk, int hd)
{
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < bsz; ++b)
        for (int s = 0; s < seq; ++s) {
            int pos = s + (positions ? positions[b] : (int)position);
            for (int h = 0; h < nq + nk; ++h) {
                uint16_t* p; const uint16_t* nw;
                if (h < nq) { p = q + (((size_t)b * seq + s) * nq + h) * hd; nw = q_norm; }
                else { if (!k) continue; p = k + (((size_t)b * seq + s) * nk + (h - nq)) * hd; nw = k_norm; }
                if (nw) {
                    double ss = 0;
                    for (int i = 0; i < hd; ++i) { double f = h2f(p[i]); ss += f * f; }
                    float rmf = (float)(1.0 / sqrt(ss / hd + (double)norm_eps));
                    uint16_t cb = f2h(norm_cbias);
                    for (int i = 0; i < hd; ++i) p[i] = hmul(hadd(nw[i], cb), f2h(h2f(p[i]) * rmf));
                }
                int half = n_freq;
                for (int t = 0; t < n_freq; ++t) {
                    float ang = inv_freq[t] * (float)pos;
                    float sn = sinf(ang) * attn_factor, cs = cosf(ang) * attn_factor;
                    int i1 = rope_mode == 2 ? t : 2 * t, i2 = rope_mode == 2 ? t + half : 2 * t + 1;
                    float v1 = h2f(p[i1]), v2 = h2f(p[i2]);
                    p[i1] = f2h(v1 * cs - v2 * sn);
                    p[i2] = f2h(v2 * cs + v1 * sn);
                }
            }
        }
}

/* -------------------------------------------------------------------------------------------------- activations */

/* z = silu(x) * y with every step in fp16: e = exp(-x) -> fp16, s = 1 + e (fp16), r = 1/s -> fp16, x*r (fp16), *y (fp16).
 * kernels/activation_kernels.cuh:22-31,142-186 (act_limit == 0). */
void orc_silu_mul(const uint16_t* x, const uint16_t* y, uint16_t* z, int64_t numel)
{
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < numel; ++i) {
        double xf = h2f(x[i]);
        uint16_t e = d2h(exp(-xf));
        uint16_t s = hadd(0x3c00, e);
        uint16_t r = d2h(1.0 / (double)h2f(s));
        z[i] = hmul(hmul(x[i], r), y[i]);
    }
}

/* z = x + y elementwise, fp16 (kernels/add.cu:44-110, half path: fp32 add, one rounding == fp16 add). */
void orc_add(const uint16_t* x, const uint16_t* y, uint16_t* z, int64_t numel)
{
    for (int64_t i = 0; i < numel; ++i) z[i] = hadd(x[i], y[i]);
}

/* argmax per row, lowest index on ties.  kernels/generator/sampling_basic.cu:21-91, kernels/reduction.cuh:9-42
 * (strict > in every comparison keeps the lower index).  logits fp16 or fp32. */
void orc_argmax(const void* logits, int fp32, int64_t* ids, int rows, int n)
{
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float best = -INFINITY; int bi = 0;
        for (int i = 0; i < n; ++i) {
            float f = fp32 ? ((const float*)logits)[(size_t)r * n + i] : h2f(((const uint16_t*)logits)[(size_t)r * n + i]);
            if (f > best) { best = f; bi = i; }
        }
        ids[r] = bi;
    }
}

/* ---------------------------------------------------------------------------------------------------- paged KV */

#define PAGE 256

/* kernels/generator/cache.cu:143-184, kernels/attention.cu:38-77: row s of sequence b goes to logical position
 * cache_seqlens[b] + s, page block_table[b][pos/256], slot pos%256.  Caches [pages,256,nkv,hd]. */
void orc_paged_kv_update(const uint16_t* k, const uint16_t* v, uint16_t* kc, uint16_t* vc, const int32_t* block_table,
                         const int32_t* seqlens, int bsz, int seq, int nkv, int hd, int pages_per_seq)
{
    size_t row = (size_t)nkv * hd;
    for (int b = 0; b < bsz; ++b)
        for (int s = 0; s < seq; ++s) {
            int pos = seqlens[b] + s;
            size_t dst = ((size_t)block_table[(size_t)b * pages_per_seq + pos / PAGE] * PAGE + pos % PAGE) * row;
            memcpy(kc + dst, k + ((size_t)b * seq + s) * row, row * 2);
            memcpy(vc + dst, v + ((size_t)b * seq + s) * row, row * 2);
        }
}

/* ---- KV quantisation codec: kernels/cache/q_cache_kernels.cuh:29-236 ---- */

static void had32(float* v)   /* unnormalised, index bits 0..4: in-register H4 then the 3 subgroup shuffle rounds */
{
    fwht(v, 32);
}

/* one group of 32 values -> `bits` uint32 words + one fp16 scale.  quant_block_x4 :61-156 (linear grid). */
static void quant_group(const uint16_t* in, uint32_t* out, uint16_t* scale, int bits)
{
    float v[32];
    for (int i = 0; i < 32; ++i) v[i] = h2f(in[i]);
    had32(v);
    float s = 0;
    for (int i = 0; i < 32; ++i) { v[i] *= 0.17677669529663688110f; float a = fabsf(v[i]); if (a > s) s = a; }
    s += 1e-10f;
    float inv_s = 1.0f / s, mf = (float)(1 << (bits - 1));
    int qmax = (1 << bits) - 1;
    uint32_t q[32];
    for (int i = 0; i < 32; ++i) {
        int qi = (int)floorf(fmaf(v[i] * inv_s, mf, mf));
        q[i] = (uint32_t)(qi < 0 ? 0 : qi > qmax ? qmax : qi);
    }
    for (int i = 0; i < bits; ++i) out[i] = 0;
    int rem = bits, wb = 0;
    for (int w = 8; w >= 1; w >>= 1) {
        if (!(bits & w)) continue;
        rem -= w;
        for (int sl = 0; sl < 8; ++sl) {
            uint32_t field = 0;
            for (int j = 0; j < 4; ++j) field |= ((q[4 * sl + j] >> rem) & ((1u << w) - 1)) << (j * w);
            int off = sl * 4 * w;
            out[wb + (off >> 5)] |= field << (off & 31);
        }
        wb += w;
    }
    *scale = f2h(s);
}

/* dequant_block_x4 :160-236 */
static void dequant_group(const uint32_t* in, uint16_t scale, uint16_t* out, int bits)
{
    uint32_t q[32];
    for (int i = 0; i < 32; ++i) q[i] = 0;
    int wb = 0;
    for (int w = 8; w >= 1; w >>= 1) {
        if (!(bits & w)) continue;
        for (int sl = 0; sl < 8; ++sl) {
            int off = sl * 4 * w;
            uint32_t word = in[wb + (off >> 5)] >> (off & 31);
            for (int j = 0; j < 4; ++j) q[4 * sl + j] = (q[4 * sl + j] << w) | ((word >> (j * w)) & ((1u << w) - 1));
        }
        wb += w;
    }
    int m = 1 << (bits - 1);
    float s = h2f(scale) * 0.17677669529663688110f;
    float sm = s * (1.0f / (float)m), mh = (float)m - 0.5f;
    float v[32];
    for (int i = 0; i < 32; ++i) v[i] = ((float)(int)q[i] - mh) * sm;
    had32(v);
    for (int i = 0; i < 32; ++i) out[i] = f2h(v[i]);
}

void orc_quant_groups(const uint16_t* in, uint32_t* out, uint16_t* scales, int64_t groups, int bits)
{
    #pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < groups; ++g) quant_group(in + g * 32, out + g * bits, scales + g, bits);
}
void orc_dequant_groups(const uint32_t* in, const uint16_t* scales, uint16_t* out, int64_t groups, int bits)
{
    #pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < groups; ++g) dequant_group(in + g * bits, scales[g], out + g * 32, bits);
}

/* quant_cache_paged (in_contiguous): kernels/cache/q_cache_kernels.cuh:292-327.
 * k_in/v_in [bsz,seq,dim]; q* [pages,256,groups*bits] uint32, s* [pages,256,groups] fp16. */
void orc_quant_cache_paged(const uint16_t* k_in, uint32_t* qk, uint16_t* sk, const uint16_t* v_in, uint32_t* qv,
                           uint16_t* sv, const int32_t* seqlens, const int32_t* block_table, int bsz, int seq,
                           int dim, int pages_per_seq, int k_bits, int v_bits)
{
    int groups = dim / 32;
    for (int b = 0; b < bsz; ++b)
        for (int s = 0; s < seq; ++s) {
            int pos = seqlens[b] + s;
            size_t tok = (size_t)block_table[(size_t)b * pages_per_seq + pos / PAGE] * PAGE + pos % PAGE;
            size_t in = ((size_t)b * seq + s) * dim;
            for (int g = 0; g < groups; ++g) {
                quant_group(k_in + in + g * 32, qk + (tok * groups + g) * k_bits, sk + tok * groups + g, k_bits);
                quant_group(v_in + in + g * 32, qv + (tok * groups + g) * v_bits, sv + tok * groups + g, v_bits);
            }
        }
}

/* dequant_cache_paged / _window: kernels/cache/q_cache_kernels.cuh:343-400.  Tokens [0, seqlens[b]+bonus) of each
 * sequence; compact != 0 writes page p of sequence b at scratch page b*pages_per_seq+p, else at the source page.
 * (sliding_window only skips whole thread blocks of old tokens in the reference; here nothing is skipped, which
 *  is a superset of what it writes.) */
void orc_dequant_cache_paged(const uint32_t* qk, const uint16_t* sk, uint16_t* k_out, const uint32_t* qv,
                             const uint16_t* sv, uint16_t* v_out, const int32_t* seqlens, const int32_t* block_table,
                             int bsz, int dim, int pages_per_seq, int k_bits, int v_bits, int compact, int bonus)
{
    int groups = dim / 32;
    #pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < bsz; ++b)
        for (int pos = 0; pos < seqlens[b] + bonus; ++pos) {
            size_t page = (size_t)block_table[(size_t)b * pages_per_seq + pos / PAGE];
            size_t tok = page * PAGE + pos % PAGE;
            size_t otok = compact ? ((size_t)b * pages_per_seq + pos / PAGE) * PAGE + pos % PAGE : tok;
            for (int g = 0; g < groups; ++g) {
                dequant_group(qk + (tok * groups + g) * k_bits, sk[tok * groups + g], k_out + (otok * groups + g) * 32, k_bits);
                dequant_group(qv + (tok * groups + g) * v_bits, sv[tok * groups + g], v_out + (otok * groups + g) * 32, v_bits);
            }
        }
}

/* --------------------------------------------------------------------------------------------- paged attention */

/* o[b,i,h,:] = softmax_j(scale * q[b,i,h,:].k[b,j,h/G,:]) v[b,j,h/G,:] over keys j <= total_k - q_len + i, where
 * total_k = cache_seqlens[b] + kv_append (the rows are already in the cache).  Rows with no visible key give zeros.
 * kernels/attention.cu:97-269 (decode), kernels/attention_mma_kernel.cuh:164-339 (q_len > 1), host :1716-1870.
 * The softmax and both products are done in double here (the reference uses fp32 with __expf and, on its
 * tensor-core path, rounds P to fp16 before PV; both lie inside the parity tolerance).
 * Ragged extension: cu_q != NULL gives per-sequence query row ranges [cu_q[b], cu_q[b+1]) in a packed q/o of
 * shape [rows,nq,hd]; then q_len of sequence b = cu_q[b+1]-cu_q[b] and total_k = cache_seqlens[b] + q_len.
 * quantised KV: bits > 0 reads qk/sk/qv/sv (layout of orc_quant_cache_paged) instead of kc/vc. */
void orc_attn_paged(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const uint32_t* qk, const uint16_t* sk,
                    const uint32_t* qv, const uint16_t* sv, int bits, const int32_t* block_table,
                    const int32_t* seqlens, const int32_t* cu_q, uint16_t* o, int bsz, int q_len, int kv_append,
                    int nq, int nkv, int hd, int pages_per_seq, int causal, float sm_scale)
{
    int G = nq / nkv, dim = nkv * hd, groups = dim / 32;
    float scale = sm_scale == 0.0f ? 1.0f / sqrtf((float)hd) : sm_scale;
    #pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < bsz * nkv; ++bh) {
        int b = bh / nkv, kvh = bh % nkv;
        int ql = cu_q ? cu_q[b + 1] - cu_q[b] : q_len;
        int row0 = cu_q ? cu_q[b] : b * q_len;
        int total_k = seqlens[b] + (cu_q ? ql : kv_append);
        if (ql == 0) continue;
        float* kf = (float*)malloc((size_t)(total_k > 0 ? total_k : 1) * hd * sizeof(float));
        float* vf = (float*)malloc((size_t)(total_k > 0 ? total_k : 1) * hd * sizeof(float));
        uint16_t tmp[32];
        for (int j = 0; j < total_k; ++j) {
            size_t tok = (size_t)block_table[(size_t)b * pages_per_seq + j / PAGE] * PAGE + j % PAGE;
            if (bits == 0) {
                for (int d = 0; d < hd; ++d) {
                    kf[(size_t)j * hd + d] = h2f(kc[(tok * nkv + kvh) * hd + d]);
                    vf[(size_t)j * hd + d] = h2f(vc[(tok * nkv + kvh) * hd + d]);
                }
            } else {
                for (int gg = 0; gg < hd / 32; ++gg) {
                    size_t g = tok * groups + (size_t)kvh * (hd / 32) + gg;
                    dequant_group(qk + g * bits, sk[g], tmp, bits);
                    for (int d = 0; d < 32; ++d) kf[(size_t)j * hd + gg * 32 + d] = h2f(tmp[d]);
                    dequant_group(qv + g * bits, sv[g], tmp, bits);
                    for (int d = 0; d < 32; ++d) vf[(size_t)j * hd + gg * 32 + d] = h2f(tmp[d]);
                }
            }
        }
        double* p = (double*)malloc((size_t)(total_k > 0 ? total_k : 1) * sizeof(double));
        for (int i = 0; i < ql; ++i)
            for (int g = 0; g < G; ++g) {
                int h = kvh * G + g;
                const uint16_t* qp = q + ((size_t)(row0 + i) * nq + h) * hd;
                uint16_t* op = o + ((size_t)(row0 + i) * nq + h) * hd;
                int vis = causal ? total_k - ql + i + 1 : total_k;
                if (vis > total_k) vis = total_k;
                if (vis <= 0) { for (int d = 0; d < hd; ++d) op[d] = 0; continue; }
                double mx = -INFINITY;
                for (int j = 0; j < vis; ++j) {
                    double s = 0;
                    for (int d = 0; d < hd; ++d) s += (double)h2f(qp[d]) * kf[(size_t)j * hd + d];
                    p[j] = s * scale; if (p[j] > mx) mx = p[j];
                }
                double l = 0;
                for (int j = 0; j < vis; ++j) { p[j] = exp(p[j] - mx); l += p[j]; }
                for (int d = 0; d < hd; ++d) {
                    double acc = 0;
                    for (int j = 0; j < vis; ++j) acc += p[j] * vf[(size_t)j * hd + d];
                    op[d] = d2h(acc / l);
                }
            }
        free(p); free(kf); free(vf);
    }
}

/* fp16 table -> fp32 rows.  src/modules.rs:430-436 (index_select + to_kind(Float)). */
void orc_embed(const int64_t* ids, const uint16_t* table, float* out, int rows, int dim)
{
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < dim; ++i) out[(size_t)r * dim + i] = h2f(table[(size_t)ids[r] * dim + i]);
}

/* the harness sets the thread count itself: a launcher may have pinned OMP_NUM_THREADS to 1 */
void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
