// Sampler-side ops of the reference's op surface (src/ffi.rs:128-139,166-167): repetition / presence / frequency
// penalties over a token history, Gumbel noise and Gumbel-max sampling on the reference's Philox stream, the page
// permutation used when a pool is defragmented, and two small element-wise ops of the hybrid models.
#include <algorithm>
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------- penalties
// kernels/generator/rep_pen.cu:24-91,135-210.  One CTA owns a span of the vocabulary in shared memory, walks the tail of
// the history that can still carry weight (the last sustain + decay tokens) and then rewrites its span of the logits.
// weight(dist) = 1 for dist <= sustain, else clamp(1 - (dist - sustain) / decay, 0, 1); duplicates of a token take the
// largest weight (repetition, presence) or add up (frequency).
constexpr int PEN_SPAN = 4096;
constexpr int PEN_THREADS = 512;

__device__ __forceinline__ float history_weight(int dist, int sustain, int decay)
{
    if (dist <= sustain) return 1.0f;
    float f = decay > 0 ? 1.0f - ((float)dist - (float)sustain) / (float)decay : 1.0f;
    return fminf(fmaxf(f, 0.0f), 1.0f);
}

// non-negative floats order like their bit patterns
__device__ __forceinline__ void smem_max_nonneg(float* addr, float v)
{
    atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

template <bool FP16_IN, bool FREQ>
__global__ void __launch_bounds__(PEN_THREADS) penalties_kernel(const void* __restrict__ in, float* __restrict__ out,
                                                                const int64_t* __restrict__ past, int past_len, int vocab,
                                                                float p0, float p1, int sustain, int decay)
{
    __shared__ float s_max[PEN_SPAN];                 // repetition weight, or presence penalty
    __shared__ float s_sum[FREQ ? PEN_SPAN : 1];      // frequency penalty
    const int lo = blockIdx.x * PEN_SPAN, hi = min(lo + PEN_SPAN, vocab);
    for (int i = threadIdx.x; i < PEN_SPAN; i += PEN_THREADS) { s_max[i] = 0.0f; if (FREQ) s_sum[i] = 0.0f; }
    __syncthreads();
    // positions i <= past_len - sustain - decay carry no weight (rep_pen.cu:51-52)
    const int first = max(0, past_len - sustain - decay + 1);
    for (int i = first + threadIdx.x; i < past_len; i += PEN_THREADS) {
        const int tok = (int)past[i];
        if (tok < lo || tok >= hi) continue;
        const float w = history_weight(past_len - i, sustain, decay);
        if (FREQ) { atomicAdd(&s_sum[tok - lo], w * p1); smem_max_nonneg(&s_max[tok - lo], w * p0); }
        else smem_max_nonneg(&s_max[tok - lo], w);
    }
    __syncthreads();
    for (int i = lo + threadIdx.x; i < hi; i += PEN_THREADS) {
        float v = FP16_IN ? __half2float(reinterpret_cast<const half*>(in)[i]) : reinterpret_cast<const float*>(in)[i];
        if (FREQ) {
            v -= s_sum[i - lo];
            v -= s_max[i - lo];
        } else {
            // blend between the logit and its penalised value (rep_pen.cu:84-88; the 1e-30 terms are the reference's)
            const float w = v > 0.0f ? v / p0 : v * p0;
            const float f = s_max[i - lo] + 1e-30f;
            const float f1 = (1.0f - f) + 1e-30f;
            v = v * f1 + w * f;
        }
        out[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------- Philox / Gumbel
// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11) laid out the way the
// reference's generator consumes it (kernels/generator/gumbel.cu:47-66, sampling_basic.cu:93-129): key = (seed, 0),
// counter = (draw / 4, 0, subsequence, 0), the four words of a block are handed out in order, and a word x becomes the
// uniform x * 2^-32 + 2^-33 in (0, 1].
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k)
{
    #pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t h0 = __umulhi(0xD2511F53u, c.x), l0 = 0xD2511F53u * c.x;
        const uint32_t h1 = __umulhi(0xCD9E8D57u, c.z), l1 = 0xCD9E8D57u * c.z;
        c = make_uint4(h1 ^ c.y ^ k.x, l1, h0 ^ c.w ^ k.y, l0);
        k.x += 0x9E3779B9u; k.y += 0xBB67AE85u;
    }
    return c;
}
__device__ __forceinline__ float philox_uniform(uint32_t seed, uint32_t subsequence, uint32_t draw)
{
    const uint4 o = philox4x32_10(make_uint4(draw >> 2, 0u, subsequence, 0u), make_uint2(seed, 0u));
    const uint32_t w = (draw & 3) == 0 ? o.x : ((draw & 3) == 1 ? o.y : ((draw & 3) == 2 ? o.z : o.w));
    return (float)w * 2.3283064e-10f + 1.1641532e-10f;
}
// -log(-log(u)) with the reference's clamps and its fast logarithm (gumbel.cu:12-16)
__device__ __forceinline__ float gumbel_of(float u)
{
    u = fminf(u, 0.99999994f);
    return -__logf(fmaxf(-__logf(fmaxf(u, 1e-20f)), 1e-20f));
}

__global__ void __launch_bounds__(256) gumbel_noise_kernel(const float* __restrict__ in, float* __restrict__ out, long long numel,
                                                           uint32_t seed)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= numel) return;
    out[i] = in[i] + gumbel_of(philox_uniform(seed, (uint32_t)i, 0));          // element i = first draw of subsequence i
}

// Gumbel-max sampling, one CTA per row (sampling_basic.cu:93-129): column c takes draw 2 (c / 2048) + (c & 1) of
// subsequence (c / 2) % 1024 - every row sees the same noise - and the row's argmax (lowest index on ties) is written.
// The reference limits the columns pair by pair (sampling_basic.cu:38-62): of the pair (c, c + 1), c even, the first
// counts when c < max_logit - 1 and the second when c < max_logit; for an odd limit that drops column max_logit - 1 and
// admits column max_logit.  Reproduced as it is.
template <bool FP32>
__global__ void __launch_bounds__(1024) gumbel_sample_kernel(const void* __restrict__ logits, int64_t* __restrict__ ids, int n,
                                                             int max_logit, uint32_t seed)
{
    const size_t row = blockIdx.x;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int end = min(n, max_logit + 1);
    for (int c = threadIdx.x; c < end; c += 1024) {
        if ((c & 1) ? (c - 1 >= max_logit) : (c >= max_logit - 1)) continue;
        float v = FP32 ? reinterpret_cast<const float*>(logits)[row * n + c]
                       : __half2float(reinterpret_cast<const half*>(logits)[row * n + c]);
        v += gumbel_of(philox_uniform(seed, (uint32_t)((c >> 1) & 1023), (uint32_t)(2 * (c >> 11) + (c & 1))));
        if (v > best) { best = v; best_i = c; }
    }
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = best; s_i[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = s_v[threadIdx.x]; best_i = s_i[threadIdx.x];
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (threadIdx.x == 0) ids[row] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

// ---------------------------------------------------------------------------------------------- page permutation
// kernels/generator/cache.cu:11-85: for i in order: (page[a] or temp) <- (page[b] or temp), pairs (a, b) = order[2i, 2i+1],
// -1 standing for the temporary page.  The copies of the list depend on one another only at equal byte offsets, so a
// thread that owns a set of 16-byte offsets can walk the whole list on its own, without any barrier.
__global__ void __launch_bounds__(256) cache_rotate_kernel(uint8_t* __restrict__ cache, const int32_t* __restrict__ order,
                                                           uint8_t* __restrict__ temp, size_t page_bytes, int n_order)
{
    const size_t chunks = page_bytes / 16;
    for (size_t c = (size_t)blockIdx.x * 256 + threadIdx.x; c < chunks; c += (size_t)gridDim.x * 256) {
        for (int i = 0; i < n_order; ++i) {
            const int a = order[2 * i], b = order[2 * i + 1];
            uint4* dst = reinterpret_cast<uint4*>(a >= 0 ? cache + page_bytes * (size_t)a : temp) + c;
            const uint4* src = reinterpret_cast<const uint4*>(b >= 0 ? cache + page_bytes * (size_t)b : temp) + c;
            *dst = *src;
        }
    }
}

// ---------------------------------------------------------------------------------------------- small element-wise ops
// x *= sigmoid(y), all steps in fp16 (kernels/activation_kernels.cuh:132-139,300-315)
__global__ void __launch_bounds__(256) mul_sigmoid_kernel(half2* __restrict__ x, const half2* __restrict__ y, long long pairs)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= pairs) return;
    const half2 one = __float2half2_rn(1.0f);
    const half2 s = h2rcp(__hadd2(one, h2exp(__hneg2(y[i]))));
    x[i] = __hmul2(x[i], s);
}

// qg [rows, heads, 2, head_dim] -> q, g [rows, heads, head_dim] (kernels/activation.cu:721-738), 16 bytes per thread
__global__ void __launch_bounds__(256) deinterleave_qg_kernel(const uint4* __restrict__ qg, uint4* __restrict__ q, uint4* __restrict__ g,
                                                              int hd8, long long n8)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n8) return;
    const long long head = i / hd8, d = i - head * hd8;
    q[i] = qg[head * 2 * hd8 + d];
    g[i] = qg[head * 2 * hd8 + hd8 + d];
}

}  // namespace

extern "C" int exl3_apply_rep_pens(exl3_ctx* ctx, exl3_stream stream, const void* in_logits, int in_fp32, void* out_logits,
                                   const int64_t* past_ids, float rep_p, int sustain_range, int decay_range, int rows, int vocab,
                                   int past_len)
{
    EXL3_REQUIRE(ctx && in_logits && out_logits && (past_ids || past_len == 0), "apply_rep_pens: null argument");
    EXL3_REQUIRE(rows == 1, "apply_rep_pens: one row of logits (as the reference, kernels/generator/rep_pen.cu:105)");
    EXL3_REQUIRE(vocab > 0 && past_len >= 0 && sustain_range >= 0 && decay_range >= 0 && rep_p > 0.0f, "apply_rep_pens: bad argument");
    const int blocks = (vocab + PEN_SPAN - 1) / PEN_SPAN;
    if (in_fp32) penalties_kernel<false, false><<<blocks, PEN_THREADS, 0, (cudaStream_t)stream>>>(in_logits, (float*)out_logits, past_ids, past_len, vocab, rep_p, 0.0f, sustain_range, decay_range);
    else penalties_kernel<true, false><<<blocks, PEN_THREADS, 0, (cudaStream_t)stream>>>(in_logits, (float*)out_logits, past_ids, past_len, vocab, rep_p, 0.0f, sustain_range, decay_range);
    ctx->launches++;
    return exl3_check_launch(ctx, "apply_rep_pens");
}

extern "C" int exl3_apply_pres_freq_pens(exl3_ctx* ctx, exl3_stream stream, const void* in_logits, int in_fp32, void* out_logits,
                                         const int64_t* past_ids, float pres_p, float freq_p, int sustain_range, int decay_range,
                                         int rows, int vocab, int past_len)
{
    EXL3_REQUIRE(ctx && in_logits && out_logits && (past_ids || past_len == 0), "apply_pres_freq_pens: null argument");
    EXL3_REQUIRE(rows == 1, "apply_pres_freq_pens: one row of logits (as the reference)");
    EXL3_REQUIRE(vocab > 0 && past_len >= 0 && sustain_range >= 0 && decay_range >= 0 && pres_p >= 0.0f && freq_p >= 0.0f,
                 "apply_pres_freq_pens: bad argument (penalties must not be negative)");
    const int blocks = (vocab + PEN_SPAN - 1) / PEN_SPAN;
    if (in_fp32) penalties_kernel<false, true><<<blocks, PEN_THREADS, 0, (cudaStream_t)stream>>>(in_logits, (float*)out_logits, past_ids, past_len, vocab, pres_p, freq_p, sustain_range, decay_range);
    else penalties_kernel<true, true><<<blocks, PEN_THREADS, 0, (cudaStream_t)stream>>>(in_logits, (float*)out_logits, past_ids, past_len, vocab, pres_p, freq_p, sustain_range, decay_range);
    ctx->launches++;
    return exl3_check_launch(ctx, "apply_pres_freq_pens");
}

extern "C" int exl3_gumbel_noise_f32(exl3_ctx* ctx, exl3_stream stream, const float* logits_in, float* logits_out, int64_t numel,
                                     uint32_t random)
{
    EXL3_REQUIRE(ctx && logits_in && logits_out && numel >= 0 && numel <= 0xffffffffLL, "gumbel_noise_f32: bad argument");
    if (numel == 0) return EXL3_OK;
    gumbel_noise_kernel<<<(unsigned)((numel + 255) / 256), 256, 0, (cudaStream_t)stream>>>(logits_in, logits_out, numel, random);
    ctx->launches++;
    return exl3_check_launch(ctx, "gumbel_noise_f32");
}

extern "C" int exl3_gumbel_sample(exl3_ctx* ctx, exl3_stream stream, const void* logits, int fp32, int64_t* ids, int rows, int n,
                                  int max_logit, uint32_t random)
{
    EXL3_REQUIRE(ctx && logits && ids && rows >= 0 && n > 0 && max_logit >= 0, "gumbel_sample: bad argument");
    if (rows == 0) return EXL3_OK;
    const int lim = (max_logit == 0 || max_logit > n) ? n : max_logit;
    if (fp32) gumbel_sample_kernel<true><<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, ids, n, lim, random);
    else gumbel_sample_kernel<false><<<rows, 1024, 0, (cudaStream_t)stream>>>(logits, ids, n, lim, random);
    ctx->launches++;
    return exl3_check_launch(ctx, "gumbel_sample");
}

extern "C" int exl3_cache_rotate(exl3_ctx* ctx, exl3_stream stream, void* cache, const int32_t* order, void* temp, int pages,
                                 int n_order, size_t page_bytes)
{
    EXL3_REQUIRE(ctx && cache && temp && (order || n_order == 0) && pages > 0 && n_order >= 0, "cache_rotate: bad argument");
    EXL3_REQUIRE(page_bytes > 0 && page_bytes % 16 == 0 && aligned16(cache) && aligned16(temp),
                 "cache_rotate: pages must be multiples of 16 bytes, 16-byte aligned");
    if (n_order == 0) return EXL3_OK;
    const size_t chunks = page_bytes / 16;
    const unsigned grid = (unsigned)std::min<size_t>((chunks + 255) / 256, (size_t)ctx->num_sms * 8);
    cache_rotate_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((uint8_t*)cache, order, (uint8_t*)temp, page_bytes, n_order);
    ctx->launches++;
    return exl3_check_launch(ctx, "cache_rotate");
}

extern "C" int exl3_mul_sigmoid_(exl3_ctx* ctx, exl3_stream stream, void* x, const void* y, int64_t numel)
{
    EXL3_REQUIRE(ctx && x && y && numel >= 0 && numel % 2 == 0, "mul_sigmoid_: bad argument");
    if (numel == 0) return EXL3_OK;
    mul_sigmoid_kernel<<<(unsigned)((numel / 2 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((half2*)x, (const half2*)y, numel / 2);
    ctx->launches++;
    return exl3_check_launch(ctx, "mul_sigmoid_");
}

extern "C" int exl3_deinterleave_qg(exl3_ctx* ctx, exl3_stream stream, const void* qg, void* q, void* g, int rows, int heads, int head_dim)
{
    EXL3_REQUIRE(ctx && qg && q && g && rows >= 0 && heads > 0 && head_dim > 0 && head_dim % 8 == 0, "deinterleave_qg: bad argument");
    EXL3_REQUIRE(aligned16(qg) && aligned16(q) && aligned16(g), "deinterleave_qg: pointers must be 16-byte aligned");
    const long long n8 = (long long)rows * heads * (head_dim / 8);
    if (n8 == 0) return EXL3_OK;
    deinterleave_qg_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)qg, (uint4*)q, (uint4*)g, head_dim / 8, n8);
    ctx->launches++;
    return exl3_check_launch(ctx, "deinterleave_qg");
}
