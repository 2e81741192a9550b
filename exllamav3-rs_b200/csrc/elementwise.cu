// Memory-bound row ops of the decode step: Hadamard-128, RMSNorm (+ fused residual add), RoPE (+ fused per-head
// RMSNorm), SiLU*mul, add, argmax, embedding gather.  Each op states the reference kernel whose arithmetic it follows.
#include "common.cuh"

namespace {

constexpr float R128 = 0.088388347648f;   // 1/sqrt(128), the constant the reference multiplies by

__device__ __forceinline__ void had4(float& v0, float& v1, float& v2, float& v3)
{
    float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
    v0 = s0 + s1; v1 = d0 + d1; v2 = s0 - s1; v3 = d0 - d1;
}

// butterflies over lane bits `from`..`to` (exclusive) for four values per lane
__device__ __forceinline__ void had_lanes(float& v0, float& v1, float& v2, float& v3, int lane, int rounds)
{
    #pragma unroll
    for (int r = 0; r < 5; ++r) {
        if (r >= rounds) break;
        const int i = 1 << r;
        float p0 = __shfl_xor_sync(0xffffffffu, v0, i), p1 = __shfl_xor_sync(0xffffffffu, v1, i);
        float p2 = __shfl_xor_sync(0xffffffffu, v2, i), p3 = __shfl_xor_sync(0xffffffffu, v3, i);
        const bool up = lane & i;
        v0 = (up ? -v0 : v0) + p0; v1 = (up ? -v1 : v1) + p1;
        v2 = (up ? -v2 : v2) + p2; v3 = (up ? -v3 : v3) + p3;
    }
}

// ---------------------------------------------------------------------------------------------- had_r_128
// One warp per 128-element block; lane t holds elements 4t..4t+3 (reference: kernels/quant/hadamard_inner.cuh:93-212).
template <typename T>
__global__ void __launch_bounds__(256) had128_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                     const half* __restrict__ pre, const half* __restrict__ post,
                                                     float r_scale, long long blocks, int blocks_per_row)
{
    const int lane = threadIdx.x & 31;
    long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for (; w < blocks; w += stride) {
        const int cb = (int)(w % blocks_per_row);
        float v0, v1, v2, v3;
        if constexpr (sizeof(T) == 2) {
            uint2 raw = reinterpret_cast<const uint2*>(x + w * 128)[lane];
            half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
            if (pre) {
                uint2 sr = reinterpret_cast<const uint2*>(pre + cb * 128)[lane];
                a = __hmul2(a, *reinterpret_cast<half2*>(&sr.x));
                b = __hmul2(b, *reinterpret_cast<half2*>(&sr.y));
            }
            v0 = __low2float(a); v1 = __high2float(a); v2 = __low2float(b); v3 = __high2float(b);
        } else {
            float4 f = reinterpret_cast<const float4*>(x + w * 128)[lane];
            v0 = f.x; v1 = f.y; v2 = f.z; v3 = f.w;
            if (pre) {
                uint2 sr = reinterpret_cast<const uint2*>(pre + cb * 128)[lane];
                half2 sa = *reinterpret_cast<half2*>(&sr.x), sb = *reinterpret_cast<half2*>(&sr.y);
                v0 *= __low2float(sa); v1 *= __high2float(sa); v2 *= __low2float(sb); v3 *= __high2float(sb);
            }
        }
        had4(v0, v1, v2, v3);
        had_lanes(v0, v1, v2, v3, lane, 5);
        v0 *= r_scale; v1 *= r_scale; v2 *= r_scale; v3 *= r_scale;
        if constexpr (sizeof(T) == 2) {
            half2 a = __floats2half2_rn(v0, v1), b = __floats2half2_rn(v2, v3);
            if (post) {
                uint2 sr = reinterpret_cast<const uint2*>(post + cb * 128)[lane];
                a = __hmul2(a, *reinterpret_cast<half2*>(&sr.x));
                b = __hmul2(b, *reinterpret_cast<half2*>(&sr.y));
            }
            uint2 o; o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
            reinterpret_cast<uint2*>(y + w * 128)[lane] = o;
        } else {
            if (post) {
                uint2 sr = reinterpret_cast<const uint2*>(post + cb * 128)[lane];
                half2 sa = *reinterpret_cast<half2*>(&sr.x), sb = *reinterpret_cast<half2*>(&sr.y);
                v0 *= __low2float(sa); v1 *= __high2float(sa); v2 *= __low2float(sb); v3 *= __high2float(sb);
            }
            reinterpret_cast<float4*>(y + w * 128)[lane] = make_float4(v0, v1, v2, v3);
        }
    }
}

// ------------------------------------------------------------------------------------------------- RMSNorm
__device__ __forceinline__ float block_sum(float v, float* sh)
{
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    v = lane < nw ? sh[lane] : 0.0f;
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One CTA per row, up to 8 float4 per thread kept in registers between the two phases.
// Arithmetic follows kernels/norm.cu:160-304: fp32 sum of squares, rsqrtf(sum/dim + eps) * cscale, x * (w + cbias) * rmf.
template <typename TI, typename TO, bool RES_IN>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const TI* __restrict__ x, const half* __restrict__ w,
                                                        TO* __restrict__ y, float* __restrict__ r, float eps,
                                                        float cbias, float cscale, int dim)
{
    __shared__ float sh[32];
    const int cols = dim >> 2;
    const size_t row = blockIdx.x;
    float4 v[8];
    float sum = 0.0f;
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < cols) {
            float4 f;
            if constexpr (sizeof(TI) == 2) {
                uint2 raw = reinterpret_cast<const uint2*>(x + row * dim)[c];
                half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
                f = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
            } else {
                f = reinterpret_cast<const float4*>(x + row * dim)[c];
            }
            if constexpr (RES_IN) {
                float4 q = reinterpret_cast<const float4*>(r + row * dim)[c];
                f.x += q.x; f.y += q.y; f.z += q.z; f.w += q.w;
                reinterpret_cast<float4*>(r + row * dim)[c] = f;
            }
            sum = fmaf(f.x, f.x, sum); sum = fmaf(f.y, f.y, sum); sum = fmaf(f.z, f.z, sum); sum = fmaf(f.w, f.w, sum);
            v[i] = f;
        }
    }
    sum = block_sum(sum, sh);
    const float rmf = rsqrtf(sum / (float)dim + eps) * cscale;
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < cols) {
            float4 f = v[i];
            if (w) {
                uint2 raw = reinterpret_cast<const uint2*>(w)[c];
                half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
                f.x = f.x * (__low2float(a) + cbias) * rmf;  f.y = f.y * (__high2float(a) + cbias) * rmf;
                f.z = f.z * (__low2float(b) + cbias) * rmf;  f.w = f.w * (__high2float(b) + cbias) * rmf;
            } else {
                f.x *= rmf; f.y *= rmf; f.z *= rmf; f.w *= rmf;
            }
            if constexpr (sizeof(TO) == 2) {
                half2 a = __floats2half2_rn(f.x, f.y), b = __floats2half2_rn(f.z, f.w);
                uint2 o; o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
                reinterpret_cast<uint2*>(y + row * dim)[c] = o;
            } else {
                reinterpret_cast<float4*>(y + row * dim)[c] = f;
            }
        }
    }
}

// 128-point Hadamard transform of a block whose element 4 * lane + j sits in v[j] of lane `lane`, after the fp16 sign
// multiply: same arithmetic as the large-M GEMM's input transform (fp16 product, fp32 butterflies, one fp16 rounding).
__device__ __forceinline__ uint2 had128_signed_lane(half2 a, half2 b, const half* __restrict__ suh, int col, int lane)
{
    const uint2 sr = reinterpret_cast<const uint2*>(suh)[col];
    a = __hmul2(a, *reinterpret_cast<const half2*>(&sr.x));
    b = __hmul2(b, *reinterpret_cast<const half2*>(&sr.y));
    float v0 = __low2float(a), v1 = __high2float(a), v2 = __low2float(b), v3 = __high2float(b);
    const float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
    v0 = s0 + s1; v1 = d0 + d1; v2 = s0 - s1; v3 = d0 - d1;
    #pragma unroll
    for (int i = 1; i < 32; i <<= 1) {
        const float p0 = __shfl_xor_sync(0xffffffffu, v0, i), p1 = __shfl_xor_sync(0xffffffffu, v1, i);
        const float p2 = __shfl_xor_sync(0xffffffffu, v2, i), p3 = __shfl_xor_sync(0xffffffffu, v3, i);
        const bool up = lane & i;
        v0 = (up ? -v0 : v0) + p0; v1 = (up ? -v1 : v1) + p1;
        v2 = (up ? -v2 : v2) + p2; v3 = (up ? -v3 : v3) + p3;
    }
    constexpr float R128 = 0.088388347648f;
    a = __floats2half2_rn(v0 * R128, v1 * R128);
    b = __floats2half2_rn(v2 * R128, v3 * R128);
    uint2 o; o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
    return o;
}

// rms_norm_kernel whose fp16 result goes straight through the input transform of the EXL3 tensors that read it (up to
// three: q/k/v or gate/up, each with its own sign vector) instead of to memory: the norm's own output and the separate
// transform launch drop out.  A warp's 32 float4 columns of one pass are one 128-block (dim % 128 == 0).
template <typename TI, bool RES_IN>
__global__ void __launch_bounds__(1024) rms_norm_had_kernel(const TI* __restrict__ x, const half* __restrict__ w, float* __restrict__ r,
                                                            float eps, float cbias, float cscale, int dim, const exl3_pre_act pre)
{
    __shared__ float sh[32];
    const int cols = dim >> 2, lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    float4 v[8];
    float sum = 0.0f;
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < cols) {
            float4 f;
            if constexpr (sizeof(TI) == 2) {
                uint2 raw = reinterpret_cast<const uint2*>(x + row * dim)[c];
                half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
                f = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
            } else {
                f = reinterpret_cast<const float4*>(x + row * dim)[c];
            }
            if constexpr (RES_IN) {
                float4 q = reinterpret_cast<const float4*>(r + row * dim)[c];
                f.x += q.x; f.y += q.y; f.z += q.z; f.w += q.w;
                reinterpret_cast<float4*>(r + row * dim)[c] = f;
            }
            sum = fmaf(f.x, f.x, sum); sum = fmaf(f.y, f.y, sum); sum = fmaf(f.z, f.z, sum); sum = fmaf(f.w, f.w, sum);
            v[i] = f;
        }
    }
    sum = block_sum(sum, sh);
    const float rmf = rsqrtf(sum / (float)dim + eps) * cscale;
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < cols) {                                         // warp-uniform: cols % 32 == 0
            float4 f = v[i];
            if (w) {
                uint2 raw = reinterpret_cast<const uint2*>(w)[c];
                half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
                f.x = f.x * (__low2float(a) + cbias) * rmf;  f.y = f.y * (__high2float(a) + cbias) * rmf;
                f.z = f.z * (__low2float(b) + cbias) * rmf;  f.w = f.w * (__high2float(b) + cbias) * rmf;
            } else {
                f.x *= rmf; f.y *= rmf; f.z *= rmf; f.w *= rmf;
            }
            const half2 a = __floats2half2_rn(f.x, f.y), b = __floats2half2_rn(f.z, f.w);      // what rms_norm_kernel stores
            #pragma unroll
            for (int sgm = 0; sgm < 3; ++sgm)
                if (sgm < pre.nseg)
                    reinterpret_cast<uint2*>(pre.a_had[sgm] + row * dim)[c] = had128_signed_lane(a, b, pre.suh[sgm], c, lane);
        }
    }
}

// ---------------------------------------------------------------------------------------------------- RoPE
// One warp per (row, head); lane holds elements lane + 32*i.  Arithmetic follows kernels/rope.cu:55-255: optional
// RMSNorm (value rounded to fp16, weight + bias in fp16, fp16 product), then the rotation in fp32 with __sinf/__cosf of
// inv_freq[t] * float(pos), rounded to fp16.
template <int EPL>   // elements per lane = hd / 32
__global__ void __launch_bounds__(256) rope_kernel(const half* q, const half* k, half* out_q, half* out_k,
                                                   const float* __restrict__ inv_freq, int n_freq, uint32_t position,
                                                   const int32_t* __restrict__ positions,
                                                   const int32_t* __restrict__ row_pos, const half* __restrict__ q_norm,
                                                   const half* __restrict__ k_norm, float norm_eps, float norm_cbias,
                                                   int rope_mode, float attn_factor, int rows, int seq, int nq, int nk)
{
    constexpr int HD = EPL * 32;
    const int lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int heads = nq + nk;
    if (gw >= (long long)rows * heads) return;
    const int row = (int)(gw / heads), h = (int)(gw % heads);
    const half* p; half* po; const half* nw;
    if (h < nq) { p = q + ((size_t)row * nq + h) * HD; po = out_q + ((size_t)row * nq + h) * HD; nw = q_norm; }
    else        { p = k + ((size_t)row * nk + (h - nq)) * HD; po = out_k + ((size_t)row * nk + (h - nq)) * HD; nw = k_norm; }
    int pos;
    if (row_pos) pos = row_pos[row];
    else         pos = (row % seq) + (positions ? positions[row / seq] : (int)position);

    half x[EPL];
    #pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] = p[lane + 32 * i];

    if (nw) {
        float ss = 0.0f;
        #pragma unroll
        for (int i = 0; i < EPL; ++i) { float f = __half2float(x[i]); ss += f * f; }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rmf = rsqrtf(ss / (float)HD + norm_eps);
        const half cb = __float2half_rn(norm_cbias);
        #pragma unroll
        for (int i = 0; i < EPL; ++i)
            x[i] = __hmul(__hadd(nw[lane + 32 * i], cb), __float2half_rn(__half2float(x[i]) * rmf));
    }

    const float pf = __int2float_rn(pos);
    if (rope_mode == EXL3_ROPE_NEOX) {
        // pair (t, t + n_freq); n_freq % 32 == 0 keeps both on the same lane
        const int off = n_freq >> 5;
        #pragma unroll
        for (int i = 0; i < EPL / 2; ++i) {
            if (i < off) {
                const int t = lane + 32 * i;
                float ang = inv_freq[t] * pf;
                float sn = __sinf(ang) * attn_factor, cs = __cosf(ang) * attn_factor;
                #pragma unroll
                for (int j = 0; j < EPL; ++j) {
                    if (j == i + off) {
                        float v1 = __half2float(x[i]), v2 = __half2float(x[j]);
                        x[i] = __float2half_rn(v1 * cs - v2 * sn);
                        x[j] = __float2half_rn(v2 * cs + v1 * sn);
                    }
                }
            }
        }
    } else if (rope_mode == EXL3_ROPE_GPTJ) {
        // pair (2t, 2t+1): neighbouring lanes
        #pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = lane + 32 * i;
            float mine = __half2float(x[i]);
            float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            if (e < 2 * n_freq) {
                float ang = inv_freq[e >> 1] * pf;
                float sn = __sinf(ang) * attn_factor, cs = __cosf(ang) * attn_factor;
                x[i] = (e & 1) ? __float2half_rn(mine * cs + other * sn) : __float2half_rn(mine * cs - other * sn);
            }
        }
    }
    #pragma unroll
    for (int i = 0; i < EPL; ++i) po[lane + 32 * i] = x[i];
}

// --------------------------------------------------------------------------------------------- activations
// z = silu(x) * y entirely in fp16: kernels/activation_kernels.cuh:22-31 (h2exp, h2rcp) and :142-186.
__global__ void __launch_bounds__(256) silu_mul_kernel(const half2* __restrict__ x, const half2* __restrict__ y,
                                                       half2* __restrict__ z, long long n4)
{
    long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    uint4 xr = reinterpret_cast<const uint4*>(x)[i], yr = reinterpret_cast<const uint4*>(y)[i], o;
    const half2 one = __float2half2_rn(1.0f);
    const uint32_t* xp = &xr.x; const uint32_t* yp = &yr.x; uint32_t* op = &o.x;
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
        half2 a = *reinterpret_cast<const half2*>(xp + j), b = *reinterpret_cast<const half2*>(yp + j);
        half2 r = h2rcp(__hadd2(one, h2exp(__hneg2(a))));
        half2 s = __hmul2(__hmul2(a, r), b);
        op[j] = *reinterpret_cast<uint32_t*>(&s);
    }
    reinterpret_cast<uint4*>(z)[i] = o;
}

__global__ void __launch_bounds__(256) silu_mul_tail_kernel(const half* x, const half* y, half* z, long long from,
                                                            long long numel)
{
    long long i = from + (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= numel) return;
    half a = x[i];
    half r = hrcp(__hadd(__float2half_rn(1.0f), hexp(__hneg(a))));
    z[i] = __hmul(__hmul(a, r), y[i]);
}

// silu_mul_kernel whose result goes straight through the input transform of the EXL3 tensor that reads it (down_proj):
// one warp per 128-block of a row, lane = 4 consecutive elements.
constexpr int SH_BLOCKS = 4;          // 128-blocks per warp: their loads are all in flight before the first is used
__global__ void __launch_bounds__(256) silu_mul_had_kernel(const half* __restrict__ x, const half* __restrict__ y,
                                                           const half* __restrict__ suh, half* __restrict__ a_had, long long blocks, int bpr)
{
    const int lane = threadIdx.x & 31;
    const long long blk0 = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * SH_BLOCKS;
    if (blk0 >= blocks) return;
    uint2 xr[SH_BLOCKS], yr[SH_BLOCKS];
    #pragma unroll
    for (int u = 0; u < SH_BLOCKS; ++u) {
        const long long blk = blk0 + u < blocks ? blk0 + u : blocks - 1;         // the tail repeats the last block
        xr[u] = reinterpret_cast<const uint2*>(x + blk * 128)[lane];
        yr[u] = reinterpret_cast<const uint2*>(y + blk * 128)[lane];
    }
    const half2 one = __float2half2_rn(1.0f);
    #pragma unroll
    for (int u = 0; u < SH_BLOCKS; ++u) {
        const long long blk = blk0 + u;
        if (blk >= blocks) break;                                                // warp-uniform
        half2 z[2];
        #pragma unroll
        for (int j = 0; j < 2; ++j) {
            const half2 a = *reinterpret_cast<const half2*>(&xr[u].x + j), b = *reinterpret_cast<const half2*>(&yr[u].x + j);
            const half2 rr = h2rcp(__hadd2(one, h2exp(__hneg2(a))));
            z[j] = __hmul2(__hmul2(a, rr), b);
        }
        const int col = (int)(blk % bpr) * 32 + lane;           // uint2 index inside the sign vector
        reinterpret_cast<uint2*>(a_had + blk * 128)[lane] = had128_signed_lane(z[0], z[1], suh, col, lane);
    }
}

__global__ void __launch_bounds__(256) add_kernel(const half* __restrict__ x, const half* __restrict__ y,
                                                  half* __restrict__ z, long long numel)
{
    long long i = ((long long)blockIdx.x * 256 + threadIdx.x) * 2;
    if (i + 1 < numel) {
        half2 a = *reinterpret_cast<const half2*>(x + i), b = *reinterpret_cast<const half2*>(y + i);
        *reinterpret_cast<half2*>(z + i) = __hadd2(a, b);
    } else if (i < numel) {
        z[i] = __hadd(x[i], y[i]);
    }
}

// -------------------------------------------------------------------------------------------------- argmax
// One CTA per row; every comparison keeps the lower index on ties (kernels/reduction.cuh:9-22 uses strict >).
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits, int64_t* __restrict__ ids, int n,
                                                      int max_logit)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    const T* p = logits + (size_t)blockIdx.x * n;
    float best = -INFINITY; int bi = 0;
    for (int i = threadIdx.x; i < max_logit; i += blockDim.x) {
        float f;
        if constexpr (sizeof(T) == 2) f = __half2float(p[i]); else f = p[i];
        if (f > best) { best = f; bi = i; }
    }
    auto better = [](float v, int i, float bv, int b) { return v > bv || (v == bv && i < b); };
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY; bi = lane < nw ? si[lane] : 0x7fffffff;
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) ids[blockIdx.x] = (best == -INFINITY) ? 0 : bi;
    }
}

__global__ void __launch_bounds__(256) embed_kernel(const int64_t* __restrict__ ids, const half* __restrict__ table,
                                                    float* __restrict__ out, int rows, int dim, int vocab)
{
    const int per_row = dim >> 3;
    long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)rows * per_row) return;
    const int row = (int)(i / per_row), c = (int)(i % per_row);
    long long id = ids[row];
    if (id < 0 || id >= vocab) id = 0;
    uint4 raw = reinterpret_cast<const uint4*>(table + (size_t)id * dim)[c];
    const half2* h = reinterpret_cast<const half2*>(&raw);
    float4 a = make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1]));
    float4 b = make_float4(__low2float(h[2]), __high2float(h[2]), __low2float(h[3]), __high2float(h[3]));
    float4* o = reinterpret_cast<float4*>(out + (size_t)row * dim) + 2 * c;
    o[0] = a; o[1] = b;
}

}  // namespace

// ================================================================================================== C-ABI

extern "C" int exl3_had_r_128(exl3_ctx* ctx, exl3_stream stream, const void* x, void* y, const void* pre_scale,
                              const void* post_scale, float scale, int rows, int cols, int fp32)
{
    EXL3_REQUIRE(ctx && x && y, "had_r_128: null argument");
    EXL3_REQUIRE(rows >= 0 && cols > 0 && cols % 128 == 0, "had_r_128: cols % 128 == 0 required");
    EXL3_REQUIRE(aligned16(x) && aligned16(y), "had_r_128: pointers must be 16-byte aligned");
    if (rows == 0) return EXL3_OK;
    // the reference applies pre_scale when given, else post_scale (hadamard.cu:113-141)
    if (pre_scale) post_scale = nullptr;
    const long long blocks = (long long)rows * (cols / 128);
    const int grid = (int)((blocks + 7) / 8 < 148 * 16 ? (blocks + 7) / 8 : 148 * 16);
    const float r_scale = scale * R128;
    cudaStream_t st = (cudaStream_t)stream;
    if (fp32) had128_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (float*)y, (const half*)pre_scale,
                                                         (const half*)post_scale, r_scale, blocks, cols / 128);
    else      had128_kernel<half><<<grid, 256, 0, st>>>((const half*)x, (half*)y, (const half*)pre_scale,
                                                        (const half*)post_scale, r_scale, blocks, cols / 128);
    ctx->launches++;
    return exl3_check_launch(ctx, "had_r_128");
}

static int rms_norm_impl(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w, void* y,
                         int y_fp32, float* r, float eps, float cbias, float cscale, int rows, int dim)
{
    EXL3_REQUIRE(ctx && x && y, "rms_norm: null argument");
    EXL3_REQUIRE(rows >= 0 && dim > 0 && dim % 4 == 0, "rms_norm: dim % 4 == 0 required");
    EXL3_REQUIRE(dim <= 32768, "rms_norm: dim > 32768 is not supported");
    EXL3_REQUIRE(aligned16(x) && aligned16(y) && aligned16(w) && aligned16(r), "rms_norm: pointers must be 16-byte aligned");
    if (rows == 0) return EXL3_OK;
    const int cols = dim / 4;
    int threads = cols <= 2048 ? 256 : 1024;
    if (cols < 256) threads = ((cols + 31) / 32) * 32;
    cudaStream_t st = (cudaStream_t)stream;
    const half* wp = (const half*)w;
#define RN_LAUNCH(TI, TO)                                                                                              \
    do {                                                                                                               \
        if (r) rms_norm_kernel<TI, TO, true><<<rows, threads, 0, st>>>((const TI*)x, wp, (TO*)y, r, eps, cbias, cscale, dim); \
        else   rms_norm_kernel<TI, TO, false><<<rows, threads, 0, st>>>((const TI*)x, wp, (TO*)y, r, eps, cbias, cscale, dim); \
    } while (0)
    if (x_fp32 && y_fp32) RN_LAUNCH(float, float);
    else if (x_fp32)      RN_LAUNCH(float, half);
    else if (y_fp32)      RN_LAUNCH(half, float);
    else                  RN_LAUNCH(half, half);
#undef RN_LAUNCH
    ctx->launches++;
    return exl3_check_launch(ctx, "rms_norm");
}

extern "C" int exl3_rms_norm(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w, void* y,
                             int y_fp32, float eps, float constant_bias, float constant_scale, int rows, int dim)
{
    return rms_norm_impl(ctx, stream, x, x_fp32, w, y, y_fp32, nullptr, eps, constant_bias, constant_scale, rows, dim);
}

extern "C" int exl3_rms_norm_res_in(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w,
                                    void* y, int y_fp32, float* r, float eps, float constant_bias,
                                    float constant_scale, int rows, int dim)
{
    EXL3_REQUIRE(r, "rms_norm_res_in: null residual");
    return rms_norm_impl(ctx, stream, x, x_fp32, w, y, y_fp32, r, eps, constant_bias, constant_scale, rows, dim);
}

extern "C" int exl3_rope(exl3_ctx* ctx, exl3_stream stream, void* q, void* out_q, void* k, void* out_k, const float* inv_freq, int n_freq,
                         uint32_t position, const int32_t* positions, const int32_t* row_pos, const void* q_norm,
                         const void* k_norm, float norm_eps, float norm_constant_bias, int rope_mode,
                         float attn_factor, int bsz, int seq, int nq, int nk, int hd)
{
    EXL3_REQUIRE(ctx && q && inv_freq, "rope: null argument");
    EXL3_REQUIRE(bsz >= 0 && seq >= 0 && nq > 0 && nk >= 0, "rope: bad shape");
    EXL3_REQUIRE(k || nk == 0, "rope: k is null but nk > 0");
    if (hd != 64 && hd != 128 && hd != 256) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "rope: head_dim must be 64, 128 or 256");
    EXL3_REQUIRE(n_freq > 0 && 2 * n_freq <= hd, "rope: 2*n_freq must be <= head_dim");
    if (rope_mode == EXL3_ROPE_NEOX && n_freq % 32 != 0)
        return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "rope: NEOX mode needs n_freq % 32 == 0");
    if (rope_mode != EXL3_ROPE_NEOX && rope_mode != EXL3_ROPE_GPTJ && rope_mode != EXL3_ROPE_NONE)
        return exl3_fail(ctx, EXL3_ERR_INVALID, "rope: unknown rope_mode");
    const int rows = bsz * seq;
    if (rows == 0) return EXL3_OK;
    const long long warps = (long long)rows * (nq + (k ? nk : 0));
    const int grid = (int)((warps + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    const int nk_eff = k ? nk : 0;
#define ROPE_LAUNCH(E)                                                                                                 \
    rope_kernel<E><<<grid, 256, 0, st>>>((const half*)q, (const half*)k, (half*)(out_q ? out_q : q), (half*)(out_k ? out_k : k), inv_freq, n_freq, position, positions, row_pos, \
                                         (const half*)q_norm, (const half*)k_norm, norm_eps, norm_constant_bias,       \
                                         rope_mode, attn_factor, rows, seq, nq, nk_eff)
    if (hd == 64) ROPE_LAUNCH(2); else if (hd == 128) ROPE_LAUNCH(4); else ROPE_LAUNCH(8);
#undef ROPE_LAUNCH
    ctx->launches++;
    return exl3_check_launch(ctx, "rope");
}

extern "C" int exl3_silu_mul(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z,
                             float act_limit, int64_t numel)
{
    EXL3_REQUIRE(ctx && x && y && z && numel >= 0, "silu_mul: null argument");
    if (act_limit != 0.0f) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "silu_mul: act_limit != 0 is not supported");
    EXL3_REQUIRE(aligned16(x) && aligned16(y) && aligned16(z), "silu_mul: pointers must be 16-byte aligned");
    if (numel == 0) return EXL3_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const long long n8 = numel / 8;
    if (n8) {
        silu_mul_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>((const half2*)x, (const half2*)y, (half2*)z, n8);
        ctx->launches++;
    }
    if (numel % 8) {
        silu_mul_tail_kernel<<<1, 256, 0, st>>>((const half*)x, (const half*)y, (half*)z, n8 * 8, numel);
        ctx->launches++;
    }
    return exl3_check_launch(ctx, "silu_mul");
}

extern "C" int exl3_add(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, int64_t numel)
{
    EXL3_REQUIRE(ctx && x && y && z && numel >= 0, "add: null argument");
    if (numel == 0) return EXL3_OK;
    const long long pairs = (numel + 1) / 2;
    add_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const half*)x, (const half*)y, (half*)z, numel);
    ctx->launches++;
    return exl3_check_launch(ctx, "add");
}

extern "C" int exl3_argmax_sample(exl3_ctx* ctx, exl3_stream stream, const void* logits, int fp32, int64_t* ids,
                                  int rows, int n, int max_logit)
{
    EXL3_REQUIRE(ctx && logits && ids, "argmax_sample: null argument");
    EXL3_REQUIRE(rows >= 0 && n > 0 && max_logit >= 0, "argmax_sample: bad shape");
    if (rows == 0) return EXL3_OK;
    if (max_logit == 0 || max_logit > n) max_logit = n;
    cudaStream_t st = (cudaStream_t)stream;
    if (fp32) argmax_kernel<float><<<rows, 1024, 0, st>>>((const float*)logits, ids, n, max_logit);
    else      argmax_kernel<half><<<rows, 1024, 0, st>>>((const half*)logits, ids, n, max_logit);
    ctx->launches++;
    return exl3_check_launch(ctx, "argmax_sample");
}

extern "C" int exl3_embed(exl3_ctx* ctx, exl3_stream stream, const int64_t* ids, const void* table, float* out,
                          int rows, int dim, int vocab)
{
    EXL3_REQUIRE(ctx && ids && table && out, "embed: null argument");
    EXL3_REQUIRE(rows >= 0 && dim > 0 && dim % 8 == 0 && vocab > 0, "embed: dim % 8 == 0 required");
    EXL3_REQUIRE(aligned16(table) && aligned16(out), "embed: pointers must be 16-byte aligned");
    if (rows == 0) return EXL3_OK;
    const long long items = (long long)rows * (dim / 8);
    embed_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(ids, (const half*)table, out, rows, dim, vocab);
    ctx->launches++;
    return exl3_check_launch(ctx, "embed");
}

// ---- producers that write the tensor-core GEMM's transformed activations themselves (internal: used by the step runner)

int exl3_rms_norm_pre(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w, float* r, float eps,
                      float cbias, float cscale, int rows, int dim, const exl3_pre_act* pre)
{
    EXL3_REQUIRE(ctx && x && pre && pre->nseg >= 1 && pre->nseg <= 3, "rms_norm (fused transform): bad argument");
    EXL3_REQUIRE(rows >= 0 && dim > 0 && dim % 128 == 0 && dim <= 32768, "rms_norm (fused transform): dim % 128 == 0, dim <= 32768 required");
    EXL3_REQUIRE(aligned16(x) && aligned16(w) && aligned16(r), "rms_norm (fused transform): pointers must be 16-byte aligned");
    if (rows == 0) return EXL3_OK;
    const int cols = dim / 4;
    int threads = cols <= 2048 ? 256 : 1024;
    if (cols < 256) threads = ((cols + 31) / 32) * 32;
    cudaStream_t st = (cudaStream_t)stream;
    const half* wp = (const half*)w;
    if (x_fp32) {
        if (r) rms_norm_had_kernel<float, true><<<rows, threads, 0, st>>>((const float*)x, wp, r, eps, cbias, cscale, dim, *pre);
        else   rms_norm_had_kernel<float, false><<<rows, threads, 0, st>>>((const float*)x, wp, r, eps, cbias, cscale, dim, *pre);
    } else {
        if (r) rms_norm_had_kernel<half, true><<<rows, threads, 0, st>>>((const half*)x, wp, r, eps, cbias, cscale, dim, *pre);
        else   rms_norm_had_kernel<half, false><<<rows, threads, 0, st>>>((const half*)x, wp, r, eps, cbias, cscale, dim, *pre);
    }
    ctx->launches++;
    return exl3_check_launch(ctx, "rms_norm (fused transform)");
}

int exl3_silu_mul_pre(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, int rows, int dim, const exl3_pre_act* pre)
{
    EXL3_REQUIRE(ctx && x && y && pre && pre->nseg == 1, "silu_mul (fused transform): bad argument");
    EXL3_REQUIRE(rows >= 0 && dim > 0 && dim % 128 == 0, "silu_mul (fused transform): dim % 128 == 0 required");
    EXL3_REQUIRE(aligned16(x) && aligned16(y), "silu_mul (fused transform): pointers must be 16-byte aligned");
    if (rows == 0) return EXL3_OK;
    const long long blocks = (long long)rows * (dim / 128);
    silu_mul_had_kernel<<<(unsigned)((blocks + 8 * SH_BLOCKS - 1) / (8 * SH_BLOCKS)), 256, 0, (cudaStream_t)stream>>>((const half*)x, (const half*)y, pre->suh[0], pre->a_had[0],
                                                                                      blocks, dim / 128);
    ctx->launches++;
    return exl3_check_launch(ctx, "silu_mul (fused transform)");
}
