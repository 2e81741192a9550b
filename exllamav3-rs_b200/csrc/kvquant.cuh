// Warp-level KV-cache codec: 4 groups of 32 values per warp, lane = (group sg = lane/8, sub-lane sl = lane%8) holding
// values 4sl..4sl+3 of its group.  Follows kernels/cache/q_cache_kernels.cuh:61-236 (linear grid only).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace exl3 {

constexpr float R32 = 0.17677669529663688110f;   // 1/sqrt(32)

__device__ __forceinline__ void h4(float& v0, float& v1, float& v2, float& v3)
{
    float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
    v0 = s0 + s1; v1 = d0 + d1; v2 = s0 - s1; v3 = d0 - d1;
}
// H8 across the 8 lanes of a group (lane bits 0..2)
__device__ __forceinline__ void h8_lanes(float& v0, float& v1, float& v2, float& v3, int lane)
{
    #pragma unroll
    for (int i = 1; i < 8; i <<= 1) {
        float p0 = __shfl_xor_sync(0xffffffffu, v0, i), p1 = __shfl_xor_sync(0xffffffffu, v1, i);
        float p2 = __shfl_xor_sync(0xffffffffu, v2, i), p3 = __shfl_xor_sync(0xffffffffu, v3, i);
        const bool up = lane & i;
        v0 = (up ? -v0 : v0) + p0; v1 = (up ? -v1 : v1) + p1;
        v2 = (up ? -v2 : v2) + p2; v3 = (up ? -v3 : v3) + p3;
    }
}

// the reference is built with fast-math, where 1.0f / s is the approximate reciprocal
__device__ __forceinline__ float rcp_fast(float s)
{
    float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(s)); return r;
}

// dequantise the lane's 4 values of its group into fp32 (before the inverse rotation is applied by the caller)
__device__ __forceinline__ void unpack4(const uint32_t* __restrict__ gw, int sl, int bits, uint32_t& q0, uint32_t& q1,
                                        uint32_t& q2, uint32_t& q3)
{
    q0 = q1 = q2 = q3 = 0;
    int wb = 0;
    #pragma unroll
    for (int w = 8; w >= 1; w >>= 1) {
        if (bits & w) {
            const int off = sl * 4 * w;
            const uint32_t word = gw[wb + (off >> 5)] >> (off & 31);
            const uint32_t mask = (1u << w) - 1;
            q0 = (q0 << w) | (word & mask);
            q1 = (q1 << w) | ((word >> w) & mask);
            q2 = (q2 << w) | ((word >> (2 * w)) & mask);
            q3 = (q3 << w) | ((word >> (3 * w)) & mask);
            wb += w;
        }
    }
}

// Quantise 4 groups: in -> 4*32 halfs, out -> 4*bits words, scales -> 4 halfs (only the first `active` groups exist).
__device__ __forceinline__ void quant_x4(const half* __restrict__ in, uint32_t* __restrict__ out,
                                         half* __restrict__ scales, int active, int bits)
{
    const int lane = threadIdx.x & 31, sg = lane >> 3, sl = lane & 7;
    const bool on = sg < active;
    float v0 = 0.f, v1 = 0.f, v2 = 0.f, v3 = 0.f;
    if (on) {
        uint2 raw = reinterpret_cast<const uint2*>(in)[lane];
        half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
        v0 = __low2float(a); v1 = __high2float(a); v2 = __low2float(b); v3 = __high2float(b);
    }
    h4(v0, v1, v2, v3);
    h8_lanes(v0, v1, v2, v3, lane);
    v0 *= R32; v1 *= R32; v2 *= R32; v3 *= R32;
    float s = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3))) + 1e-10f;
    #pragma unroll
    for (int i = 1; i < 8; i <<= 1) s = fmaxf(s, __shfl_xor_sync(0xffffffffu, s, i));
    const float inv_s = rcp_fast(s);
    const float mf = (float)(1 << (bits - 1));
    const int qmax = (1 << bits) - 1;
    auto q1f = [&](float v) -> uint32_t {
        int q = __float2int_rd(fmaf(v * inv_s, mf, mf));
        return (uint32_t)max(min(q, qmax), 0);
    };
    const uint32_t q0 = q1f(v0), q1 = q1f(v1), q2 = q1f(v2), q3 = q1f(v3);

    int rem = bits, wb = 0;
    #pragma unroll
    for (int w = 8; w >= 1; w >>= 1) {
        if (bits & w) {
            rem -= w;
            const uint32_t mask = (1u << w) - 1;
            uint32_t field = ((q0 >> rem) & mask) | (((q1 >> rem) & mask) << w) | (((q2 >> rem) & mask) << (2 * w)) |
                             (((q3 >> rem) & mask) << (3 * w));
            const int off = sl * 4 * w;
            uint32_t word = field << (off & 31);
            const int lanes_per_word = 8 / w;               // 1, 2, 4, 8
            #pragma unroll
            for (int o = 1; o < 8; o <<= 1)
                if (o < lanes_per_word) word |= __shfl_xor_sync(0xffffffffu, word, o);
            if (on && (sl & (lanes_per_word - 1)) == 0) out[sg * bits + wb + (off >> 5)] = word;
            wb += w;
        }
    }
    if (on && sl == 0) scales[sg] = __float2half_rn(s);
}

// Dequantise 4 groups into fp16.
__device__ __forceinline__ void dequant_x4(const uint32_t* __restrict__ in, const half* __restrict__ scales,
                                           half* __restrict__ out, int active, int bits)
{
    const int lane = threadIdx.x & 31, sg = lane >> 3, sl = lane & 7;
    const bool on = sg < active;
    uint32_t q0 = 0, q1 = 0, q2 = 0, q3 = 0;
    if (on) unpack4(in + sg * bits, sl, bits, q0, q1, q2, q3);
    const int m = 1 << (bits - 1);
    float s = on ? __half2float(scales[sg]) : 0.0f;
    s *= R32;
    const float sm = s * (1.0f / (float)m), mh = (float)m - 0.5f;
    float v0 = ((float)(int)q0 - mh) * sm, v1 = ((float)(int)q1 - mh) * sm;
    float v2 = ((float)(int)q2 - mh) * sm, v3 = ((float)(int)q3 - mh) * sm;
    h4(v0, v1, v2, v3);
    h8_lanes(v0, v1, v2, v3, lane);
    if (on) {
        half2 a = __floats2half2_rn(v0, v1), b = __floats2half2_rn(v2, v3);
        uint2 o; o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint2*>(out)[lane] = o;
    }
}

// The same without the inverse rotation: out = (code - (m - 1/2)) * scale / m, in the rotated domain the codes live in.
// For attention the rotation H32/sqrt(32) of every group is orthogonal and symmetric, so q . H(c) = H(q) . c and
// sum_j p_j H(c_j) = H(sum_j p_j c_j): the kernel rotates each query once and each output row once instead of every
// key and value (attn_paged.cuh), and this is all the per-key work that remains.
__device__ __forceinline__ void dequant_x4_norot(const uint32_t* __restrict__ in, const half* __restrict__ scales,
                                                 half* __restrict__ out, int bits)
{
    const int lane = threadIdx.x & 31, sg = lane >> 3, sl = lane & 7;
    // Codes become fp16 numbers without an integer-to-float conversion: 0x6000 | (q << 1) is the half 512 + q (spacing
    // 0.5 in [512, 1024), q <= 255); subtracting 512 + m - 1/2 and multiplying by scale / m are then both exact up to
    // the single final rounding, the same value as (q - (m - 1/2)) * scale / m computed in fp32 and rounded once.
    uint32_t p0, p1;
    if (bits == 4) {
        const uint32_t w = in[sg * 4 + (sl >> 1)] >> ((sl & 1) * 16);
        p0 = 0x60006000u | ((w & 0xFu) << 1) | ((w & 0xF0u) << 13);
        p1 = 0x60006000u | ((w & 0xF00u) >> 7) | ((w & 0xF000u) << 5);
    } else if (bits == 6) {
        // planes of 4 bits (high part of each code) and 2 bits (low part): q = (nibble << 2) | pair
        const uint32_t w4 = in[sg * 6 + (sl >> 1)] >> ((sl & 1) * 16);
        const uint32_t w2 = in[sg * 6 + 4 + (sl >> 2)] >> ((sl & 3) * 8);
        p0 = 0x60006000u | ((w4 & 0xFu) << 3) | ((w2 & 0x3u) << 1) | ((w4 & 0xF0u) << 15) | ((w2 & 0xCu) << 15);
        p1 = 0x60006000u | ((w4 & 0xF00u) >> 5) | ((w2 & 0x30u) >> 3) | ((w4 & 0xF000u) << 7) | ((w2 & 0xC0u) << 11);
    } else if (bits == 8) {
        const uint32_t w = in[sg * 8 + sl];                 // one plane of 8-bit fields: the lane's 4 codes are its 4 bytes
        p0 = 0x60006000u | ((w & 0xFFu) << 1) | ((w & 0xFF00u) << 9);
        p1 = 0x60006000u | ((w >> 15) & 0x1FEu) | ((w & 0xFF000000u) >> 7);
    } else {
        uint32_t q0, q1, q2, q3;
        unpack4(in + sg * bits, sl, bits, q0, q1, q2, q3);
        p0 = 0x60006000u | (q0 << 1) | (q1 << 17);
        p1 = 0x60006000u | (q2 << 1) | (q3 << 17);
    }
    const int m = 1 << (bits - 1);
    const half2 off = __float2half2_rn(512.0f + (float)m - 0.5f);
    const half2 sm = __half2half2(__hmul(scales[sg], __float2half_rn(1.0f / (float)m)));
    const half2 a = __hmul2(__hsub2(*reinterpret_cast<const half2*>(&p0), off), sm);
    const half2 b = __hmul2(__hsub2(*reinterpret_cast<const half2*>(&p1), off), sm);
    uint2 o; o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&b);
    reinterpret_cast<uint2*>(out)[lane] = o;
}

// 4-bit codes of one key and one 128-wide head, K and V in one warp operation: lanes 0..15 scale the 16 words of K (8
// codes each: dims 8l..8l+7), lanes 16..31 those of V.  `rk`/`rv`: the key's codes (64 bytes) with its 4 group scales
// `scale_off` bytes further on; `dk`/`dv`: the key's row of the fp16 tiles.  Same arithmetic, operation for operation,
// as dequant_x4_norot (so the results are the same bits), at half the instructions per value: one shared-memory load
// feeds eight values, and a byte of two codes becomes the half2 (512 + q0, 512 + q1) with one multiply and one logic op
// (b * 0x2002 puts b << 1 and b << 13 side by side; the mask keeps one nibble of each).
__device__ __forceinline__ void dequant4_kv_norot(const uint8_t* __restrict__ rk, const uint8_t* __restrict__ rv, int scale_off,
                                                  half* __restrict__ dk, half* __restrict__ dv)
{
    const int lane = threadIdx.x & 31, l = lane & 15;
    const uint8_t* r = (lane & 16) ? rv : rk;
    half* out = (lane & 16) ? dv : dk;
    const uint32_t w = reinterpret_cast<const uint32_t*>(r)[l];
    const half sc = reinterpret_cast<const half*>(r + scale_off)[l >> 2];
    const half2 off = __float2half2_rn(512.0f + 8.0f - 0.5f);
    const half2 sm = __half2half2(__hmul(sc, __float2half_rn(0.125f)));
    uint32_t o[4];
    #pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t b = __byte_perm(w, 0, 0x4440 + j);
        const uint32_t p = ((b * 0x2002u) & 0x001e001eu) | 0x60006000u;
        const half2 h = __hmul2(__hsub2(*reinterpret_cast<const half2*>(&p), off), sm);
        o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(out)[l] = make_uint4(o[0], o[1], o[2], o[3]);
}

// Unnormalised H32 of a group held in mma fragment order by the 4 lanes of a quad: v[blk][c] is element 8 blk + 2 t + c
// (t = lane & 3).  All 32 lanes must call it.
__device__ __forceinline__ void had32_quad(float (&v)[4][2], int t)
{
    #pragma unroll
    for (int b = 0; b < 4; ++b) { const float a = v[b][0], d = v[b][1]; v[b][0] = a + d; v[b][1] = a - d; }
    #pragma unroll
    for (int c = 0; c < 2; ++c) {
        const float s0 = v[0][c] + v[1][c], d0 = v[0][c] - v[1][c], s1 = v[2][c] + v[3][c], d1 = v[2][c] - v[3][c];
        v[0][c] = s0 + s1; v[1][c] = d0 + d1; v[2][c] = s0 - s1; v[3][c] = d0 - d1;
    }
    #pragma unroll
    for (int i = 1; i < 4; i <<= 1) {
        const bool up = t & i;
        #pragma unroll
        for (int b = 0; b < 4; ++b) {
            #pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float pv = __shfl_xor_sync(0xffffffffu, v[b][c], i);
                v[b][c] = (up ? -v[b][c] : v[b][c]) + pv;
            }
        }
    }
}

}  // namespace exl3
