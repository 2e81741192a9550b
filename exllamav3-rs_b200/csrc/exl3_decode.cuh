// EXL3 tile decoding: bit-window extraction and the three procedural codebooks.
//
// Format (reference: kernels/quant/exl3_dq.cuh:16-31, kernels/quant/codebook.cuh:56-90, kernels/quant/pack.cu:9-57):
// a 16x16 weight tile is 8*K uint32 words read MSB-first as a ring of 256*K bits.  Ring position t (0..255) has the
// 16-bit state made of ring bits [t*K+K-16, t*K+K).  Lane l of a warp owns positions 8l..8l+7, which sit at tile
// rows 2(l%4)+{0,1,8,9} and columns l/4 and l/4+8 (the mma.m16n8k16 B-fragment order).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace exl3 {

#define EXL3_HD __host__ __device__ __forceinline__

// Integer intrinsics with host stand-ins, so the window extraction can also be unit-tested on a CPU.
EXL3_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, int s)
{
#ifdef __CUDA_ARCH__
    return __funnelshift_r(lo, hi, s);
#else
    return (uint32_t)(((((uint64_t)hi) << 32) | lo) >> (s & 31));
#endif
}
EXL3_HD uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel)
{
#ifdef __CUDA_ARCH__
    return __byte_perm(a, b, sel);
#else
    uint64_t v = (((uint64_t)b) << 32) | a; uint32_t r = 0;
    for (int i = 0; i < 4; ++i) r |= (uint32_t)((v >> (8 * ((sel >> (4 * i)) & 7))) & 0xff) << (8 * i);
    return r;
#endif
}

// The 8 states of lane `lane` from the tile words at `tile` (shared or global memory), st[j] = position 8*lane+j.
template <int K>
EXL3_HD void lane_states(const uint32_t* __restrict__ tile, int lane, uint32_t (&st)[8])
{
    constexpr int NW = 8 * K;
    if constexpr (K == 4) {
        // one word per lane; the window also needs the 12 low bits of the previous word
        uint32_t b = tile[lane], a = tile[(lane + 31) & 31];
        uint32_t c = funnel_r(b, a, 16);
        uint32_t b4 = b >> 4, c4 = c >> 4;
        st[7] = byte_perm(b, 0, 0x4410);
        st[6] = byte_perm(b4, 0, 0x4410);
        st[5] = byte_perm(b, 0, 0x4421);
        st[4] = byte_perm(b4, 0, 0x4421);
        st[3] = byte_perm(c, 0, 0x4410);
        st[2] = byte_perm(c4, 0, 0x4410);
        st[1] = byte_perm(c, 0, 0x4421);
        st[0] = byte_perm(c4, 0, 0x4421);
    } else if constexpr (K == 8) {
        // two words per lane plus the low byte of the word before
        uint2 w = reinterpret_cast<const uint2*>(tile)[lane];
        uint32_t mid = w.x, lo = w.y, hi = tile[(2 * lane + NW - 1) & (NW - 1)];
        uint32_t m1 = funnel_r(lo, mid, 16), m2 = funnel_r(mid, hi, 16);
        st[7] = byte_perm(lo, 0, 0x4410);
        st[6] = byte_perm(lo, 0, 0x4421);
        st[5] = byte_perm(lo, 0, 0x4432);
        st[4] = byte_perm(m1, 0, 0x4421);
        st[3] = byte_perm(mid, 0, 0x4410);
        st[2] = byte_perm(mid, 0, 0x4421);
        st[1] = byte_perm(mid, 0, 0x4432);
        st[0] = byte_perm(m2, 0, 0x4421);
    } else {
        // generic: right-align the lane's window at its last bit, then cut 16-bit fields at compile-time offsets
        const int end = 8 * (lane + 1) * K;              // exclusive end bit of the window, 8K..256K
        const int wi = (end - 1) >> 5;                    // word holding the last bit
        const int drop = ((wi + 1) << 5) - end;           // bits right of the window inside that word
        int i1 = wi - 1; if (i1 < 0) i1 += NW;
        int i0 = wi - 2; if (i0 < 0) i0 += NW;
        uint32_t w2 = tile[wi], w1 = tile[i1];
        constexpr int DROP_MAX = (K % 2) ? 24 : 16;
        constexpr bool NEED3 = (7 * K + 16 + DROP_MAX) > 64;
        uint32_t w0 = NEED3 ? tile[i0] : 0u;
        uint32_t lo = funnel_r(w2, w1, drop);
        uint32_t mid = funnel_r(w1, w0, drop);
        uint32_t hi = w0 >> drop;
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int s = (7 - j) * K;
            uint32_t v;
            if (s + 16 <= 32)      v = lo >> s;
            else if (s < 32)       v = funnel_r(lo, mid, s);
            else if (s + 16 <= 64) v = mid >> (s - 32);
            else                   v = funnel_r(mid, hi, s - 32);
            st[j] = v & 0xffffu;
        }
    }
}

// The 8 states of a lane at 4 bpw with the two nibble shifts written as multiplies, which the FMA pipe executes; the
// permutes and the logic op of the codebook are what keeps the ALU pipe busy.
__device__ __forceinline__ void lane_states4(const uint32_t* __restrict__ tile, int lane, int lane_prev, uint32_t (&st)[8])
{
    const uint32_t b = tile[lane], a = tile[lane_prev];
    const uint32_t c = __funnelshift_r(b, a, 16);
    const uint32_t bl = b * 16u, cl = c * 16u;
    st[7] = __byte_perm(b, 0, 0x4410);
    st[6] = __byte_perm(bl, 0, 0x4421);
    st[5] = __byte_perm(b, 0, 0x4421);
    st[4] = __byte_perm(bl, 0, 0x4432);
    st[3] = __byte_perm(b, 0, 0x4432);
    st[2] = __byte_perm(cl, 0, 0x4421);
    st[1] = __byte_perm(c, 0, 0x4421);
    st[0] = __byte_perm(cl, 0, 0x4432);
}

// ---- codebooks -------------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t lop_3inst(uint32_t x)
{
    // (x & 0x8fff8fff) ^ 0x3b603b60
    asm("lop3.b32 %0, %0, 0x8fff8fff, 0x3b603b60, 0x6a;" : "+r"(x));
    return x;
}

// "raw" form of a decoded weight, cheap to produce and exact once expanded:
//   cb 0/1: a register whose two fp16 halves sum to the weight;
//   cb 2  : low half = fp16(1024 + s), high half = fp16(-1534), weight = fma(1024 + s, k_inv, k_bias).
template <int cb>
__device__ __forceinline__ uint32_t decode_raw(uint32_t s)
{
    if constexpr (cb == 0) return lop_3inst(s * 89226354u + 64248484u);
    else if constexpr (cb == 1) return lop_3inst(s * 0xCBAC1FEDu);
    else return __dp4a(s * 0x83DCD12Du, 0x01010101u, 0xE5FE6400u);   // 0xE5FE = fp16(-1534)
}

// Exact fp16 weights of two states (same arithmetic and rounding as the reference's decode_3inst_2).
template <int cb>
__device__ __forceinline__ half2 decode_pair(uint32_t s0, uint32_t s1)
{
    if constexpr (cb == 2) {
        uint32_t a = __dp4a(s0 * 0x83DCD12Du, 0x01010101u, 0x6400u);
        uint32_t b = __dp4a(s1 * 0x83DCD12Du, 0x01010101u, 0x6400u);
        uint32_t p = __byte_perm(a, b, 0x5410);
        half2 h = *reinterpret_cast<half2*>(&p);
        return __hfma2(h, __half2half2(__ushort_as_half(0x1eee)), __half2half2(__ushort_as_half(0xc931)));
    } else {
        uint32_t y0 = decode_raw<cb>(s0), y1 = decode_raw<cb>(s1);
        uint32_t lo = __byte_perm(y0, y1, 0x5410), hi = __byte_perm(y0, y1, 0x7632);
        return __hadd2(*reinterpret_cast<half2*>(&lo), *reinterpret_cast<half2*>(&hi));
    }
}

}  // namespace exl3
