// EXL3 GEMM for large M (prefill chunks, verify batches, big packed steps): a real contraction on the 5th-generation
// tensor cores.  Activations arrive by TMA (tiled, 128-byte swizzle), trellis codes by bulk copies; eight decoder
// warps turn codes into fp16 weights and write them straight into the K-major swizzled B operand tile in shared memory;
// one thread issues tcgen05.mma with both accumulators (2 x 128 rows x 256 columns, all 512 TMEM columns) resident in
// tensor memory; the epilogue reads TMEM, applies the 128-wide output Hadamard in registers and stores fp16/fp32.
//
// CTA tile: 256 rows x 256 columns, K step 64.  Roles: warp 0 = producer (TMA + bulk copies), warp 1 = MMA issuer and
// TMEM owner, warps 2..17 = decoders, then epilogue (warp w reads TMEM lanes 32*(w%4)..+31).
// Every mbarrier wait is bounded; a wait that runs out makes the CTA skip to the tear-down (TMEM is always freed) and
// sets the status word.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "exl3_decode.cuh"
#include "async_copy.cuh"

namespace exl3 {

constexpr int TC_BM = 256, TC_BN = 256, TC_BK = 64;
constexpr int TC_SA = 3, TC_SR = 3, TC_SB = 2;          // stages: activations, raw codes, decoded weights
constexpr int TC_DECODERS = 16;                          // decoder warps (one 16-column tile strip each)
constexpr int TC_THREADS = (2 + TC_DECODERS) * 32;       // 18 warps
constexpr int TC_MAX_SEG = 3;                            // weight tensors that may share one launch
constexpr int TC_A_STAGE = TC_BM * TC_BK * 2;            // 32 KB
constexpr int TC_B_STAGE = TC_BN * TC_BK * 2;            // 32 KB
constexpr float TC_R128 = 0.088388347648f;

template <int K> struct TcSmem {
    static constexpr int RAW_STAGE = (TC_BK / 16) * (TC_BN / 16) * 32 * K;      // 4 tile rows x 16 tiles x 32K bytes
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + TC_SA * TC_A_STAGE;
    static constexpr int OFF_RAW = OFF_B + TC_SB * TC_B_STAGE;
    static constexpr int OFF_SVH = OFF_RAW + TC_SR * RAW_STAGE;
    static constexpr int OFF_BAR = OFF_SVH + TC_BN * 2;
    static constexpr int N_BARS = 2 * TC_SA + 2 * TC_SR + 2 * TC_SB + 1;
    static constexpr int OFF_TMEM = OFF_BAR + N_BARS * 8;
    static constexpr int BYTES = OFF_TMEM + 16 + 1024;      // + slack to align the base to 1024 bytes
};

// Up to TC_MAX_SEG weight tensors with the same k, bits and codebook share one launch (q/k/v or gate/up of a layer):
// their 256-column blocks are laid end to end along blockIdx.x, which keeps the grid near a whole number of waves.
struct GemmTcParams {
    const uint32_t* trellis[TC_MAX_SEG];   // [k/16][n/16][8K] words
    void* C[TC_MAX_SEG];                   // [m][n] fp16 or fp32
    const half* svh[TC_MAX_SEG];           // [n] or NULL
    int n[TC_MAX_SEG];
    int blk_end[TC_MAX_SEG];               // running count of 256-column blocks
    int* status;
    int m, k, c_fp32;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], fp16 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32])
{
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8])
{
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const float (&v)[8])
{
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tc_wait_st_acc() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO), descriptor version 1
__device__ __forceinline__ uint64_t tc_smem_desc(const void* p)
{
    const uint32_t a = smem_u32(p);
    uint64_t d = 0;
    d |= (uint64_t)((a >> 4) & 0x3fff);            // start address
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzled K-major; 1 as CUTLASS sets)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}

// instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = 256
constexpr uint32_t TC_IDESC = (1u << 4) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);


// in-register unnormalised 32-point Walsh-Hadamard transform (Sylvester order)
__device__ __forceinline__ void fwht32(float (&v)[32])
{
    #pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        #pragma unroll
        for (int i = 0; i < 32; i += 2 * h) {
            #pragma unroll
            for (int j = i; j < i + h; ++j) { const float a = v[j], b = v[j + h]; v[j] = a + b; v[j + h] = a - b; }
        }
    }
}

// grid (n / 256, ceil(m / 256)); the activations come through `amap` (A_had [m][k] fp16, box 64 x 256, 128B swizzle)
template <int K, int CB>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap amap0,
                                                               const __grid_constant__ CUtensorMap amap1,
                                                               const __grid_constant__ CUtensorMap amap2, const GemmTcParams p)
{
    using SM = TcSmem<K>;
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
    uint64_t* a_full = bars;                 uint64_t* a_empty = a_full + TC_SA;
    uint64_t* r_full = a_empty + TC_SA;      uint64_t* r_empty = r_full + TC_SR;
    uint64_t* b_full = r_empty + TC_SR;      uint64_t* b_empty = b_full + TC_SB;
    uint64_t* acc_full = b_empty + TC_SB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::OFF_TMEM);
    __shared__ int s_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seg = (blockIdx.x >= p.blk_end[0]) + (blockIdx.x >= p.blk_end[1]);
    const int n0 = (blockIdx.x - (seg ? p.blk_end[seg - 1] : 0)) * TC_BN, m0 = blockIdx.y * TC_BM;
    const CUtensorMap* amap = seg == 0 ? &amap0 : (seg == 1 ? &amap1 : &amap2);
    const uint32_t* trellis = p.trellis[seg];
    const half* svh = p.svh[seg];
    const int n = p.n[seg];
    const int tiles_n = n >> 4;
    const int ksteps = p.k / TC_BK;
    const bool two_tiles = p.m - m0 > 128;               // a block with at most 128 valid rows skips its second M tile

    if (tid == 0) {
        s_failed = 0;
        for (int i = 0; i < TC_SA; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < TC_SR; ++i) { mbar_init(&r_full[i], 1); mbar_init(&r_empty[i], TC_DECODERS); }
        for (int i = 0; i < TC_SB; ++i) { mbar_init(&b_full[i], TC_DECODERS); mbar_init(&b_empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (svh) for (int i = tid; i < TC_BN; i += TC_THREADS) reinterpret_cast<half*>(smem + SM::OFF_SVH)[i] = svh[n0 + i];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        // ===== producer: activations by TMA, trellis codes by bulk copies
        if (lane == 0) {
            for (int ks = 0; ks < ksteps; ++ks) {
                const int sa = ks % TC_SA, sr = ks % TC_SR;
                if (ks >= TC_SA && !mbar_wait(&a_empty[sa], ((ks / TC_SA) - 1) & 1)) { failed = true; break; }
                mbar_expect_tx(&a_full[sa], TC_A_STAGE);
                tma_load_2d(smem + SM::OFF_A + sa * TC_A_STAGE, amap, ks * TC_BK, m0, &a_full[sa]);
                if (ks >= TC_SR && !mbar_wait(&r_empty[sr], ((ks / TC_SR) - 1) & 1)) { failed = true; break; }
                mbar_expect_tx(&r_full[sr], SM::RAW_STAGE);
                #pragma unroll
                for (int r = 0; r < TC_BK / 16; ++r)
                    bulk_g2s(smem + SM::OFF_RAW + sr * SM::RAW_STAGE + r * (TC_BN / 16) * 32 * K,
                             trellis + ((size_t)(ks * (TC_BK / 16) + r) * tiles_n + (n0 >> 4)) * 8 * K,
                             (TC_BN / 16) * 32 * K, &r_full[sr]);
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer
        if (lane == 0) {
            for (int ks = 0; ks < ksteps; ++ks) {
                const int sa = ks % TC_SA, sb = ks % TC_SB;
                if (!mbar_wait(&a_full[sa], (ks / TC_SA) & 1) || !mbar_wait(&b_full[sb], (ks / TC_SB) & 1)) { failed = true; break; }
                tc_fence_after();
                const uint64_t adesc0 = tc_smem_desc(smem + SM::OFF_A + sa * TC_A_STAGE);
                const uint64_t adesc1 = tc_smem_desc(smem + SM::OFF_A + sa * TC_A_STAGE + 128 * 128);
                const uint64_t bdesc = tc_smem_desc(smem + SM::OFF_B + sb * TC_B_STAGE);
                #pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk) {
                    const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
                    tc_mma_f16(tmem_base, adesc0 + 2 * kk, bdesc + 2 * kk, TC_IDESC, acc);          // +32 bytes per K=16
                    if (two_tiles) tc_mma_f16(tmem_base + TC_BN, adesc1 + 2 * kk, bdesc + 2 * kk, TC_IDESC, acc);
                }
                tc_commit(&a_empty[sa]);      // arrive when the MMAs above have finished reading the stage
                tc_commit(&b_empty[sb]);
            }
            if (!failed) tc_commit(acc_full);
        }
    } else {
        // ===== decoders: raw codes -> fp16 weights in the K-major swizzled B tile
        const int nt = warp - 2;                                   // 0..15: owns tile column nt of every tile row
        const int g = lane >> 2, t = lane & 3;
        for (int ks = 0; ks < ksteps; ++ks) {
            const int sr = ks % TC_SR, sb = ks % TC_SB;
            if (!mbar_wait_warp(&r_full[sr], (ks / TC_SR) & 1)) { failed = true; break; }
            if (ks >= TC_SB && !mbar_wait_warp(&b_empty[sb], ((ks / TC_SB) - 1) & 1)) { failed = true; break; }
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(smem + SM::OFF_RAW + sr * SM::RAW_STAGE);
            uint8_t* bt = smem + SM::OFF_B + sb * TC_B_STAGE;
            #pragma unroll
            for (int r = 0; r < TC_BK / 16; ++r) {
                {
                    uint32_t st[8];
                    lane_states<K>(raw + (r * (TC_BN / 16) + nt) * 8 * K, lane, st);
                    const half2 w0 = decode_pair<CB>(st[0], st[1]);      // rows 2t, 2t+1   col g
                    const half2 w1 = decode_pair<CB>(st[2], st[3]);      // rows 2t+8, +9   col g
                    const half2 w2 = decode_pair<CB>(st[4], st[5]);      // rows 2t, 2t+1   col g+8
                    const half2 w3 = decode_pair<CB>(st[6], st[7]);      // rows 2t+8, +9   col g+8
                    // B tile row = n (128 bytes = 64 k), 16-byte chunk index XOR (n & 7)
                    const int na = nt * 16 + g, nb = na + 8;
                    const int c0 = 2 * r, c1 = 2 * r + 1;                 // chunks of k = 16r + [0,8) and [8,16)
                    uint8_t* ra = bt + na * 128; uint8_t* rb = bt + nb * 128;
                    *reinterpret_cast<half2*>(ra + ((c0 ^ (na & 7)) << 4) + 4 * t) = w0;
                    *reinterpret_cast<half2*>(ra + ((c1 ^ (na & 7)) << 4) + 4 * t) = w1;
                    *reinterpret_cast<half2*>(rb + ((c0 ^ (nb & 7)) << 4) + 4 * t) = w2;
                    *reinterpret_cast<half2*>(rb + ((c1 ^ (nb & 7)) << 4) + 4 * t) = w3;
                }
            }
            fence_proxy_async();                 // make the generic-proxy stores visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) { mbar_arrive(&b_full[sb]); mbar_arrive(&r_empty[sr]); }
        }
    }

    // ===== epilogue (warps 2..17): TMEM -> registers -> output transform -> global
    if (warp >= 2 && !failed) {
        if (!mbar_wait_warp(acc_full, 0)) failed = true;
        if (!failed) {
            tc_fence_after();
            // TMEM lane quadrant q; each of the four warps of a quadrant takes one (M tile, 128-column half) pair
            const int q = warp & 3, mt = (warp - 2) >> 3, sel = ((warp - 2) >> 2) & 1;
            const half* svh_s = reinterpret_cast<const half*>(smem + SM::OFF_SVH) + sel * 128;
            if (mt == 0 || two_tiles) {
                const int row = m0 + mt * 128 + q * 32 + lane;
                const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + mt * TC_BN + sel * 128;
                // The 128-point transform of a row is split so that a thread never holds more than 32 accumulators:
                // the two outer butterfly levels (strides 32 and 64) run on 8-column slices and go back to TMEM, the five
                // inner levels run on each 32-column chunk as it is read for the store.
                if (svh) {
                    #pragma unroll
                    for (int s8 = 0; s8 < 4; ++s8) {
                        float c0[8], c1[8], c2[8], c3[8];
                        tc_ld8(tacc + s8 * 8, c0);      tc_ld8(tacc + 32 + s8 * 8, c1);
                        tc_ld8(tacc + 64 + s8 * 8, c2); tc_ld8(tacc + 96 + s8 * 8, c3);
                        tc_wait_ld();
                        #pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float s01 = c0[e] + c1[e], d01 = c0[e] - c1[e], s23 = c2[e] + c3[e], d23 = c2[e] - c3[e];
                            c0[e] = s01 + s23; c1[e] = d01 + d23; c2[e] = s01 - s23; c3[e] = d01 - d23;
                        }
                        tc_st8(tacc + s8 * 8, c0);      tc_st8(tacc + 32 + s8 * 8, c1);
                        tc_st8(tacc + 64 + s8 * 8, c2); tc_st8(tacc + 96 + s8 * 8, c3);
                    }
                    tc_wait_st_acc();
                }
                #pragma unroll 1
                for (int j = 0; j < 4; ++j) {
                    float v[32];
                    tc_ld32(tacc + j * 32, v);
                    tc_wait_ld();
                    if (svh) {
                        fwht32(v);
                        #pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] *= TC_R128;
                    }
                    if (row < p.m) {
                        const size_t off = (size_t)row * n + n0 + sel * 128 + j * 32;
                        const half* sv = svh_s + j * 32;
                        if (p.c_fp32) {
                            float4* dst = reinterpret_cast<float4*>((float*)p.C[seg] + off);
                            #pragma unroll
                            for (int e = 0; e < 32; e += 4) {
                                float4 o = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                                if (svh) {
                                    o.x *= __half2float(sv[e]); o.y *= __half2float(sv[e + 1]);
                                    o.z *= __half2float(sv[e + 2]); o.w *= __half2float(sv[e + 3]);
                                }
                                dst[e >> 2] = o;
                            }
                        } else {
                            uint4* dst = reinterpret_cast<uint4*>((half*)p.C[seg] + off);
                            #pragma unroll
                            for (int e = 0; e < 32; e += 8) {
                                uint32_t w[4];
                                #pragma unroll
                                for (int h = 0; h < 4; ++h) {
                                    half2 x = __floats2half2_rn(v[e + 2 * h], v[e + 2 * h + 1]);
                                    if (svh) x = __hmul2(x, *reinterpret_cast<const half2*>(sv + e + 2 * h));
                                    w[h] = *reinterpret_cast<uint32_t*>(&x);
                                }
                                dst[e >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            }
        }
    }

    // ===== tear-down: every path arrives here; TMEM is released by the warp that allocated it
    if (failed) s_failed = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 2);
}

}  // namespace exl3
