// EXL3 GEMM for the decode regime (1..16 rows): the weight stream sets the time, so the kernel is built around the cost
// of turning trellis codes into multiplier operands, one warp-instruction at a time.
//
// Function computed (reference: kernels/quant/exl3_gemm_kernel.cuh:14-50, exl3_gemm_inner.cuh:456-480; the reference's
// own small-m kernel is kernels/quant/exl3_gemv_kernel.cuh:138-402):
//   C = H128( fp16(H128(A o suh)/sqrt128) . W ) / sqrt128 o svh
//
// Layout of the work.  A CTA has 16 warps = 8 k-slices x 2 column halves.  Its unit of work is (128-column block,
// 1024-k chunk); inside a unit warp (ks, ch) owns the 8 x 4 weight tiles of k-slice ks (128 k) and column half ch (64
// columns).  Units are ordered column-block-major and dealt to the CTAs as contiguous ranges (stream-K), so a warp walks
// down k with its accumulators in registers and only meets the other warps when the CTA leaves a column block: the 8
// k-slices are added in a fixed order through shared memory, a block shared with a neighbouring CTA goes through a
// partial-sum slot in global memory that the last CTA to arrive adds up in owner order (deterministic), and the finisher
// applies the output Hadamard and svh.
//
// Every warp streams its own codes: a ring of TMA boxes (4 tile rows x 4 tiles) with one mbarrier per slot, issued and
// consumed by the warp itself, so the main loop has no CTA-wide barrier.  The transformed activations arrive in MMA
// fragment order (gemm_decode_prologue_kernel) and are loaded once per slot, 16 bytes per lane and tile row.
//
// Multiplier mapping.  The 16x16 tile is stored in mma.m16n8k16 B-fragment order; read as the A operand of the
// transposed product (weights^T . activations^T) the same registers are one A fragment, so a tile costs two MMAs for
// up to 8 rows (N = 8 is the batch) instead of four.  For codebooks 0/1 a weight is the fp16 sum of the two halves of
// y = lop3(x * C); y goes to the tensor core as two consecutive k entries and the activation is duplicated in the B
// fragment, so the halves are added by the MMA in fp32; codebook 2 uses (1024 + s, -1534) the same way and is scaled
// in the epilogue.  Per tile and lane at 4 bpw: 2 shared loads, 3 shifts, 8 byte permutes, 8 multiplies, 8 lop3, 2 MMAs.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "exl3_decode.cuh"
#include "async_copy.cuh"

namespace exl3 {

constexpr int GD_WARPS = 16;
constexpr int GD_THREADS = GD_WARPS * 32;
constexpr int GD_KSL = 8;                    // k-slices (128 k each) of a CTA unit
constexpr int GD_UNIT_K = GD_KSL * 128;      // k extent of a unit
constexpr int GD_SLOT_ROWS = 4;              // tile rows per TMA box
constexpr int GD_SLOT_TILES = 4;             // tiles per row of a box (one column half)
constexpr int GD_MAX_SEG = 3;
constexpr int GD_RSTRIDE = 132;              // floats per row of the reduction tiles
constexpr float GD_R128 = 0.088388347648f;
constexpr float GD_MUL1_KINV = 0.00676727294921875f;
constexpr float GD_MUL1_DELTA = -10.3828125f + 1534.0f * 0.00676727294921875f;

template <int K, int MT> struct GdSmem {
    static constexpr int ROWS = 8 * MT;                                            // batch rows held by the MMAs
    static constexpr int SLOT_BYTES = GD_SLOT_ROWS * GD_SLOT_TILES * 32 * K;       // 512 K
    static constexpr int RED_BYTES = GD_KSL * ROWS * GD_RSTRIDE * 4;               // per-slice partial tiles
    static constexpr int SC_BYTES = ROWS * GD_RSTRIDE * 4;                         // the summed tile
    static constexpr int ROOM = 227 * 1024 - RED_BYTES - SC_BYTES - 1024;
    static constexpr int DEPTH_FIT = ROOM / (GD_WARPS * SLOT_BYTES);
    static constexpr int DEPTH = DEPTH_FIT > 8 ? 8 : DEPTH_FIT;
    static_assert(DEPTH >= 2, "the code ring needs two slots per warp");
    static constexpr int OFF_RING = 0;
    static constexpr int OFF_RED = OFF_RING + GD_WARPS * DEPTH * SLOT_BYTES;
    static constexpr int OFF_SC = OFF_RED + RED_BYTES;
    static constexpr int OFF_BAR = OFF_SC + SC_BYTES;
    static constexpr int BYTES = OFF_BAR + GD_WARPS * DEPTH * 8 + 128;             // + slack to align the base to 128 bytes
};

struct GemmDecodeParams {
    const uint4* a_frag[GD_MAX_SEG];   // [MT][k/64][4][32] uint4: activations in B-fragment order, duplicated halves
    const float* rowsum[GD_MAX_SEG];   // [8*MT] sum over k of the transformed activations (codebook 2 only)
    void* C[GD_MAX_SEG];               // [m][n] fp16 or fp32
    const half* svh[GD_MAX_SEG];       // [n] or NULL
    int n[GD_MAX_SEG];
    int blk_end[GD_MAX_SEG];           // running count of 128-column blocks
    float* partial;                    // [grid][2][m][128] fp32: a CTA's first and last column block when shared
    int* counters;                     // [column blocks] arrival counters, zero on entry and on exit
    int* status;
    int m, k, c_fp32;
};

__device__ __forceinline__ void gd_tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// D (16 weight columns x 8 batch rows) += A (weights^T, 16 x 16) . B (activations^T, 16 x 8)
__device__ __forceinline__ void gd_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// Activations in fragment order.  One CTA per (batch row slot b, tensor): row b < m is transformed as in
// kernels/quant/hadamard_inner.cuh:93-147 (fp16 pre-scale multiply, fp32 butterflies, one fp16 rounding); slots past m
// are zero-filled.  Word (set, kslot, r, lane = 4 g + t, w) holds the value of batch row 8 set + g at
// k = 64 kslot + 16 r + 2 t + (w & 1) + 8 (w >> 1), duplicated into both halves.
struct GemmDecodePrologueArgs { const half* suh[GD_MAX_SEG]; uint32_t* a_frag[GD_MAX_SEG]; float* rowsum[GD_MAX_SEG]; };

__global__ void __launch_bounds__(256) gemm_decode_prologue_kernel(const half* __restrict__ A, const GemmDecodePrologueArgs args,
                                                                   int m, int k)
{
    __shared__ float sh[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x, seg = blockIdx.y;
    const half* __restrict__ suh = args.suh[seg];
    uint32_t* __restrict__ out = args.a_frag[seg];
    const int set = b >> 3, g = b & 7;
    const int q = lane & 3;                                  // position of the lane's 4 values inside a 16-k tile row
    const int t0 = 2 * (q & 1), w0 = 2 * (q >> 1);
    float part = 0.0f;
    for (int blk = warp; blk < k / 128; blk += 8) {
        uint32_t h0 = 0, h1 = 0, h2 = 0, h3 = 0;
        if (b < m) {
            uint2 raw = reinterpret_cast<const uint2*>(A + (size_t)b * k + blk * 128)[lane];
            half2 x = *reinterpret_cast<half2*>(&raw.x), y = *reinterpret_cast<half2*>(&raw.y);
            if (suh) {
                uint2 sr = reinterpret_cast<const uint2*>(suh + blk * 128)[lane];
                x = __hmul2(x, *reinterpret_cast<half2*>(&sr.x));
                y = __hmul2(y, *reinterpret_cast<half2*>(&sr.y));
            }
            float v0 = __low2float(x), v1 = __high2float(x), v2 = __low2float(y), v3 = __high2float(y);
            if (suh) {
                float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
                v0 = s0 + s1; v1 = d0 + d1; v2 = s0 - s1; v3 = d0 - d1;
                #pragma unroll
                for (int i = 1; i < 32; i <<= 1) {
                    float p0 = __shfl_xor_sync(0xffffffffu, v0, i), p1 = __shfl_xor_sync(0xffffffffu, v1, i);
                    float p2 = __shfl_xor_sync(0xffffffffu, v2, i), p3 = __shfl_xor_sync(0xffffffffu, v3, i);
                    const bool up = lane & i;
                    v0 = (up ? -v0 : v0) + p0; v1 = (up ? -v1 : v1) + p1;
                    v2 = (up ? -v2 : v2) + p2; v3 = (up ? -v3 : v3) + p3;
                }
                v0 *= GD_R128; v1 *= GD_R128; v2 *= GD_R128; v3 *= GD_R128;
            }
            h0 = __half_as_ushort(__float2half_rn(v0)); h1 = __half_as_ushort(__float2half_rn(v1));
            h2 = __half_as_ushort(__float2half_rn(v2)); h3 = __half_as_ushort(__float2half_rn(v3));
            part += __half2float(__ushort_as_half((unsigned short)h0)) + __half2float(__ushort_as_half((unsigned short)h1)) +
                    __half2float(__ushort_as_half((unsigned short)h2)) + __half2float(__ushort_as_half((unsigned short)h3));
        }
        // the lane's values sit at k = 128 blk + 4 lane + j: kslot = 2 blk + lane / 16, r = (lane / 4) % 4, and inside the
        // tile row at 4 q + j
        const size_t base = ((((size_t)set * (k / 64) + 2 * blk + (lane >> 4)) * 4 + ((lane >> 2) & 3)) * 32 + 4 * g) * 4;
        *reinterpret_cast<uint2*>(out + base + (size_t)t0 * 4 + w0) = make_uint2(h0 * 0x10001u, h1 * 0x10001u);
        *reinterpret_cast<uint2*>(out + base + (size_t)(t0 + 1) * 4 + w0) = make_uint2(h2 * 0x10001u, h3 * 0x10001u);
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) sh[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int w = 0; w < 8; ++w) s += sh[w];
        args.rowsum[seg][b] = s;
    }
}

// grid = CTAs of the stream-K split (at most one per SM), 512 threads, GdSmem<K, MT>::BYTES of dynamic shared memory.
// rmap*: the trellis of each tensor as a matrix of 64-bit words [k/16][n/16 * 4K], box 4 rows x 4 tiles.
template <int K, int CB, int MT>
__global__ void __launch_bounds__(GD_THREADS, 1) gemm_decode_kernel(const __grid_constant__ CUtensorMap rmap0,
                                                                   const __grid_constant__ CUtensorMap rmap1,
                                                                   const __grid_constant__ CUtensorMap rmap2,
                                                                   const GemmDecodeParams p)
{
    using SM = GdSmem<K, MT>;
    extern __shared__ uint8_t gd_smem_unaligned[];
    uint8_t* smem = gd_smem_unaligned + ((128u - (smem_u32(gd_smem_unaligned) & 127u)) & 127u);
    float* red = reinterpret_cast<float*>(smem + SM::OFF_RED);
    float* sc = reinterpret_cast<float*>(smem + SM::OFF_SC);
    __shared__ int s_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ks = warp & (GD_KSL - 1), ch = warp >> 3;
    const int KC = (p.k + GD_UNIT_K - 1) / GD_UNIT_K;                  // k chunks per column block
    const long long total = (long long)p.blk_end[GD_MAX_SEG - 1] * KC;
    const long long G = gridDim.x;
    const long long u0 = total * blockIdx.x / G, u1 = total * (blockIdx.x + 1) / G;
    const int nunits = (int)(u1 - u0);
    const int mrows = p.m;

    uint8_t* ring = smem + SM::OFF_RING + warp * SM::DEPTH * SM::SLOT_BYTES;
    const uint32_t ring_u32 = smem_u32(ring);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR) + warp * SM::DEPTH;
    const uint32_t bars_u32 = smem_u32(bars);
    if (lane == 0) {
        #pragma unroll
        for (int s = 0; s < SM::DEPTH; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncwarp();

    // Units are walked with two cursors (the one being multiplied and the one being requested, DEPTH - 1 slots ahead),
    // each stepped one unit at a time: (column block, k chunk) without a division in the loop.
    const int nbg0 = (int)(u0 / KC), kc0 = (int)(u0 - (long long)nbg0 * KC);
    auto seg_of = [&](int nbg) -> int { return (nbg >= p.blk_end[0]) + (nbg >= p.blk_end[1]); };
    auto col0_of = [&](int nbg, int seg) -> int { return (nbg - (seg == 0 ? 0 : (seg == 1 ? p.blk_end[0] : p.blk_end[1]))) * 128; };
    // slot j = 2 i + h of this warp: tile rows [64 kc + 8 ks + 4 h, +4) of unit i; a unit whose chunk ends before this
    // warp's k-slice has no slots for it
    auto slot_active = [&](int kc) -> bool { return (kc * GD_UNIT_K + ks * 128) < p.k; };
    const int nslots = 2 * nunits;
    int issued = 0, consumed = 0;
    int j_iss = 0, nbg_iss = nbg0, kc_iss = kc0;
    bool failed = false;
    auto issue_next = [&]() {
        if (j_iss >= nslots) return;
        if (slot_active(kc_iss) && !failed) {
            if (lane == 0) {
                const int seg = seg_of(nbg_iss);
                const int s = issued % SM::DEPTH;
                const CUtensorMap* rmap = seg == 0 ? &rmap0 : (seg == 1 ? &rmap1 : &rmap2);
                const uint32_t bar = bars_u32 + 8u * s;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)SM::SLOT_BYTES) : "memory");
                gd_tma_load_2d(ring_u32 + s * SM::SLOT_BYTES, rmap, ((col0_of(nbg_iss, seg) >> 4) + ch * GD_SLOT_TILES) * 4 * K,
                               kc_iss * (GD_UNIT_K / 16) + ks * 8 + (j_iss & 1) * GD_SLOT_ROWS, bar);
            }
            ++issued;
        }
        if (j_iss & 1) { if (++kc_iss == KC) { kc_iss = 0; ++nbg_iss; } }
        ++j_iss;
    };
    #pragma unroll 1
    for (int j = 0; j < SM::DEPTH - 1; ++j) issue_next();

    float acc[MT][GD_SLOT_TILES][4];
    #pragma unroll
    for (int s = 0; s < MT; ++s)
        #pragma unroll
        for (int c = 0; c < GD_SLOT_TILES; ++c)
            #pragma unroll
            for (int e = 0; e < 4; ++e) acc[s][c][e] = 0.0f;

    const int lane_prev = (lane + 31) & 31;
    int nbg = nbg0, kc = kc0 - 1;
    #pragma unroll 1
    for (int i = 0; i < nunits; ++i) {
        if (++kc == KC) { kc = 0; ++nbg; }
        const int seg = seg_of(nbg);
        const int n0 = col0_of(nbg, seg);
        const bool active = slot_active(kc);
        const uint4* afr = (seg == 0 ? p.a_frag[0] : (seg == 1 ? p.a_frag[1] : p.a_frag[2]));
        #pragma unroll 1
        for (int h = 0; h < 2; ++h) {
            // the slot freed by the previous iteration is refilled first (all lanes have consumed its words)
            __syncwarp();
            issue_next();
            if (!active || failed) continue;
            // this slot's activations: batch rows 8 set + g, k = 64 kslot + 16 r + {2t, 2t+1, 2t+8, 2t+9}
            const int kslot = kc * (GD_UNIT_K / 64) + ks * 2 + h;
            uint4 af[MT][GD_SLOT_ROWS];
            #pragma unroll
            for (int s = 0; s < MT; ++s)
                #pragma unroll
                for (int r = 0; r < GD_SLOT_ROWS; ++r)
                    af[s][r] = __ldg(afr + (((size_t)s * (p.k / 64) + kslot) * 4 + r) * 32 + lane);
            const int s_idx = consumed % SM::DEPTH;
            const bool ok = mbar_wait_sleep_warp(&bars[s_idx], (consumed / SM::DEPTH) & 1);
            ++consumed;
            if (!ok) { failed = true; continue; }
            const uint32_t* sb = reinterpret_cast<const uint32_t*>(ring + s_idx * SM::SLOT_BYTES);
            #pragma unroll
            for (int r = 0; r < GD_SLOT_ROWS; ++r) {
                #pragma unroll
                for (int c = 0; c < GD_SLOT_TILES; ++c) {
                    uint32_t st[8], y[8];
                    if constexpr (K == 4) lane_states4(sb + (r * GD_SLOT_TILES + c) * 8 * K, lane, lane_prev, st);
                    else lane_states<K>(sb + (r * GD_SLOT_TILES + c) * 8 * K, lane, st);
                    #pragma unroll
                    for (int q = 0; q < 8; ++q) y[q] = decode_raw<CB>(st[q]);
                    #pragma unroll
                    for (int s = 0; s < MT; ++s) {
                        gd_mma(acc[s][c], y[0], y[4], y[1], y[5], af[s][r].x, af[s][r].y);
                        gd_mma(acc[s][c], y[2], y[6], y[3], y[7], af[s][r].z, af[s][r].w);
                    }
                }
            }
        }

        const bool block_done = kc == KC - 1 || i == nunits - 1;
        if (!block_done) continue;

        // ---- the CTA leaves column block nbg: per-slice tiles -> shared memory, then added in slice order
        #pragma unroll
        for (int s = 0; s < MT; ++s)
            #pragma unroll
            for (int c = 0; c < GD_SLOT_TILES; ++c) {
                float* dst = red + ((size_t)ks * SM::ROWS + s * 8 + 2 * t) * GD_RSTRIDE + ch * 64 + c * 16 + g;
                dst[0] = acc[s][c][0]; dst[GD_RSTRIDE] = acc[s][c][1];
                dst[8] = acc[s][c][2]; dst[GD_RSTRIDE + 8] = acc[s][c][3];
                acc[s][c][0] = acc[s][c][1] = acc[s][c][2] = acc[s][c][3] = 0.0f;
            }
        if (__syncthreads_or(failed)) { failed = true; break; }
        for (int e = tid; e < SM::ROWS * 32; e += GD_THREADS) {
            const int row = e >> 5, c4 = e & 31;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            #pragma unroll
            for (int s = 0; s < GD_KSL; ++s) {
                const float4 v = *reinterpret_cast<const float4*>(red + ((size_t)s * SM::ROWS + row) * GD_RSTRIDE + c4 * 4);
                a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
            }
            *reinterpret_cast<float4*>(sc + row * GD_RSTRIDE + c4 * 4) = a;
        }
        __syncthreads();

        // CTAs that own a part of this block: those whose unit range meets [nbg * KC, (nbg + 1) * KC)
        const long long first = (long long)nbg * KC;
        auto owner = [&](long long u) -> int { return (int)(((u + 1) * G + total - 1) / total - 1); };
        const int c_first = owner(first), c_last = owner(first + KC - 1);
        const int ncontrib = c_last - c_first + 1;
        bool finish = true;
        if (ncontrib > 1) {
            // a CTA shares at most its first and its last column block: slot 0 and slot 1 of its pair
            auto slot_of = [&](int cta) -> float* {
                const long long fb = (total * cta / G) / KC;
                return p.partial + ((size_t)cta * 2 + (fb == nbg ? 0 : 1)) * mrows * 128;
            };
            float* mine = slot_of(blockIdx.x);
            for (int e = tid; e < mrows * 32; e += GD_THREADS) {
                const int row = e >> 5, c4 = e & 31;
                *reinterpret_cast<float4*>(mine + row * 128 + c4 * 4) = *reinterpret_cast<const float4*>(sc + row * GD_RSTRIDE + c4 * 4);
            }
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const int old = atomicAdd(&p.counters[nbg], 1);
                s_flag = (old == ncontrib - 1);
                if (s_flag) p.counters[nbg] = 0;
            }
            __syncthreads();
            finish = s_flag != 0;
            if (finish) {
                __threadfence();
                for (int e = tid; e < mrows * 32; e += GD_THREADS) {
                    const int row = e >> 5, c4 = e & 31;
                    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int s = c_first; s <= c_last; ++s) {           // owner order: independent of arrival order
                        const float4 v = __ldcg(reinterpret_cast<const float4*>(slot_of(s) + row * 128 + c4 * 4));
                        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                    }
                    *reinterpret_cast<float4*>(sc + row * GD_RSTRIDE + c4 * 4) = a;
                }
                __syncthreads();
            }
        }
        if (finish) {
            // output transform: one warp per row, lane holds 4 consecutive columns
            const half* svh = seg == 0 ? p.svh[0] : (seg == 1 ? p.svh[1] : p.svh[2]);
            void* Cout = seg == 0 ? p.C[0] : (seg == 1 ? p.C[1] : p.C[2]);
            const int n = seg == 0 ? p.n[0] : (seg == 1 ? p.n[1] : p.n[2]);
            for (int row = warp; row < mrows; row += GD_WARPS) {
                float4 v = *reinterpret_cast<const float4*>(sc + row * GD_RSTRIDE + lane * 4);
                if constexpr (CB == 2) {
                    const float* rsum = seg == 0 ? p.rowsum[0] : (seg == 1 ? p.rowsum[1] : p.rowsum[2]);
                    const float rs = rsum[row] * GD_MUL1_DELTA;
                    v.x = fmaf(v.x, GD_MUL1_KINV, rs); v.y = fmaf(v.y, GD_MUL1_KINV, rs);
                    v.z = fmaf(v.z, GD_MUL1_KINV, rs); v.w = fmaf(v.w, GD_MUL1_KINV, rs);
                }
                const size_t off = (size_t)row * n + n0 + lane * 4;
                if (svh) {
                    float s0 = v.x + v.y, d0 = v.x - v.y, s1 = v.z + v.w, d1 = v.z - v.w;
                    v.x = s0 + s1; v.y = d0 + d1; v.z = s0 - s1; v.w = d0 - d1;
                    #pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        float p0 = __shfl_xor_sync(0xffffffffu, v.x, o), p1 = __shfl_xor_sync(0xffffffffu, v.y, o);
                        float p2 = __shfl_xor_sync(0xffffffffu, v.z, o), p3 = __shfl_xor_sync(0xffffffffu, v.w, o);
                        const bool up = lane & o;
                        v.x = (up ? -v.x : v.x) + p0; v.y = (up ? -v.y : v.y) + p1;
                        v.z = (up ? -v.z : v.z) + p2; v.w = (up ? -v.w : v.w) + p3;
                    }
                    v.x *= GD_R128; v.y *= GD_R128; v.z *= GD_R128; v.w *= GD_R128;
                    uint2 sr = *reinterpret_cast<const uint2*>(svh + n0 + lane * 4);
                    half2 sa2 = *reinterpret_cast<half2*>(&sr.x), sb2 = *reinterpret_cast<half2*>(&sr.y);
                    if (p.c_fp32) {
                        v.x *= __low2float(sa2); v.y *= __high2float(sa2); v.z *= __low2float(sb2); v.w *= __high2float(sb2);
                        *reinterpret_cast<float4*>((float*)Cout + off) = v;
                    } else {
                        half2 a = __hmul2(__floats2half2_rn(v.x, v.y), sa2), b = __hmul2(__floats2half2_rn(v.z, v.w), sb2);
                        uint2 o2; o2.x = *reinterpret_cast<uint32_t*>(&a); o2.y = *reinterpret_cast<uint32_t*>(&b);
                        *reinterpret_cast<uint2*>((half*)Cout + off) = o2;
                    }
                } else {
                    if (p.c_fp32) *reinterpret_cast<float4*>((float*)Cout + off) = v;
                    else {
                        half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
                        uint2 o2; o2.x = *reinterpret_cast<uint32_t*>(&a); o2.y = *reinterpret_cast<uint32_t*>(&b);
                        *reinterpret_cast<uint2*>((half*)Cout + off) = o2;
                    }
                }
            }
        }
        __syncthreads();      // the reduction tiles are reused by the next column block
    }
    // A wait that ran out: no new copies are issued after it, but boxes already requested may still land; give them the
    // same bounded time before the CTA's shared memory is released.
    if (failed) {
        while (consumed < issued) {
            mbar_wait_sleep_warp(&bars[consumed % SM::DEPTH], (consumed / SM::DEPTH) & 1, 1u << 12);
            ++consumed;
        }
        if (tid == 0) atomicExch(p.status, 1);
    }
}

}  // namespace exl3
