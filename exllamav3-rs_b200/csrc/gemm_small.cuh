// EXL3 GEMM for small and medium M (the HBM-bound decode path): trellis tiles staged to shared memory by the bulk-copy
// engine, decoded in registers and multiplied with mma.sync m16n8k16.
//
// Function computed (reference: kernels/quant/exl3_gemm_kernel.cuh:14-50, exl3_gemm_inner.cuh:456-480):
//   C = H128( fp16(H128(A o suh)/sqrt128) . W ) / sqrt128 o svh
//
// Decode trick.  For codebooks 0/1 a weight is the fp16 sum of the two halves of one 32-bit register y; for codebook 2
// it is k_inv*(h - 1534) + delta with h = fp16 in the low half of y and -1534 in its high half.  Instead of adding the
// halves on the CUDA cores, y is fed to the tensor core as two consecutive k-entries of the B fragment and the
// activation is duplicated in the two matching k-entries of the A fragment, so the MMA forms a*(lo+hi) in fp32.
// One 16x16 weight tile then costs four m16n8k16 MMAs (16 real k = 32 MMA k) and no repacking instructions.
#pragma once
#include "common.cuh"
#include "exl3_decode.cuh"
#include "async_copy.cuh"

namespace exl3 {

constexpr int GS_KS = 8;            // weight-tile rows (16 k each) per pipeline stage: one 128-wide Hadamard block
constexpr int GS_STAGES = 4;
constexpr int GS_ASTRIDE = GS_KS * 16 + 8;   // words per activation row in shared memory (+8: conflict-free LDS.64)
constexpr float GS_R128 = 0.088388347648f;
// codebook 2: weight = K_INV*(h-1534) + DELTA, DELTA = k_bias + 1534*k_inv with the fp16 constants of the reference
constexpr float GS_MUL1_KINV = 0.00676727294921875f;
constexpr float GS_MUL1_DELTA = -10.3828125f + 1534.0f * 0.00676727294921875f;

struct GemmSmallParams {
    const uint32_t* a_dup;     // [m][k] words, each = (a, a) as two fp16: the Hadamard-transformed activations
    const float* rowsum;       // [m] sum over k of the transformed activations (codebook 2 only)
    const uint32_t* trellis;   // [k/16][n/16][8K] words
    float* partial;            // [grid][2][m][128] fp32: a CTA's partial sums of its first and of its last column block, when
                               // those are shared with a neighbouring CTA (a CTA's range of units is contiguous, so no other
                               // block of it can be)
    int* counters;             // [n/128] arrival counters, zero on entry and on exit
    void* C;                   // [m][n] fp16 or fp32
    const half* svh;           // [n] or NULL
    int* status;
    int m, k, n, c_fp32;
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int K, int MT>
struct GemmSmallSmem {
    static constexpr int B_STAGE_WORDS = GS_KS * 8 * 8 * K;            // GS_KS tile rows x 8 tiles x 8K words
    static constexpr int STAGE_WORDS = B_STAGE_WORDS;                   // only the codes are staged; activations come via L1
    static constexpr int C_WORDS = MT * 16 * 132;                        // epilogue tile [rows][128+4] fp32 (own region)
    // as many stages (up to GS_STAGES) as fit in the 227 KB a CTA may use
    static constexpr int STAGES = ((GS_STAGES * STAGE_WORDS + C_WORDS) * 4 + 256 <= 227 * 1024) ? GS_STAGES
                                : (((GS_STAGES - 1) * STAGE_WORDS + C_WORDS) * 4 + 256 <= 227 * 1024) ? GS_STAGES - 1 : 2;
    static constexpr int PIPE_WORDS = STAGES * STAGE_WORDS;
    static constexpr int BYTES = (PIPE_WORDS + C_WORDS) * 4 + STAGES * 8 + 16;
};

// Persistent stream-K kernel.  The work is the list of (column block, 128-k stage) units in column-block-major order;
// CTA c of G owns units [total*c/G, total*(c+1)/G).  Its bulk-copy pipeline runs through that range without draining at
// column-block boundaries.  When a CTA leaves a column block it either finishes it (sole owner) or publishes its
// partial sums; the last of the block's owners to arrive adds the partials in owner order (deterministic) and applies
// the output transform.  256 threads = 8 warps, warp w owns the 16 columns of tile w of the current 128-column block.
template <int K, int CB, int MT>
__global__ void __launch_bounds__(256) gemm_small_kernel(const GemmSmallParams p)
{
    using SM = GemmSmallSmem<K, MT>;
    extern __shared__ __align__(128) uint32_t smem[];
    float* sc = reinterpret_cast<float*>(smem + SM::PIPE_WORDS);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::PIPE_WORDS + SM::C_WORDS);
    __shared__ int s_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tiles_n = p.n >> 4;
    const int NST = p.k >> 7;                                 // 128-k stages per column block
    const long long total = (long long)(p.n >> 7) * NST;
    const long long G = gridDim.x;
    const long long u0 = total * blockIdx.x / G, u1 = total * (blockIdx.x + 1) / G;
    const int nunits = (int)(u1 - u0);
    const int mrows = p.m < MT * 16 ? p.m : MT * 16;

    if (tid == 0) {
        #pragma unroll
        for (int s = 0; s < SM::STAGES; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    // producer: one thread issues all bulk copies of a unit
    auto issue = [&](int i) {
        const long long u = u0 + i;
        const int nb = (int)(u / NST), st = (int)(u - (long long)nb * NST);
        const int slot = i % SM::STAGES;
        uint32_t* sb = smem + slot * SM::STAGE_WORDS;
        const int kt0 = st * GS_KS;
        mbar_expect_tx(&bars[slot], GS_KS * 8 * 8 * K * 4);
        #pragma unroll
        for (int r = 0; r < GS_KS; ++r)
            bulk_g2s(sb + r * 64 * K, p.trellis + ((size_t)(kt0 + r) * tiles_n + nb * 8) * 8 * K, 64 * K * 4, &bars[slot]);
    };
    // CTA that owns unit u
    auto owner = [&](long long u) -> int { return (int)(((u + 1) * G + total - 1) / total - 1); };

    if (tid == 0) {
        for (int s = 0; s < SM::STAGES - 1 && s < nunits; ++s) issue(s);
    }

    float acc[MT][2][4];
    #pragma unroll
    for (int i = 0; i < MT; ++i)
        #pragma unroll
        for (int j = 0; j < 2; ++j)
            #pragma unroll
            for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.0f;

    bool failed = false;
    for (int i = 0; i < nunits; ++i) {
        const int slot = i % SM::STAGES;
        if (tid == 0 && i + SM::STAGES - 1 < nunits) issue(i + SM::STAGES - 1);
        const bool ok = mbar_wait_sleep(&bars[slot], (i / SM::STAGES) & 1);
        if (ok) {
            const uint32_t* sb = smem + slot * SM::STAGE_WORDS + warp * 8 * K;
            // The duplicated activations are read straight from global memory: all eight warps of all resident CTAs
            // read the same few KB per stage, so these loads hit L1; keeping them out of shared memory lets several more
            // CTAs share an SM.  Rows past m repeat the last row (their products are never stored).
            const int kst = (int)((u0 + i) % NST);
            const uint32_t* abase = p.a_dup + (size_t)kst * 128 + 2 * t;
            #pragma unroll 2
            for (int r = 0; r < GS_KS; ++r) {
                uint32_t st[8], y[8];
                lane_states<K>(sb + r * 64 * K, lane, st);
                #pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = decode_raw<CB>(st[j]);
                #pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int row0 = min(mt * 16 + g, mrows - 1), row1 = min(mt * 16 + g + 8, mrows - 1);
                    const uint32_t* ar0 = abase + (size_t)row0 * p.k + r * 16;
                    const uint32_t* ar1 = abase + (size_t)row1 * p.k + r * 16;
                    uint2 lo0 = __ldg(reinterpret_cast<const uint2*>(ar0));         // rows g   : k 2t, 2t+1
                    uint2 hi0 = __ldg(reinterpret_cast<const uint2*>(ar0 + 8));     // k 2t+8, 2t+9
                    uint2 lo1 = make_uint2(0u, 0u), hi1 = make_uint2(0u, 0u);       // rows g+8 (absent when m <= 8)
                    if (mt * 16 + 8 < mrows) {
                        lo1 = __ldg(reinterpret_cast<const uint2*>(ar1));
                        hi1 = __ldg(reinterpret_cast<const uint2*>(ar1 + 8));
                    }
                    mma16816(acc[mt][0], lo0.x, lo1.x, lo0.y, lo1.y, y[0], y[1]);
                    mma16816(acc[mt][0], hi0.x, hi1.x, hi0.y, hi1.y, y[2], y[3]);
                    mma16816(acc[mt][1], lo0.x, lo1.x, lo0.y, lo1.y, y[4], y[5]);
                    mma16816(acc[mt][1], hi0.x, hi1.x, hi0.y, hi1.y, y[6], y[7]);
                }
            }
        }
        // all warps are done with this slot (it is refilled at the top of the next iteration); a wait that ran out
        // anywhere in the CTA ends the loop for everyone
        if (__syncthreads_or(!ok)) { failed = true; break; }

        const long long u = u0 + i;
        const int nb = (int)(u / NST);
        const bool block_done = (u + 1) % NST == 0 || i == nunits - 1;
        if (!block_done) continue;

        // ---- leave column block nb: accumulators -> shared tile [rows][132] fp32
        #pragma unroll
        for (int mt = 0; mt < MT; ++mt)
            #pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int col = warp * 16 + j * 8 + 2 * t;
                *reinterpret_cast<float2*>(sc + (mt * 16 + g) * 132 + col) = make_float2(acc[mt][j][0], acc[mt][j][1]);
                *reinterpret_cast<float2*>(sc + (mt * 16 + g + 8) * 132 + col) = make_float2(acc[mt][j][2], acc[mt][j][3]);
                acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.0f;
            }
        __syncthreads();

        const long long first = (long long)nb * NST;
        const int c_first = owner(first), c_last = owner(first + NST - 1);
        const int ncontrib = c_last - c_first + 1;
        bool finish = true;
        if (ncontrib > 1) {
            // slot 0 of a CTA's pair holds its first column block, slot 1 its last
            auto slot_of = [&](int cta) -> float* {
                const long long fb = (total * cta / G) / NST;
                return p.partial + ((size_t)cta * 2 + (fb == nb ? 0 : 1)) * p.m * 128;
            };
            float* mine = slot_of(blockIdx.x);
            for (int e = tid; e < mrows * 32; e += 256) {
                const int row = e >> 5, c4 = e & 31;
                *reinterpret_cast<float4*>(mine + row * 128 + c4 * 4) = *reinterpret_cast<const float4*>(sc + row * 132 + c4 * 4);
            }
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const int old = atomicAdd(&p.counters[nb], 1);
                s_flag = (old == ncontrib - 1);
                if (s_flag) p.counters[nb] = 0;
            }
            __syncthreads();
            finish = s_flag != 0;
            if (finish) {
                __threadfence();
                for (int e = tid; e < mrows * 32; e += 256) {
                    const int row = e >> 5, c4 = e & 31;
                    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int s = c_first; s <= c_last; ++s) {   // owner order: independent of arrival order
                        float4 v = __ldcg(reinterpret_cast<const float4*>(slot_of(s) + (size_t)row * 128 + c4 * 4));
                        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                    }
                    *reinterpret_cast<float4*>(sc + row * 132 + c4 * 4) = a;
                }
                __syncthreads();
            }
        }
        if (finish) {
            // output transform: one warp per row, lane holds 4 consecutive columns
            for (int row = warp; row < mrows; row += 8) {
                float4 v = *reinterpret_cast<const float4*>(sc + row * 132 + lane * 4);
                if constexpr (CB == 2) {
                    const float rs = p.rowsum[row] * GS_MUL1_DELTA;
                    v.x = fmaf(v.x, GS_MUL1_KINV, rs); v.y = fmaf(v.y, GS_MUL1_KINV, rs);
                    v.z = fmaf(v.z, GS_MUL1_KINV, rs); v.w = fmaf(v.w, GS_MUL1_KINV, rs);
                }
                const size_t off = (size_t)row * p.n + nb * 128 + lane * 4;
                if (p.svh) {
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
                    v.x *= GS_R128; v.y *= GS_R128; v.z *= GS_R128; v.w *= GS_R128;
                    uint2 sr = *reinterpret_cast<const uint2*>(p.svh + nb * 128 + lane * 4);
                    half2 sa2 = *reinterpret_cast<half2*>(&sr.x), sb2 = *reinterpret_cast<half2*>(&sr.y);
                    if (p.c_fp32) {
                        v.x *= __low2float(sa2); v.y *= __high2float(sa2); v.z *= __low2float(sb2); v.w *= __high2float(sb2);
                        *reinterpret_cast<float4*>((float*)p.C + off) = v;
                    } else {
                        half2 a = __hmul2(__floats2half2_rn(v.x, v.y), sa2), b = __hmul2(__floats2half2_rn(v.z, v.w), sb2);
                        uint2 o2; o2.x = *reinterpret_cast<uint32_t*>(&a); o2.y = *reinterpret_cast<uint32_t*>(&b);
                        *reinterpret_cast<uint2*>((half*)p.C + off) = o2;
                    }
                } else {
                    if (p.c_fp32) *reinterpret_cast<float4*>((float*)p.C + off) = v;
                    else {
                        half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
                        uint2 o2; o2.x = *reinterpret_cast<uint32_t*>(&a); o2.y = *reinterpret_cast<uint32_t*>(&b);
                        *reinterpret_cast<uint2*>((half*)p.C + off) = o2;
                    }
                }
            }
        }
        __syncthreads();      // the shared tile is reused by the next column block
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
}

}  // namespace exl3
