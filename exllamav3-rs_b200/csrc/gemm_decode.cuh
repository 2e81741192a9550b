// EXL3 GEMM for the decode regime (1..16 rows): the weight stream sets the time, so the kernel is built around the cost
// of turning trellis codes into multiplier operands, one warp-instruction at a time.
//
// Function computed (reference: kernels/quant/exl3_gemm_kernel.cuh:14-50, exl3_gemm_inner.cuh:456-480; the reference's
// own small-m kernel is kernels/quant/exl3_gemv_kernel.cuh:138-402):
//   C = H128( fp16(H128(A o suh)/sqrt128) . W ) / sqrt128 o svh
//
// Layout of the work.  A CTA has 16 warps = 8 k-slices x 2 column halves.  Its unit of work is (128-column block,
// 512-k chunk); inside a unit warp (ks, ch) owns the 4 x 4 weight tiles of k-slice ks (64 k) and column half ch (64
// columns).  Units are ordered column-block-major and dealt to the CTAs as contiguous ranges: whole column blocks per CTA
// when that costs at most one unit more than an even split (no traffic between CTAs), else an even split (stream-K).  A
// warp walks down k with its accumulators in registers and only meets the other warps when the CTA leaves a column
// block: the 8 k-slices are added in a fixed order through shared memory by the warp that arrives last, a block shared
// with a neighbouring CTA goes through a partial-sum slot in global memory that the last CTA to arrive adds up in owner
// order (deterministic), and the finisher applies the output Hadamard and svh.
//
// The two warps of a k-slice share a ring of slots; one warp of a fifth warpgroup is the producer for all eight rings
// (setmaxnreg moves that group's registers to the decoders): lane l of it keeps k-slice l's ring full (one TMA box of 4
// tile rows x 8 tiles of codes per slot and, for up to 8 rows, one bulk copy of the slot's activations in MMA fragment
// order, written by gemm_decode_prologue_kernel), signalled through one "full" and one "empty" mbarrier per slot.  A
// decoder's main loop is: wait, decode and multiply its 16 tiles, release - no CTA-wide barrier and no address arithmetic.
//
// Multiplier mapping.  The 16x16 tile is stored in mma.m16n8k16 B-fragment order; read as the A operand of the
// transposed product (weights^T . activations^T) the same registers are one A fragment, so a tile costs two MMAs for
// up to 8 rows (N = 8 is the batch) instead of four.  For codebooks 0/1 a weight is the fp16 sum of the two halves of
// y = lop3(x * C); y goes to the tensor core as two consecutive k entries and the activation is duplicated in the B
// fragment, so the halves are added by the MMA in fp32; codebook 2 uses (1024 + s, -1534) the same way and is scaled
// in the epilogue.  Measured per tile at 4 bpw (MCG codebook, 1 row): 38.6 warp instructions, of which 18.9 on the ALU pipe
// (shifts, permutes, lop3), 4.9 integer multiplies, 2.3 shared loads and 2 MMAs.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "exl3_decode.cuh"
#include "async_copy.cuh"

namespace exl3 {

#ifdef GD_TRACE
// timeline of one launch (debug builds only): per CTA and warp [start, first data, loop end, end] in nanoseconds
__device__ unsigned long long g_gd_trace[148 * 16 * 8];
__device__ __forceinline__ unsigned long long gd_now() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define GD_STAMP(slot) do { if (lane == 0 && warp < 16 && blockIdx.x < 148) g_gd_trace[(blockIdx.x * 16 + warp) * 8 + (slot)] = gd_now(); } while (0)
#define GD_ACC(slot, v) do { if (lane == 0 && warp < 16 && blockIdx.x < 148) g_gd_trace[(blockIdx.x * 16 + warp) * 8 + (slot)] += (v); } while (0)
#define GD_T0() const unsigned long long gd_t0_ = gd_now()
#define GD_DT() (gd_now() - gd_t0_)
#else
#define GD_STAMP(slot) do { } while (0)
#define GD_ACC(slot, v) do { } while (0)
#define GD_T0() do { } while (0)
#define GD_DT() 0
#endif

constexpr int GD_WARPS = 16;                 // decoder warps
constexpr int GD_THREADS = (GD_WARPS + 4) * 32;            // + the producer's warpgroup (one of its four warps works)
constexpr int GD_KSL = 8;                    // k-slices of a CTA unit
constexpr int GD_SLOT_ROWS = 4;              // tile rows per TMA box = one k-slice (64 k)
constexpr int GD_UNIT_K = GD_KSL * GD_SLOT_ROWS * 16;      // k extent of a unit: 512
constexpr int GD_SLOT_TILES = 4;             // tiles per row of a box (one column half)
constexpr int GD_MAX_SEG = 3;
constexpr int GD_RSTRIDE = 132;              // floats per row of the reduction tiles
constexpr float GD_R128 = 0.088388347648f;
constexpr float GD_MUL1_KINV = 0.00676727294921875f;
constexpr float GD_MUL1_DELTA = -10.3828125f + 1534.0f * 0.00676727294921875f;

template <int K, int MT> struct GdSmem {
    static constexpr int ROWS = 8 * MT;                                            // batch rows held by the MMAs
    static constexpr int CODE_BYTES = GD_SLOT_ROWS * 2 * GD_SLOT_TILES * 32 * K;   // 4 tile rows x 8 tiles: 1024 K
    // up to 8 rows: the slot also carries its activations (4 tile rows x 32 lanes x 16 bytes); with two row sets there is
    // no room for that and the decoders load them from global memory
    static constexpr int ACT_BYTES = MT == 1 ? GD_SLOT_ROWS * 32 * 16 : 0;
    static constexpr int SLOT_BYTES = CODE_BYTES + ACT_BYTES;
    static constexpr int RED_BYTES = GD_KSL * ROWS * GD_RSTRIDE * 4;               // per-slice partial tiles
    static constexpr int ROOM = 227 * 1024 - RED_BYTES - 2048;                     // barriers, alignment slack, static shared memory
    static constexpr int DEPTH_FIT = ROOM / (GD_KSL * SLOT_BYTES);
    static constexpr int DEPTH = DEPTH_FIT > 8 ? 8 : DEPTH_FIT;
    static_assert(DEPTH >= 2, "a ring needs two slots");
    static constexpr int OFF_RING = 0;
    static constexpr int OFF_RED = OFF_RING + GD_KSL * DEPTH * SLOT_BYTES;
    static constexpr int OFF_BAR = OFF_RED + RED_BYTES;                            // full[8][DEPTH], empty[8][DEPTH]
    static constexpr int BYTES = OFF_BAR + 2 * GD_KSL * DEPTH * 8 + 128;           // + slack to align the base to 128 bytes
};

struct GemmDecodeParams {
    const uint4* a_frag[GD_MAX_SEG];   // [MT][k/64][4][32] uint4: activations in B-fragment order, duplicated halves
    const float* rowsum[GD_MAX_SEG];   // [rowsum_parts][8*MT] partial sums over k of the transformed activations (codebook 2 only)
    int rowsum_parts;                  // k ranges the input transform was split into (their sums are added in order)
    void* C[GD_MAX_SEG];               // [m][n] fp16 or fp32
    const half* svh[GD_MAX_SEG];       // [n] or NULL
    int n[GD_MAX_SEG];
    int blk_end[GD_MAX_SEG];           // running count of 128-column blocks
    float* partial;                    // [grid][2][m][128] fp32: a CTA's first and last column block when shared
    int* counters;                     // [column blocks] arrival counters, zero on entry and on exit
    int* status;
    int m, k, c_fp32;
    int aligned;                       // 1: every CTA owns whole column blocks (no block is shared), 0: stream-K over units
    // Table mode (the kernel's MULTI form, exl3_mgemm): `slots` products over tensors picked from device-resident tables.
    // Slot j uses tensor indices[j] (j itself when indices is NULL; a negative entry leaves the slot untouched), reads
    // the activations a_frag[0] + j * slot stride and writes C[0] + j * m * n, scaled by weights[j] when given.  All
    // tensors have n[0] columns; the column blocks of slot j are blocks [j * n/128, (j + 1) * n/128).
    const uint32_t* const* trellis_tab;
    const half* const* svh_tab;
    const int64_t* indices;
    const half* weights;
    int slots;
    long long c_slot_stride;           // elements between the outputs of consecutive slots
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

// One slot = 4 tile rows x 4 tiles of one warp: decode and multiply.
template <int K, int CB, int MT>
__device__ __forceinline__ void gd_slot(const uint32_t* __restrict__ sb, int ch, int lane, int lane_prev, uint4 (&af)[MT][GD_SLOT_ROWS],
                                        float (&acc)[MT][GD_SLOT_TILES][4])
{
    if constexpr (MT == 1) {
        // activations of the slot, behind its codes: [tile row][lane] 16 bytes each
        const uint4* sa = reinterpret_cast<const uint4*>(sb + GD_SLOT_ROWS * 2 * GD_SLOT_TILES * 8 * K);
        #pragma unroll
        for (int r = 0; r < GD_SLOT_ROWS; ++r) af[0][r] = sa[r * 32 + lane];
    }
    #pragma unroll
    for (int r = 0; r < GD_SLOT_ROWS; ++r) {
        #pragma unroll
        for (int c = 0; c < GD_SLOT_TILES; ++c) {
            const uint32_t* tile = sb + ((r * 2 + ch) * GD_SLOT_TILES + c) * 8 * K;      // this warp's half of the 8-tile row
            uint32_t y[8];
            {
                uint32_t st[8];
                if constexpr (K == 4) lane_states4(tile, lane, lane_prev, st);
                else lane_states<K>(tile, lane, st);
                #pragma unroll
                for (int q = 0; q < 8; ++q) y[q] = decode_raw<CB>(st[q]);
            }
            #pragma unroll
            for (int s = 0; s < MT; ++s) {
                gd_mma(acc[s][c], y[0], y[4], y[1], y[5], af[s][r].x, af[s][r].y);
                gd_mma(acc[s][c], y[2], y[6], y[3], y[7], af[s][r].z, af[s][r].w);
            }
        }
    }
}

// Activations in fragment order.  One CTA per (batch row slot b, tensor): row b < m is transformed as in
// kernels/quant/hadamard_inner.cuh:93-147 (fp16 pre-scale multiply, fp32 butterflies, one fp16 rounding); slots past m
// are zero-filled.  Word (set, kslot, r, lane = 4 g + t, w) holds the value of batch row 8 set + g at
// k = 64 kslot + 16 r + 2 t + (w & 1) + 8 (w >> 1), duplicated into both halves.
struct GemmDecodePrologueArgs { const half* suh[GD_MAX_SEG]; uint32_t* a_frag[GD_MAX_SEG]; float* rowsum[GD_MAX_SEG]; };

// one CTA: batch-row slot b of one tensor's activations
constexpr int GD_PRO_SPLIT = 4;      // CTAs along k per row slot in the input transform of the single-tensor paths

__device__ __forceinline__ void gd_prologue_row(const half* __restrict__ Arow, const half* __restrict__ suh, uint32_t* __restrict__ out,
                                                float* __restrict__ rowsum, int b, bool valid, int k, int part_idx = 0, int parts = 1)
{
    __shared__ float sh[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int set = b >> 3, g = b & 7;
    const int q = lane & 3;                                  // position of the lane's 4 values inside a 16-k tile row
    const int t0 = 2 * (q & 1), w0 = 2 * (q >> 1);
    float part = 0.0f;
    const int per = (k / 128 + parts - 1) / parts;             // 128-blocks of this CTA's k range
    const int blk_end = min(k / 128, (part_idx + 1) * per);
    for (int blk = part_idx * per + warp; blk < blk_end; blk += 8) {
        uint32_t h0 = 0, h1 = 0, h2 = 0, h3 = 0;
        if (valid) {
            uint2 raw = reinterpret_cast<const uint2*>(Arow + blk * 128)[lane];
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
        rowsum[(size_t)part_idx * gridDim.x + b] = s;
    }
}

static __global__ void __launch_bounds__(256) gemm_decode_prologue_kernel(const half* __restrict__ A, const GemmDecodePrologueArgs args,
                                                                   int m, int k)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b = blockIdx.x, seg = blockIdx.y;
    gd_prologue_row(A + (size_t)b * k, args.suh[seg], args.a_frag[seg], args.rowsum[seg], b, b < m, k, blockIdx.z, gridDim.z);
}

// Table mode: grid (row slots, product slots).  Slot j transforms rows of A[j] (or of A[0] when a_slot_stride is 0) with
// the sign vector of the tensor it uses; an unused slot (negative index) gets zeros.
static __global__ void __launch_bounds__(256) gemm_decode_prologue_multi_kernel(const half* __restrict__ A, size_t a_slot_stride,
                                                                         const half* const* __restrict__ suh_tab,
                                                                         const int64_t* __restrict__ indices, uint32_t* a_frag,
                                                                         float* rowsum, int rows_per_slot, int m, int k)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b = blockIdx.x, j = blockIdx.y;
    const int mat = indices ? (int)indices[j] : j;
    const half* suh = mat >= 0 ? suh_tab[mat] : nullptr;
    gd_prologue_row(A + j * a_slot_stride + (size_t)b * k, suh, a_frag + (size_t)j * (rows_per_slot / 8) * (k / 64) * 4 * 32 * 4,
                    rowsum + (size_t)j * rows_per_slot, b, b < m && mat >= 0, k);
}

// Output transform of one row of a 128-column block held by a warp (lane = 4 consecutive columns): codebook-2 affine
// map, 128-point Hadamard, svh, store.
template <int CB>
__device__ __forceinline__ void gd_store_row(float4 v, int lane, float rowsum, const half* __restrict__ svh, void* Cout, size_t off,
                                             int col0, int c_fp32, float r128 = GD_R128)
{
    if constexpr (CB == 2) {
        const float rs = rowsum * GD_MUL1_DELTA;
        v.x = fmaf(v.x, GD_MUL1_KINV, rs); v.y = fmaf(v.y, GD_MUL1_KINV, rs);
        v.z = fmaf(v.z, GD_MUL1_KINV, rs); v.w = fmaf(v.w, GD_MUL1_KINV, rs);
    }
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
        v.x *= r128; v.y *= r128; v.z *= r128; v.w *= r128;
        uint2 sr = *reinterpret_cast<const uint2*>(svh + col0 + lane * 4);
        half2 sa2 = *reinterpret_cast<half2*>(&sr.x), sb2 = *reinterpret_cast<half2*>(&sr.y);
        if (c_fp32) {
            v.x *= __low2float(sa2); v.y *= __high2float(sa2); v.z *= __low2float(sb2); v.w *= __high2float(sb2);
            *reinterpret_cast<float4*>((float*)Cout + off) = v;
        } else {
            half2 a = __hmul2(__floats2half2_rn(v.x, v.y), sa2), b = __hmul2(__floats2half2_rn(v.z, v.w), sb2);
            uint2 o2; o2.x = *reinterpret_cast<uint32_t*>(&a); o2.y = *reinterpret_cast<uint32_t*>(&b);
            *reinterpret_cast<uint2*>((half*)Cout + off) = o2;
        }
    } else {
        if (c_fp32) *reinterpret_cast<float4*>((float*)Cout + off) = v;
        else {
            half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
            uint2 o2; o2.x = *reinterpret_cast<uint32_t*>(&a); o2.y = *reinterpret_cast<uint32_t*>(&b);
            *reinterpret_cast<uint2*>((half*)Cout + off) = o2;
        }
    }
}

// grid = CTAs of the split (at most one per SM), 20 warps (16 decoders, the producer and its three idle warpgroup mates), GdSmem<K, MT>::BYTES of dynamic shared memory.
// rmap*: the trellis of each tensor as a matrix of 64-bit words [k/16][n/16 * 4K], box 4 rows x 4 tiles.
//
// Leaving a column block does not stop the CTA: every decoder drops its accumulators into the reduction tile and goes on
// with the next block; the one that arrives last adds the 8 k-slices, exchanges partial sums with the neighbouring CTAs
// where the block is shared, transforms and stores, and then hands the tile back (an mbarrier the other warps test before
// their next drop, several units later).  While that warp waits on the arrival counter of the exchange, the other warps
// of its scheduler use its issue slots.
template <int K, int CB, int MT, bool MULTI = false>
__global__ void __launch_bounds__(GD_THREADS, 1) gemm_decode_kernel(const __grid_constant__ CUtensorMap rmap0,
                                                                   const __grid_constant__ CUtensorMap rmap1,
                                                                   const __grid_constant__ CUtensorMap rmap2,
                                                                   const GemmDecodeParams p)
{
    using SM = GdSmem<K, MT>;
    extern __shared__ uint8_t gd_smem_unaligned[];
    uint8_t* smem = gd_smem_unaligned + ((128u - (smem_u32(gd_smem_unaligned) & 127u)) & 127u);
    float* red = reinterpret_cast<float*>(smem + SM::OFF_RED);
    uint64_t* full_bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
    uint64_t* empty_bars = full_bars + GD_KSL * SM::DEPTH;
    __shared__ int s_drops;
    __shared__ __align__(8) uint64_t s_red_free;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KC = (p.k + GD_UNIT_K - 1) / GD_UNIT_K;                  // k chunks per column block
    const int blocks = p.blk_end[GD_MAX_SEG - 1];
    const long long total = (long long)blocks * KC;
    const long long G = gridDim.x;
    // this CTA's contiguous range of units (column-block-major): whole blocks, or an even share of all units
    const long long u0 = p.aligned ? (long long)(blocks * (long long)blockIdx.x / G) * KC : total * blockIdx.x / G;
    const long long u1 = p.aligned ? (long long)(blocks * (long long)(blockIdx.x + 1) / G) * KC : total * (blockIdx.x + 1) / G;
    const int nunits = (int)(u1 - u0);
    const int mrows = p.m;
    const int nbg0 = (int)(u0 / KC), kc0 = (int)(u0 - (long long)nbg0 * KC);
    const int bpm = p.n[0] >> 7;                                       // column blocks per tensor (table mode)
    auto seg_of = [&](int nbg) -> int {
        if constexpr (MULTI) return nbg / bpm;
        else return (nbg >= p.blk_end[0]) + (nbg >= p.blk_end[1]);
    };
    auto col0_of = [&](int nbg, int seg) -> int {
        if constexpr (MULTI) return (nbg - seg * bpm) * 128;
        else return (nbg - (seg == 0 ? 0 : (seg == 1 ? p.blk_end[0] : p.blk_end[1]))) * 128;
    };
    // table mode: the tensor a slot uses, or -1
    auto mat_of = [&](int seg) -> int { return p.indices ? (int)p.indices[seg] : seg; };
    const size_t afrag_slot = (size_t)MT * (p.k / 64) * GD_SLOT_ROWS * 32;        // uint4 per slot of activations (table mode)

    GD_STAMP(0);
#ifdef GD_TRACE
    if (lane == 0 && warp < 16 && blockIdx.x < 148) { for (int q = 4; q < 7; ++q) g_gd_trace[(blockIdx.x * 16 + warp) * 8 + q] = 0; }
#endif
    if (tid == 0) {
        for (int i = 0; i < GD_KSL * SM::DEPTH; ++i) { mbar_init(&full_bars[i], 1); mbar_init(&empty_bars[i], 2); }
        mbar_init(&s_red_free, 1);
        s_drops = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // Twenty warps start with 96 registers each; the producer's warpgroup hands most of its share back and the four decoder
    // warpgroups take 120 each (the register file holds 20 x 32 x 96 + 16 x 32 x 24 + 4 x 32 x (24 - 96) <= 65536).
    bool failed = false;
    if (warp >= GD_WARPS) asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 120;");
    if (warp > GD_WARPS) {
        // idle warps of the producer's warpgroup
    } else if (warp == GD_WARPS) {
        // ===== producer: lane l < 8 serves k-slice l (decoder warps l and l + 8, the two column halves).  Unit i of the CTA
        // is slot i % DEPTH of every ring.  The lanes share one instruction stream but each keeps its own cursor: in every
        // pass a lane whose next slot is free requests its next unit, so a pair that runs ahead is fed ahead and one that
        // has fallen behind (the warp that finishes a column block) holds nobody else up.  A unit whose k chunk ends before
        // the slice (ragged last chunk) still takes the slot: nothing is copied and the lane arrives on the "full" barrier
        // itself.
        const bool serving = lane < GD_KSL;
        const int ks = lane & (GD_KSL - 1);
        const uint32_t ring = smem_u32(smem + SM::OFF_RING + ks * SM::DEPTH * SM::SLOT_BYTES);
        const uint32_t fb = smem_u32(full_bars + ks * SM::DEPTH);
        uint64_t* eb = empty_bars + ks * SM::DEPTH;
        const int kslot_stride = GD_SLOT_ROWS * 32;                                 // uint4 per activation slot
        int i = serving ? 0 : nunits, nbg = nbg0, kc = kc0, slot = 0, round = 0;
        bool waited = false;                   // the wait for the activations' producer (first use only)
        uint32_t idle = 0;
        while (__any_sync(0xffffffffu, i < nunits)) {
            const bool go = i < nunits && (round == 0 || mbar_try_wait(&eb[slot], (round - 1) & 1));
            if (go) {
                const uint32_t bar = fb + 8u * slot;
                const int seg = seg_of(nbg);
                const int mat = MULTI ? mat_of(seg) : 0;
                if (kc * GD_UNIT_K + ks * (GD_SLOT_ROWS * 16) < p.k && mat >= 0) {
                    const uint32_t dst = ring + slot * SM::SLOT_BYTES;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)SM::SLOT_BYTES) : "memory");
                    if constexpr (MULTI) {
                        // the tensor comes out of a device table: four row copies of 8 tiles each instead of one tiled box
                        const uint32_t* src = p.trellis_tab[mat] +
                            ((size_t)(kc * (GD_UNIT_K / 16) + ks * GD_SLOT_ROWS) * (p.n[0] >> 4) + (col0_of(nbg, seg) >> 4)) * 8 * K;
                        #pragma unroll
                        for (int r = 0; r < GD_SLOT_ROWS; ++r)
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(dst + (uint32_t)(r * (SM::CODE_BYTES / GD_SLOT_ROWS))), "l"(src + (size_t)r * (p.n[0] >> 4) * 8 * K),
                                           "r"((uint32_t)(SM::CODE_BYTES / GD_SLOT_ROWS)), "r"(bar) : "memory");
                    } else {
                        const CUtensorMap* rmap = seg == 0 ? &rmap0 : (seg == 1 ? &rmap1 : &rmap2);
                        gd_tma_load_2d(dst, rmap, (col0_of(nbg, seg) >> 4) * 4 * K, kc * (GD_UNIT_K / 16) + ks * GD_SLOT_ROWS, bar);
                    }
                    if constexpr (SM::ACT_BYTES > 0) {
                        // The launch may overlap the tail of the kernel that writes the activations (programmatic dependent
                        // launch): the codes above do not depend on it, the activations do.
                        if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
                        const uint4* afr = MULTI ? p.a_frag[0] + (size_t)seg * afrag_slot
                                                 : (seg == 0 ? p.a_frag[0] : (seg == 1 ? p.a_frag[1] : p.a_frag[2]));
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst + (uint32_t)SM::CODE_BYTES), "l"(afr + (size_t)(kc * GD_KSL + ks) * kslot_stride),
                                       "r"((uint32_t)SM::ACT_BYTES), "r"(bar) : "memory");
                    }
                } else {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
                }
                if (++slot == SM::DEPTH) { slot = 0; ++round; }
                if (++kc == KC) { kc = 0; ++nbg; }
                ++i;
            }
            // nothing to do for any lane: leave the issue slots to the decoders for a moment; give up after about 4 s
            if (!__any_sync(0xffffffffu, go)) {
                __nanosleep(200);
                if (++idle > (1u << 24)) { failed = true; break; }
            } else idle = 0;
        }
    } else {
        // ===== decoders
        const int g = lane >> 2, t = lane & 3;
        const int ks = warp & (GD_KSL - 1), ch = warp >> 3;
        const uint8_t* ring = smem + SM::OFF_RING + ks * SM::DEPTH * SM::SLOT_BYTES;
        uint64_t* full = full_bars + ks * SM::DEPTH;
        uint64_t* empty = empty_bars + ks * SM::DEPTH;

        float acc[MT][GD_SLOT_TILES][4];
        #pragma unroll
        for (int s = 0; s < MT; ++s)
            #pragma unroll
            for (int c = 0; c < GD_SLOT_TILES; ++c)
                #pragma unroll
                for (int e = 0; e < 4; ++e) acc[s][c][e] = 0.0f;

        if constexpr (SM::ACT_BYTES == 0) asm volatile("griddepcontrol.wait;" ::: "memory");      // these warps read the activations themselves

        const int lane_prev = (lane + 31) & 31;
        int nbg = nbg0, kc = kc0 - 1, slot = 0, par = 0;
        int events = 0;                                     // column blocks this CTA has left so far
        #pragma unroll 1
        for (int i = 0; i < nunits; ++i) {
            if (++kc == KC) { kc = 0; ++nbg; }
            const bool active = kc * GD_UNIT_K + ks * (GD_SLOT_ROWS * 16) < p.k && (!MULTI || mat_of(seg_of(nbg)) >= 0);
            if (!failed) {
                uint4 af[MT][GD_SLOT_ROWS];
                if (SM::ACT_BYTES == 0 && active) {
                    // batch rows 8 set + g, k = 64 kslot + 16 r + {2t, 2t+1, 2t+8, 2t+9}
                    const int seg = seg_of(nbg);
                    const uint4* afr = MULTI ? p.a_frag[0] + (size_t)seg * afrag_slot
                                             : (seg == 0 ? p.a_frag[0] : (seg == 1 ? p.a_frag[1] : p.a_frag[2]));
                    const int kslot = kc * GD_KSL + ks;
                    #pragma unroll
                    for (int s = 0; s < MT; ++s)
                        #pragma unroll
                        for (int r = 0; r < GD_SLOT_ROWS; ++r)
                            af[s][r] = __ldg(afr + (((size_t)s * (p.k / 64) + kslot) * 4 + r) * 32 + lane);
                }
                GD_T0();
                const bool ok = mbar_wait_sleep_warp(&full[slot], par);
                if (i > 0) GD_ACC(4, GD_DT());
                if (i == 0) GD_STAMP(1);
                if (ok) {
                    if (active) gd_slot<K, CB, MT>(reinterpret_cast<const uint32_t*>(ring + slot * SM::SLOT_BYTES), ch, lane, lane_prev, af, acc);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[slot]);              // every lane of this warp has read the slot
                } else failed = true;
                if (++slot == SM::DEPTH) { slot = 0; par ^= 1; }
            }

            const bool block_done = kc == KC - 1 || i == nunits - 1;
            if (i == nunits - 1) GD_STAMP(2);
            if (!block_done) continue;

            // ---- the CTA leaves column block nbg.  The reduction tile is free again once the warp that finished the
            // previous block has read it (that was several units ago unless this is the CTA's last, short block).
            if (events > 0 && !mbar_wait_sleep_warp(&s_red_free, (events - 1) & 1)) failed = true;
            ++events;
            #pragma unroll
            for (int s = 0; s < MT; ++s)
                #pragma unroll
                for (int c = 0; c < GD_SLOT_TILES; ++c) {
                    float* dst = red + ((size_t)ks * SM::ROWS + s * 8 + 2 * t) * GD_RSTRIDE + ch * 64 + c * 16 + g;
                    dst[0] = acc[s][c][0]; dst[GD_RSTRIDE] = acc[s][c][1];
                    dst[8] = acc[s][c][2]; dst[GD_RSTRIDE + 8] = acc[s][c][3];
                    acc[s][c][0] = acc[s][c][1] = acc[s][c][2] = acc[s][c][3] = 0.0f;
                }
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = atomicAdd(&s_drops, 1) == GD_WARPS - 1;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (!last) continue;

            // ---- this warp arrived last: it finishes the block on its own
            GD_T0();
            if (lane == 0) s_drops = 0;
            __threadfence_block();
            const int seg = seg_of(nbg);
            const int n0 = col0_of(nbg, seg);
            const half* svh = seg == 0 ? p.svh[0] : (seg == 1 ? p.svh[1] : p.svh[2]);
            void* Cout = seg == 0 ? p.C[0] : (seg == 1 ? p.C[1] : p.C[2]);
            int n = seg == 0 ? p.n[0] : (seg == 1 ? p.n[1] : p.n[2]);
            const float* rsum = seg == 0 ? p.rowsum[0] : (seg == 1 ? p.rowsum[1] : p.rowsum[2]);
            float r128 = GD_R128;
            bool store = true;
            if constexpr (MULTI) {
                const int mat = mat_of(seg);
                store = mat >= 0;                         // an unused slot's rows of C are left as they are
                n = p.n[0];
                svh = store ? p.svh_tab[mat] : nullptr;
                Cout = p.c_fp32 ? (void*)((float*)p.C[0] + (size_t)seg * p.c_slot_stride) : (void*)((half*)p.C[0] + (size_t)seg * p.c_slot_stride);
                rsum = p.rowsum[0] + (size_t)seg * SM::ROWS;
                if (p.weights) r128 *= __half2float(p.weights[seg]);
            }
            auto rs_of = [&](int row) -> float {
                float a = 0.f;
                for (int z = 0; z < p.rowsum_parts; ++z) a += rsum[(size_t)z * SM::ROWS + row];
                return a;
            };
            // sum of the 8 k-slices of one row, in slice order; lane = 4 consecutive columns
            auto row_sum = [&](int row) -> float4 {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                #pragma unroll
                for (int s = 0; s < GD_KSL; ++s) {
                    const float4 v = *reinterpret_cast<const float4*>(red + ((size_t)s * SM::ROWS + row) * GD_RSTRIDE + lane * 4);
                    a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                }
                return a;
            };
            // CTAs that own a part of this block: those whose unit range meets [nbg * KC, (nbg + 1) * KC)
            int c_first = blockIdx.x, c_last = blockIdx.x;
            if (!p.aligned) {
                const long long first = (long long)nbg * KC;
                auto owner = [&](long long u) -> int { return (int)(((u + 1) * G + total - 1) / total - 1); };
                c_first = owner(first); c_last = owner(first + KC - 1);
            }
            const int ncontrib = c_last - c_first + 1;
            if (ncontrib == 1) {
                for (int row = 0; row < mrows && store; ++row)
                    gd_store_row<CB>(row_sum(row), lane, CB == 2 ? rs_of(row) : 0.f, svh, Cout, (size_t)row * n + n0 + lane * 4, n0, p.c_fp32, r128);
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_red_free);
            } else {
                // a CTA shares at most its first and its last column block: slot 0 and slot 1 of its pair
                auto slot_of = [&](int cta) -> float* {
                    const long long fb = (total * cta / G) / KC;
                    return p.partial + ((size_t)cta * 2 + (fb == nbg ? 0 : 1)) * mrows * 128;
                };
                float* mine = slot_of(blockIdx.x);
                for (int row = 0; row < mrows; ++row)
                    *reinterpret_cast<float4*>(mine + row * 128 + lane * 4) = row_sum(row);
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_red_free);              // the tile has been read: the other warps may drop again
                // one arrival per CTA: the release half publishes this warp's partial sums (ordered before it by the warp
                // barrier above), the acquire half makes the other owners' visible to the CTA that arrives last
                int fin = 0;
                if (lane == 0) {
                    int old;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + nbg) : "memory");
                    fin = old == ncontrib - 1;
                    if (fin) p.counters[nbg] = 0;
                }
                fin = __shfl_sync(0xffffffffu, fin, 0);
                if (fin) {
                    __syncwarp();
                    // all owners' partial sums of up to 8 rows are requested before the first is used
                    for (int row0 = 0; row0 < mrows; row0 += 8) {
                        float4 a[8];
                        #pragma unroll
                        for (int r = 0; r < 8; ++r) a[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int s = c_first; s <= c_last; ++s) {           // owner order: independent of arrival order
                            const float* src = slot_of(s) + lane * 4;
                            #pragma unroll
                            for (int r = 0; r < 8; ++r)
                                if (row0 + r < mrows) {
                                    const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (row0 + r) * 128));
                                    a[r].x += v.x; a[r].y += v.y; a[r].z += v.z; a[r].w += v.w;
                                }
                        }
                        #pragma unroll
                        for (int r = 0; r < 8; ++r)
                            if (row0 + r < mrows && store)
                                gd_store_row<CB>(a[r], lane, CB == 2 ? rs_of(row0 + r) : 0.f, svh, Cout, (size_t)(row0 + r) * n + n0 + lane * 4, n0, p.c_fp32, r128);
                    }
                }
            }
            GD_ACC(5, GD_DT());
        }
        GD_STAMP(3);
    }
    // A wait that ran out ends the CTA's work; the status word tells the host.  (Copies still in flight belong to slots
    // whose barrier nobody waits on any more; they were requested at most a ring's depth ahead and land within microseconds,
    // long before the bounded waits of the other warps give up and the CTA can exit.)
    if (__syncthreads_or(failed) && tid == 0) atomicExch(p.status, 1);
}

}  // namespace exl3
