// EXL3 GEMM for large M (prefill chunks, verify batches, big packed steps): a real contraction on the 5th-generation
// tensor cores.  Activations arrive by TMA (tiled, 128-byte swizzle), trellis codes by bulk copies; sixteen decoder
// warps turn codes into fp16 weights and write them straight into the K-major swizzled B operand tile in shared memory;
// one thread issues tcgen05.mma with both accumulators (2 x 128 rows x 256 columns, all 512 TMEM columns) resident in
// tensor memory; the epilogue reads TMEM, applies the 128-wide output Hadamard and stores fp16/fp32.
//
// Two forms of the same kernel (template parameter CTAS):
//   CTAS = 1  one CTA owns 256 rows x 256 columns and decodes all 256 columns of the weight slab.
//   CTAS = 2  a cluster of two CTAs (one SM pair) owns 512 rows x 256 columns.  Each CTA decodes only its 128-column half
//             of the slab and holds the accumulators of its own 2 x 128 rows; the leader CTA issues
//             tcgen05.mma.cta_group::2 (M = 256 across the pair), which reads each CTA's half of B from that CTA's shared
//             memory.  The decode work per multiply is halved, which is what bounds the CTAS = 1 form.
// K step 64.  Roles: warp 0 = activation producer (TMA), warp 1 = MMA issuer (leader CTA only) and TMEM owner,
// warps 2..17 = decoders, then epilogue (warp w reads TMEM lanes 32*(w%4)..+31), warp 18 = trellis-code producer.
// Every mbarrier wait is bounded; a wait that runs out makes the CTA skip to the tear-down (TMEM is always freed) and
// sets the status word.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "exl3_decode.cuh"
#include "async_copy.cuh"

namespace exl3 {

constexpr int TC_BM = 256, TC_BN = 256, TC_BK = 64;     // rows per CTA, columns per slab, K step
constexpr int TC_DECODERS = 16;                          // decoder warps
constexpr int TC_THREADS = (3 + TC_DECODERS) * 32;       // 19 warps: two producers, the MMA issuer, the decoders
constexpr int TC_MAX_SEG = 3;                            // weight tensors that may share one launch
constexpr int TC_A_TILE = 128 * TC_BK * 2;               // one 128-row activation tile of a stage: 16 KB
constexpr int TC_A_STAGE = 2 * TC_A_TILE;                // 32 KB
constexpr float TC_R128 = 0.088388347648f;

template <int K, int CTAS, int BN = 256> struct TcSmem {
    static constexpr int SA = CTAS == 2 ? 4 : 3;         // stages: activations,
    static constexpr int SB = CTAS == 2 ? 4 : 2;         //         decoded weights,
    static constexpr int NB = BN / CTAS;                 // columns this CTA decodes
    static constexpr int B_STAGE = NB * TC_BK * 2;
    static constexpr int RAW_ROW = (NB / 16) * 32 * K;   // one tile row of codes: NB/16 tiles x 32K bytes
    static constexpr int RAW_STAGE = (TC_BK / 16) * RAW_ROW;
    // raw codes come from HBM with the longest latency of the three rings and are the smallest: a deep ring keeps
    // enough bytes in flight (a pair CTA has about 32 KB left for it, one CTA alone 24 KB)
    static constexpr int SR_ROOM = (CTAS == 2 ? 32 : 24) * 1024 / RAW_STAGE;
    static constexpr int SR = SR_ROOM > 8 ? 8 : (SR_ROOM < 3 ? 3 : SR_ROOM);
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + SA * TC_A_STAGE;
    static constexpr int OFF_RAW = OFF_B + SB * B_STAGE;
    static constexpr int OFF_SVH = OFF_RAW + SR * RAW_STAGE;
    static constexpr int OFF_BAR = OFF_SVH + BN * 2;
    static constexpr int N_BARS = 4 * SA + 2 * SR + 2 * SB + 2;      // the A ring has 2 * SA slots for one-tile blocks
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
    int blk_end[TC_MAX_SEG];               // running count of 256-column slabs
    int* status;
    int m, k, c_fp32;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// shared -> global tensor store (rows and columns past the tensor's extent are clipped), committed as a bulk group
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// one lane of a converged warp
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// D[tmem] (+)= A[smem desc] * B[smem desc], fp16 inputs, fp32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// ---- the same operations for a CTA pair (cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// all threads of both CTAs
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tile lands in this CTA's shared memory, its bytes are counted on the leader CTA's barrier (rank bit of the address cleared)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar) & 0xFEFFFFFFu) : "memory");
}
// arrive on the barrier at the same offset in CTA `cta` of the cluster.  The data this signals lies in the arriving CTA's own
// shared memory and was fenced into the async proxy by each writing lane; a cluster-scope release on top of that was
// measured to cost a quarter of the kernel's time and is what no 2-CTA pipeline needs for SM-local shared memory.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta)
{
    asm volatile("{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\t"
                 "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(bar)), "r"(cta) : "memory");
}
// bounded wait that acquires at cluster scope (the arrivals or bytes may come from the other CTA); each poll may sleep
// up to `ns` nanoseconds inside the instruction and returns early when the phase completes
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 20), uint32_t ns = 2000)
{
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
        if (ok) return true;
    }
    return false;
}
// the same with plain polls: for the one thread whose wake-up latency is on the critical path
__device__ __forceinline__ bool mbar_spin_cluster(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 24))
{
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// arrive on the barrier at this offset in both CTAs of the pair when the MMAs issued so far have completed
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
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

// instruction descriptor: D fp32, A/B fp16, both K-major, N = 256, M = 128 (one CTA) or 256 (a CTA pair)
constexpr uint32_t tc_idesc(int n, int m) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }


// Exact fp16 weights of two states, as decode_pair, with one ALU-pipe instruction less: the two halves of each raw
// register are added with half-selecting operands (both halves of the result hold the weight) and one permute merges the
// two sums, instead of two permutes and one packed add (256-row GEMM at 5120 x 17408: 51.4 -> 48.6 us).
template <int CB>
__device__ __forceinline__ half2 tc_decode_pair(uint32_t s0, uint32_t s1)
{
    if constexpr (CB == 2) return decode_pair<CB>(s0, s1);
    else {
        const uint32_t y0 = decode_raw<CB>(s0), y1 = decode_raw<CB>(s1);
        const half2 a = *reinterpret_cast<const half2*>(&y0), b = *reinterpret_cast<const half2*>(&y1);
        const half2 w0 = __hadd2(__low2half2(a), __high2half2(a));
        const half2 w1 = __hadd2(__low2half2(b), __high2half2(b));
        return __lows2half2(w0, w1);
    }
}

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


// CTAS = 1: grid (slabs, ceil(m / 256)).  CTAS = 2: grid (2 * slabs, ceil(m / 512)), cluster (2,1,1).
// The activations come through `amap*` (A_had [m][k] fp16, box 64 x 128, 128-byte swizzle), one map per weight tensor.
// BN = columns per slab: 256, or 128 (pair form only) for launches whose 256-column slabs would leave most SMs without
// work (one row block, at most a quarter as many slabs as SMs): the decode work of a tensor then spreads over twice the CTAs.
template <int K, int CB, int CTAS, int BN = 256>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap amap0,
                                                               const __grid_constant__ CUtensorMap amap1,
                                                               const __grid_constant__ CUtensorMap amap2,
                                                               const __grid_constant__ CUtensorMap rmap0,
                                                               const __grid_constant__ CUtensorMap rmap1,
                                                               const __grid_constant__ CUtensorMap rmap2,
                                                               const __grid_constant__ CUtensorMap cmap0,
                                                               const __grid_constant__ CUtensorMap cmap1,
                                                               const __grid_constant__ CUtensorMap cmap2, const GemmTcParams p)
{
    using SM = TcSmem<K, CTAS, BN>;
    constexpr bool PAIR = CTAS == 2;
    constexpr uint32_t IDESC = tc_idesc(BN, 128 * CTAS);
    constexpr int NT = SM::NB / 16;                       // tile columns this CTA decodes (16, 8 or 4)
    // decoder warps per group: a group takes a K step together, four tiles per warp where the stage has enough of them
    constexpr int GW = (TC_BK / 16) * NT / 4 < 8 ? (TC_BK / 16) * NT / 4 : 8;
    constexpr int NG = TC_DECODERS / GW;                  // groups, taking K steps in turn
    extern __shared__ uint8_t smem_unaligned[];
    // aligned to 1024 bytes by an offset from the array, not through an integer, so that the compiler still knows the
    // pointer is in shared memory (32-bit addresses, ld/st.shared) instead of falling back to generic accesses
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::OFF_BAR);
    uint64_t* a_full = bars;                  uint64_t* a_empty = a_full + 2 * SM::SA;
    uint64_t* r_full = a_empty + 2 * SM::SA;      uint64_t* r_empty = r_full + SM::SR;
    uint64_t* b_full = r_empty + SM::SR;      uint64_t* b_empty = b_full + SM::SB;
    uint64_t* acc_full = b_empty + SM::SB;    uint64_t* drain = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::OFF_TMEM);
    __shared__ int s_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = PAIR ? (int)cluster_ctarank() : 0;                  // 0 = leader of the pair
    const int slab = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int seg = (slab >= p.blk_end[0]) + (slab >= p.blk_end[1]);
    const int n0 = (slab - (seg == 0 ? 0 : (seg == 1 ? p.blk_end[0] : p.blk_end[1]))) * BN;     // first column of the slab
    const int nd0 = n0 + rank * SM::NB;                                  // first column this CTA decodes
    const int m0 = blockIdx.y * (TC_BM * CTAS);
    const int row_t0 = m0 + rank * 128, row_t1 = row_t0 + 128 * CTAS;    // first rows of this CTA's two M tiles
    const CUtensorMap* amap = seg == 0 ? &amap0 : (seg == 1 ? &amap1 : &amap2);
    const CUtensorMap* rmap = seg == 0 ? &rmap0 : (seg == 1 ? &rmap1 : &rmap2);       // trellis as [k/16][row of uint64]
    const CUtensorMap* cmap = seg == 0 ? &cmap0 : (seg == 1 ? &cmap1 : &cmap2);       // fp16 output [m][n], box 64 x 32, 128-byte swizzle
    // (selected with compares: indexing the parameter arrays with `seg` would put a copy of them in local memory)
    const uint32_t* trellis = seg == 0 ? p.trellis[0] : (seg == 1 ? p.trellis[1] : p.trellis[2]);
    const half* svh = seg == 0 ? p.svh[0] : (seg == 1 ? p.svh[1] : p.svh[2]);
    void* Cout = seg == 0 ? p.C[0] : (seg == 1 ? p.C[1] : p.C[2]);
    const int n = seg == 0 ? p.n[0] : (seg == 1 ? p.n[1] : p.n[2]);
    const int tiles_n = n >> 4;
    const int ksteps = p.k / TC_BK;
    const bool two_tiles = p.m - m0 > 128 * CTAS;          // otherwise the second M tile (of both CTAs) has no valid row
    // The activation ring holds SA steps of two tiles, or twice as many steps of one tile: a block with one tile spends half
    // the tensor-core time per step, and the TMA round trip (about 2000 cycles) must still be covered by the steps in flight.
    const int a_slots = two_tiles ? SM::SA : 2 * SM::SA;
    const uint32_t a_slot_bytes = two_tiles ? TC_A_STAGE : TC_A_TILE;

    if (tid == 0) {
        s_failed = 0;
        for (int i = 0; i < 2 * SM::SA; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < SM::SR; ++i) { mbar_init(&r_full[i], 1); mbar_init(&r_empty[i], GW); }
        for (int i = 0; i < SM::SB; ++i) { mbar_init(&b_full[i], GW * CTAS); mbar_init(&b_empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_init(drain, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    // (the last slab of a tensor with n % 256 == 128 has one valid half: its other half decodes zero-filled codes into
    // columns that are never stored)
    if (svh) for (int i = tid; i < BN; i += TC_THREADS)
        reinterpret_cast<half*>(smem + SM::OFF_SVH)[i] = n0 + i < n ? svh[n0 + i] : __float2half(0.f);
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();               // the other CTA's barriers are initialised before anything arrives
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    // The two producers are single threads on different schedulers (warps 0 and 18).  One thread doing both jobs took
    // about 1000 cycles per K step (some fifty dependent instructions, each arbitrated against four decoder warps) and
    // was what the tensor core ended up waiting for.
    if (warp == 0) {
        // ===== activation producer: one or two tiled TMA loads per K step
        if (lane == 0) {
            const uint32_t a_bytes = (two_tiles ? 2u : 1u) * TC_A_TILE * CTAS;     // what lands on the leader's barrier
            int sa = 0;
            uint32_t par_ae = 1;                                  // a_empty is waited from the second round on
            for (int ks = 0; ks < ksteps; ++ks) {
                if (ks >= a_slots && !mbar_wait(&a_empty[sa], par_ae)) { failed = true; break; }
                uint8_t* at = smem + SM::OFF_A + sa * a_slot_bytes;
                if constexpr (PAIR) {
                    if (rank == 0) mbar_expect_tx(&a_full[sa], a_bytes);
                    tma_load_2d_pair(at, amap, ks * TC_BK, row_t0, &a_full[sa]);
                    if (two_tiles) tma_load_2d_pair(at + TC_A_TILE, amap, ks * TC_BK, row_t1, &a_full[sa]);
                } else {
                    mbar_expect_tx(&a_full[sa], a_bytes);
                    tma_load_2d(at, amap, ks * TC_BK, row_t0, &a_full[sa]);
                    if (two_tiles) tma_load_2d(at + TC_A_TILE, amap, ks * TC_BK, row_t1, &a_full[sa]);
                }
                if (++sa == a_slots) { sa = 0; par_ae ^= 1; }
            }
        }
    } else if (warp == 2 + TC_DECODERS) {
        // ===== code producer: a stage of trellis codes = 4 tile rows x RAW_ROW bytes.  The pair form fetches it with one
        // tiled TMA load (box of 4 rows), the one-CTA form with four bulk copies issued by four lanes at once.
        const size_t row_words = (size_t)tiles_n * 8 * K;                      // one tile row of the whole tensor
        const uint32_t* src_lane = trellis + (size_t)(lane & 3) * row_words + (size_t)(nd0 >> 4) * 8 * K;
        const uint32_t dst_lane = smem_u32(smem + SM::OFF_RAW) + (lane & 3) * SM::RAW_ROW;
        if (PAIR ? lane == 0 : lane < TC_BK / 16) {
            int sr = 0;
            uint32_t par_re = 1;                                  // r_empty is waited from the second round on
            for (int kr = 0; kr < ksteps; ++kr) {
                if (kr >= SM::SR && !mbar_wait(&r_empty[sr], par_re)) { failed = true; break; }
                if (lane == 0) mbar_expect_tx(&r_full[sr], SM::RAW_STAGE);
                if constexpr (PAIR) {
                    tma_load_2d(smem + SM::OFF_RAW + sr * SM::RAW_STAGE, rmap, (nd0 >> 4) * 4 * K, kr * (TC_BK / 16), &r_full[sr]);
                } else {
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(dst_lane + sr * SM::RAW_STAGE), "l"(src_lane + (size_t)kr * (TC_BK / 16) * row_words),
                                   "r"((uint32_t)SM::RAW_ROW), "r"(smem_u32(&r_full[sr])) : "memory");
                }
                if (++sr == SM::SR) { sr = 0; par_re ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer (leader CTA).  The whole warp runs the loop with warp-uniform values, so that descriptors and
        // addresses stay in uniform registers (where tcgen05.mma takes them from); one elected lane issues.
        if (rank == 0) {
            const bool leader = elect_one();
            constexpr uint32_t HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);     // SBO 1024, version 1, SWIZZLE_128B
            const uint32_t a_lo = (smem_u32(smem + SM::OFF_A) >> 4) | (1u << 16);
            const uint32_t b_lo = (smem_u32(smem + SM::OFF_B) >> 4) | (1u << 16);
            auto mk = [](uint32_t lo) { return ((uint64_t)HI << 32) | lo; };
            int sa = 0, sb = 0;
            uint32_t par_a = 0, par_b = 0;
            for (int ks = 0; ks < ksteps; ++ks) {
                bool ok = PAIR ? mbar_spin_cluster(&a_full[sa], par_a) : mbar_wait(&a_full[sa], par_a);
                ok = ok && (PAIR ? mbar_spin_cluster(&b_full[sb], par_b) : mbar_wait(&b_full[sb], par_b));
                if (!__all_sync(0xffffffffu, ok)) { failed = true; break; }
                tc_fence_after();
                const uint32_t a0 = a_lo + sa * (a_slot_bytes >> 4), b0 = b_lo + sb * (SM::B_STAGE >> 4);
                if (leader) {
                    #pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk) {
                        const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (PAIR) {
                            tc_mma_f16_pair(tmem_base, mk(a0 + 2 * kk), mk(b0 + 2 * kk), IDESC, acc);      // +32 bytes per K=16
                            if (two_tiles) tc_mma_f16_pair(tmem_base + BN, mk(a0 + (TC_A_TILE >> 4) + 2 * kk), mk(b0 + 2 * kk), IDESC, acc);
                        } else {
                            tc_mma_f16(tmem_base, mk(a0 + 2 * kk), mk(b0 + 2 * kk), IDESC, acc);
                            if (two_tiles) tc_mma_f16(tmem_base + BN, mk(a0 + (TC_A_TILE >> 4) + 2 * kk), mk(b0 + 2 * kk), IDESC, acc);
                        }
                    }
                    // arrive when the MMAs above have finished reading the stage (in both CTAs of a pair)
                    if constexpr (PAIR) { tc_commit_pair(&a_empty[sa]); tc_commit_pair(&b_empty[sb]); }
                    else { tc_commit(&a_empty[sa]); tc_commit(&b_empty[sb]); }
                }
                __syncwarp();
                if (++sa == a_slots) { sa = 0; par_a ^= 1; }
                if (++sb == SM::SB) { sb = 0; par_b ^= 1; }
            }
            if (leader) {
                if (!failed) {
                    if constexpr (PAIR) tc_commit_pair(acc_full); else tc_commit(acc_full);
                } else {
                    // leave no MMA in flight behind: the tear-down lets the other CTA go, whose shared memory they read
                    if constexpr (PAIR) tc_commit_pair(drain); else tc_commit(drain);
                    mbar_wait(drain, 0);
                }
            }
            __syncwarp();
        }
    } else if (warp < 2 + TC_DECODERS) {
        // ===== decoders: raw codes -> fp16 weights in the K-major swizzled B tile.
        // The 16 warps form NG groups (two of 8 warps, or four of 4 on 128-column slabs; every group has a warp on each
        // scheduler) that take K steps in turn: while one group waits on its barriers, fences and arrives, the others
        // decode, so the schedulers stay busy (with all 16 warps in lockstep on every stage, the waits of a stage cost as
        // much as its decode work; with two tiles per warp and stage they cost a third of it).
        constexpr int TPW = (TC_BK / 16) * NT / GW;                // tiles per warp and stage: 4, or 8 (one CTA per slab)
        constexpr int TB = 4;                                      // tiles decoded together (register budget)
        static_assert(TPW % TB == 0 && SM::SR >= NG, "decoder groups");
        const int dw = warp - 2;
        const int grp = (dw >> 2) % NG;
        const int wi = (dw & 3) + 4 * (dw / (4 * NG));             // 0..GW-1 inside the group
        const int g = lane >> 2, t = lane & 3;
        // Tile (r, nt) of a stage: tile row r covers k = 16r..16r+15, i.e. 16-byte chunks 2r and 2r+1 of a 128-byte B
        // row; B row = column 16nt + g (and + 8, 1024 bytes further on); the chunk index is XORed with (row & 7) = g.
        uint32_t raw_off[TPW], st_off[TPW][2];
        #pragma unroll
        for (int i = 0; i < TPW; ++i) {
            const int idx = wi + GW * i, r = idx / NT, nt = idx % NT;
            raw_off[i] = (r * NT + nt) * 8 * K;
            st_off[i][0] = (nt * 16 + g) * 128 + (((2 * r) ^ g) << 4) + 4 * t;
            st_off[i][1] = (nt * 16 + g) * 128 + (((2 * r + 1) ^ g) << 4) + 4 * t;
        }
        uint32_t bfull_addr = smem_u32(&b_full[0]);
        if constexpr (PAIR) asm volatile("mapa.shared::cluster.u32 %0, %0, 0;" : "+r"(bfull_addr));
        int sr = grp % SM::SR, sb = grp % SM::SB;
        uint32_t par_r = 0, par_b = 1;                             // b_empty is waited from the second round on
        for (int ks = grp; ks < ksteps; ks += NG) {
            if (!mbar_wait_sleep_warp(&r_full[sr], par_r)) { failed = true; break; }
            if (ks >= SM::SB && !mbar_wait_sleep_warp(&b_empty[sb], par_b)) { failed = true; break; }
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(smem + SM::OFF_RAW + sr * SM::RAW_STAGE);
            uint8_t* bt = smem + SM::OFF_B + sb * SM::B_STAGE;
            #pragma unroll
            for (int h = 0; h < TPW; h += TB) {
                uint32_t st[TB][8];
                #pragma unroll
                for (int i = 0; i < TB; ++i) {
                    if constexpr (K == 4) lane_states4(raw + raw_off[h + i], lane, (lane + 31) & 31, st[i]);
                    else lane_states<K>(raw + raw_off[h + i], lane, st[i]);
                }
                #pragma unroll
                for (int i = 0; i < TB; ++i) {
                    const half2 w0 = tc_decode_pair<CB>(st[i][0], st[i][1]);      // rows 2t, 2t+1   col g
                    const half2 w1 = tc_decode_pair<CB>(st[i][2], st[i][3]);      // rows 2t+8, +9   col g
                    const half2 w2 = tc_decode_pair<CB>(st[i][4], st[i][5]);      // rows 2t, 2t+1   col g+8
                    const half2 w3 = tc_decode_pair<CB>(st[i][6], st[i][7]);      // rows 2t+8, +9   col g+8
                    *reinterpret_cast<half2*>(bt + st_off[h + i][0]) = w0;
                    *reinterpret_cast<half2*>(bt + st_off[h + i][1]) = w1;
                    *reinterpret_cast<half2*>(bt + st_off[h + i][0] + 1024) = w2;
                    *reinterpret_cast<half2*>(bt + st_off[h + i][1] + 1024) = w3;
                }
            }
            // make the generic-proxy stores visible to the tensor core's reads, then tell the issuer
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bfull_addr + 8u * sb) : "memory");
                mbar_arrive(&r_empty[sr]);
            }
            sr += NG; if (sr >= SM::SR) { sr -= SM::SR; par_r ^= 1; }
            sb += NG; if (sb >= SM::SB) { sb -= SM::SB; par_b ^= 1; }
        }
    }

    // ===== epilogue (warps 2..17): TMEM -> registers -> output transform -> global.  Each CTA stores its own rows.
    if (warp >= 2 && warp < 2 + TC_DECODERS && !failed) {
        if (!mbar_wait_warp(acc_full, 0)) failed = true;
        if (!failed) {
            tc_fence_after();
            // TMEM lane quadrant q; each of the four warps of a quadrant takes one (M tile, 128-column half) pair
            const int q = warp & 3, mt = (warp - 2) >> 3, sel = ((warp - 2) >> 2) & 1;
            const half* svh_s = reinterpret_cast<const half*>(smem + SM::OFF_SVH) + sel * 128;
            if ((mt == 0 || two_tiles) && sel * 128 < BN && n0 + sel * 128 < n) {
                const int row = (mt ? row_t1 : row_t0) + q * 32 + lane;
                const uint32_t tacc = tmem_base + ((uint32_t)(q * 32) << 16) + mt * BN + sel * 128;
                uint8_t* stage_w = smem + SM::OFF_A + (warp - 2) * 8192;        // 8 KB of the idle activation ring per warp
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
                        if (p.c_fp32) {
                            const size_t off = (size_t)row * n + n0 + sel * 128 + j * 32;
                            const half* sv = svh_s + j * 32;
                            float4* dst = reinterpret_cast<float4*>((float*)Cout + off);
                            #pragma unroll
                            for (int e = 0; e < 32; e += 4) {
                                float4 o = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                                if (svh) {
                                    o.x *= __half2float(sv[e]); o.y *= __half2float(sv[e + 1]);
                                    o.z *= __half2float(sv[e + 2]); o.w *= __half2float(sv[e + 3]);
                                }
                                dst[e >> 2] = o;
                            }
                        }
                    }
                    if (!p.c_fp32) {
                        // fp16 output: this warp's 32 rows x 128 columns go through shared memory (two boxes of 64 columns,
                        // rows of 128 bytes, 16-byte chunks XORed with row & 7) and leave by two tensor stores.  Written
                        // by each thread to its own row, a store instruction touched 32 rows - 32 half-used sectors - and
                        // the 256 such instructions of a CTA took 12 500 cycles, 12 % of a 512-row item.  The activation
                        // and weight rings are free by now: the accumulators are complete.
                        const half* sv = svh_s + j * 32;
                        uint8_t* box = stage_w + (j >> 1) * 4096 + lane * 128;
                        #pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint32_t w[4];
                            #pragma unroll
                            for (int h = 0; h < 4; ++h) {
                                half2 x = __floats2half2_rn(v[e + 2 * h], v[e + 2 * h + 1]);
                                if (svh) x = __hmul2(x, *reinterpret_cast<const half2*>(sv + e + 2 * h));
                                w[h] = *reinterpret_cast<uint32_t*>(&x);
                            }
                            const int chunk = (j & 1) * 4 + (e >> 3);
                            *reinterpret_cast<uint4*>(box + ((chunk ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                        if (j & 1) {                                // a box of 64 columns is complete: it leaves while the next is computed
                            fence_proxy_async();
                            __syncwarp();
                            const int row_w = (mt ? row_t1 : row_t0) + q * 32;          // first row of this warp
                            if (lane == 0 && row_w < p.m) {
                                tma_store_2d(cmap, stage_w + (j >> 1) * 4096, n0 + sel * 128 + (j >> 1) * 64, row_w);
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            }
                        }
                    }
                }
                if (!p.c_fp32) {
                    // the CTA may not leave (and free its shared memory) before the stores have read it
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
                }
            }
        }
    }

    // ===== tear-down: every path arrives here; TMEM is released by the warp that allocated it, and in a pair only after
    // both CTAs are done with their accumulators and with each other's barriers and shared memory
    if (failed) s_failed = 1;
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 2);
}

}  // namespace exl3
