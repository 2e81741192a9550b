// Paged flash attention on tcgen05 for sequences with many packed (query, head) rows (prefill chunks, wide verify).
//
// One CTA = one work item (sequence, 256-row block, KV split) of one kv head.  The 256 rows are two blocks of 128 (the
// TMEM lane count) that share every K/V tile and take turns on the tensor core: while it computes S or PV for one block,
// the softmax warps of the other block work.  K and V tiles of 128 keys come straight out of the paged pools by 4-D TMA
// (a tile never crosses a 256-token page) through one ring of five 32 KB buffers (K0 V0 K1 V1 ...).  S = Q K^T (one
// 128-column buffer per block) and O += P V live in tensor memory (2 x 128 + 2 x 128 = 512 columns); P is written
// back as packed fp16 over the last 64 columns of its S buffer and is the A operand of the PV MMA straight from
// tensor memory, so it costs no shared-memory traffic and no proxy fence.  Four softmax warps per block own one row
// per thread (TMEM lane), so the row maximum and sum need no shuffles.  O is rescaled lazily: the running maximum used in the exponent only moves when the true maximum
// has grown by more than 2^8, which keeps the TMEM read-modify-write of O rare.
// All MMAs are 128 x 128 x 16 (64 tensor-core cycles): the issue cost of one tcgen05.mma from a single thread was
// measured at about 65 cycles, which smaller MMAs (64-key tiles) cannot hide.
// Roles by warpgroup: warps 0..3 = softmax / epilogue of block 0, warps 4..7 = the same for block 1, warp 8 = TMA
// producer, warp 9 = MMA issuer and TMEM owner (10 and 11 idle).  The service warpgroup hands most of its registers
// to the softmax warpgroups (setmaxnreg), which need over 200 to keep 64 scores and their exponentials in flight.
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA leaves through the tear-down.
#pragma once
#include "attn_paged.cuh"
#include "gemm_tc.cuh"

namespace exl3 {

constexpr int ATC_ROWS = 128, ATC_NB = 2, ATC_CTA_ROWS = ATC_ROWS * ATC_NB, ATC_TN = 128, ATC_D = 128;
constexpr int ATC_KV_SLOTS = 5;                               // ring of K / V tile buffers
constexpr int ATC_THREADS = ATC_NB * 128 + 128;                // two softmax warpgroups + one service warpgroup
constexpr int ATC_Q_BYTES = ATC_ROWS * ATC_D * 2;             // per block, 32 KB: two 64-wide d blocks of 16 KB
constexpr int ATC_KV_SLOT = ATC_TN * ATC_D * 2;               // one K or V tile, 32 KB: two 64-wide d blocks of 16 KB
constexpr int ATC_OFF_Q = 0;
constexpr int ATC_OFF_KV = ATC_OFF_Q + ATC_NB * ATC_Q_BYTES;
constexpr int ATC_OFF_BAR = ATC_OFF_KV + ATC_KV_SLOTS * ATC_KV_SLOT;
// q_full[NB], kv_full/kv_empty[slots], s_full[NB], p_full[NB], o_full
constexpr int ATC_NBARS = ATC_NB + 2 * ATC_KV_SLOTS + 2 * ATC_NB + 1;
constexpr int ATC_SMEM = ATC_OFF_BAR + ATC_NBARS * 8 + 16 + 1024;
constexpr float ATC_RESCALE_THRESHOLD = 8.0f;                 // log2 units

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float (&v)[32])
{
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major (N contiguous), 128-byte swizzled B tile: 64-element N atoms `lbo` bytes apart, 8-row K groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_smem_desc_mn(const void* p, uint32_t lbo)
{
    const uint32_t a = smem_u32(p);
    uint64_t d = 0;
    d |= (uint64_t)((a >> 4) & 0x3fff);
    d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

constexpr uint32_t ATC_IDESC_S  = (1u << 4) | ((uint32_t)(ATC_TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);            // N = 128 keys
constexpr uint32_t ATC_IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(ATC_D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); // B MN-major, N = 128



// D[tmem] (+)= A[tmem, packed fp16] * B[smem desc]
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_st32u(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}

__device__ __forceinline__ void tc_st16u(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two exponentials per special-function operation: 2^x of an fp16 pair (the result is used as fp16 anyway)
__device__ __forceinline__ uint32_t ex2_h2(uint32_t x)
{
    uint32_t y;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
#ifndef ATC_EXP_F16X2
#define ATC_EXP_F16X2 0
#endif
// registers of a softmax thread / of a service thread after the split: 256 x 184 + 128 x 120 <= 64 K.  (Holding all 128
// scores of a row through the maximum and both exponential passes - one TMEM read and one wait per tile instead of
// three - needs about 230 registers; at 184 it spills and ran at 278 us against 162 us on 4 x 256 query rows.)
#define ATC_REG_SOFTMAX 184
#define ATC_REG_SERVICE 120
__device__ __forceinline__ float fmax3(float a, float b, float c)
{
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}


// grid (max_items, nkv); kmap / vmap: 4-D maps of the pools {D, nkv, 256, pages}, box {64, 1, 128, 1}, 128B swizzle.
// The plan's chunk must be a multiple of 128 keys.
__global__ void __launch_bounds__(ATC_THREADS, 1) attn_tc_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                const __grid_constant__ CUtensorMap vmap, const AttnParams p)
{
    // grid max_items * nkv: the CTAs of one item are neighbours in launch order, items come longest first
    if ((int)(blockIdx.x / p.nkv) >= p.plan->n_items) return;
    const int item_idx = p.order[blockIdx.x / p.nkv];
    extern __shared__ uint8_t smem_unaligned[];
    // aligned to 1024 bytes by an offset from the array, not through an integer, so that the compiler still knows the
    // pointer is in shared memory (32-bit addresses, ld/st.shared) instead of falling back to generic accesses
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ATC_OFF_BAR);
    uint64_t* q_full = bars;                               // [NB]
    uint64_t* kv_full = q_full + ATC_NB;                   uint64_t* kv_empty = kv_full + ATC_KV_SLOTS;
    uint64_t* s_full = kv_empty + ATC_KV_SLOTS;            // [NB]
    uint64_t* p_full = s_full + ATC_NB;
    uint64_t* o_full = p_full + ATC_NB;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
    __shared__ int s_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x % p.nkv;
    const int G = p.nq / p.nkv;
    const int chunk = p.plan->chunk;
    const AttnItem item = p.items[item_idx];
    const int b = item.b;
    const int row_base = p.cu_q ? p.cu_q[b] : b * p.q_len;
    const int ql = p.cu_q ? p.cu_q[b + 1] - row_base : p.q_len;
    const int total_k = p.seqlens[b] + (p.cu_q ? ql : p.kv_append);
    const int splits = p.seq_splits[b];
    const int r0 = item.rb * ATC_CTA_ROWS;
    const int i_last = min(ql - 1, (r0 + ATC_CTA_ROWS - 1) / G);
    const int vis_max = p.causal ? min(total_k, total_k - ql + i_last + 1) : total_k;
    const int k_begin = item.split * chunk;
    const int k_end = min(min(k_begin + chunk, total_k), vis_max);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + ATC_TN - 1) / ATC_TN : 0;
    const int32_t* bt = p.block_table + (size_t)b * p.pps;
    // the second block is skipped when the item's rows end inside the first one
    const int nb = (ql * G - r0 > ATC_ROWS) ? 2 : 1;

    if (tid == 0) {
        s_failed = 0;
        for (int i = 0; i < ATC_NB; ++i) {
            mbar_init(&q_full[i], 4); mbar_init(&p_full[i], 4); mbar_init(&s_full[i], 1);
        }
        for (int i = 0; i < ATC_KV_SLOTS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
        mbar_init(o_full, 1);
        mbar_fence_init();
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;             // S of block i: columns i*128 (P over its last 64); O of block i: 256 + i*128
    bool failed = false;

    if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ATC_REG_SERVICE));
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(ATC_REG_SOFTMAX));
    if (warp == 8) {
        // ===== producer: K and V tiles by TMA out of the paged pools; ring item 2j = K of tile j, 2j+1 = V of tile j
        if (lane == 0) {
            for (int it = 0; it < 2 * n_tiles; ++it) {
                const int slot = it % ATC_KV_SLOTS;
                if (it >= ATC_KV_SLOTS && !mbar_wait_sleep(&kv_empty[slot], ((it / ATC_KV_SLOTS) - 1) & 1)) { failed = true; break; }
                const int k0 = k_begin + (it >> 1) * ATC_TN;
                const int page = bt[k0 >> 8], tok = k0 & 255;
                uint8_t* st = smem + ATC_OFF_KV + slot * ATC_KV_SLOT;
                const CUtensorMap* map = (it & 1) ? &vmap : &kmap;
                mbar_expect_tx(&kv_full[slot], ATC_KV_SLOT);
                tma_load_4d(st, map, 0, kvh, tok, page, &kv_full[slot]);
                tma_load_4d(st + ATC_TN * 128, map, 64, kvh, tok, page, &kv_full[slot]);
            }
        }
    } else if (warp == 9) {
        // ===== MMA issuer: after P(j) of a block is ready, S(j+1) then PV(j) of that block; the two blocks interleave.
        // The whole warp runs the loop with warp-uniform values (so that descriptors and addresses can live in uniform
        // registers, which is where tcgen05.mma takes them from); one elected lane issues.
        if (n_tiles > 0) {
            const bool leader = elect_one();
            constexpr uint32_t HI_K = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);   // SBO, version 1, SWIZZLE_128B
            constexpr uint32_t LBO_K = 1u << 16;                                          // K-major: unused, 1 as CUTLASS sets
            constexpr uint32_t LBO_V = (uint32_t)((ATC_TN * 128) >> 4) << 16;             // MN-major: the next 64-wide d atom
            auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            const uint32_t q_lo = (smem_u32(smem + ATC_OFF_Q) >> 4) | LBO_K;
            const uint32_t kv_lo = smem_u32(smem + ATC_OFF_KV) >> 4;
            // An MMA of 128 x 128 x 16 is issued every 65 cycles or so whatever its N (measured; with both operands in
            // shared memory it reads 8 KB, which is also about 64 cycles of the SM's shared-memory bandwidth).
            auto s_mma = [&](int blk, int slot, int kk) {
                const uint32_t a0 = q_lo + blk * (ATC_Q_BYTES >> 4), b0 = (kv_lo + slot * (ATC_KV_SLOT >> 4)) | LBO_K;
                const uint32_t ao = ((kk >> 2) * (ATC_ROWS * 128) + (kk & 3) * 32) >> 4;
                const uint32_t bo = ((kk >> 2) * (ATC_TN * 128) + (kk & 3) * 32) >> 4;
                tc_mma_f16(tmem_base + blk * 128, mk(a0 + ao, HI_K), mk(b0 + bo, HI_K), ATC_IDESC_S, kk > 0 ? 1u : 0u);
            };
            // P(blk): 128 lanes x 64 columns (64..127 of the S buffer) of packed fp16 pairs, 8 columns per K step of 16 keys
            auto pv_mma = [&](int blk, int slot, int kk, bool acc) {
                const uint32_t b0 = (kv_lo + slot * (ATC_KV_SLOT >> 4)) | LBO_V;
                tc_mma_f16_ts(tmem_base + 256 + blk * 128, tmem_base + blk * 128 + 64 + kk * 8, mk(b0 + kk * (2048 >> 4), HI_K), ATC_IDESC_PV, acc ? 1u : 0u);
            };
            for (int blk = 0; blk < nb && !failed; ++blk)
                if (!mbar_wait_sleep_warp(&q_full[blk], 0)) failed = true;
            if (!failed && !mbar_wait_sleep_warp(&kv_full[0], 0)) failed = true;        // K of tile 0: ring item 0
            if (!failed) {
                tc_fence_after();
                if (leader) {
                    for (int blk = 0; blk < nb; ++blk) {
                        #pragma unroll
                        for (int kk = 0; kk < ATC_D / 16; ++kk) s_mma(blk, 0, kk);
                        tc_commit(&s_full[blk]);
                    }
                    tc_commit(&kv_empty[0]);
                }
                __syncwarp();
            }
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int itv = 2 * j + 1, slot_v = itv % ATC_KV_SLOTS;                  // V of tile j
                const int itk = 2 * j + 2, slot_k = itk % ATC_KV_SLOTS;                  // K of tile j + 1
                const bool more = j + 1 < n_tiles;
                for (int blk = 0; blk < nb; ++blk) {
                    if (!mbar_wait_warp(&p_full[blk], j & 1)) { failed = true; break; }     // plain polls: a sleeping wait wakes up hundreds of cycles late
                    if (blk == 0 && (!mbar_wait_sleep_warp(&kv_full[slot_v], (itv / ATC_KV_SLOTS) & 1) ||
                                     (more && !mbar_wait_sleep_warp(&kv_full[slot_k], (itk / ATC_KV_SLOTS) & 1)))) { failed = true; break; }
                    tc_fence_after();
                    if (leader) {
                        // PV(j) reads P(j) out of the S buffer before S(j+1) overwrites it: the tensor core runs them in order
                        #pragma unroll
                        for (int kk = 0; kk < ATC_TN / 16; ++kk) pv_mma(blk, slot_v, kk, j > 0 || kk > 0);
                        if (blk == nb - 1) tc_commit(&kv_empty[slot_v]);
                        if (more) {
                            #pragma unroll
                            for (int kk = 0; kk < ATC_D / 16; ++kk) s_mma(blk, slot_k, kk);
                            tc_commit(&s_full[blk]);                 // also means PV(j) is done: O may be rescaled
                            if (blk == nb - 1) tc_commit(&kv_empty[slot_k]);
                        }
                    }
                    __syncwarp();
                }
            }
            if (!failed && leader) tc_commit(o_full);
        }
    } else if (warp < 8 && (warp >> 2) < nb) {
        // ===== softmax warps: one packed (query, head) row per thread
        const int blk = warp >> 2;
        const int q = warp & 3;                                  // TMEM lane quadrant this warp may access
        const int lr = q * 32 + lane;                            // row inside the block
        const int row = r0 + blk * ATC_ROWS + lr;
        const int qidx = row / G;
        const bool valid = row < ql * G;
        const int head = kvh * G + (row - qidx * G);
        const int lim = valid ? (p.causal ? min(total_k, total_k - ql + qidx + 1) : total_k) : 0;
        {   // Q row -> shared memory in the K-major 128B-swizzled operand layout (two 64-wide d blocks)
            const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)(row_base + qidx) * p.nq + head) * ATC_D);
            uint8_t* qs = smem + ATC_OFF_Q + blk * ATC_Q_BYTES;
            #pragma unroll
            for (int c = 0; c < 16; ++c) {
                const uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(qs + (c >> 3) * (ATC_ROWS * 128) + lr * 128 + (((c & 7) ^ (lr & 7)) << 4)) = v;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_full[blk]);
        }
        float m_used = -INFINITY, m_true = -INFINITY, l_run = 0.f;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const uint32_t tmem_s = tmem_base + lane_addr + blk * 128;
        const uint32_t tmem_o = tmem_base + lane_addr + 256 + blk * 128;
        const float scale = p.scale_log2;
        // one 64-key half of the S tile: TMEM -> registers, masked
        auto load_half = [&](int h, int nvis, float (&sv)[64]) {
            float (&lo)[32] = *reinterpret_cast<float (*)[32]>(&sv[0]);
            float (&hi)[32] = *reinterpret_cast<float (*)[32]>(&sv[32]);
            tc_ld32(tmem_s + h * 64, lo);
            tc_ld32(tmem_s + h * 64 + 32, hi);
            tc_wait_ld();
            if (nvis < (h + 1) * 64) {
                #pragma unroll
                for (int e = 0; e < 64; ++e) sv[e] = h * 64 + e < nvis ? sv[e] : -INFINITY;
            }
        };
        auto half_max = [&](const float (&sv)[64]) {
            float mx0 = -INFINITY, mx1 = -INFINITY;
            #pragma unroll
            for (int e = 0; e < 64; e += 4) { mx0 = fmax3(mx0, sv[e], sv[e + 1]); mx1 = fmax3(mx1, sv[e + 2], sv[e + 3]); }
            return fmaxf(mx0, mx1);
        };
        // P = 2^(s * scale - m_used) as fp16 pairs, summed in fp32 (masked scores are -inf and give 0)
        auto half_exp = [&](const float (&sv)[64], float nref, uint32_t (&pw)[32], float& l0, float& l1) {
#if ATC_EXP_F16X2
            // The exponent s * scale - m is formed in fp32 and rounded to fp16 (it lies in (-inf, threshold]: a rounding
            // step of 2^-11 |x| moves 2^x by the factor 2^(2^-11 |x|), i.e. by at most 2.6e-4 of the row's largest
            // weight, the size of P's own fp16 rounding).  The special-function unit then takes both exponentials of a
            // pair in one operation - it has 16 lanes per SM against 128 exponentials per row and tile - and returns
            // them already packed.  Row sums: groups of four pairs are added in fp16 (at most 2^11), then in fp32.
            #pragma unroll
            for (int e = 0; e < 64; e += 8) {
                __half2 acc = __float2half2_rn(0.f);
                #pragma unroll
                for (int u = 0; u < 8; u += 2) {
                    const uint32_t w = ex2_h2(pack_h2(fmaf(sv[e + u], scale, nref), fmaf(sv[e + u + 1], scale, nref)));
                    pw[(e + u) >> 1] = w;
                    acc = __hadd2(acc, *reinterpret_cast<const __half2*>(&w));
                }
                l0 += __low2float(acc); l1 += __high2float(acc);
            }
#else
            #pragma unroll
            for (int e = 0; e < 64; e += 2) {
                const float e0 = ex2_approx(fmaf(sv[e], scale, nref)), e1 = ex2_approx(fmaf(sv[e + 1], scale, nref));
                l0 += e0; l1 += e1;
                pw[e >> 1] = pack_h2(e0, e1);
            }
#endif
        };
        for (int j = 0; j < n_tiles; ++j) {
            if (!mbar_wait_warp(&s_full[blk], j & 1)) { failed = true; break; }
            tc_fence_after();
            const int kbase = k_begin + j * ATC_TN;
            const int nvis = min(lim, k_end) - kbase;            // keys of this tile the row may see (may be <= 0)
            // The row maximum needs all 128 scores, the exponentials are then taken half by half: the second half stays
            // in registers from the maximum pass, the first is read from TMEM again (cheaper than holding 128 scores).
            float sv[64];
            load_half(0, nvis, sv);
            const float mxa = half_max(sv);                      // raw scores: the scale is positive, so max commutes with it
            load_half(1, nvis, sv);
            m_true = fmaxf(m_true, fmaxf(mxa, half_max(sv)) * scale);
            // lazy reference update: this row moves its reference when the true maximum ran ahead by more than the
            // threshold (or when it sees its first key); rows that already contributed to O rescale their O row.
            const bool move = m_true > m_used + ATC_RESCALE_THRESHOLD || (m_used == -INFINITY && m_true > -INFINITY);
            const bool rescale = move && m_used != -INFINITY && j > 0;
            const float corr = rescale ? ex2_approx(m_used - m_true) : 1.0f;
            if (move) m_used = m_true;
            const float nref = (m_used == -INFINITY) ? 0.f : -m_used;
            // P goes over the SECOND half of the S buffer (columns 64..127, column 64 + c = keys 2c, 2c+1): that half is
            // already in registers, so its exponentials can be stored before the first half is read again, and no more
            // than 64 scores and 32 packed words are live at a time.
            uint32_t pw[32];
            float l0 = 0.f, l1 = 0.f;
            half_exp(sv, nref, pw, l0, l1);
            tc_st32u(tmem_s + 64 + 32, pw);
            load_half(0, nvis, sv);
            half_exp(sv, nref, pw, l0, l1);
            tc_st32u(tmem_s + 64, pw);
            if (__any_sync(0xffffffffu, rescale)) {
                // PV(j-1) is complete: S(j) was committed after it.  The TMEM accesses are warp-wide; rows that do not
                // rescale multiply by 1.
                tc_fence_after();
                #pragma unroll
                for (int c = 0; c < ATC_D / 32; ++c) {
                    float part[32];
                    tc_ld32(tmem_o + c * 32, part);
                    tc_wait_ld();
                    #pragma unroll
                    for (int e = 0; e < 32; ++e) part[e] *= corr;
                    tc_st32(tmem_o + c * 32, part);
                }
                tc_wait_st();
            }
            l_run = l_run * corr + (l0 + l1);
            // the last tile of a split may reach past the end of the sequence: those V rows hold whatever is in the pool
            // (possibly NaN bit patterns), and 0 * NaN would poison O, so they are cleared before PV reads them.  Block 0
            // does it: its P is waited for first, and the tensor core runs the PV of block 1 after that of block 0.
            if (blk == 0 && kbase + ATC_TN > k_end) {
                const int it = 2 * j + 1, slot = it % ATC_KV_SLOTS;
                if (!mbar_wait_sleep_warp(&kv_full[slot], (it / ATC_KV_SLOTS) & 1)) { failed = true; break; }
                uint8_t* vst = smem + ATC_OFF_KV + slot * ATC_KV_SLOT;
                const int first_bad = k_end - kbase;                        // 1..127
                for (int i = lr; i < (ATC_TN - first_bad) * 16; i += 128) {
                    const int key = first_bad + (i >> 4), c = i & 15;      // 16 chunks of 16 bytes per key over both d blocks
                    *reinterpret_cast<uint4*>(vst + (c >> 3) * (ATC_TN * 128) + key * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[blk]);
        }
        // ===== epilogue: O (TMEM) -> output or split-KV partial, 32 columns at a time
        failed = __any_sync(0xffffffffu, failed);
        if (!failed && n_tiles > 0 && !mbar_wait_sleep_warp(o_full, 0)) failed = true;
        if (!failed) {
            tc_fence_after();
            const float inv = (splits == 1) ? (l_run > 0.f ? 1.0f / l_run : 0.f) : 1.0f;
            half* orow = p.o + ((size_t)(row_base + qidx) * p.nq + head) * ATC_D;
            float* pp = p.partial + (((size_t)item_idx * p.nkv + kvh) * ATC_CTA_ROWS + blk * ATC_ROWS + lr) * (ATC_D + 2);
            #pragma unroll 1
            for (int c = 0; c < ATC_D / 32; ++c) {
                float ov[32];
                if (n_tiles > 0) {
                    tc_ld32(tmem_o + c * 32, ov);
                    tc_wait_ld();
                } else {
                    #pragma unroll
                    for (int e = 0; e < 32; ++e) ov[e] = 0.f;
                }
                if (valid) {
                    if (splits == 1) {
                        uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
                        #pragma unroll
                        for (int e = 0; e < 4; ++e)
                            dst[e] = make_uint4(pack_h2(ov[e * 8] * inv, ov[e * 8 + 1] * inv), pack_h2(ov[e * 8 + 2] * inv, ov[e * 8 + 3] * inv),
                                                pack_h2(ov[e * 8 + 4] * inv, ov[e * 8 + 5] * inv), pack_h2(ov[e * 8 + 6] * inv, ov[e * 8 + 7] * inv));
                    } else {
                        #pragma unroll
                        for (int e = 0; e < 32; e += 2) *reinterpret_cast<float2*>(pp + c * 32 + e) = make_float2(ov[e], ov[e + 1]);
                    }
                }
            }
            if (valid && splits != 1) { pp[ATC_D] = m_used; pp[ATC_D + 1] = l_run; }
        }
    }

    if (failed) s_failed = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 3);
}

}  // namespace exl3
