// Paged flash attention on tcgen05 for sequences with many packed (query, head) rows (prefill chunks, wide verify).
//
// One CTA = one work item (sequence, 128-row block, KV split) of one kv head.  K and V tiles of 64 keys come straight
// out of the paged pools by 4-D TMA (a tile never crosses a 256-token page), S = Q K^T and O += P V run on the tensor
// core with S (double-buffered) and O in tensor memory; four softmax warps own one row per thread (TMEM lane), so the
// row maximum and sum need no shuffles.  O is rescaled lazily: the running maximum used in the exponent only moves
// when the true maximum has grown by more than 2^8, which keeps the TMEM read-modify-write of O rare.
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..5 = softmax / epilogue.
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA leaves through the tear-down.
#pragma once
#include "attn_paged.cuh"
#include "gemm_tc.cuh"

namespace exl3 {

constexpr int ATC_ROWS = 128, ATC_TN = 64, ATC_D = 128;
constexpr int ATC_KV_STAGES = 3;
constexpr int ATC_THREADS = 192;
constexpr int ATC_Q_BYTES = ATC_ROWS * ATC_D * 2;             // 32 KB: two 64-wide d blocks of 16 KB
constexpr int ATC_KV_STAGE = 4 * ATC_TN * 128;                // K d0, K d1, V d0, V d1: 8 KB each
constexpr int ATC_P_BYTES = ATC_ROWS * ATC_TN * 2;            // 16 KB
constexpr int ATC_OFF_Q = 0;
constexpr int ATC_OFF_KV = ATC_OFF_Q + ATC_Q_BYTES;
constexpr int ATC_OFF_P = ATC_OFF_KV + ATC_KV_STAGES * ATC_KV_STAGE;
constexpr int ATC_OFF_BAR = ATC_OFF_P + 2 * ATC_P_BYTES;
constexpr int ATC_NBARS = 1 + 3 * ATC_KV_STAGES + 2 + 2 + 2 + 1;    // q_full, k_full/v_full/kv_empty, s_full, p_full, p_empty, o_full
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

constexpr uint32_t ATC_IDESC_S  = (1u << 4) | ((uint32_t)(ATC_TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);            // N = 64 keys
constexpr uint32_t ATC_IDESC_PV = (1u << 4) | (1u << 16) | ((uint32_t)(ATC_D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24); // B MN-major, N = 128


// grid (max_items, nkv); kmap / vmap: 4-D maps of the pools {D, nkv, 256, pages}, box {64, 1, 64, 1}, 128B swizzle
__global__ void __launch_bounds__(ATC_THREADS, 1) attn_tc_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                const __grid_constant__ CUtensorMap vmap, const AttnParams p)
{
    const int item_idx = blockIdx.x;
    if (item_idx >= p.plan->n_items) return;
    extern __shared__ uint8_t smem_unaligned[];
    // aligned to 1024 bytes by an offset from the array, not through an integer, so that the compiler still knows the
    // pointer is in shared memory (32-bit addresses, ld/st.shared) instead of falling back to generic accesses
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ATC_OFF_BAR);
    uint64_t* q_full = bars;
    uint64_t* k_full = q_full + 1;                 uint64_t* v_full = k_full + ATC_KV_STAGES;
    uint64_t* kv_empty = v_full + ATC_KV_STAGES;   uint64_t* s_full = kv_empty + ATC_KV_STAGES;
    uint64_t* p_full = s_full + 2;                 uint64_t* p_empty = p_full + 2;
    uint64_t* o_full = p_empty + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
    __shared__ int s_failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y;
    const int G = p.nq / p.nkv;
    const int chunk = p.plan->chunk;
    const AttnItem item = p.items[item_idx];
    const int b = item.b;
    const int row_base = p.cu_q ? p.cu_q[b] : b * p.q_len;
    const int ql = p.cu_q ? p.cu_q[b + 1] - row_base : p.q_len;
    const int total_k = p.seqlens[b] + (p.cu_q ? ql : p.kv_append);
    const int splits = p.seq_splits[b];
    const int r0 = item.rb * ATC_ROWS;
    const int i_last = min(ql - 1, (r0 + ATC_ROWS - 1) / G);
    const int vis_max = p.causal ? min(total_k, total_k - ql + i_last + 1) : total_k;
    const int k_begin = item.split * chunk;
    const int k_end = min(min(k_begin + chunk, total_k), vis_max);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + ATC_TN - 1) / ATC_TN : 0;
    const int32_t* bt = p.block_table + (size_t)b * p.pps;

    if (tid == 0) {
        s_failed = 0;
        mbar_init(q_full, 4);
        for (int i = 0; i < ATC_KV_STAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&kv_empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&p_empty[i], 1); }
        mbar_init(o_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 2 * ATC_TN;
    bool failed = false;

    if (warp == 0) {
        // ===== producer: K and V tiles by TMA out of the paged pools
        if (lane == 0) {
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % ATC_KV_STAGES;
                if (j >= ATC_KV_STAGES && !mbar_wait(&kv_empty[s], ((j / ATC_KV_STAGES) - 1) & 1)) { failed = true; break; }
                const int k0 = k_begin + j * ATC_TN;
                const int page = bt[k0 >> 8], tok = k0 & 255;
                uint8_t* st = smem + ATC_OFF_KV + s * ATC_KV_STAGE;
                mbar_expect_tx(&k_full[s], 2 * ATC_TN * 128);
                tma_load_4d(st, &kmap, 0, kvh, tok, page, &k_full[s]);
                tma_load_4d(st + ATC_TN * 128, &kmap, 64, kvh, tok, page, &k_full[s]);
                mbar_expect_tx(&v_full[s], 2 * ATC_TN * 128);
                tma_load_4d(st + 2 * ATC_TN * 128, &vmap, 0, kvh, tok, page, &v_full[s]);
                tma_load_4d(st + 3 * ATC_TN * 128, &vmap, 64, kvh, tok, page, &v_full[s]);
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer
        if (lane == 0 && n_tiles > 0) {
            auto issue_s = [&](int j) -> bool {
                const int s = j % ATC_KV_STAGES;
                if (!mbar_wait(&k_full[s], (j / ATC_KV_STAGES) & 1)) return false;
                tc_fence_after();
                const uint8_t* kst = smem + ATC_OFF_KV + s * ATC_KV_STAGE;
                #pragma unroll
                for (int kk = 0; kk < ATC_D / 16; ++kk) {
                    const uint64_t ad = tc_smem_desc(smem + ATC_OFF_Q + (kk >> 2) * (ATC_ROWS * 128) + (kk & 3) * 32);
                    const uint64_t bd = tc_smem_desc(kst + (kk >> 2) * (ATC_TN * 128) + (kk & 3) * 32);
                    tc_mma_f16(tmem_base + (j & 1) * ATC_TN, ad, bd, ATC_IDESC_S, kk > 0 ? 1u : 0u);
                }
                tc_commit(&s_full[j & 1]);
                return true;
            };
            if (!mbar_wait(q_full, 0)) failed = true;
            if (!failed && !issue_s(0)) failed = true;
            if (!failed && n_tiles > 1 && !issue_s(1)) failed = true;
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int s = j % ATC_KV_STAGES;
                if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1) || !mbar_wait(&v_full[s], (j / ATC_KV_STAGES) & 1)) { failed = true; break; }
                tc_fence_after();
                const uint8_t* vst = smem + ATC_OFF_KV + s * ATC_KV_STAGE + 2 * ATC_TN * 128;
                #pragma unroll
                for (int kk = 0; kk < ATC_TN / 16; ++kk) {
                    const uint64_t ad = tc_smem_desc(smem + ATC_OFF_P + (j & 1) * ATC_P_BYTES + kk * 32);
                    const uint64_t bd = tc_smem_desc_mn(vst + kk * 2048, ATC_TN * 128);
                    tc_mma_f16(tmem_o, ad, bd, ATC_IDESC_PV, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tc_commit(&kv_empty[s]);
                tc_commit(&p_empty[j & 1]);
                if (j + 2 < n_tiles && !issue_s(j + 2)) { failed = true; break; }
            }
            if (!failed) tc_commit(o_full);
        }
    } else {
        // ===== softmax warps: one packed (query, head) row per thread
        const int q = warp & 3;
        const int lr = q * 32 + lane;
        const int row = r0 + lr;
        const int qidx = row / G;
        const bool valid = row < ql * G;
        const int head = kvh * G + (row - qidx * G);
        const int lim = valid ? (p.causal ? min(total_k, total_k - ql + qidx + 1) : total_k) : 0;
        {   // Q row -> shared memory in the K-major 128B-swizzled operand layout (two 64-wide d blocks)
            const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)(row_base + qidx) * p.nq + head) * ATC_D);
            #pragma unroll
            for (int c = 0; c < 16; ++c) {
                const uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(smem + ATC_OFF_Q + (c >> 3) * (ATC_ROWS * 128) + lr * 128 + (((c & 7) ^ (lr & 7)) << 4)) = v;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        float m_used = -INFINITY, m_true = -INFINITY, l_run = 0.f;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        for (int j = 0; j < n_tiles; ++j) {
            if (!mbar_wait_warp(&s_full[j & 1], (j >> 1) & 1)) { failed = true; break; }
            tc_fence_after();
            float sv[ATC_TN];
            {
                float part[32];
                tc_ld32(tmem_base + lane_addr + (j & 1) * ATC_TN, part);
                tc_wait_ld();
                #pragma unroll
                for (int e = 0; e < 32; ++e) sv[e] = part[e];
                tc_ld32(tmem_base + lane_addr + (j & 1) * ATC_TN + 32, part);
                tc_wait_ld();
                #pragma unroll
                for (int e = 0; e < 32; ++e) sv[32 + e] = part[e];
            }
            const int kbase = k_begin + j * ATC_TN;
            const int nvis = min(lim, k_end) - kbase;            // keys of this tile the row may see (may be <= 0)
            float mx = -INFINITY;
            if (nvis >= ATC_TN) {
                #pragma unroll
                for (int e = 0; e < ATC_TN; ++e) { sv[e] *= p.scale_log2; mx = fmaxf(mx, sv[e]); }
            } else {
                #pragma unroll
                for (int e = 0; e < ATC_TN; ++e) { sv[e] = e < nvis ? sv[e] * p.scale_log2 : -INFINITY; mx = fmaxf(mx, sv[e]); }
            }
            m_true = fmaxf(m_true, mx);
            // lazy reference update: this row moves its reference when the true maximum ran ahead by more than the
            // threshold (or when it sees its first key); rows that already contributed to O rescale their O row.
            const bool move = m_true > m_used + ATC_RESCALE_THRESHOLD || (m_used == -INFINITY && m_true > -INFINITY);
            const bool rescale = move && m_used != -INFINITY && j > 0;
            if (__any_sync(0xffffffffu, rescale)) {
                // the TMEM accesses are warp-wide; rows that do not rescale multiply by 1.  PV(j-1) must have finished.
                if (!mbar_wait_warp(&p_empty[(j - 1) & 1], ((j - 1) >> 1) & 1)) { failed = true; break; }
                tc_fence_after();
                const float corr = rescale ? exp2f(m_used - m_true) : 1.0f;
                #pragma unroll
                for (int c = 0; c < ATC_D / 32; ++c) {
                    float part[32];
                    tc_ld32(tmem_o + lane_addr + c * 32, part);
                    tc_wait_ld();
                    #pragma unroll
                    for (int e = 0; e < 32; ++e) part[e] *= corr;
                    tc_st32(tmem_o + lane_addr + c * 32, part);
                }
                tc_wait_st();
                l_run *= corr;
            }
            if (move) m_used = m_true;
            // the last tile of a split may reach past the end of the sequence: those V rows hold whatever is in the pool
            // (possibly NaN bit patterns), and 0 * NaN would poison O, so they are cleared before PV reads them
            if (kbase + ATC_TN > k_end) {
                const int sj = j % ATC_KV_STAGES;
                if (!mbar_wait_warp(&v_full[sj], (j / ATC_KV_STAGES) & 1)) { failed = true; break; }
                uint8_t* vst = smem + ATC_OFF_KV + sj * ATC_KV_STAGE + 2 * ATC_TN * 128;
                const int first_bad = k_end - kbase;                        // 1..63
                for (int i = (warp - 2) * 32 + lane; i < (ATC_TN - first_bad) * 16; i += 128) {
                    const int key = first_bad + (i >> 4), c = i & 15;      // 16 chunks of 16 bytes per key over both d blocks
                    *reinterpret_cast<uint4*>(vst + (c >> 3) * (ATC_TN * 128) + key * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
            }
            const float mref = (m_used == -INFINITY) ? 0.f : m_used;
            if (j >= 2 && !mbar_wait_warp(&p_empty[j & 1], ((j >> 1) - 1) & 1)) { failed = true; break; }
            uint8_t* prow = smem + ATC_OFF_P + (j & 1) * ATC_P_BYTES + lr * 128;
            #pragma unroll
            for (int c = 0; c < ATC_TN / 8; ++c) {
                uint32_t w[4];
                #pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float e0 = exp2f(sv[c * 8 + 2 * h] - mref), e1 = exp2f(sv[c * 8 + 2 * h + 1] - mref);
                    l_run += e0 + e1;
                    w[h] = pack_h2(e0, e1);
                }
                *reinterpret_cast<uint4*>(prow + ((c ^ (lr & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[j & 1]);
        }
        // ===== epilogue: O (TMEM) -> output or split-KV partial
        failed = __any_sync(0xffffffffu, failed);
        if (!failed) {
            float ov[ATC_D];
            if (n_tiles > 0) {
                if (!mbar_wait_warp(o_full, 0)) failed = true;
                tc_fence_after();
                if (!failed) {
                    #pragma unroll
                    for (int c = 0; c < ATC_D / 32; ++c) {
                        float part[32];
                        tc_ld32(tmem_o + lane_addr + c * 32, part);
                        tc_wait_ld();
                        #pragma unroll
                        for (int e = 0; e < 32; ++e) ov[c * 32 + e] = part[e];
                    }
                }
            } else {
                #pragma unroll
                for (int e = 0; e < ATC_D; ++e) ov[e] = 0.f;
            }
            if (!failed && valid) {
                if (splits == 1) {
                    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
                    uint4* dst = reinterpret_cast<uint4*>(p.o + ((size_t)(row_base + qidx) * p.nq + head) * ATC_D);
                    #pragma unroll
                    for (int c = 0; c < 16; ++c)
                        dst[c] = make_uint4(pack_h2(ov[c * 8] * inv, ov[c * 8 + 1] * inv), pack_h2(ov[c * 8 + 2] * inv, ov[c * 8 + 3] * inv),
                                            pack_h2(ov[c * 8 + 4] * inv, ov[c * 8 + 5] * inv), pack_h2(ov[c * 8 + 6] * inv, ov[c * 8 + 7] * inv));
                } else {
                    float* pp = p.partial + (((size_t)item_idx * p.nkv + kvh) * ATC_ROWS + lr) * (ATC_D + 2);
                    #pragma unroll
                    for (int e = 0; e < ATC_D; e += 2) *reinterpret_cast<float2*>(pp + e) = make_float2(ov[e], ov[e + 1]);
                    pp[ATC_D] = m_used; pp[ATC_D + 1] = l_run;
                }
            }
        }
    }

    if (failed) s_failed = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 3);
}

}  // namespace exl3
