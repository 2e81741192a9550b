// Paged flash attention on tcgen05, second arrangement: one CTA = one work item (sequence, 128-row block, KV split) of one
// kv head, H = 2 or 4 softmax threads per row and a double-buffered S.
//
// Why.  In the 256-row kernel (attn_tc.cuh) a softmax thread owns a whole row of a 128-key tile: it reads its 128 scores
// from tensor memory in three round trips (the row maximum needs all of them, registers hold 64) and takes 128
// exponentials, and the tensor core idles through that (tensor pipe 34 % busy, long-scoreboard stalls 4.3 per issued
// instruction).  Here the H threads of a row take 128 / H keys each: one round trip, the row maximum and sum exchanged
// through shared memory between the H warps that share a TMEM lane quadrant.  S has two buffers, so S(j+1) = Q K(j+1)^T is
// computed while the threads work on tile j, and PV(j) follows as soon as P(j) is written.
//
// Measured per tile in steady state (clock64 in one CTA, 8192-key context): 2150 cycles, the same for H = 2 and H = 4:
// row maximum 200, rendezvous of the row's warps 200, exponentials 1250 (the special-function unit's 16 per clock and SM
// would allow 1024), P store 140, wait for and request of the next scores 220, loop 140; the issuer sees P 375 cycles
// after it was announced and needs 410 + 710 cycles to issue PV(j) and S(j+2).  The tensor core (1024 cycles of work per
// tile) is never what the softmax threads wait for.  Four 256-row chunks, 145 us: about half of that is the tile loop,
// the rest the start and end of each CTA (4.2 CTAs per SM) and, before the work list was ordered longest first, the tail.
//
// TMEM: S0 columns 0..127, S1 128..255 (P of a tile over the last 64 columns of its S buffer, packed fp16), O 256..383.
// Warps 0..4H-1: softmax, lane quadrant = warp % 4, key part = warp / 4; then the TMA producer and the MMA issuer (which
// owns the TMEM allocation).  K/V tiles by 4-D TMA out of the paged pools through a ring of five 32 KB buffers in the
// order the issuer consumes them: K0 K1 V0 K2 V1 K3 ...  Every wait is bounded; a wait that runs out sets the status word.
#pragma once
#include "attn_tc.cuh"

namespace exl3 {

constexpr int A2_ROWS = 128, A2_TN = 128, A2_D = 128;
constexpr int A2_KV_SLOTS = 5;
constexpr int A2_MAX_H = 4;                                           // softmax threads per row: 2 or 4
constexpr int a2_threads(int H) { return (4 * H + 2) * 32; }
constexpr int A2_Q_BYTES = A2_ROWS * A2_D * 2;
constexpr int A2_KV_SLOT = A2_TN * A2_D * 2;
constexpr int A2_OFF_Q = 0;
constexpr int A2_OFF_KV = A2_OFF_Q + A2_Q_BYTES;
constexpr int A2_OFF_X = A2_OFF_KV + A2_KV_SLOTS * A2_KV_SLOT;        // exchange of row maxima / sums: [2 buffers][H parts][128] floats
constexpr int A2_OFF_BAR = A2_OFF_X + 2 * A2_MAX_H * A2_ROWS * 4;
// q_full, kv_full/kv_empty[slots], s_full[2], p_full[2], pv_done, o_full, pair[4]
constexpr int A2_NBARS = 1 + 2 * A2_KV_SLOTS + 2 + 2 + 1 + 1 + 4;
constexpr int A2_SMEM = A2_OFF_BAR + A2_NBARS * 8 + 16 + 1024;

// Rendezvous of the two warps that own a lane quadrant, with a bounded wait like every other wait here (a named barrier
// would leave one warp waiting for ever if its partner had left through a time-out).  False on time-out.
__device__ __forceinline__ bool a2_pair_sync(uint64_t* bar, uint32_t& phase, int lane)
{
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    const bool ok = mbar_wait_warp(bar, phase);
    phase ^= 1;
    return ok;
}

template <int H>
__global__ void __launch_bounds__(a2_threads(H), 1) attn_tc2_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                    const __grid_constant__ CUtensorMap vmap, const AttnParams p)
{
    static_assert(H == 2 || H == 4, "two or four softmax threads per row");
    constexpr int NSW = 4 * H;                     // softmax warps; warp NSW = TMA producer, NSW + 1 = MMA issuer and TMEM owner
    constexpr int KPT = A2_TN / H;                 // keys of a tile, and columns of O, per softmax thread
    // grid max_items * nkv: the CTAs of one item are neighbours in launch order, items come longest first
    if ((int)(blockIdx.x / p.nkv) >= p.plan->n_items) return;
    const int item_idx = p.order[blockIdx.x / p.nkv];
    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + A2_OFF_BAR);
    uint64_t* q_full = bars;
    uint64_t* kv_full = q_full + 1;                        uint64_t* kv_empty = kv_full + A2_KV_SLOTS;
    uint64_t* s_full = kv_empty + A2_KV_SLOTS;             // [2]
    uint64_t* p_full = s_full + 2;                         // [2]
    uint64_t* pv_done = p_full + 2;
    uint64_t* o_full = pv_done + 1;
    uint64_t* pair_bar = o_full + 1;                       // [4]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pair_bar + 4);
    float* xch = reinterpret_cast<float*>(smem + A2_OFF_X);
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
    const int r0 = item.rb * A2_ROWS;
    const int i_last = min(ql - 1, (r0 + A2_ROWS - 1) / G);
    const int vis_max = p.causal ? min(total_k, total_k - ql + i_last + 1) : total_k;
    const int k_begin = item.split * chunk;
    const int k_end = min(min(k_begin + chunk, total_k), vis_max);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + A2_TN - 1) / A2_TN : 0;
    const int32_t* bt = p.block_table + (size_t)b * p.pps;

    // Softmax thread = (row, part h of a tile's keys).  Its 128 / H dims of the Q row are requested here, before the
    // barriers and the TMEM allocation are set up: a global-memory round trip on a busy GPU is as long as that set-up.
    constexpr int QCH = 16 / H;                                  // 16-byte chunks per thread
    const int sm_q = warp & 3, sm_h = warp >> 2;
    const int sm_lr = sm_q * 32 + lane;
    const int sm_row = r0 + sm_lr;
    const int sm_qidx = sm_row / G;
    const bool sm_valid = warp < NSW && sm_row < ql * G;
    const int sm_head = kvh * G + (sm_row - sm_qidx * G);
    uint4 qv[QCH];
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)(row_base + sm_qidx) * p.nq + sm_head) * A2_D) + sm_h * QCH;
        #pragma unroll
        for (int c = 0; c < QCH; ++c) qv[c] = sm_valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
    }

    if (tid == 0) {
        s_failed = 0;
        mbar_init(q_full, NSW);
        for (int i = 0; i < 2; ++i) { mbar_init(&p_full[i], NSW); mbar_init(&s_full[i], 1); }
        for (int i = 0; i < A2_KV_SLOTS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
        mbar_init(pv_done, 1);
        mbar_init(o_full, 1);
        for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], H);
        mbar_fence_init();
    }
    if (warp == NSW + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    // H = 2: 64 scores per softmax thread fit the launch allocation of 168 registers; the service warps keep 152 (their
    // code - descriptors, ring cursors - spills below about 140).  H = 4: 576 threads, 112 registers each, 32 scores.
    if constexpr (H == 2) { if (warp >= NSW) asm volatile("setmaxnreg.dec.sync.aligned.u32 152;"); }

    if (warp == NSW) {
        // ===== producer: ring items in the order the issuer takes them: K0, K1, then V(j), K(j+2) for every tile j
        if (lane == 0 && n_tiles > 0) {
            int it = 0;
            auto load = [&](int tile, bool is_v) -> bool {
                const int slot = it % A2_KV_SLOTS;
                if (it >= A2_KV_SLOTS && !mbar_wait_sleep(&kv_empty[slot], ((it / A2_KV_SLOTS) - 1) & 1)) return false;
                const int k0 = k_begin + tile * A2_TN;
                const int page = bt[k0 >> 8], tok = k0 & 255;
                uint8_t* st = smem + A2_OFF_KV + slot * A2_KV_SLOT;
                const CUtensorMap* map = is_v ? &vmap : &kmap;
                mbar_expect_tx(&kv_full[slot], A2_KV_SLOT);
                tma_load_4d(st, map, 0, kvh, tok, page, &kv_full[slot]);
                tma_load_4d(st + A2_TN * 128, map, 64, kvh, tok, page, &kv_full[slot]);
                ++it;
                return true;
            };
            bool ok = load(0, false);
            if (ok && n_tiles > 1) ok = load(1, false);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = load(j, true);
                if (ok && j + 2 < n_tiles) ok = load(j + 2, false);
            }
            if (!ok) failed = true;
        }
    } else if (warp == NSW + 1) {
        // ===== MMA issuer.  The whole warp runs the loop with warp-uniform values; one elected lane issues.
        if (n_tiles > 0) {
            const bool leader = elect_one();
            constexpr uint32_t HI_K = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);   // SBO, version 1, SWIZZLE_128B
            constexpr uint32_t LBO_K = 1u << 16;
            constexpr uint32_t LBO_V = (uint32_t)((A2_TN * 128) >> 4) << 16;
            auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            const uint32_t q_lo = (smem_u32(smem + A2_OFF_Q) >> 4) | LBO_K;
            const uint32_t kv_lo = smem_u32(smem + A2_OFF_KV) >> 4;
            int it = 0;                                                     // ring items consumed so far
            // S(tile) into S buffer sb from the K tile that is ring item `it`
            auto s_tile = [&](int sb) -> bool {
                const int slot = it % A2_KV_SLOTS;
                if (!mbar_wait_sleep_warp(&kv_full[slot], (it / A2_KV_SLOTS) & 1)) return false;
                tc_fence_after();
                if (leader) {
                    const uint32_t b0 = (kv_lo + slot * (A2_KV_SLOT >> 4)) | LBO_K;
                    #pragma unroll
                    for (int kk = 0; kk < A2_D / 16; ++kk) {
                        const uint32_t ao = ((kk >> 2) * (A2_ROWS * 128) + (kk & 3) * 32) >> 4;
                        const uint32_t bo = ((kk >> 2) * (A2_TN * 128) + (kk & 3) * 32) >> 4;
                        tc_mma_f16(tmem_base + sb * 128, mk(q_lo + ao, HI_K), mk(b0 + bo, HI_K), ATC_IDESC_S, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(&s_full[sb]);
                    tc_commit(&kv_empty[slot]);
                }
                __syncwarp();
                ++it;
                return true;
            };
            if (!mbar_wait_sleep_warp(q_full, 0)) failed = true;
            if (!failed && !s_tile(0)) failed = true;
            if (!failed && n_tiles > 1 && !s_tile(1)) failed = true;
            for (int j = 0; j < n_tiles && !failed; ++j) {
                const int sb = j & 1;
                const int slot = it % A2_KV_SLOTS;                          // V of tile j
                if (!mbar_wait_warp(&p_full[sb], (j >> 1) & 1) ||
                    !mbar_wait_sleep_warp(&kv_full[slot], (it / A2_KV_SLOTS) & 1)) { failed = true; break; }
                tc_fence_after();
                if (leader) {
                    const uint32_t b0 = (kv_lo + slot * (A2_KV_SLOT >> 4)) | LBO_V;
                    #pragma unroll
                    for (int kk = 0; kk < A2_TN / 16; ++kk)
                        tc_mma_f16_ts(tmem_base + 256, tmem_base + sb * 128 + 64 + kk * 8, mk(b0 + kk * (2048 >> 4), HI_K), ATC_IDESC_PV,
                                      (j > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(pv_done);                                     // O holds tiles 0..j: it may be rescaled or read
                    tc_commit(&kv_empty[slot]);
                }
                __syncwarp();
                ++it;
                // S(j+2) goes into the buffer P(j) was read from: the tensor core runs PV(j) first
                if (j + 2 < n_tiles && !s_tile(sb)) { failed = true; break; }
            }
            if (!failed && leader) tc_commit(o_full);
        }
    } else if (warp < NSW) {
        // ===== softmax: thread = (row, part h of the tile's keys)
        const int q = sm_q, h = sm_h, lr = sm_lr, qidx = sm_qidx, head = sm_head;
        const bool valid = sm_valid;
        const int lim = valid ? (p.causal ? min(total_k, total_k - ql + qidx + 1) : total_k) : 0;
        {   // Q row part -> shared memory, K-major 128B-swizzled (two 64-wide d blocks)
            const int c0 = h * QCH;                              // first chunk of the row's 16
            uint8_t* qs = smem + A2_OFF_Q + (c0 >> 3) * (A2_ROWS * 128) + lr * 128;
            #pragma unroll
            for (int c = 0; c < QCH; ++c) *reinterpret_cast<uint4*>(qs + ((((c0 & 7) + c) ^ (lr & 7)) << 4)) = qv[c];
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        float m_used = -INFINITY, m_true = -INFINITY, l_part = 0.f;
        uint32_t pair_phase = 0;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const uint32_t tmem_o = tmem_base + lane_addr + 256 + h * KPT;      // this thread's columns of O
        const float scale = p.scale_log2;
        // The scores of tile j+1 are requested before P(j) is announced: a TMEM read issued after the issuer has queued
        // PV(j) and S(j+2) waits behind those 1024 tensor-core cycles (per-tile time 2770 cycles with the read at the top of
        // the loop).  S(j+1) was issued before PV(j), so waiting for it here cannot hold anything up.
        float sv[KPT];
        auto request_scores = [&](int j) -> bool {
            const int sb = j & 1;
            if (!mbar_wait_warp(&s_full[sb], (j >> 1) & 1)) return false;
            tc_fence_after();
            #pragma unroll
            for (int c = 0; c < KPT / 32; ++c)
                tc_ld32(tmem_base + lane_addr + sb * 128 + h * KPT + c * 32, *reinterpret_cast<float (*)[32]>(&sv[c * 32]));
            return true;
        };
        if (n_tiles > 0) {
            if (!request_scores(0)) failed = true;
            tc_wait_ld();
        }
        for (int j = 0; j < n_tiles && !failed; ++j) {
            const int sb = j & 1;
            const uint32_t tmem_s = tmem_base + lane_addr + sb * 128;
            const int kbase = k_begin + j * A2_TN;
            const int nvis = min(lim, k_end) - kbase - h * KPT;      // keys of this thread's part the row may see (may be <= 0)
            if (nvis < KPT) {
                #pragma unroll
                for (int e = 0; e < KPT; ++e) sv[e] = e < nvis ? sv[e] : -INFINITY;
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
            #pragma unroll
            for (int e = 0; e < KPT; e += 4) { mx0 = fmax3(mx0, sv[e], sv[e + 1]); mx1 = fmax3(mx1, sv[e + 2], sv[e + 3]); }
            // row maximum over all parts: the partners are the same lane of the other warps of this lane quadrant
            float* xm = xch + (size_t)sb * A2_MAX_H * A2_ROWS;
            xm[h * A2_ROWS + lr] = fmaxf(mx0, mx1);
            if (!a2_pair_sync(&pair_bar[q], pair_phase, lane)) { failed = true; break; }
            float mrow = xm[lr];
            #pragma unroll
            for (int hh = 1; hh < H; ++hh) mrow = fmaxf(mrow, xm[hh * A2_ROWS + lr]);
            m_true = fmaxf(m_true, mrow * scale);                   // raw scores: the scale is positive
            // lazy reference update, decided identically by both threads of the row
            const bool move = m_true > m_used + ATC_RESCALE_THRESHOLD || (m_used == -INFINITY && m_true > -INFINITY);
            const bool rescale = move && m_used != -INFINITY && j > 0;
            const float corr = rescale ? ex2_approx(m_used - m_true) : 1.0f;
            if (move) m_used = m_true;
            const float nref = (m_used == -INFINITY) ? 0.f : -m_used;
            uint32_t pw[KPT / 2];
            float l0 = 0.f, l1 = 0.f;
            #pragma unroll
            for (int e = 0; e < KPT; e += 2) {
                const float e0 = ex2_approx(fmaf(sv[e], scale, nref)), e1 = ex2_approx(fmaf(sv[e + 1], scale, nref));
                l0 += e0; l1 += e1;
                pw[e >> 1] = pack_h2(e0, e1);
            }
            // P over the last 64 columns of the S buffer (column 64 + c = keys 2c, 2c+1).  The partners have read their
            // scores out of those columns before they reached the barrier above.
            if constexpr (H == 2) tc_st32u(tmem_s + 64 + h * 32, pw);
            else tc_st16u(tmem_s + 64 + h * 16, pw);
            if (__any_sync(0xffffffffu, rescale)) {
                // O holds tiles 0..j-1 once PV(j-1) has completed (its commit is completion j-1 of pv_done)
                if (!mbar_wait_warp(pv_done, (j - 1) & 1)) { failed = true; break; }
                tc_fence_after();
                #pragma unroll
                for (int c = 0; c < KPT / 32; ++c) {
                    float part[32];
                    tc_ld32(tmem_o + c * 32, part);
                    tc_wait_ld();
                    #pragma unroll
                    for (int e = 0; e < 32; ++e) part[e] *= corr;
                    tc_st32(tmem_o + c * 32, part);
                }
            }
            l_part = l_part * corr + (l0 + l1);
            // rows of V past the end of the sequence may hold anything (0 * NaN would poison O): cleared before PV reads them
            if (h == 0 && kbase + A2_TN > k_end) {
                // V of tile j is ring item 2 + 2j for j < n_tiles - 1 ... the last tile's V is the last item: 2 n_tiles - 1
                const int itv = 2 * n_tiles - 1, slot = itv % A2_KV_SLOTS;
                if (!mbar_wait_sleep_warp(&kv_full[slot], (itv / A2_KV_SLOTS) & 1)) { failed = true; break; }
                uint8_t* vst = smem + A2_OFF_KV + slot * A2_KV_SLOT;
                const int first_bad = k_end - kbase;                        // 1..127
                for (int i = lr; i < (A2_TN - first_bad) * 16; i += 128) {
                    const int key = first_bad + (i >> 4), c = i & 15;
                    *reinterpret_cast<uint4*>(vst + (c >> 3) * (A2_TN * 128) + key * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            tc_wait_st();
            const bool more = j + 1 < n_tiles;
            if (more && !request_scores(j + 1)) { failed = true; break; }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[sb]);
            if (more) tc_wait_ld();
        }
        // ===== epilogue: row sums of the two halves, then O (TMEM) -> output or split-KV partial, this thread's 64 columns
        failed = __any_sync(0xffffffffu, failed);
        float l_run = l_part;
        if (!failed) {
            float* xl = xch;                                     // the maxima buffers are idle now
            bool ok = a2_pair_sync(&pair_bar[q], pair_phase, lane);      // both warps are past their last read of them
            xl[h * A2_ROWS + lr] = l_part;
            ok = a2_pair_sync(&pair_bar[q], pair_phase, lane) && ok;
            l_run = xl[lr];
            #pragma unroll
            for (int hh = 1; hh < H; ++hh) l_run += xl[hh * A2_ROWS + lr];
            if (!ok) failed = true;
        }
        if (!failed && n_tiles > 0 && !mbar_wait_sleep_warp(o_full, 0)) failed = true;
        // Split-KV partials ([128 rows][D + 2] floats per item and kv head) go through shared memory: written by each
        // thread straight to its own row, a store instruction touched 32 rows = 32 sectors for 256 bytes, and the 32 such
        // instructions per thread took 6400 cycles per CTA; staged, a warp writes whole rows.  The K/V ring is idle by now
        // (the last PV product has completed, nothing is in flight).
        constexpr int SROW = A2_D + 4;                            // staging row stride in floats: 16-byte aligned, conflict-free
        float* stage = reinterpret_cast<float*>(smem + A2_OFF_KV);
        static_assert(A2_ROWS * (A2_D + 4) * 4 <= A2_KV_SLOTS * A2_KV_SLOT, "staging fits the K/V ring");
        if (!failed) {
            tc_fence_after();
            const float inv = (splits == 1) ? (l_run > 0.f ? 1.0f / l_run : 0.f) : 1.0f;
            half* orow = p.o + ((size_t)(row_base + qidx) * p.nq + head) * A2_D + h * KPT;
            float oall[KPT];
            if (n_tiles > 0) {
                #pragma unroll
                for (int c = 0; c < KPT / 32; ++c) tc_ld32(tmem_o + c * 32, *reinterpret_cast<float (*)[32]>(&oall[c * 32]));
                tc_wait_ld();
            } else {
                #pragma unroll
                for (int e = 0; e < KPT; ++e) oall[e] = 0.f;
            }
            #pragma unroll
            for (int c = 0; c < KPT / 32; ++c) {
                const float* ov = &oall[c * 32];
                if (splits == 1) {
                    if (valid) {
                        uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
                        #pragma unroll
                        for (int e = 0; e < 4; ++e)
                            dst[e] = make_uint4(pack_h2(ov[e * 8] * inv, ov[e * 8 + 1] * inv), pack_h2(ov[e * 8 + 2] * inv, ov[e * 8 + 3] * inv),
                                                pack_h2(ov[e * 8 + 4] * inv, ov[e * 8 + 5] * inv), pack_h2(ov[e * 8 + 6] * inv, ov[e * 8 + 7] * inv));
                    }
                } else {
                    float4* dst = reinterpret_cast<float4*>(stage + lr * SROW + h * KPT + c * 32);
                    #pragma unroll
                    for (int e = 0; e < 8; ++e) dst[e] = make_float4(ov[4 * e], ov[4 * e + 1], ov[4 * e + 2], ov[4 * e + 3]);
                }
            }
            if (splits != 1 && h == 0) { stage[lr * SROW + A2_D] = m_used; stage[lr * SROW + A2_D + 1] = l_run; }
        }
        if (splits != 1) {                                        // CTA-uniform
            // every softmax warp comes here exactly once, whatever its `failed`
            asm volatile("bar.sync 1, %0;" ::"n"(NSW * 32) : "memory");
            if (!failed) {
                float* pbase = p.partial + ((size_t)item_idx * p.nkv + kvh) * A2_ROWS * (A2_D + 2);
                const int n_valid = min(A2_ROWS, ql * G - r0);    // valid rows of this block are its first ones
                for (int r = warp; r < n_valid; r += NSW) {
                    const float2* srow = reinterpret_cast<const float2*>(stage + r * SROW);
                    float2* drow = reinterpret_cast<float2*>(pbase + (size_t)r * (A2_D + 2));
                    drow[lane] = srow[lane];
                    drow[lane + 32] = srow[lane + 32];
                    if (lane == 0) drow[64] = srow[64];
                }
            }
        }
    }

    if (failed) s_failed = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == NSW + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 3);
}

}  // namespace exl3
