// Decode-class paged attention over 4-bit quantised KV pools (k_bits = v_bits = 4, head_dim 128, at most 16 packed
// (query, head) rows per CTA): the kernel behind exl3_bighead_attn_paged_q for the common cache format.
// Reference semantics: kernels/attention.cu:97-269,1716-1870 with the cache codec of
// kernels/cache/q_cache_kernels.cuh:61-236 (a code c of a group of 32 rotated values stands for (c - 7.5) * scale / 8).
//
// What differs from the generic quantised kernel (attn_paged.cuh), which scales every code into fp16 tiles in shared
// memory before the MMAs read them back:
//  * a tile of 64 keys (codes and scales of one kv head: 10 KB) arrives by four tiled TMA copies issued by one thread;
//  * K never goes through a decoded tile: the thread that owns key g of an MMA column block reads the 16 bytes of one
//    group (lane t of the quad = group t), turns every 32-bit word into four fp16 pairs with a shift and one logic
//    operation each ((w << 6) & 0x03C003C0 | 0x4C004C00 = the halves 16 + n0, 16 + n4), subtracts 23.5, multiplies by
//    the group scale and feeds the pairs to the tensor core as they are; the query fragments are laid out in the same
//    dimension order (and rotated by H32 once per work unit, since q . H(c) = H(q) . c);
//  * V is unpacked to 16 + n only (no subtraction, no scale) into a per-warp fp16 tile; the scale of (key, group) is
//    multiplied into the softmax weights instead (four A operands, one per group) and the offset 23.5 * sum_k P s comes
//    from one extra MMA per group against a column of ones, subtracted once per work unit;
//  * the softmax scale, 1/sqrt(32) of the rotation and the codec's 1/8 are folded into the query, the output's into the
//    final normalisation.
// Work distribution, split-KV partials and the combine kernel are those of attn_paged.cuh.
#pragma once
#include <cuda.h>
#include "attn_paged.cuh"
#include "async_copy.cuh"

namespace exl3 {

constexpr int AQ_TK = 64;                 // keys per tile
constexpr int AQ_STAGES = 4;
constexpr int AQ_THREADS = 128;
constexpr int AQ_CODES = AQ_TK * 64;      // bytes of K (or V) codes per tile: 64 bytes per key and head
constexpr int AQ_SCALES = AQ_TK * 16;     // scales of two neighbouring heads per key (the copy must be 16 bytes wide)
constexpr int AQ_STAGE = 2 * AQ_CODES + 2 * AQ_SCALES;
constexpr int AQ_VROW = (128 + 8) * 2;    // bytes per key row of a warp's unpacked V tile (padding keeps ldmatrix conflict-free)
constexpr int AQ_OFF_V = AQ_STAGES * AQ_STAGE;
constexpr int AQ_OFF_BAR = AQ_OFF_V + 4 * 16 * AQ_VROW;
constexpr int AQ_PIPE = AQ_OFF_BAR + 64;
constexpr int AQ_MERGE = 4 * 16 * (128 + 4) * 4;
constexpr int AQ_SMEM = AQ_PIPE > AQ_MERGE ? AQ_PIPE : AQ_MERGE;
static_assert(AQ_MERGE <= AQ_OFF_BAR, "the merge buffer must not reach the barriers");

__device__ __forceinline__ void aq_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ float aq_ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// the four fp16 pairs (16 + n_i, 16 + n_{i+4}), i = 0..3, of a word of eight 4-bit codes
__device__ __forceinline__ void aq_unpack(uint32_t w, uint32_t (&x)[4])
{
    constexpr uint32_t M = 0x03C003C0u, E = 0x4C004C00u;
    x[0] = ((w << 6) & M) | E;
    x[1] = ((w << 2) & M) | E;
    x[2] = ((w >> 2) & M) | E;
    x[3] = ((w >> 6) & M) | E;
}

__global__ void __launch_bounds__(AQ_THREADS, 3)
attn_q4_decode_kernel(const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_qv,
                      const __grid_constant__ CUtensorMap map_sk, const __grid_constant__ CUtensorMap map_sv, const AttnParams p)
{
    constexpr int D = 128, ROWS = 16, DBLK = 16;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + AQ_OFF_BAR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = p.nq / p.nkv;
    const int n_items = p.plan->n_items, chunk = p.plan->chunk;
    if (tid == 0) {
        #pragma unroll
        for (int s = 0; s < AQ_STAGES; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    uint8_t* vt = smem_raw + AQ_OFF_V + warp * 16 * AQ_VROW;       // this warp's unpacked V rows
    uint32_t tiles_done = 0;                                        // tiles consumed by this CTA so far: stage and parity

    __shared__ int s_unit;
    const int n_units = n_items * p.nkv;
    for (;;) {
        __syncthreads();                                   // the previous unit's merge buffer and s_unit are free
        if (tid == 0) s_unit = atomicAdd(const_cast<int*>(&p.plan->next), 1);
        __syncthreads();
        const int unit = s_unit;
        if (unit >= n_units) break;
        const int item_idx = p.order[unit / p.nkv], kvh = unit % p.nkv;
        const AttnItem item = p.items[item_idx];
        const int b = item.b;
        const int row_base = p.cu_q ? p.cu_q[b] : b * p.q_len;
        const int ql = p.cu_q ? p.cu_q[b + 1] - row_base : p.q_len;
        const int total_k = p.seqlens[b] + (p.cu_q ? ql : p.kv_append);
        const int splits = p.seq_splits[b];
        const int r0 = item.rb * ROWS;
        const int i_last = min(ql - 1, (r0 + ROWS - 1) / G);
        const int vis_max = p.causal ? min(total_k, total_k - ql + i_last + 1) : total_k;
        const int k_begin = item.split * chunk;
        const int k_end = min(min(k_begin + chunk, total_k), vis_max);
        const int32_t* bt = p.block_table + (size_t)b * p.pps;
        const int n_tiles = k_end > k_begin ? (k_end - k_begin + AQ_TK - 1) / AQ_TK : 0;

        // ---- tile loads: one thread, four tiled copies per tile (a tile of 64 keys lies inside one 256-token page)
        auto issue = [&](int tile) {
            const int k0 = k_begin + tile * AQ_TK;
            const int tok0 = bt[k0 >> 8] * EXL3_PAGE + (k0 & 255);
            const uint32_t s = (tiles_done + tile) % AQ_STAGES;
            const uint32_t dst = smem_u32(smem_raw + s * AQ_STAGE), bar = smem_u32(&full[s]);
            mbar_expect_tx(&full[s], AQ_STAGE);
            aq_tma_2d(dst, &map_qk, kvh * 16, tok0, bar);
            aq_tma_2d(dst + AQ_CODES, &map_qv, kvh * 16, tok0, bar);
            aq_tma_2d(dst + 2 * AQ_CODES, &map_sk, (kvh >> 1) * 8, tok0, bar);
            aq_tma_2d(dst + 2 * AQ_CODES + AQ_SCALES, &map_sv, (kvh >> 1) * 8, tok0, bar);
        };
        if (tid == 0) {
            // the stages were last written and read through the generic proxy (merge buffer of the previous unit)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            #pragma unroll
            for (int pre = 0; pre < AQ_STAGES - 1; ++pre)
                if (pre < n_tiles) issue(pre);
        }

        // ---- per-thread row bookkeeping: rows g and g + 8
        int qi[2], lim[2];
        bool rvalid[2];
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r0 + g + 8 * h;
            qi[h] = row / G;
            rvalid[h] = row < ql * G;
            lim[h] = rvalid[h] ? (p.causal ? min(total_k, total_k - ql + qi[h] + 1) : total_k) : 0;
        }
        int wlim = min(rvalid[0] ? lim[0] : 0x7fffffff, rvalid[1] ? lim[1] : 0x7fffffff);
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) wlim = min(wlim, __shfl_xor_sync(0xffffffffu, wlim, o));

        // ---- Q: lane t of a quad takes group t (dims 32t .. 32t+31) of rows g and g+8, rotates it (H32, in registers),
        // scales it and packs it in the order the K words unpack to: MMA k-step ks = 2u + v covers word u of the group,
        // a0/a1 = dims (8u + 2v, 8u + 2v + 4), a2/a3 = dims (8u + 2v + 1, 8u + 2v + 5)
        uint32_t qf[8][4];
        {
            const float qs = p.scale_log2 * R32 * 0.125f;
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = r0 + g + 8 * h;
                const int head = kvh * G + (row - qi[h] * G);
                float v[32];
                if (rvalid[h]) {
                    const uint4* qp = reinterpret_cast<const uint4*>(p.q + ((size_t)(row_base + qi[h]) * p.nq + head) * D + 32 * t);
                    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint4 raw = qp[c];
                        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
                        #pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const half2 x = *reinterpret_cast<const half2*>(&w[e]);
                            v[8 * c + 2 * e] = __low2float(x); v[8 * c + 2 * e + 1] = __high2float(x);
                        }
                    }
                } else {
                    #pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = 0.f;
                }
                #pragma unroll
                for (int st = 1; st < 32; st <<= 1) {
                    #pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        if ((e & st) == 0) { const float a = v[e], c = v[e | st]; v[e] = a + c; v[e | st] = a - c; }
                    }
                }
                #pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const int d = 8 * (ks >> 1) + 2 * (ks & 1);
                    qf[ks][h] = pack_h2(v[d] * qs, v[d + 4] * qs);
                    qf[ks][h + 2] = pack_h2(v[d + 1] * qs, v[d + 5] * qs);
                }
            }
        }

        float o_acc[DBLK][4];
        #pragma unroll
        for (int i = 0; i < DBLK; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
        float csum[4][4];                                     // per group: sum over keys of P * scale (rows g, g+8 in [0], [2])
        #pragma unroll
        for (int j = 0; j < 4; ++j) { csum[j][0] = csum[j][1] = csum[j][2] = csum[j][3] = 0.f; }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        const int sc_off = (kvh & 1) * 8;                     // this head's 4 scales inside the 16-byte pair

        bool failed = false;
        for (int tile = 0; tile < n_tiles; ++tile) {
            const uint32_t seq = tiles_done + tile;
            const uint32_t stage = seq % AQ_STAGES;
            const bool ok = mbar_wait(&full[stage], (seq / AQ_STAGES) & 1);
            // one barrier per tile: the tile is visible to everyone, and everyone is done with the previous tile, whose
            // stage the next load may now overwrite
            if (__syncthreads_or(!ok)) { failed = true; break; }
            if (tid == 0 && tile + AQ_STAGES - 1 < n_tiles) issue(tile + AQ_STAGES - 1);

            const uint8_t* sb = smem_raw + stage * AQ_STAGE;
            const int kbase = k_begin + tile * AQ_TK + warp * 16;      // first key of this warp's 16

            // ---- S = Q K^T straight from the codes
            float s_acc[2][4];
            #pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                s_acc[nb][0] = s_acc[nb][1] = s_acc[nb][2] = s_acc[nb][3] = 0.f;
                const int kl = warp * 16 + nb * 8 + g;                 // key inside the tile
                const uint4 kw = *reinterpret_cast<const uint4*>(sb + kl * 64 + t * 16);
                half sc = *reinterpret_cast<const half*>(sb + 2 * AQ_CODES + kl * 16 + sc_off + 2 * t);
                if (kbase + nb * 8 + g >= k_end) sc = __float2half(0.f);        // rows of the page past the sequence: any bits
                const half2 sc2 = __half2half2(sc);
                const half2 off = __float2half2_rn(23.5f);
                const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
                #pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint32_t x[4];
                    aq_unpack(w[u], x);
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const half2 y = __hmul2(__hsub2(*reinterpret_cast<const half2*>(&x[e]), off), sc2);
                        x[e] = *reinterpret_cast<const uint32_t*>(&y);
                    }
                    mma_f16(s_acc[nb], qf[2 * u][0], qf[2 * u][1], qf[2 * u][2], qf[2 * u][3], x[0], x[1]);
                    mma_f16(s_acc[nb], qf[2 * u + 1][0], qf[2 * u + 1][1], qf[2 * u + 1][2], qf[2 * u + 1][3], x[2], x[3]);
                }
            }

            // ---- V: this warp's 16 keys as 16 + n, fp16, into its own tile (columns of every 8 in the order 0 4 1 5 2 6 3 7)
            #pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int kl = 2 * i + (lane >> 4);
                const uint32_t w = *reinterpret_cast<const uint32_t*>(sb + AQ_CODES + (warp * 16 + kl) * 64 + (lane & 15) * 4);
                uint32_t x[4];
                aq_unpack(w, x);
                *reinterpret_cast<uint4*>(vt + kl * AQ_VROW + (lane & 15) * 16) = make_uint4(x[0], x[1], x[2], x[3]);
            }

            // ---- mask, online softmax in base 2 (the scores already carry the softmax scale)
            const bool need_mask = kbase + 16 > wlim || kbase + 16 > k_end;      // warp-uniform
            float mx[2] = {-INFINITY, -INFINITY};
            if (need_mask) {
                #pragma unroll
                for (int nb = 0; nb < 2; ++nb)
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int h = e >> 1;
                        const int key = kbase + nb * 8 + 2 * t + (e & 1);
                        const float v = (key < lim[h] && key < k_end) ? s_acc[nb][e] : -INFINITY;
                        s_acc[nb][e] = v;
                        mx[h] = fmaxf(mx[h], v);
                    }
            } else {
                #pragma unroll
                for (int nb = 0; nb < 2; ++nb)
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s_acc[nb][e]);
            }
            float corr[2];
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                corr[h] = (m_new == -INFINITY) ? 1.0f : aq_ex2(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= corr[h];
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
                #pragma unroll
                for (int i = 0; i < DBLK; ++i) { o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0]; o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1]; }
                #pragma unroll
                for (int j = 0; j < 4; ++j) { csum[j][0] *= corr[0]; csum[j][2] *= corr[1]; }
            }
            const float mref0 = (m_run[0] == -INFINITY) ? 0.f : m_run[0], mref1 = (m_run[1] == -INFINITY) ? 0.f : m_run[1];
            uint32_t pf[2][2];
            #pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                const float e0 = aq_ex2(s_acc[nb][0] - mref0), e1 = aq_ex2(s_acc[nb][1] - mref0);
                const float e2 = aq_ex2(s_acc[nb][2] - mref1), e3 = aq_ex2(s_acc[nb][3] - mref1);
                l_run[0] += e0 + e1; l_run[1] += e2 + e3;
                pf[nb][0] = pack_h2(e0, e1); pf[nb][1] = pack_h2(e2, e3);
            }

            // ---- the V scales of this lane's four keys (2t, 2t+1, 2t+8, 2t+9 of the warp's 16), as pairs per group
            uint2 sv4[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int kl = 2 * t + (i & 1) + 8 * (i >> 1);
                sv4[i] = *reinterpret_cast<const uint2*>(sb + 2 * AQ_CODES + AQ_SCALES + (warp * 16 + kl) * 16 + sc_off);
                if (kbase + kl >= k_end) sv4[i] = make_uint2(0u, 0u);
            }
            __syncwarp();                                              // the V tile is complete

            // ---- O += (P * scale_group) (16 + n), group by group; csum collects sum_k P * scale_group
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo01 = (j & 2) ? sv4[0].y : sv4[0].x, hi01 = (j & 2) ? sv4[1].y : sv4[1].x;
                const uint32_t lo23 = (j & 2) ? sv4[2].y : sv4[2].x, hi23 = (j & 2) ? sv4[3].y : sv4[3].x;
                const uint32_t s01 = __byte_perm(lo01, hi01, (j & 1) ? 0x7632 : 0x5410);
                const uint32_t s23 = __byte_perm(lo23, hi23, (j & 1) ? 0x7632 : 0x5410);
                const half2 h01 = *reinterpret_cast<const half2*>(&s01), h23 = *reinterpret_cast<const half2*>(&s23);
                const half2 a0h = __hmul2(*reinterpret_cast<const half2*>(&pf[0][0]), h01);
                const half2 a1h = __hmul2(*reinterpret_cast<const half2*>(&pf[0][1]), h01);
                const half2 a2h = __hmul2(*reinterpret_cast<const half2*>(&pf[1][0]), h23);
                const half2 a3h = __hmul2(*reinterpret_cast<const half2*>(&pf[1][1]), h23);
                const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&a0h), a1 = *reinterpret_cast<const uint32_t*>(&a1h);
                const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&a2h), a3 = *reinterpret_cast<const uint32_t*>(&a3h);
                mma_f16(csum[j], a0, a1, a2, a3, 0x3C003C00u, 0x3C003C00u);
                const uint8_t* vrow = vt + (lane & 15) * AQ_VROW + (lane >> 4) * 16 + j * 64;
                #pragma unroll
                for (int d2 = 0; d2 < 2; ++d2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(b0, b1, b2, b3, vrow + d2 * 32);
                    mma_f16(o_acc[4 * j + 2 * d2], a0, a1, a2, a3, b0, b1);
                    mma_f16(o_acc[4 * j + 2 * d2 + 1], a0, a1, a2, a3, b2, b3);
                }
            }
            __syncwarp();                                              // before the next tile's unpack overwrites the V tile
        }
        if (failed) {
            if (tid == 0) atomicCAS(p.status, 0, 4);
            return;                                                    // uniform: every thread saw the same barrier result
        }
        tiles_done += n_tiles;
        __syncthreads();                                               // all warps are done with the stages: the merge buffer may overwrite them

        // ---- take the offset out: value = (16 + n - 23.5) * scale / 8; the 1/8 goes into the normalisation below
        #pragma unroll
        for (int i = 0; i < DBLK; ++i) {
            o_acc[i][0] -= 23.5f * csum[i >> 2][0]; o_acc[i][1] -= 23.5f * csum[i >> 2][0];
            o_acc[i][2] -= 23.5f * csum[i >> 2][2]; o_acc[i][3] -= 23.5f * csum[i >> 2][2];
        }
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }

        // ---- merge the four key slices through shared memory: [warp][16 rows][D+4] fp32, cols D, D+1 = m, l
        float* ms = reinterpret_cast<float*>(smem_raw);
        constexpr int MS = D + 4;
        {
            float* mine = ms + warp * 16 * MS;
            #pragma unroll
            for (int db = 0; db < DBLK; ++db) {
                *reinterpret_cast<float2*>(mine + g * MS + db * 8 + 2 * t) = make_float2(o_acc[db][0], o_acc[db][1]);
                *reinterpret_cast<float2*>(mine + (g + 8) * MS + db * 8 + 2 * t) = make_float2(o_acc[db][2], o_acc[db][3]);
            }
            if (t == 0) {
                mine[g * MS + D] = m_run[0]; mine[g * MS + D + 1] = l_run[0];
                mine[(g + 8) * MS + D] = m_run[1]; mine[(g + 8) * MS + D + 1] = l_run[1];
            }
        }
        __syncthreads();
        // one warp per output row; lane = (group lane / 8, values 4 (lane % 8) .. + 3) as in the cache codec.  Those four
        // dims sit at every second column of their block of 8 (columns hold dims 0 4 1 5 2 6 3 7).
        for (int lr = warp; lr < ROWS; lr += 4) {
            const int row = r0 + lr;
            if (row >= ql * G) break;
            float mm = -INFINITY;
            #pragma unroll
            for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ms[(w * 16 + lr) * MS + D]);
            float ll = 0.f;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const int col0 = (lane >> 1) * 8 + (lane & 1);
            #pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float* src = ms + (w * 16 + lr) * MS;
                const float mw = src[D];
                const float sc = (mw == -INFINITY) ? 0.f : aq_ex2(mw - mm);
                ll += src[D + 1] * sc;
                #pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] += src[col0 + 2 * e] * sc;
            }
            h4(acc[0], acc[1], acc[2], acc[3]);
            h8_lanes(acc[0], acc[1], acc[2], acc[3], lane);
            #pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] *= R32 * 0.125f;
            const int qidx = row / G, head = kvh * G + (row - qidx * G);
            if (splits == 1) {
                const float inv = ll > 0.f ? 1.0f / ll : 0.f;
                half* op = p.o + ((size_t)(row_base + qidx) * p.nq + head) * D + lane * 4;
                *reinterpret_cast<uint2*>(op) = make_uint2(pack_h2(acc[0] * inv, acc[1] * inv), pack_h2(acc[2] * inv, acc[3] * inv));
            } else {
                float* pp = p.partial + (((size_t)item_idx * p.nkv + kvh) * ROWS + lr) * (D + 2);
                *reinterpret_cast<float2*>(pp + lane * 4) = make_float2(acc[0], acc[1]);
                *reinterpret_cast<float2*>(pp + lane * 4 + 2) = make_float2(acc[2], acc[3]);
                if (lane == 0) { pp[D] = mm; pp[D + 1] = ll; }
            }
        }
    }
}

}  // namespace exl3
