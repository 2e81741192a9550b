// Paged GQA flash attention over block tables for mixed decode / verify / prefill-chunk rows.
//
// Semantics (reference: kernels/attention.cu:97-269,1716-1870, kernels/attention_mma_kernel.cuh:37-380):
//   o[b,i,h,:] = softmax_j(scale * q[b,i,h,:] . k[b,j,h/G,:]) v[b,j,h/G,:]  over keys j <= total_k(b) - q_len(b) + i,
// keys read from pages [pages,256,nkv,D] through block_table.  The M dimension of the MMA tiles packs (query, head)
// pairs of one kv head: row = i*G + g, so a 1-query decode row with G sibling heads and an 8-row verify batch both fill
// 16-row tiles.  KV is split by the REAL length of each sequence (device-built work list), partial results are
// merged by a combine kernel.
#pragma once
#include "common.cuh"
#include "kvquant.cuh"

namespace exl3 {

constexpr int AT_TK = 64;          // keys per shared-memory tile
constexpr int AT_THREADS = 128;    // 4 warps
constexpr int AT_STAGES = 2;        // K/V tile stages per CTA (3 stages leave room for 2 CTAs per SM instead of 3: measured 10 % slower)

struct AttnItem { int b, rb, split, pad; };

struct AttnPlan {          // device-resident, written by attn_plan_kernel
    int n_items;
    int chunk;             // keys per split
    int next;              // work counter of the persistent kernel: next (item, kv head) unit to hand out; zeroed per launch
    int pad1;
};

struct AttnParams {
    const half* q;                 // [rows, nq, D]
    half* o;                       // [rows, nq, D]
    const half* kc; const half* vc;            // fp16 pools [pages,256,nkv,D]
    const uint32_t* qk; const half* sk;        // quantised pools (QUANT): [pages,256,groups*bits], [pages,256,groups]
    const uint32_t* qv; const half* sv;
    const int32_t* block_table;    // [bsz, pps]
    const int32_t* seqlens;        // [bsz]  tokens in the cache BEFORE this step's append (NULL: none, all keys are "appended")
    const int32_t* cu_q;           // [bsz+1] or NULL (then rows of sequence b = [b*q_len, (b+1)*q_len))
    const AttnPlan* plan;
    const AttnItem* items;
    const int* order;              // [n_items] item indices, longest first: the order in which CTAs / work units take them
    const int* seq_base;           // [bsz] first item of sequence b
    const int* seq_splits;         // [bsz]
    float* partial;                // [n_items][nkv][ROWS][D+2]
    int* status;                   // context status word (bounded waits)
    int bsz, q_len, kv_append, nq, nkv, pps, pages, causal, k_bits, v_bits;
    int contig_kv;                 // > 0: kc/vc are plain [bsz, contig_kv, nkv, D] tensors, no block table (mma.sync fp16 kernel only)
    float scale_log2;              // sm_scale * log2(e)
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b)
{
    half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Shared memory: per stage a K tile and a V tile [AT_TK][D+8] fp16; quantised pools (QB > 0: codes of at most QB bits)
// stage the raw codes and scales instead and decode them into one pair of fp16 tiles.
template <int D, int QB>
struct AttnSmem {
    static constexpr bool QUANT = QB > 0;
    static constexpr int ROWB = (D + 8) * 2;                       // bytes per key row (padding keeps ldmatrix conflict-free)
    static constexpr int TILE = AT_TK * ROWB;
    static constexpr int RAW_ROW = QUANT ? (D / 32) * QB * 4 + 16 : 0;  // QB-bit codes of D/32 groups + scales, per key
    // 64 bytes between the K and the V rows of a stage: the 4-bit decoder reads a key's K words with lanes 0..15 and its V
    // words with lanes 16..31, which must fall into different banks
    static constexpr int RAW = AT_TK * RAW_ROW + 64;
    static constexpr int STAGE = QUANT ? 2 * RAW : 2 * TILE;      // QUANT stages the raw bytes; tiles are decoded in place below
    static constexpr int DECODED = QUANT ? 2 * TILE : 0;
    static constexpr int PIPE = AT_STAGES * STAGE + DECODED;
    static constexpr int MERGE = 4 * 16 * (D + 4) * 4;             // cross-warp merge / output staging, fp32
    static constexpr int BYTES = PIPE > MERGE ? PIPE : MERGE;
};

// WM x WN = 4 warps: WM 16-row tiles, WN key slices of every tile.  (4,1): prefill/verify rows, (1,4): decode rows.
#ifndef AT_Q4_DECODE_BLOCKS
#define AT_Q4_DECODE_BLOCKS 4         // resident CTAs per SM the 4-bit decode-class kernel is compiled for (register cap)
#endif
template <int D, int WM, int WN, int QB>
__global__ void __launch_bounds__(AT_THREADS, (QB == 4 && WN == 4) ? AT_Q4_DECODE_BLOCKS : 1) attn_paged_kernel(const AttnParams p)
{
    using SM = AttnSmem<D, QB>;
    constexpr bool QUANT = QB > 0;
    constexpr int ROWS = 16 * WM;
    constexpr int KEYS_W = AT_TK / WN;          // keys of a tile handled by one warp
    constexpr int NBLK = KEYS_W / 8;            // n8 blocks of S per warp
    constexpr int DBLK = D / 8;                 // n8 blocks of O
    constexpr int KSTEPS = D / 16;
    extern __shared__ __align__(128) uint8_t smem_raw[];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp / WN, wn = warp % WN;
    const int G = p.nq / p.nkv;
    const int n_items = p.plan->n_items, chunk = p.plan->chunk;

    // Work units = (item, kv head), handed out through a counter: items differ in length (last splits, causal cuts), and a
    // fixed assignment left a quarter of the SM time idle at the end of the kernel.
    __shared__ int s_unit;
    const int n_units = n_items * p.nkv;
    for (;;) {
        __syncthreads();                                   // everyone is done with the previous unit (and with s_unit)
        if (tid == 0) s_unit = atomicAdd(const_cast<int*>(&p.plan->next), 1);
        __syncthreads();
        const int unit = s_unit;
        if (unit >= n_units) break;
        const int item_idx = p.order[unit / p.nkv], kvh = unit % p.nkv;
        const AttnItem item = p.items[item_idx];
        const int b = item.b;
        const int row_base = p.cu_q ? p.cu_q[b] : b * p.q_len;
        const int ql = p.cu_q ? p.cu_q[b + 1] - row_base : p.q_len;
        const int total_k = (p.seqlens ? p.seqlens[b] : 0) + (p.cu_q ? ql : p.kv_append);
        const int splits = p.seq_splits[b];
        const int r0 = item.rb * ROWS;                       // first packed (query, head) row of this CTA
        // keys this row block can see at all (causal, bottom-right aligned)
        const int i_last = min(ql - 1, (r0 + ROWS - 1) / G);
        const int vis_max = p.causal ? min(total_k, total_k - ql + i_last + 1) : total_k;
        const int k_begin = item.split * chunk;
        const int k_end = min(min(k_begin + chunk, total_k), vis_max);
        const int32_t* bt = p.block_table + (size_t)b * p.pps;      // not dereferenced for plain tensors

        // ---- per-thread row bookkeeping: rows g and g+8 of this warp's 16-row tile
        int qi[2], lim[2];      // query index and last visible key (exclusive) per row
        bool rvalid[2];
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r0 + wm * 16 + g + 8 * h;
            qi[h] = row / G;
            rvalid[h] = row < ql * G;
            lim[h] = rvalid[h] ? (p.causal ? min(total_k, total_k - ql + qi[h] + 1) : total_k) : 0;
        }

        // smallest visibility limit among this warp's valid rows: tiles entirely below it need no masking
        int wlim = min(rvalid[0] ? lim[0] : 0x7fffffff, rvalid[1] ? lim[1] : 0x7fffffff);
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) wlim = min(wlim, __shfl_xor_sync(0xffffffffu, wlim, o));

        // ---- Q fragments (A operand), straight from global memory
        uint32_t qf[KSTEPS][4];
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r0 + wm * 16 + g + 8 * h;
            const int head = kvh * G + (row - qi[h] * G);
            const half* qp = p.q + ((size_t)(row_base + qi[h]) * p.nq + head) * D;
            #pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                qf[ks][h]     = rvalid[h] ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * t) : 0u;
                qf[ks][h + 2] = rvalid[h] ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + 2 * t) : 0u;
            }
        }

        if constexpr (QUANT) {
            // Quantised pools hold codes of the rotated vectors H(k), H(v) (H = H32 / sqrt(32) per group of 32 dims).
            // Instead of rotating every key and value back, the query is rotated once here (q . H(c) = H(q) . c) and the
            // output row once at the end; the tiles below then hold the scaled codes as they are.
            #pragma unroll
            for (int gq = 0; gq < D / 32; ++gq) {
                #pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float v[4][2];
                    #pragma unroll
                    for (int b4 = 0; b4 < 4; ++b4) {
                        const half2 x = *reinterpret_cast<const half2*>(&qf[2 * gq + (b4 >> 1)][h + 2 * (b4 & 1)]);
                        v[b4][0] = __low2float(x); v[b4][1] = __high2float(x);
                    }
                    had32_quad(v, t);
                    #pragma unroll
                    for (int b4 = 0; b4 < 4; ++b4)
                        qf[2 * gq + (b4 >> 1)][h + 2 * (b4 & 1)] = pack_h2(v[b4][0] * R32, v[b4][1] * R32);
                }
            }
        }

        float o_acc[DBLK][4];
        #pragma unroll
        for (int i = 0; i < DBLK; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        const int n_tiles = k_end > k_begin ? (k_end - k_begin + AT_TK - 1) / AT_TK : 0;

        // ---- tile loader: AT_TK keys of kv head kvh, starting at key k0
        auto load_tile = [&](int tile, int stage) {
            const int k0 = k_begin + tile * AT_TK;
            uint8_t* sbase = smem_raw + stage * SM::STAGE;
            if constexpr (!QUANT) {
                // A tile of 64 keys starts at a multiple of 64, so it lies inside one 256-token page: one block-table
                // lookup per tile.  Thread layout: 16-byte chunk tid % 16 of keys tid / 16 + 8 i (D = 128: 16 chunks per
                // key row).  Keys past the end of the split repeat the last valid key (masked later).
                static_assert(D == 128, "loader assumes 16 chunks per key row");
                const size_t tok0 = p.contig_kv ? (size_t)b * p.contig_kv + k0 : (size_t)bt[k0 >> 8] * EXL3_PAGE + (k0 & 255);
                const int kmax = k_end - 1 - k0;
                const int ch = tid & 15, key0 = tid >> 4;
                const size_t rstride = (size_t)p.nkv * D;
                const half* kb = p.kc + (tok0 * p.nkv + kvh) * D + ch * 8;
                const half* vb = p.vc + (tok0 * p.nkv + kvh) * D + ch * 8;
                uint8_t* dk = sbase + ch * 16;
                #pragma unroll
                for (int i = 0; i < AT_TK / 8; ++i) {
                    const int key = key0 + 8 * i;
                    const size_t so = (size_t)min(key, kmax) * rstride;
                    cp_async16(dk + key * SM::ROWB, kb + so);
                    cp_async16(dk + SM::TILE + key * SM::ROWB, vb + so);
                }
            } else {
                // A tile of 64 keys lies inside one page (as above).  Per key and head the codes are bits x 16 bytes (4 groups
                // x bits words) and the scales 8 bytes; two threads share a key: both copy code chunks, one the K scales,
                // the other the V scales.
                static_assert(D == 128, "loader assumes 4 groups per head");
                const int groups = p.nkv * (D / 32);
                const size_t tok0 = (size_t)bt[k0 >> 8] * EXL3_PAGE + (k0 & 255);
                const int key = tid >> 1, half_id = tid & 1;
                const size_t tok = tok0 + min(key, k_end - 1 - k0);
                const uint8_t* ksrc = reinterpret_cast<const uint8_t*>(p.qk + (tok * groups + kvh * 4) * p.k_bits);
                const uint8_t* vsrc = reinterpret_cast<const uint8_t*>(p.qv + (tok * groups + kvh * 4) * p.v_bits);
                uint8_t* kdst = sbase + key * SM::RAW_ROW;
                uint8_t* vdst = sbase + SM::RAW + key * SM::RAW_ROW;
                const int kb = QB == 4 ? 4 : p.k_bits, vb = QB == 4 ? 4 : p.v_bits;
                #pragma unroll
                for (int ch = half_id; ch < kb; ch += 2) cp_async16(kdst + ch * 16, ksrc + ch * 16);
                #pragma unroll
                for (int ch = half_id; ch < vb; ch += 2) cp_async16(vdst + ch * 16, vsrc + ch * 16);
                const half* ssrc = (half_id ? p.sv : p.sk) + tok * groups + kvh * 4;
                cp_async8((half_id ? vdst : kdst) + SM::RAW_ROW - 16, ssrc);
            }
        };

        #pragma unroll
        for (int pre = 0; pre < AT_STAGES - 1; ++pre) {            // tiles 0 .. S-2 in flight before the loop
            if (pre < n_tiles) load_tile(pre, pre);
            cp_async_commit();
        }
        int stage = 0;
        for (int tile = 0; tile < n_tiles; ++tile) {
            const int ahead = tile + AT_STAGES - 1;
            if (ahead < n_tiles) load_tile(ahead, (stage + AT_STAGES - 1) % AT_STAGES);
            cp_async_commit();
            cp_async_wait<AT_STAGES - 1>();
            __syncthreads();

            const uint8_t* ktile; const uint8_t* vtile;
            if constexpr (QUANT) {
                // scale the staged codes into fp16 tiles (rotated domain): one warp-op = 4 groups = the D=128 values of one key
                uint8_t* dk = smem_raw + AT_STAGES * SM::STAGE;
                uint8_t* dv = dk + SM::TILE;
                const uint8_t* raw = smem_raw + stage * SM::STAGE;
                if (QB == 4) {
                    static_assert(!QUANT || D == 128, "the 4-bit path scales one 128-wide head per half warp");
                    #pragma unroll 4
                    for (int key = warp; key < AT_TK; key += 4)
                        dequant4_kv_norot(raw + key * SM::RAW_ROW, raw + SM::RAW + key * SM::RAW_ROW, SM::RAW_ROW - 16,
                                          reinterpret_cast<half*>(dk + key * SM::ROWB), reinterpret_cast<half*>(dv + key * SM::ROWB));
                } else
                #pragma unroll 4                                   // independent keys in flight: the chain per key is latency-bound
                for (int key = warp; key < AT_TK; key += 4) {
                    #pragma unroll
                    for (int part = 0; part < D / 128; ++part) {
                        const uint8_t* rk = raw + key * SM::RAW_ROW;
                        const uint8_t* rv = raw + SM::RAW + key * SM::RAW_ROW;
                        dequant_x4_norot(reinterpret_cast<const uint32_t*>(rk) + part * 4 * p.k_bits,
                                         reinterpret_cast<const half*>(rk + SM::RAW_ROW - 16) + part * 4,
                                         reinterpret_cast<half*>(dk + key * SM::ROWB) + part * 128, p.k_bits);
                        dequant_x4_norot(reinterpret_cast<const uint32_t*>(rv) + part * 4 * p.v_bits,
                                         reinterpret_cast<const half*>(rv + SM::RAW_ROW - 16) + part * 4,
                                         reinterpret_cast<half*>(dv + key * SM::ROWB) + part * 128, p.v_bits);
                    }
                }
                __syncthreads();
                ktile = dk; vtile = dv;
            } else {
                ktile = smem_raw + stage * SM::STAGE;
                vtile = ktile + SM::TILE;
            }

            const int kbase = k_begin + tile * AT_TK + wn * KEYS_W;      // first key of this warp's slice
            // ---- S = Q K^T for the warp's key slice
            float s_acc[NBLK][4];
            #pragma unroll
            for (int nb = 0; nb < NBLK; ++nb) { s_acc[nb][0] = s_acc[nb][1] = s_acc[nb][2] = s_acc[nb][3] = 0.f; }
            #pragma unroll
            for (int nb = 0; nb < NBLK; ++nb) {
                const uint8_t* krow = ktile + (wn * KEYS_W + nb * 8 + (lane & 7)) * SM::ROWB + (lane >> 3) * 16;
                #pragma unroll
                for (int ks = 0; ks < KSTEPS; ks += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(b0, b1, b2, b3, krow + ks * 32);
                    mma_f16(s_acc[nb], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    mma_f16(s_acc[nb], qf[ks + 1][0], qf[ks + 1][1], qf[ks + 1][2], qf[ks + 1][3], b2, b3);
                }
            }
            // ---- scale, mask, online softmax (base 2)
            const bool need_mask = kbase + KEYS_W > wlim || kbase + KEYS_W > k_end;      // warp-uniform
            float mx[2] = {-INFINITY, -INFINITY};
            if (need_mask) {
                #pragma unroll
                for (int nb = 0; nb < NBLK; ++nb)
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int h = e >> 1;
                        const int key = kbase + nb * 8 + 2 * t + (e & 1);
                        float v = s_acc[nb][e] * p.scale_log2;
                        v = (key < lim[h] && key < k_end) ? v : -INFINITY;
                        s_acc[nb][e] = v;
                        mx[h] = fmaxf(mx[h], v);
                    }
            } else {
                #pragma unroll
                for (int nb = 0; nb < NBLK; ++nb)
                    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = s_acc[nb][e] * p.scale_log2;
                        s_acc[nb][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
            }
            float corr[2];
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                corr[h] = (m_new == -INFINITY) ? 1.0f : exp2f(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= corr[h];
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
                #pragma unroll
                for (int i = 0; i < DBLK; ++i) { o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0]; o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1]; }
            }
            // rows that have seen no key yet keep m = -inf: use 0 as the reference so that exp2(-inf - 0) = 0
            const float mref0 = (m_run[0] == -INFINITY) ? 0.f : m_run[0], mref1 = (m_run[1] == -INFINITY) ? 0.f : m_run[1];
            uint32_t pf[NBLK][2];
            #pragma unroll
            for (int nb = 0; nb < NBLK; ++nb) {
                const float e0 = exp2f(s_acc[nb][0] - mref0), e1 = exp2f(s_acc[nb][1] - mref0);
                const float e2 = exp2f(s_acc[nb][2] - mref1), e3 = exp2f(s_acc[nb][3] - mref1);
                l_run[0] += e0 + e1; l_run[1] += e2 + e3;
                pf[nb][0] = pack_h2(e0, e1); pf[nb][1] = pack_h2(e2, e3);
            }
            // ---- O += P V
            #pragma unroll
            for (int kk = 0; kk < KEYS_W / 16; ++kk) {
                const uint8_t* vrow = vtile + (wn * KEYS_W + kk * 16 + (lane & 15)) * SM::ROWB + (lane >> 4) * 16;
                #pragma unroll
                for (int db = 0; db < DBLK; db += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(b0, b1, b2, b3, vrow + db * 16);
                    mma_f16(o_acc[db], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b0, b1);
                    mma_f16(o_acc[db + 1], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b2, b3);
                }
            }
            __syncthreads();      // the stage is refilled by the next iteration's loads
            stage = stage + 1 == AT_STAGES ? 0 : stage + 1;
        }
        cp_async_wait<0>();
        __syncthreads();

        // ---- row sums across the 4 lanes that share a row
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }

        // ---- merge the WN key slices through shared memory: layout [warp][16 rows][D+4] fp32, cols D..D+1 = m, l
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
        // one warp per output row: lane covers D/32 consecutive dims
        for (int lr = warp; lr < ROWS; lr += 4) {
            const int row = r0 + lr;
            if (row >= ql * G) break;
            const int tile_m = lr >> 4, rr = lr & 15;
            float mm = -INFINITY;
            #pragma unroll
            for (int w = 0; w < WN; ++w) mm = fmaxf(mm, ms[((tile_m * WN + w) * 16 + rr) * MS + D]);
            float ll = 0.f;
            float acc[D / 32];
            #pragma unroll
            for (int e = 0; e < D / 32; ++e) acc[e] = 0.f;
            #pragma unroll
            for (int w = 0; w < WN; ++w) {
                const float* src = ms + ((tile_m * WN + w) * 16 + rr) * MS;
                const float mw = src[D];
                const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
                ll += src[D + 1] * sc;
                #pragma unroll
                for (int e = 0; e < D / 32; ++e) acc[e] += src[lane * (D / 32) + e] * sc;
            }
            if constexpr (QUANT) {
                // back out of the rotated domain: lane = (group lane / 8, values 4 (lane % 8) .. +3), as in the KV codec
                static_assert(!QUANT || D == 128, "one warp = the 4 groups of a 128-wide head");
                h4(acc[0], acc[1], acc[2], acc[3]);
                h8_lanes(acc[0], acc[1], acc[2], acc[3], lane);
                #pragma unroll
                for (int e = 0; e < D / 32; ++e) acc[e] *= R32;
            }
            const int qidx = row / G, head = kvh * G + (row - qidx * G);
            if (splits == 1) {
                const float inv = ll > 0.f ? 1.0f / ll : 0.f;
                half* op = p.o + ((size_t)(row_base + qidx) * p.nq + head) * D + lane * (D / 32);
                #pragma unroll
                for (int e = 0; e < D / 32; e += 2)
                    *reinterpret_cast<uint32_t*>(op + e) = pack_h2(acc[e] * inv, acc[e + 1] * inv);
            } else {
                float* pp = p.partial + (((size_t)item_idx * p.nkv + kvh) * ROWS + lr) * (D + 2);
                #pragma unroll
                for (int e = 0; e < D / 32; ++e) pp[lane * (D / 32) + e] = acc[e];
                if (lane == 0) { pp[D] = mm; pp[D + 1] = ll; }
            }
        }
        __syncthreads();
    }
}

}  // namespace exl3
