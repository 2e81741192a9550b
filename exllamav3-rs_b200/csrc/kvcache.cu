// Paged KV-cache write path: fp16 append, quantise on write, dequantise (bulk and compact window).
//
// Quantised format (reference: kernels/cache/q_cache_kernels.cuh:61-236): per token the nkv*hd values are split into
// groups of 32; a group is rotated by H32/sqrt(32), scaled by its absmax (stored as fp16) and quantised on the
// midpoint grid to `bits` bits; the codes of a group are stored as bit planes of widths 8,4,2,1 (the binary expansion
// of `bits`, most significant plane first), each plane holding for sub-lane sl (values 4sl..4sl+3) the field
// p0 | p1<<w | p2<<2w | p3<<3w at bit offset sl*4w.
#include "common.cuh"
#include "kvquant.cuh"

namespace {

// sequence/row lookup shared by the write kernels: rectangular [bsz,seq] or ragged via cu_q
__device__ __forceinline__ bool locate_row(const int32_t* cu_q, int b, int s, int seq, long long& in_row)
{
    if (cu_q) {
        const int q0 = cu_q[b], ql = cu_q[b + 1] - q0;
        if (s >= ql) return false;
        in_row = q0 + s;
    } else {
        in_row = (long long)b * seq + s;
    }
    return true;
}

__global__ void __launch_bounds__(256) kv_append_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v,
                                                        uint4* __restrict__ kc, uint4* __restrict__ vc,
                                                        const int32_t* __restrict__ block_table,
                                                        const int32_t* __restrict__ seqlens,
                                                        const int32_t* __restrict__ cu_q, int seq, int chunks,
                                                        int pages, int pps)
{
    const int b = blockIdx.z, s = blockIdx.y;
    long long in_row;
    if (!locate_row(cu_q, b, s, seq, in_row)) return;
    const int pos = seqlens[b] + s;
    const int lp = pos >> 8;
    if (lp >= pps) return;
    const int page = block_table[(size_t)b * pps + lp];
    if (page < 0 || page >= pages) return;
    const size_t dst = ((size_t)page * EXL3_PAGE + (pos & 255)) * chunks;
    for (int c = blockIdx.x * 256 + threadIdx.x; c < chunks; c += gridDim.x * 256) {
        kc[dst + c] = k[(size_t)in_row * chunks + c];
        vc[dst + c] = v[(size_t)in_row * chunks + c];
    }
}

// one warp per 4 groups of one token; grid (chunk blocks, seq, bsz)
__global__ void __launch_bounds__(256) quant_paged_kernel(const half* __restrict__ k_in, uint32_t* __restrict__ qk,
                                                          half* __restrict__ sk, const half* __restrict__ v_in,
                                                          uint32_t* __restrict__ qv, half* __restrict__ sv,
                                                          const int32_t* __restrict__ seqlens,
                                                          const int32_t* __restrict__ block_table,
                                                          const int32_t* __restrict__ cu_q, int seq, int groups,
                                                          int pages, int pps, int k_bits, int v_bits)
{
    const int b = blockIdx.z, s = blockIdx.y;
    long long in_row;
    if (!locate_row(cu_q, b, s, seq, in_row)) return;
    const int pos = seqlens[b] + s;
    const int lp = pos >> 8;
    if (lp >= pps) return;
    const int page = block_table[(size_t)b * pps + lp];
    if (page < 0 || page >= pages) return;
    const size_t tok = (size_t)page * EXL3_PAGE + (pos & 255);
    const int g0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * 4;
    if (g0 >= groups) return;
    const int active = min(4, groups - g0);
    const size_t base = tok * groups + g0;
    const size_t in_base = ((size_t)in_row * groups + g0) * 32;
    exl3::quant_x4(k_in + in_base, qk + base * k_bits, sk + base, active, k_bits);
    exl3::quant_x4(v_in + in_base, qv + base * v_bits, sv + base, active, v_bits);
}

// one warp per 4 groups of one token, 32 (token, chunk) items per warp; grid (blocks, bsz)
__global__ void __launch_bounds__(256) dequant_paged_kernel(const uint32_t* __restrict__ qk, const half* __restrict__ sk,
                                                            half* __restrict__ k_out, const uint32_t* __restrict__ qv,
                                                            const half* __restrict__ sv, half* __restrict__ v_out,
                                                            const int32_t* __restrict__ seqlens,
                                                            const int32_t* __restrict__ block_table, int groups,
                                                            int pages, int out_pages, int pps, int k_bits, int v_bits,
                                                            int compact, int bonus, int window)
{
    const int b = blockIdx.y;
    const int chunks = (groups + 3) >> 2;
    int max_tok = seqlens[b] + bonus;
    if (max_tok > pps * EXL3_PAGE) max_tok = pps * EXL3_PAGE;
    const int first_tok = window > 0 ? max(0, max_tok - window) : 0;
    long long item = ((long long)blockIdx.x * 32) * 8 + (threadIdx.x >> 5);
    for (int it = 0; it < 32; ++it, item += 8) {
        const int tok_idx = (int)(item / chunks);
        if (tok_idx >= max_tok) break;
        if (tok_idx < first_tok) continue;
        const int g0 = (int)(item - (long long)tok_idx * chunks) * 4;
        const int active = min(4, groups - g0);
        const int lp = tok_idx >> 8;
        const int page = block_table[(size_t)b * pps + lp];
        if (page < 0 || page >= pages) continue;
        const size_t tok = (size_t)page * EXL3_PAGE + (tok_idx & 255);
        const size_t opage = compact ? (size_t)b * pps + lp : (size_t)page;
        if (opage >= (size_t)out_pages) continue;
        const size_t otok = opage * EXL3_PAGE + (tok_idx & 255);
        const size_t base = tok * groups + g0, obase = (otok * groups + g0) * 32;
        exl3::dequant_x4(qk + base * k_bits, sk + base, k_out + obase, active, k_bits);
        exl3::dequant_x4(qv + base * v_bits, sv + base, v_out + obase, active, v_bits);
    }
}

}  // namespace

extern "C" int exl3_paged_kv_cache_update(exl3_ctx* ctx, exl3_stream stream, const void* k, const void* v,
                                          void* k_cache, void* v_cache, const int32_t* block_table,
                                          const int32_t* cache_seqlens, const int32_t* cu_q, int bsz, int seq, int nkv,
                                          int hd, int pages, int pages_per_seq)
{
    EXL3_REQUIRE(ctx && k && v && k_cache && v_cache && block_table && cache_seqlens, "paged_kv_cache_update: null argument");
    EXL3_REQUIRE(bsz >= 0 && seq >= 0 && nkv > 0 && hd > 0 && (nkv * hd) % 8 == 0 && pages > 0 && pages_per_seq > 0,
                 "paged_kv_cache_update: bad shape");
    EXL3_REQUIRE(aligned16(k) && aligned16(v) && aligned16(k_cache) && aligned16(v_cache),
                 "paged_kv_cache_update: pointers must be 16-byte aligned");
    EXL3_REQUIRE(bsz <= 65535 && seq <= 65535, "paged_kv_cache_update: bsz and seq must be <= 65535");
    if (bsz == 0 || seq == 0) return EXL3_OK;
    const int chunks = nkv * hd / 8;
    dim3 grid((chunks + 255) / 256, seq, bsz);
    kv_append_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)k, (const uint4*)v, (uint4*)k_cache,
                                                             (uint4*)v_cache, block_table, cache_seqlens, cu_q, seq,
                                                             chunks, pages, pages_per_seq);
    ctx->launches++;
    return exl3_check_launch(ctx, "paged_kv_cache_update");
}

extern "C" int exl3_quant_cache_paged(exl3_ctx* ctx, exl3_stream stream, const void* k_in, void* k_out,
                                      void* k_out_scales, const void* v_in, void* v_out, void* v_out_scales,
                                      const int32_t* cache_seqlens, const int32_t* block_table, const int32_t* cu_q,
                                      int bsz, int seq, int dim, int pages, int pages_per_seq, int k_bits, int v_bits,
                                      int page_size, float compand_a, int in_contiguous)
{
    EXL3_REQUIRE(ctx && k_in && k_out && k_out_scales && v_in && v_out && v_out_scales && cache_seqlens && block_table,
                 "quant_cache_paged: null argument");
    EXL3_REQUIRE(page_size == EXL3_PAGE, "quant_cache_paged: page_size must be 256");
    EXL3_REQUIRE(dim > 0 && dim % 32 == 0, "quant_cache_paged: dim % 32 == 0 required");
    EXL3_REQUIRE(k_bits >= 2 && k_bits <= 8 && v_bits >= 2 && v_bits <= 8, "quant_cache_paged: bits must be 2..8");
    EXL3_REQUIRE(bsz >= 0 && seq >= 0 && bsz <= 65535 && seq <= 65535 && pages > 0 && pages_per_seq > 0, "quant_cache_paged: bad shape");
    if (compand_a > 0.0f) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "quant_cache_paged: compand_a > 0 is not supported");
    if (!in_contiguous) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "quant_cache_paged: in_contiguous = 0 is not supported");
    if (bsz == 0 || seq == 0) return EXL3_OK;
    const int groups = dim / 32;
    dim3 grid((groups + 31) / 32, seq, bsz);
    quant_paged_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const half*)k_in, (uint32_t*)k_out, (half*)k_out_scales,
                                                               (const half*)v_in, (uint32_t*)v_out, (half*)v_out_scales,
                                                               cache_seqlens, block_table, cu_q, seq, groups, pages,
                                                               pages_per_seq, k_bits, v_bits);
    ctx->launches++;
    return exl3_check_launch(ctx, "quant_cache_paged");
}

static int dequant_impl(exl3_ctx* ctx, exl3_stream stream, const void* k_in, const void* k_in_scales, void* k_out,
                        const void* v_in, const void* v_in_scales, void* v_out, const int32_t* cache_seqlens,
                        const int32_t* block_table, int bsz, int dim, int pages, int out_pages, int pps, int k_bits,
                        int v_bits, int page_size, int compact, int bonus, int window, float compand_a)
{
    EXL3_REQUIRE(ctx && k_in && k_in_scales && k_out && v_in && v_in_scales && v_out && cache_seqlens && block_table,
                 "dequant_cache_paged: null argument");
    EXL3_REQUIRE(page_size == EXL3_PAGE, "dequant_cache_paged: page_size must be 256");
    EXL3_REQUIRE(dim > 0 && dim % 32 == 0, "dequant_cache_paged: dim % 32 == 0 required");
    EXL3_REQUIRE(k_bits >= 2 && k_bits <= 8 && v_bits >= 2 && v_bits <= 8, "dequant_cache_paged: bits must be 2..8");
    EXL3_REQUIRE(bsz >= 0 && bsz <= 65535 && pages > 0 && pps > 0 && bonus >= 0, "dequant_cache_paged: bad shape");
    if (compand_a > 0.0f) return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, "dequant_cache_paged: compand_a > 0 is not supported");
    if (bsz == 0) return EXL3_OK;
    const int groups = dim / 32;
    const long long items = (long long)pps * EXL3_PAGE * ((groups + 3) / 4);
    dim3 grid((unsigned)((items + 255) / 256), bsz);
    dequant_paged_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint32_t*)k_in, (const half*)k_in_scales,
                                                                 (half*)k_out, (const uint32_t*)v_in,
                                                                 (const half*)v_in_scales, (half*)v_out, cache_seqlens,
                                                                 block_table, groups, pages, out_pages, pps, k_bits,
                                                                 v_bits, compact, bonus, window);
    ctx->launches++;
    return exl3_check_launch(ctx, "dequant_cache_paged");
}

extern "C" int exl3_dequant_cache_paged(exl3_ctx* ctx, exl3_stream stream, const void* k_in, const void* k_in_scales,
                                        void* k_out, const void* v_in, const void* v_in_scales, void* v_out,
                                        const int32_t* cache_seqlens, const int32_t* block_table, int bsz, int dim,
                                        int pages, int pages_per_seq, int k_bits, int v_bits, int page_size,
                                        int sliding_window, float compand_a)
{
    return dequant_impl(ctx, stream, k_in, k_in_scales, k_out, v_in, v_in_scales, v_out, cache_seqlens, block_table, bsz,
                        dim, pages, pages, pages_per_seq, k_bits, v_bits, page_size, 0, 0, sliding_window, compand_a);
}

extern "C" int exl3_dequant_cache_paged_window(exl3_ctx* ctx, exl3_stream stream, const void* k_in,
                                               const void* k_in_scales, void* k_out, const void* v_in,
                                               const void* v_in_scales, void* v_out, const int32_t* cache_seqlens,
                                               const int32_t* block_table, int bsz, int dim, int pages,
                                               int pages_per_seq, int k_bits, int v_bits, int page_size, int bonus_len,
                                               float compand_a)
{
    return dequant_impl(ctx, stream, k_in, k_in_scales, k_out, v_in, v_in_scales, v_out, cache_seqlens, block_table, bsz,
                        dim, pages, bsz * pages_per_seq, pages_per_seq, k_bits, v_bits, page_size, 1, bonus_len, 0,
                        compand_a);
}
