// Step runner: one forward pass of a dense EXL3 transformer over a packed ragged batch, with the per-row descriptors
// built on the device.  Op order and dtypes follow the reference's forward_paged_batched (src/model.rs:1171-1194),
// TransformerBlock::forward (src/modules.rs:1020-1035), Attention::forward (:634-789), GatedMlp::forward (:932-940)
// and finalize_head (src/model.rs:1038-1050): fp32 residual stream, fp16 activations, residual adds fused into the
// next RMSNorm.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(1024) build_desc_kernel(const int32_t* __restrict__ q_lens,
                                                          const int32_t* __restrict__ seqlens, int bsz, int rows,
                                                          int32_t* __restrict__ cu_q, int32_t* __restrict__ row_pos,
                                                          int32_t* __restrict__ last_row)
{
    __shared__ int s_scan[1024];
    __shared__ int s_carry;
    const int tid = threadIdx.x;
    if (tid == 0) { s_carry = 0; cu_q[0] = 0; }
    __syncthreads();
    for (int b0 = 0; b0 < bsz; b0 += 1024) {
        const int b = b0 + tid;
        const int ql = b < bsz ? q_lens[b] : 0;
        s_scan[tid] = ql;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            int v = tid >= o ? s_scan[tid - o] : 0;
            __syncthreads();
            s_scan[tid] += v;
            __syncthreads();
        }
        if (b < bsz) {
            const int end = s_carry + s_scan[tid];
            cu_q[b + 1] = end;
            last_row[b] = (ql > 0 && end <= rows) ? end - 1 : -1;
            const int start = end - ql, pos0 = seqlens[b];
            for (int i = 0; i < ql && start + i < rows; ++i) row_pos[start + i] = pos0 + i;
        }
        __syncthreads();
        if (tid == 1023) s_carry += s_scan[1023];
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256) advance_kernel(int32_t* seqlens, const int32_t* q_lens, int bsz)
{
    const int b = blockIdx.x * 256 + threadIdx.x;
    if (b < bsz) seqlens[b] += q_lens[b];
}

// out[i] = in[idx[i]] (16-byte chunks); rows with idx < 0 are zero-filled
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                          const int32_t* __restrict__ idx, int n_out, int chunks)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)n_out * chunks) return;
    const int r = (int)(i / chunks), c = (int)(i % chunks);
    const int src = idx[r];
    out[i] = src >= 0 ? in[(size_t)src * chunks + c] : make_uint4(0, 0, 0, 0);
}

struct Scratch {
    int32_t *cu_q, *row_pos, *last_row;
    float *resid, *resid_last;
    half *a_in, *q, *k, *v, *attn_o, *proj, *gate, *up, *act, *pend_last, *y_last;
    float* logits;
};

size_t carve(const exl3_model* m, int max_rows, int max_bsz, int head_rows, uint8_t* base, Scratch* s)
{
    size_t off = 0;
    auto take = [&](size_t bytes) -> void* {
        off = (off + 255) & ~(size_t)255;
        void* p = base ? base + off : nullptr;
        off += bytes;
        return p;
    };
    const size_t R = max_rows, B = max_bsz;
    Scratch t;
    t.cu_q = (int32_t*)take((B + 1) * 4);
    t.row_pos = (int32_t*)take(R * 4);
    t.last_row = (int32_t*)take(B * 4);
    t.resid = (float*)take(R * m->hidden * 4);
    t.resid_last = (float*)take(B * m->hidden * 4);
    t.a_in = (half*)take(R * m->hidden * 2);
    t.q = (half*)take(R * m->nq * m->hd * 2);
    t.k = (half*)take(R * m->nkv * m->hd * 2);
    t.v = (half*)take(R * m->nkv * m->hd * 2);
    t.attn_o = (half*)take(R * m->nq * m->hd * 2);
    t.proj = (half*)take(R * m->hidden * 2);
    t.gate = (half*)take(R * m->inter * 2);
    t.up = (half*)take(R * m->inter * 2);
    t.act = (half*)take(R * m->inter * 2);
    t.pend_last = (half*)take(B * m->hidden * 2);
    t.y_last = (half*)take(B * m->hidden * 2);
    t.logits = (float*)take((size_t)head_rows * (size_t)m->vocab * 4);
    if (s) *s = t;
    return (off + 255) & ~(size_t)255;
}

int linear(exl3_ctx* ctx, exl3_stream st, const exl3_linear& w, const void* x, void* y, int rows, int c_fp32)
{
    return exl3_gemm(ctx, st, x, w.trellis, y, w.suh, nullptr, w.svh, rows, w.k, w.n, w.K, c_fp32, w.cb == 1, w.cb == 2);
}

}  // namespace

extern "C" size_t exl3_step_scratch_bytes(const exl3_model* model, int max_rows, int max_bsz, int all_rows)
{
    if (!model || max_rows <= 0 || max_bsz <= 0) return 0;
    return carve(model, max_rows, max_bsz, all_rows ? max_rows : max_bsz, nullptr, nullptr);
}

extern "C" int exl3_step_build_descriptors(exl3_ctx* ctx, exl3_stream stream, const int32_t* q_lens,
                                           const int32_t* cache_seqlens, int bsz, int rows, int32_t* cu_q,
                                           int32_t* row_pos, int32_t* last_row)
{
    EXL3_REQUIRE(ctx && q_lens && cache_seqlens && cu_q && row_pos && last_row, "step_build_descriptors: null argument");
    EXL3_REQUIRE(bsz > 0 && rows >= 0, "step_build_descriptors: bad shape");
    build_desc_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(q_lens, cache_seqlens, bsz, rows, cu_q, row_pos, last_row);
    ctx->launches++;
    return exl3_check_launch(ctx, "step_build_descriptors");
}

#define STEP_TRY(expr) do { int rc_ = (expr); if (rc_ != EXL3_OK) return rc_; } while (0)

// Stage boundaries of a profiled step: an event per boundary on the step's stream, read back when the step has been
// issued.  Mirrors the reference's per-stage accumulators (EXL3_TRUNK_PROF, src/model.rs:72-116,158-187), which bracket
// the stages with device synchronisations; here the step runs as it always does and only the last event is waited for.
namespace {
struct StageProf {
    exl3_ctx* ctx; cudaStream_t st; int n;
    void mark(int stage)
    {
        if (n < ctx->prof_ev_n && cudaEventRecord(ctx->prof_ev[n], st) == cudaSuccess) { ctx->prof_stage[n] = stage; ++n; }
    }
};
}  // namespace
#define STAGE(id) do { if (prof) prof->mark(id); } while (0)

static int step_forward_impl(exl3_ctx* ctx, exl3_stream stream, const exl3_model* m, const exl3_batch* b,
                             void* scratch, size_t scratch_bytes, int64_t* out_tokens, float* logits, StageProf* prof);

extern "C" int exl3_step_forward(exl3_ctx* ctx, exl3_stream stream, const exl3_model* m, const exl3_batch* b,
                                 void* scratch, size_t scratch_bytes, int64_t* out_tokens, float* logits)
{
    EXL3_REQUIRE(ctx && m, "step_forward: null argument");
    StageProf sp{ctx, (cudaStream_t)stream, 0};
    StageProf* prof = nullptr;
    if (ctx->stage_prof && m->n_layers > 0) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing((cudaStream_t)stream, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone) {
            const int need = 3 + 5 * m->n_layers;           // start, embedding, five per layer, head
            if (ctx->prof_ev_n < need) {
                for (int i = 0; i < ctx->prof_ev_n; ++i) cudaEventDestroy(ctx->prof_ev[i]);
                delete[] ctx->prof_ev; delete[] ctx->prof_stage;
                ctx->prof_ev = new cudaEvent_t[need]; ctx->prof_stage = new int[need]; ctx->prof_ev_n = 0;
                for (int i = 0; i < need; ++i) {
                    if (cudaEventCreate(&ctx->prof_ev[i]) != cudaSuccess) break;
                    ctx->prof_ev_n = i + 1;
                }
            }
            if (ctx->prof_ev_n >= need) prof = &sp;
        } else cudaGetLastError();
    }
    STAGE(0);
    const int rc = step_forward_impl(ctx, stream, m, b, scratch, scratch_bytes, out_tokens, logits, prof);
    if (prof && rc == EXL3_OK && sp.n > 1 && cudaEventSynchronize(ctx->prof_ev[sp.n - 1]) == cudaSuccess) {
        for (int i = 1; i < sp.n; ++i) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, ctx->prof_ev[i - 1], ctx->prof_ev[i]) == cudaSuccess) ctx->stage_ms[ctx->prof_stage[i]] += ms;
        }
        ctx->stage_steps++;
    }
    return rc;
}

static int step_forward_impl(exl3_ctx* ctx, exl3_stream stream, const exl3_model* m, const exl3_batch* b,
                             void* scratch, size_t scratch_bytes, int64_t* out_tokens, float* logits, StageProf* prof)
{
    EXL3_REQUIRE(ctx && m && b && scratch && out_tokens, "step_forward: null argument");
    EXL3_REQUIRE(m->layers && m->n_layers > 0 && m->embed && m->final_norm && m->inv_freq, "step_forward: incomplete model");
    EXL3_REQUIRE(b->ids && b->q_lens && b->cache_seqlens && b->block_table, "step_forward: incomplete batch");
    EXL3_REQUIRE(b->bsz > 0 && b->rows > 0 && b->max_q_len > 0 && b->pages_per_seq > 0, "step_forward: bad batch shape");
    EXL3_REQUIRE(aligned16(scratch), "step_forward: scratch must be 16-byte aligned");
    EXL3_REQUIRE(m->kv_bits == 0 || (m->kv_bits >= 2 && m->kv_bits <= 8), "step_forward: kv_bits must be 0 or 2..8");
    Scratch s;
    const size_t need = carve(m, b->rows, b->bsz, b->all_rows ? b->rows : b->bsz, (uint8_t*)scratch, &s);
    // attention work lists are built by the first layer and kept for the others; the flag drops on every way out
    struct PlanKeep {
        exl3_ctx* c;
        explicit PlanKeep(exl3_ctx* ctx_) : c(ctx_) { c->plan_keep = 1; c->plan_valid[0] = c->plan_valid[1] = 0; }
        ~PlanKeep() { c->plan_keep = 0; c->plan_valid[0] = c->plan_valid[1] = 0; }
    } plan_keep(ctx);
    if (need > scratch_bytes) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "step_forward: scratch buffer too small");
    cudaStream_t st = (cudaStream_t)stream;
    const int rows = b->rows, bsz = b->bsz, hidden = m->hidden;

    STEP_TRY(exl3_step_build_descriptors(ctx, stream, b->q_lens, b->cache_seqlens, bsz, rows, s.cu_q, s.row_pos, s.last_row));
    STEP_TRY(exl3_embed(ctx, stream, b->ids, m->embed, s.resid, rows, hidden, m->vocab));

    STAGE(0);                           // descriptors and embedding
    const half* pending = nullptr;      // output of the previous block's MLP, added to the residual by the next norm
    // (measured on the 27B-class shard: 84.6 against 85.3 ms at 1052 rows, but 22.7 against 22.5 ms at 32 rows, where the norm's
    // one CTA per row leaves the three transforms of a row to 32 CTAs: fused from 128 rows on)
    const bool fuse_pre = ctx->fuse_transform != 0 && rows >= 128;
    for (int l = 0; l < m->n_layers; ++l) {
        const exl3_layer& L = m->layers[l];
        {
            // with enough rows for the tensor-core GEMM the norm writes the transformed activations of q/k/v itself
            const exl3_linear* w[3] = {&L.q_proj, &L.k_proj, &L.v_proj};
            void* out[3] = {s.q, s.k, s.v};
            exl3_pre_act pre;
            if (fuse_pre && exl3_tc_pre_buffers(ctx, 3, w, rows, &pre)) {
                if (pending) STEP_TRY(exl3_rms_norm_pre(ctx, stream, pending, 0, L.attn_norm, s.resid, m->norm_eps, 0.f, 1.f, rows, hidden, &pre));
                else         STEP_TRY(exl3_rms_norm_pre(ctx, stream, s.resid, 1, L.attn_norm, nullptr, m->norm_eps, 0.f, 1.f, rows, hidden, &pre));
                STEP_TRY(exl3_gemm_fanout_pre(ctx, stream, 3, w, out, rows, 0));
            } else {
                if (pending) STEP_TRY(exl3_rms_norm_res_in(ctx, stream, pending, 0, L.attn_norm, s.a_in, 0, s.resid, m->norm_eps, 0.f, 1.f, rows, hidden));
                else         STEP_TRY(exl3_rms_norm(ctx, stream, s.resid, 1, L.attn_norm, s.a_in, 0, m->norm_eps, 0.f, 1.f, rows, hidden));
                STEP_TRY(exl3_gemm_fanout(ctx, stream, s.a_in, 3, w, out, rows, 0));
            }
        }
        STAGE(1);                       // attention norm + q/k/v
        STEP_TRY(exl3_rope(ctx, stream, s.q, nullptr, s.k, nullptr, m->inv_freq, m->n_freq, 0, nullptr, s.row_pos, L.q_norm, L.k_norm,
                           m->norm_eps, 0.f, m->rope_mode, m->attn_factor, 1, rows, m->nq, m->nkv, m->hd));
        if (m->kv_bits == 0)
            STEP_TRY(exl3_bighead_attn_paged(ctx, stream, s.q, s.k, s.v, L.k_cache, L.v_cache, b->block_table,
                                             b->cache_seqlens, s.cu_q, s.attn_o, bsz, b->max_q_len, rows, m->nq, m->nkv,
                                             m->hd, m->pages, b->pages_per_seq, 256, 1, 0.f));
        else
            STEP_TRY(exl3_bighead_attn_paged_q(ctx, stream, s.q, s.k, s.v, L.qk, L.sk, L.qv, L.sv, b->block_table,
                                               b->cache_seqlens, s.cu_q, s.attn_o, bsz, b->max_q_len, rows, m->nq,
                                               m->nkv, m->hd, m->pages, b->pages_per_seq, m->kv_bits, m->kv_bits, 256, 1,
                                               0.f, 0.f));
        STAGE(2);                       // rope, KV write, attention
        STEP_TRY(linear(ctx, stream, L.o_proj, s.attn_o, s.proj, rows, 0));
        STAGE(3);                       // o_proj
        {
            const exl3_linear* w[2] = {&L.gate_proj, &L.up_proj};
            void* out[2] = {s.gate, s.up};
            exl3_pre_act pre;
            if (fuse_pre && exl3_tc_pre_buffers(ctx, 2, w, rows, &pre)) {
                STEP_TRY(exl3_rms_norm_pre(ctx, stream, s.proj, 0, L.mlp_norm, s.resid, m->norm_eps, 0.f, 1.f, rows, hidden, &pre));
                STEP_TRY(exl3_gemm_fanout_pre(ctx, stream, 2, w, out, rows, 0));
            } else {
                STEP_TRY(exl3_rms_norm_res_in(ctx, stream, s.proj, 0, L.mlp_norm, s.a_in, 0, s.resid, m->norm_eps, 0.f, 1.f, rows, hidden));
                STEP_TRY(exl3_gemm_fanout(ctx, stream, s.a_in, 2, w, out, rows, 0));
            }
        }
        STAGE(4);                       // MLP norm + gate/up
        {
            const exl3_linear* w[1] = {&L.down_proj};
            void* out[1] = {s.proj};
            exl3_pre_act pre;
            if (fuse_pre && exl3_tc_pre_buffers(ctx, 1, w, rows, &pre)) {
                STEP_TRY(exl3_silu_mul_pre(ctx, stream, s.gate, s.up, rows, m->inter, &pre));
                STEP_TRY(exl3_gemm_fanout_pre(ctx, stream, 1, w, out, rows, 0));
            } else {
                STEP_TRY(exl3_silu_mul(ctx, stream, s.gate, s.up, s.act, 0.f, (int64_t)rows * m->inter));
                STEP_TRY(linear(ctx, stream, L.down_proj, s.act, s.proj, rows, 0));
            }
        }
        STAGE(5);                       // activation + down_proj
        pending = s.proj;
    }

    if (b->all_rows) {
        // head over every packed row (the speculative verify round reads the argmax after each draft token,
        // src/generator.rs:1649-1790): final norm into the free activation buffer, lm_head, argmax per row
        STEP_TRY(exl3_rms_norm_res_in(ctx, stream, pending, 0, m->final_norm, s.a_in, 0, s.resid, m->norm_eps, 0.f, 1.f, rows, hidden));
        float* lga = logits ? logits : s.logits;
        STEP_TRY(linear(ctx, stream, m->lm_head, s.a_in, lga, rows, 1));
        STEP_TRY(exl3_argmax_sample(ctx, stream, lga, 1, out_tokens, rows, m->vocab, 0));
        if (b->advance) {
            advance_kernel<<<(bsz + 255) / 256, 256, 0, st>>>(b->cache_seqlens, b->q_lens, bsz);
            ctx->launches++;
            STEP_TRY(exl3_check_launch(ctx, "step advance"));
        }
        STAGE(6);                       // final norm, lm_head, argmax
        return EXL3_OK;
    }
    // head: only the last row of every sequence (src/model.rs:1038-1050 last_only), logits in fp32
    {
        const long long it = (long long)bsz * (hidden * 4 / 16);
        gather_rows_kernel<<<(unsigned)((it + 255) / 256), 256, 0, st>>>((const uint4*)s.resid, (uint4*)s.resid_last, s.last_row, bsz, hidden * 4 / 16);
        const long long ih = (long long)bsz * (hidden * 2 / 16);
        gather_rows_kernel<<<(unsigned)((ih + 255) / 256), 256, 0, st>>>((const uint4*)pending, (uint4*)s.pend_last, s.last_row, bsz, hidden * 2 / 16);
        ctx->launches += 2;
        STEP_TRY(exl3_check_launch(ctx, "step gather"));
    }
    STEP_TRY(exl3_rms_norm_res_in(ctx, stream, s.pend_last, 0, m->final_norm, s.y_last, 0, s.resid_last, m->norm_eps, 0.f, 1.f, bsz, hidden));
    float* lg = logits ? logits : s.logits;
    STEP_TRY(linear(ctx, stream, m->lm_head, s.y_last, lg, bsz, 1));
    STEP_TRY(exl3_argmax_sample(ctx, stream, lg, 1, out_tokens, bsz, m->vocab, 0));
    if (b->advance) {
        advance_kernel<<<(bsz + 255) / 256, 256, 0, st>>>(b->cache_seqlens, b->q_lens, bsz);
        ctx->launches++;
        STEP_TRY(exl3_check_launch(ctx, "step advance"));
    }
    STAGE(6);                           // final norm, lm_head, argmax
    return EXL3_OK;
}
