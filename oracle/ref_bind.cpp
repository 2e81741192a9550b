// Raw-pointer binding over the reference's own CUDA ops, for the tests only (never part of the product library).
//
// The reference exposes its ops to Rust as `exl3_shim_*` functions that take `at::Tensor*` handles
// (csrc/exl3_shim.cpp).  The tests here work with device pointers, so this file wraps a pointer + shape in a
// non-owning at::Tensor (at::from_blob) and forwards to the same kernel host functions, with the same fixed
// arguments the reference shim passes (csrc/exl3_shim.cpp:44-53,79-91,101-129,140-164,226-277).
// Ops run on torch's current stream of the current device.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAFunctions.h>
#include <cstdint>
#include <cstdio>
#include <exception>

#include "norm.cuh"
#include "rope.cuh"
#include "hgemm.cuh"
#include "attention.cuh"
#include "activation.cuh"
#include "add.cuh"
#include "softcap.cuh"
#include "quant/exl3_gemm.cuh"
#include "quant/hadamard.cuh"
#include "quant/reconstruct.cuh"
#include "generator/cache.cuh"
#include "generator/sampling_basic.cuh"
#include "generator/rep_pen.cuh"
#include "generator/gumbel.cuh"
#include "cache/q_cache.cuh"

extern "C" void exl3_set_mma_attn(int on);

namespace {
at::Tensor wrap(const void* p, std::initializer_list<int64_t> shape, at::ScalarType dt)
{
    auto opts = at::TensorOptions().dtype(dt).device(at::kCUDA, c10::cuda::current_device());
    return at::from_blob(const_cast<void*>(p), at::IntArrayRef(shape.begin(), shape.size()), opts);
}
c10::optional<at::Tensor> owrap(const void* p, std::initializer_list<int64_t> shape, at::ScalarType dt)
{
    if (!p) return c10::nullopt;
    return wrap(p, shape, dt);
}
template <typename F> int guarded(F&& f)
{
    try { f(); return 0; }
    catch (const std::exception& e) { fprintf(stderr, "ref op failed: %s\n", e.what()); return -1; }
    catch (...) { return -1; }
}
}  // namespace

extern "C" {

// returns the reference's kernel tag (0 or 90 = success), -1 on exception
int ref_exl3_gemm(const void* A, const void* B, void* C, const void* suh, void* A_had, const void* svh,
                  int m, int k, int n, int K, int c_fp32, int mcg, int mul1, int force_shape_idx)
{
    int tag = -1;
    int rc = guarded([&] {
        auto a = wrap(A, {m, k}, at::kHalf);
        auto b = wrap(B, {k / 16, n / 16, 16 * K}, at::kShort);
        auto c = wrap(C, {m, n}, c_fp32 ? at::kFloat : at::kHalf);
        tag = exl3_gemm(a, b, c, owrap(suh, {k}, at::kHalf), owrap(A_had, {m, k}, at::kHalf),
                        owrap(svh, {n}, at::kHalf), force_shape_idx, mcg != 0, mul1 != 0, 0);
    });
    return rc ? rc : tag;
}

// exl3_shim_mgemm (csrc/exl3_shim.cpp:57-75): tables are int64 tensors of device pointers; indices int64 [1, bszm],
// weights fp16 [1, bszm] (both optional)
int ref_exl3_mgemm(const void* A, const void* B_tab, void* C, const void* suh_tab, void* A_had, const void* svh_tab,
                   const void* indices, const void* weights, int num_mats, int bszm_in, int bszm_out, int m, int k, int n,
                   int K, int c_fp32, int mcg, int mul1, int num_tokens)
{
    int tag = -1;
    int rc = guarded([&] {
        const int bszm = bszm_in > bszm_out ? bszm_in : bszm_out;
        auto a = wrap(A, {bszm_in, m, k}, at::kHalf);
        auto b = wrap(B_tab, {num_mats}, at::kLong);
        auto c = wrap(C, {bszm_out, m, n}, c_fp32 ? at::kFloat : at::kHalf);
        auto su = wrap(suh_tab, {num_mats}, at::kLong);
        auto sv = wrap(svh_tab, {num_mats}, at::kLong);
        auto ah = wrap(A_had, {bszm, m, k}, at::kHalf);
        tag = exl3_mgemm(a, b, c, su, ah, sv, owrap(indices, {1, bszm}, at::kLong), owrap(weights, {1, bszm}, at::kHalf), K, -1,
                         mcg != 0, mul1 != 0, -1, -1, 0, num_tokens, {}, {});
    });
    return rc ? rc : tag;
}

int ref_reconstruct(void* out, const void* packed, int k, int n, int K, int mcg, int mul1)
{
    return guarded([&] {
        reconstruct(wrap(out, {k, n}, at::kHalf), wrap(packed, {k / 16, n / 16, 16 * K}, at::kShort), K, mcg != 0, mul1 != 0);
    });
}

int ref_had_r_128(const void* x, void* y, const void* pre, const void* post, float scale, int rows, int cols, int fp32)
{
    return guarded([&] {
        auto dt = fp32 ? at::kFloat : at::kHalf;
        had_r_128(wrap(x, {rows, cols}, dt), wrap(y, {rows, cols}, dt), owrap(pre, {cols}, at::kHalf),
                  owrap(post, {cols}, at::kHalf), scale);
    });
}

int ref_hgemm(const void* a, const void* b, void* c, int m, int k, int n, int c_fp32)
{
    return guarded([&] {
        hgemm(wrap(a, {m, k}, at::kHalf), wrap(b, {k, n}, at::kHalf), wrap(c, {m, n}, c_fp32 ? at::kFloat : at::kHalf));
    });
}

int ref_rms_norm(const void* x, int x_fp32, const void* w, void* y, int y_fp32, float eps, float cbias, float cscale,
                 int rows, int dim)
{
    return guarded([&] {
        rms_norm(wrap(x, {rows, dim}, x_fp32 ? at::kFloat : at::kHalf), owrap(w, {dim}, at::kHalf),
                 wrap(y, {rows, dim}, y_fp32 ? at::kFloat : at::kHalf), eps, cbias, cscale, false, false);
    });
}

int ref_rms_norm_res_in(const void* x, int x_fp32, const void* w, void* y, int y_fp32, void* r, int r_fp32, float eps,
                        float cbias, float cscale, int rows, int dim)
{
    return guarded([&] {
        rms_norm_res_in(wrap(x, {rows, dim}, x_fp32 ? at::kFloat : at::kHalf), owrap(w, {dim}, at::kHalf),
                        wrap(y, {rows, dim}, y_fp32 ? at::kFloat : at::kHalf),
                        wrap(r, {rows, dim}, r_fp32 ? at::kFloat : at::kHalf), eps, cbias, cscale);
    });
}

int ref_rope(void* q, void* k, const void* inv_freq, int n_freq, uint32_t position, const void* positions,
             const void* q_norm, const void* k_norm, float norm_eps, float norm_cbias, int rope_mode, float attn_factor,
             int bsz, int seq, int nq, int nk, int hd)
{
    return guarded([&] {
        auto tq = wrap(q, {bsz, seq, nq, hd}, at::kHalf);
        c10::optional<at::Tensor> tk = owrap(k, {bsz, seq, nk, hd}, at::kHalf);
        c10::optional<at::Tensor> ok = tk;
        rope(tq, tq, tk, ok, wrap(inv_freq, {n_freq}, at::kFloat), position, owrap(positions, {bsz}, at::kInt),
             c10::nullopt, rope_mode, attn_factor, owrap(q_norm, {hd}, at::kHalf), owrap(k_norm, {hd}, at::kHalf),
             norm_eps, norm_cbias, 0.0f, 1, 1, 0);
    });
}

int ref_paged_kv_cache_update(const void* k, const void* v, void* kc, void* vc, const void* bt, const void* seqlens,
                              int bsz, int seq, int nkv, int hd, int pages, int pps)
{
    return guarded([&] {
        auto tkc = wrap(kc, {pages, 256, nkv, hd}, at::kHalf), tvc = wrap(vc, {pages, 256, nkv, hd}, at::kHalf);
        auto tbt = wrap(bt, {bsz, pps}, at::kInt), tsl = wrap(seqlens, {bsz}, at::kInt);
        paged_kv_cache_update(wrap(k, {bsz, seq, nkv, hd}, at::kHalf), wrap(v, {bsz, seq, nkv, hd}, at::kHalf),
                              tkc, tvc, tbt, tsl);
    });
}

int ref_bighead_attn_paged(const void* q, const void* k, const void* v, void* kc, void* vc, const void* bt,
                           const void* seqlens, void* o, int bsz, int q_len, int kv_append, int nq, int nkv, int hd,
                           int pages, int pps, int kv_chunk, int causal, float sm_scale)
{
    return guarded([&] {
        bighead_attn_paged(wrap(q, {bsz, q_len, nq, hd}, at::kHalf), wrap(k, {bsz, kv_append, nkv, hd}, at::kHalf),
                           wrap(v, {bsz, kv_append, nkv, hd}, at::kHalf), wrap(kc, {pages, 256, nkv, hd}, at::kHalf),
                           wrap(vc, {pages, 256, nkv, hd}, at::kHalf), wrap(bt, {bsz, pps}, at::kInt),
                           wrap(seqlens, {bsz}, at::kInt), wrap(o, {bsz, q_len, nq, hd}, at::kHalf), kv_chunk,
                           causal != 0, sm_scale);
    });
}

int ref_bighead_attn(const void* q, const void* k, const void* v, void* o, int bsz, int q_len, int kv_len, int nq, int nkv,
                     int hd, int kv_chunk, int causal, float sm_scale)
{
    return guarded([&] {
        bighead_attn(wrap(q, {bsz, q_len, nq, hd}, at::kHalf), wrap(k, {bsz, kv_len, nkv, hd}, at::kHalf),
                     wrap(v, {bsz, kv_len, nkv, hd}, at::kHalf), wrap(o, {bsz, q_len, nq, hd}, at::kHalf), kv_chunk,
                     causal != 0, sm_scale);
    });
}

int ref_bighead_attn_paged_q(const void* q, const void* k, const void* v, void* qk, void* sk, void* qv, void* sv,
                             const void* bt, const void* seqlens, void* o, int bsz, int q_len, int kv_append, int nq,
                             int nkv, int hd, int pages, int pps, int k_bits, int v_bits, int kv_chunk, int causal,
                             float sm_scale)
{
    return guarded([&] {
        int groups = nkv * hd / 32;
        bighead_attn_paged_q(wrap(q, {bsz, q_len, nq, hd}, at::kHalf), wrap(k, {bsz, kv_append, nkv, hd}, at::kHalf),
                             wrap(v, {bsz, kv_append, nkv, hd}, at::kHalf),
                             wrap(qk, {pages, 256, groups * k_bits}, at::kInt), wrap(sk, {pages, 256, groups}, at::kHalf),
                             wrap(qv, {pages, 256, groups * v_bits}, at::kInt), wrap(sv, {pages, 256, groups}, at::kHalf),
                             wrap(bt, {bsz, pps}, at::kInt), wrap(seqlens, {bsz}, at::kInt),
                             wrap(o, {bsz, q_len, nq, hd}, at::kHalf), kv_chunk, causal != 0, sm_scale, 0.0f);
    });
}

int ref_quant_cache_paged(const void* k_in, void* qk, void* sk, const void* v_in, void* qv, void* sv,
                          const void* seqlens, const void* bt, int bsz, int seq, int nkv, int hd, int pages, int pps,
                          int k_bits, int v_bits)
{
    return guarded([&] {
        int groups = nkv * hd / 32;
        quant_cache_paged(wrap(k_in, {bsz, seq, nkv, hd}, at::kHalf), wrap(qk, {pages, 256, groups * k_bits}, at::kInt),
                          wrap(sk, {pages, 256, groups}, at::kHalf), wrap(v_in, {bsz, seq, nkv, hd}, at::kHalf),
                          wrap(qv, {pages, 256, groups * v_bits}, at::kInt), wrap(sv, {pages, 256, groups}, at::kHalf),
                          wrap(seqlens, {bsz}, at::kInt), wrap(bt, {bsz, pps}, at::kInt), 256, seq, 0.0f, true);
    });
}

// window != 0: compact output (dequant_cache_paged_window, `arg` = bonus_len); else in-place pages (`arg` = sliding_window)
int ref_dequant_cache_paged(const void* qk, const void* sk, void* k_out, const void* qv, const void* sv, void* v_out,
                            const void* seqlens, const void* bt, int bsz, int nkv, int hd, int pages, int out_pages,
                            int pps, int k_bits, int v_bits, int window, int arg)
{
    return guarded([&] {
        int groups = nkv * hd / 32;
        auto tqk = wrap(qk, {pages, 256, groups * k_bits}, at::kInt), tsk = wrap(sk, {pages, 256, groups}, at::kHalf);
        auto tqv = wrap(qv, {pages, 256, groups * v_bits}, at::kInt), tsv = wrap(sv, {pages, 256, groups}, at::kHalf);
        auto tko = wrap(k_out, {out_pages, 256, nkv, hd}, at::kHalf), tvo = wrap(v_out, {out_pages, 256, nkv, hd}, at::kHalf);
        auto tsl = wrap(seqlens, {bsz}, at::kInt), tbt = wrap(bt, {bsz, pps}, at::kInt);
        if (window) dequant_cache_paged_window(tqk, tsk, tko, tqv, tsv, tvo, tsl, tbt, 256, arg, 0.0f);
        else        dequant_cache_paged(tqk, tsk, tko, tqv, tsv, tvo, tsl, tbt, 256, arg, 0.0f);
    });
}

int ref_silu_mul(const void* x, const void* y, void* z, int64_t rows, int64_t cols)
{
    return guarded([&] {
        auto tz = wrap(z, {rows, cols}, at::kHalf);
        silu_mul(wrap(x, {rows, cols}, at::kHalf), wrap(y, {rows, cols}, at::kHalf), tz, 0.0f);
    });
}

// act: 0 gelu_mul, 1 relu2_mul (kernels/activation.cu:246-333)
int ref_act_mul(int act, const void* x, const void* y, void* z, float act_limit, int64_t rows, int64_t cols)
{
    return guarded([&] {
        auto tz = wrap(z, {rows, cols}, at::kHalf);
        if (act == 0) gelu_mul(wrap(x, {rows, cols}, at::kHalf), wrap(y, {rows, cols}, at::kHalf), tz, act_limit);
        else relu2_mul(wrap(x, {rows, cols}, at::kHalf), wrap(y, {rows, cols}, at::kHalf), tz, act_limit);
    });
}

int ref_softcap(const void* x, void* y, float factor, int64_t rows, int64_t cols, int fp32)
{
    return guarded([&] {
        softcap(wrap(x, {rows, cols}, fp32 ? at::kFloat : at::kHalf), wrap(y, {rows, cols}, fp32 ? at::kFloat : at::kHalf), factor);
    });
}

int ref_apply_rep_pens(const void* in, int in_fp32, void* out, const void* past, float rep_p, int sustain, int decay, int vocab, int past_len)
{
    return guarded([&] {
        apply_rep_pens(wrap(in, {1, vocab}, in_fp32 ? at::kFloat : at::kHalf), wrap(out, {1, vocab}, at::kFloat),
                       wrap(past, {1, past_len}, at::kLong), rep_p, sustain, decay);
    });
}

int ref_apply_pres_freq_pens(const void* in, int in_fp32, void* out, const void* past, float pres_p, float freq_p, int sustain,
                             int decay, int vocab, int past_len)
{
    return guarded([&] {
        apply_pres_freq_pens(wrap(in, {1, vocab}, in_fp32 ? at::kFloat : at::kHalf), wrap(out, {1, vocab}, at::kFloat),
                             wrap(past, {1, past_len}, at::kLong), pres_p, freq_p, sustain, decay);
    });
}

int ref_gumbel_noise_f32(const void* in, void* out, int64_t numel, uint32_t random)
{
    return guarded([&] {
        auto to = wrap(out, {numel}, at::kFloat);
        gumbel_noise_f32(wrap(in, {numel}, at::kFloat), to, random);
    });
}

int ref_gumbel_sample(const void* logits, void* ids, int rows, int n, int max_logit, uint32_t random)
{
    return guarded([&] {
        auto ti = wrap(ids, {rows, 1}, at::kLong);
        gumbel_sample(wrap(logits, {rows, n}, at::kHalf), ti, max_logit, random);
    });
}

int ref_cache_rotate(void* cache, const void* order, void* temp, int pages, int n_order, int64_t page_bytes)
{
    return guarded([&] {
        cache_rotate(wrap(cache, {pages, page_bytes}, at::kByte), wrap(order, {2 * n_order}, at::kInt), wrap(temp, {page_bytes}, at::kByte));
    });
}

int ref_mul_sigmoid_(void* x, const void* y, int64_t numel)
{
    return guarded([&] {
        auto tx = wrap(x, {numel}, at::kHalf);
        mul_sigmoid_(tx, wrap(y, {numel}, at::kHalf));
    });
}

int ref_deinterleave_qg(const void* qg, void* q, void* g, int rows, int heads, int head_dim)
{
    return guarded([&] {
        auto tq = wrap(q, {rows, heads * head_dim}, at::kHalf), tg = wrap(g, {rows, heads * head_dim}, at::kHalf);
        deinterleave_qg(wrap(qg, {rows, heads * 2 * head_dim}, at::kHalf), tq, tg, head_dim);
    });
}

int ref_add(const void* x, const void* y, void* z, int64_t rows, int64_t cols)
{
    return guarded([&] {
        auto tz = wrap(z, {rows, cols}, at::kHalf);
        add(wrap(x, {rows, cols}, at::kHalf), wrap(y, {rows, cols}, at::kHalf), tz);
    });
}

int ref_argmax_sample(const void* logits, void* ids, int rows, int n, int max_logit)
{
    return guarded([&] {
        auto tids = wrap(ids, {rows, 1}, at::kLong);
        argmax_sample(wrap(logits, {rows, n}, at::kHalf), tids, max_logit);
    });
}

void ref_set_mma_attn(int on) { exl3_set_mma_attn(on); }

}  // extern "C"
