/*
 * exl3_abi.h — C-ABI of libexl3b200.so: the EXL3 decode-step ops for NVIDIA B200 (sm_100a).
 *
 * This is the drop-in boundary for the reference's op surface: every function below replaces one
 * `exl3_shim_*` symbol that the reference's Rust side declares in src/ffi.rs:17-203 and implements in
 * csrc/exl3_shim.cpp.  The op names and semantics are the same; what changes is the calling convention:
 *
 *   reference:  void exl3_shim_<op>(void* tensor_handle, ...)      (at::Tensor* handles, libtorch underneath)
 *   this ABI:   int  exl3_<op>(exl3_ctx*, exl3_stream, <device pointers>, <shapes>, <scalars>)
 *
 * Conventions
 *   - every pointer named below is a DEVICE pointer unless its comment says "host";
 *   - tensors are dense row-major with the shapes given; fp16 is IEEE binary16 ("half");
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - the return value is 0 on success or a negative EXL3_ERR_* code; nothing throws, nothing calls libtorch,
 *     cuBLAS or a CPU fallback;
 *   - buffers are borrowed for the duration of the call (asynchronous work is ordered on `stream`);
 *   - a context owns the per-device scratch the reference keeps in hidden globals (kernels/quant/exl3_devctx.cu:59-70):
 *     split-K partial sums, arrival counters, attention split-KV partials, the device status word.
 *     One context per device per caller thread; calls on one context must be issued from one thread at a time,
 *     and kernels of two calls that share a context must not overlap on the GPU (use one stream per context).
 */
#ifndef EXL3_ABI_H
#define EXL3_ABI_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EXL3_API __attribute__((visibility("default")))
#else
#define EXL3_API
#endif

typedef struct exl3_ctx exl3_ctx;
typedef struct exl3_pool exl3_pool;       /* KV pools + page table, see the end of this file */
typedef void* exl3_stream;

enum {
    EXL3_OK               = 0,
    EXL3_ERR_INVALID      = -1,   /* bad shape / null pointer / misaligned pointer */
    EXL3_ERR_UNSUPPORTED  = -2,   /* a (head_dim, GQA ratio, bits, mode) combination that is not built */
    EXL3_ERR_WORKSPACE    = -3,   /* context scratch too small for this call */
    EXL3_ERR_CUDA         = -4,   /* a CUDA runtime call failed; see exl3_last_error */
    EXL3_ERR_DEVICE_WAIT  = -5,   /* a bounded device-side wait ran out (reported by exl3_ctx_poll_status) */
    EXL3_ERR_NOMEM        = -6
};

/* rope_mode values, as src/ffi.rs:217-219 / kernels/rope.cuh:6-8 */
enum { EXL3_ROPE_NONE = 0, EXL3_ROPE_GPTJ = 1, EXL3_ROPE_NEOX = 2 };

/* ------------------------------------------------------------------------------------------------ context */

/* Create the per-device context (allocates scratch with cudaMalloc on `device`).  `workspace_bytes` = 0 picks the
 * default (512 MiB).  Replaces the reference's DevCtx singleton (kernels/quant/exl3_devctx.cuh:18-40). */
EXL3_API int  exl3_ctx_create(int device, size_t workspace_bytes, exl3_ctx** out);
EXL3_API void exl3_ctx_destroy(exl3_ctx* ctx);
/* host string describing the last error on this context (never NULL) */
EXL3_API const char* exl3_last_error(const exl3_ctx* ctx);
/* Synchronises `stream`, then returns and clears the device status word: 0 or EXL3_ERR_DEVICE_WAIT. */
EXL3_API int  exl3_ctx_poll_status(exl3_ctx* ctx, exl3_stream stream);
/* Self-test of the failure path: launches a kernel whose single bounded wait (`polls` polls, at most 2^20) can never be
 * satisfied.  The kernel gives up, records it in the status word and ends normally; the next exl3_ctx_poll_status
 * returns EXL3_ERR_DEVICE_WAIT and later calls on the context work as before.  No counterpart in the reference (its
 * waits are unbounded spins, kernels/quant/exl3_gemm_inner.cuh barrier code). */
EXL3_API int  exl3_selftest_bounded_wait(exl3_ctx* ctx, exl3_stream stream, uint32_t polls);
/* Per-stage device times of exl3_step_forward, the counterpart of the reference's EXL3_TRUNK_PROF accumulators
 * (src/model.rs:72-116,158-187).  While enabled, a step that is not being captured into a graph records an event at each
 * stage boundary and waits for the last one before it returns.  Stages: 0 descriptors + embedding, 1 attention norm +
 * q/k/v, 2 rope + KV write + attention, 3 o_proj, 4 MLP norm + gate/up, 5 activation + down_proj, 6 head. */
#define EXL3_STAGES 7
EXL3_API int exl3_ctx_stage_profile(exl3_ctx* ctx, int enable);
/* ms[EXL3_STAGES]: milliseconds summed over the `*steps` profiled steps since the last reset. */
EXL3_API int exl3_ctx_stage_times(exl3_ctx* ctx, double* ms, int* steps, int reset);
/* number of kernels this context has launched since creation (for launch accounting in benchmarks) */
EXL3_API uint64_t exl3_ctx_launch_count(const exl3_ctx* ctx);
EXL3_API const char* exl3_version(void);

/* ---------------------------------------------------------------------------------------- EXL3 linear ops */

/* exl3_shim_gemm (src/ffi.rs:18-27, csrc/exl3_shim.cpp:44-53 -> kernels/quant/exl3_gemm.cu:110-339).
 * C[m,n] = H128( fp16(H128(A o suh)/sqrt128) . W ) / sqrt128 o svh, W decoded from `trellis` [k/16, n/16, 16*K] int16.
 * A [m,k] fp16; C fp16 (c_fp32 = 0) or fp32; suh [k], svh [n] fp16; A_had: accepted for signature compatibility and
 * ignored (the transformed activations live in the context's scratch in a kernel-specific layout; pass NULL).  K = bits per weight 1..8; mcg/mul1 select the codebook (both set is an error).
 * k % 128 == 0, n % 128 == 0.  Returns 0 (the reference returns a kernel tag where 0 and 90 mean success). */
EXL3_API int exl3_gemm(exl3_ctx* ctx, exl3_stream stream, const void* A, const void* trellis, void* C, const void* suh,
              void* A_had, const void* svh, int m, int k, int n, int K, int c_fp32, int mcg, int mul1);

/* No counterpart in the reference.  The same product as exl3_gemm for up to 16 rows, for callers that cannot allocate
 * device memory (code running inside an allocator or memory-pool callback, latency-critical loops that must avoid the
 * device synchronisation an allocation may trigger, plug-ins held to a fixed memory budget): it takes no context and
 * calls no cudaMalloc / cudaFree or other allocating routine.  Its scratch is an 8 MiB array built into the library
 * image, present on every GPU that loads the library until the process exits.
 * Limits: m <= 16, k <= 32768, n <= 524288 (larger sizes return EXL3_ERR_WORKSPACE and print the limits to stderr).
 * Warm-up: the first call on a device looks up the array's device address, and the first call per device for each
 * (bits, codebook) pair configures that kernel (with lazy module loading the CUDA runtime may load code and reserve
 * memory at that moment).  Make one call per pair you will use at start-up, outside any stream capture and outside the
 * region that must not allocate; later calls only launch.
 * All calls on a device share the one array, which still holds the previous call's contents (the entry point clears the
 * parts that must start at zero on `stream`): two calls whose kernels can overlap on the GPU - different streams without
 * an ordering between them - race on it.  Call with the target device current. */
EXL3_API int exl3_gemm_noalloc(exl3_stream stream, const void* A, const void* trellis, void* C, const void* suh,
                               const void* svh, int m, int k, int n, int K, int c_fp32, int mcg, int mul1);
/* No counterpart in the reference.  Status of the exl3_gemm_noalloc calls issued so far on the current device:
 * synchronises `stream`, returns EXL3_ERR_DEVICE_WAIT (and clears the word) if a bounded device-side wait ran out in any
 * of them - their output is then incomplete - and EXL3_OK otherwise.  Allocates nothing. */
EXL3_API int exl3_gemm_noalloc_poll_status(exl3_stream stream);

/* exl3_shim_reconstruct (src/ffi.rs:162, csrc/exl3_shim.cpp:162-164 -> kernels/quant/reconstruct.cu:375-386).
 * Dense fp16 W[k,n] from the packed tensor; bit-exact with the reference. */
EXL3_API int exl3_reconstruct(exl3_ctx* ctx, exl3_stream stream, void* unpacked, const void* trellis, int k, int n, int K,
                     int mcg, int mul1);

/* exl3_shim_had_r_128 (src/ffi.rs:159-161, csrc/exl3_shim.cpp:157-159 -> kernels/quant/hadamard.cu:88-173).
 * y = (x.view(-1,128) @ H128) * scale/sqrt(128) with an optional per-column fp16 pre_scale or post_scale [cols].
 * x,y [rows,cols] both fp16 (fp32 = 0) or both fp32; cols % 128 == 0; in place allowed. */
EXL3_API int exl3_had_r_128(exl3_ctx* ctx, exl3_stream stream, const void* x, void* y, const void* pre_scale,
                   const void* post_scale, float scale, int rows, int cols, int fp32);

/* ------------------------------------------------------------------------------------- norm / rope / act */

/* exl3_shim_rms_norm (src/ffi.rs:43-50 -> kernels/norm.cu:313-360). x fp16|fp32 [rows,dim], w fp16 [dim] or NULL,
 * y fp16|fp32.  y = x * (w + constant_bias) * rsqrt(mean(x^2) + eps) * constant_scale.  dim % 4 == 0. */
EXL3_API int exl3_rms_norm(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w, void* y, int y_fp32,
                  float eps, float constant_bias, float constant_scale, int rows, int dim);

/* exl3_shim_rms_norm_res_in (src/ffi.rs:114-117 -> kernels/norm.cu RES_IN): r += x (r fp32 [rows,dim], stored),
 * then y = norm(r) as above. */
EXL3_API int exl3_rms_norm_res_in(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w, void* y,
                         int y_fp32, float* r, float eps, float constant_bias, float constant_scale, int rows, int dim);

/* exl3_shim_rope (src/ffi.rs:51-65, csrc/exl3_shim.cpp:79-91 -> kernels/rope.cu:279-440).  q [bsz,seq,nq,hd] and
 * k [bsz,seq,nk,hd] (k may be NULL) are written to out_q / out_k; NULL for either means in place (the reference's callers
 * pass the input tensor again for that).  Optional per-head RMSNorm with fp16 weights q_norm/k_norm [hd] first, then the
 * rotation of the first 2*n_freq dims; token t of sequence b rotates by position t + positions[b] (positions int32
 * [bsz], device) or t + position when positions is NULL.
 * Ragged form: row_pos (int32 [rows], device) non-NULL -> q,k are packed [rows,...] (bsz*seq = rows) and row r rotates
 * by row_pos[r] (positions/position ignored). */
EXL3_API int exl3_rope(exl3_ctx* ctx, exl3_stream stream, void* q, void* out_q, void* k, void* out_k, const float* inv_freq,
              int n_freq, uint32_t position, const int32_t* positions, const int32_t* row_pos, const void* q_norm,
              const void* k_norm, float norm_eps, float norm_constant_bias, int rope_mode, float attn_factor,
              int bsz, int seq, int nq, int nk, int hd);

/* exl3_shim_silu_mul (src/ffi.rs:125 -> kernels/activation.cu:24-100): z = silu(x) * y in fp16 arithmetic.
 * act_limit must be 0. */
EXL3_API int exl3_silu_mul(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, float act_limit,
                  int64_t numel);
/* exl3_shim_add (src/ffi.rs:124 -> kernels/add.cu:44-110): z = x + y, fp16. */
EXL3_API int exl3_add(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, int64_t numel);

/* exl3_shim_argmax_sample (src/ffi.rs:136 -> kernels/generator/sampling_basic.cu:65-172): ids[r] = argmax of
 * logits[r, 0:max_logit) (max_logit 0 = n), lowest index on ties.  logits fp16 (fp32 = 0) or fp32; ids int64 [rows]. */
EXL3_API int exl3_argmax_sample(exl3_ctx* ctx, exl3_stream stream, const void* logits, int fp32, int64_t* ids, int rows, int n,
                       int max_logit);

/* Token embedding gather, fp16 table [vocab,dim] -> fp32 rows (replaces tch index_select + to_kind(Float),
 * src/modules.rs:430-436).  ids int64 [rows]. */
EXL3_API int exl3_embed(exl3_ctx* ctx, exl3_stream stream, const int64_t* ids, const void* table, float* out, int rows,
               int dim, int vocab);

/* ---------------------------------------------------------------------------------------------- paged KV */

/* exl3_shim_paged_kv_cache_update (src/ffi.rs:76-83, csrc/exl3_shim.cpp:101-106 -> kernels/generator/cache.cu:143-243).
 * Row s of sequence b (k,v [bsz,seq,nkv,hd] fp16) is written at logical position cache_seqlens[b]+s of caches
 * [pages,256,nkv,hd] through block_table [bsz,pages_per_seq] int32.
 * Ragged form: cu_q (int32 [bsz+1], device) non-NULL -> k,v are packed [rows,nkv,hd] and sequence b owns rows
 * [cu_q[b], cu_q[b+1]); `seq` is then only an upper bound on rows per sequence. */
EXL3_API int exl3_paged_kv_cache_update(exl3_ctx* ctx, exl3_stream stream, const void* k, const void* v, void* k_cache,
                               void* v_cache, const int32_t* block_table, const int32_t* cache_seqlens,
                               const int32_t* cu_q, int bsz, int seq, int nkv, int hd, int pages, int pages_per_seq);

/* exl3_shim_bighead_attn_paged (src/ffi.rs:84-96, csrc/exl3_shim.cpp:110-118 -> kernels/attention.cu:1716-2075).
 * Appends k,v (as above; kv_append may be 0 with k = v = NULL) then computes causal GQA attention of
 * q [bsz,q_len,nq,hd] over the first cache_seqlens[b]+kv_append cached keys; query i sees keys
 * j <= total - q_len + i.  sm_scale 0 = 1/sqrt(hd).  o like q.  kv_chunk_size is accepted and ignored (split sizes
 * are derived on the device from the real lengths).
 * Ragged form: cu_q non-NULL -> q,o [rows,nq,hd], k,v [rows,nkv,hd] packed; sequence b owns rows [cu_q[b], cu_q[b+1])
 * and appends exactly those rows.  Then `q_len` is an upper bound on the rows of any one sequence and `kv_append`
 * carries the total number of packed rows (cu_q[bsz]). */
EXL3_API int exl3_bighead_attn_paged(exl3_ctx* ctx, exl3_stream stream, const void* q, const void* k, const void* v,
                            void* k_cache, void* v_cache, const int32_t* block_table, const int32_t* cache_seqlens,
                            const int32_t* cu_q, void* o, int bsz, int q_len, int kv_append, int nq, int nkv, int hd,
                            int pages, int pages_per_seq, int kv_chunk_size, int causal, float sm_scale);

/* exl3_shim_bighead_attn_paged_q (src/ffi.rs:97-113, csrc/exl3_shim.cpp:122-129 -> kernels/attention.cu:2086-2290).
 * Same against the quantised pools: qk/qv [pages,256,groups*bits] int32, sk/sv [pages,256,groups] fp16,
 * groups = nkv*hd/32.  Fresh rows are quantised in first.  compand_a must be 0. */
EXL3_API int exl3_bighead_attn_paged_q(exl3_ctx* ctx, exl3_stream stream, const void* q, const void* k, const void* v, void* qk,
                              void* sk, void* qv, void* sv, const int32_t* block_table, const int32_t* cache_seqlens,
                              const int32_t* cu_q, void* o, int bsz, int q_len, int kv_append, int nq, int nkv, int hd,
                              int pages, int pages_per_seq, int k_bits, int v_bits, int kv_chunk_size, int causal,
                              float sm_scale, float compand_a);

/* exl3_shim_quant_cache_paged (src/ffi.rs:141-146, csrc/exl3_shim.cpp:231-240 -> kernels/cache/q_cache.cu:146-258).
 * k_in,v_in [bsz,seq,nkv*hd] fp16 contiguous (in_contiguous must be 1) -> codes/scales at cache_seqlens[b]+s.
 * page_size must be 256; bits 2..8; compand_a must be 0.  cu_q: ragged form as above. */
EXL3_API int exl3_quant_cache_paged(exl3_ctx* ctx, exl3_stream stream, const void* k_in, void* k_out, void* k_out_scales,
                           const void* v_in, void* v_out, void* v_out_scales, const int32_t* cache_seqlens,
                           const int32_t* block_table, const int32_t* cu_q, int bsz, int seq, int dim, int pages,
                           int pages_per_seq, int k_bits, int v_bits, int page_size, float compand_a,
                           int in_contiguous);

/* exl3_shim_dequant_cache_paged (src/ffi.rs:147-152 -> kernels/cache/q_cache.cu:271-350): tokens [0, cache_seqlens[b])
 * of every sequence are dequantised into fp16 pools k_out/v_out [pages,256,dim] at their physical positions.
 * sliding_window > 0 may skip tokens older than the window. */
EXL3_API int exl3_dequant_cache_paged(exl3_ctx* ctx, exl3_stream stream, const void* k_in, const void* k_in_scales, void* k_out,
                             const void* v_in, const void* v_in_scales, void* v_out, const int32_t* cache_seqlens,
                             const int32_t* block_table, int bsz, int dim, int pages, int pages_per_seq, int k_bits,
                             int v_bits, int page_size, int sliding_window, float compand_a);

/* exl3_shim_dequant_cache_paged_window (src/ffi.rs:153-158 -> kernels/cache/q_cache.cu:352-435): as above but page p
 * of sequence b is written compactly at scratch page b*pages_per_seq+p, tokens [0, cache_seqlens[b]+bonus_len). */
EXL3_API int exl3_dequant_cache_paged_window(exl3_ctx* ctx, exl3_stream stream, const void* k_in, const void* k_in_scales,
                                    void* k_out, const void* v_in, const void* v_in_scales, void* v_out,
                                    const int32_t* cache_seqlens, const int32_t* block_table, int bsz, int dim,
                                    int pages, int pages_per_seq, int k_bits, int v_bits, int page_size,
                                    int bonus_len, float compand_a);

/* ------------------------------------------------------------------------------- graphs, streams, memory */

/* exl3_graph_* (src/ffi.rs:193-197, csrc/exl3_shim.cpp:287-344): capture on the context's side stream and replay.
 * capture_begin switches capture on for the side stream (returned by exl3_side_stream); launch ops on it, then
 * capture_end.  All return 0 on success, 1 on failure like the reference. */
typedef struct exl3_graph exl3_graph;
EXL3_API exl3_graph* exl3_graph_new(exl3_ctx* ctx);
EXL3_API void exl3_graph_free(exl3_graph* g);
EXL3_API int  exl3_graph_capture_begin(exl3_graph* g);
EXL3_API int  exl3_graph_capture_end(exl3_graph* g);
EXL3_API int  exl3_graph_replay(exl3_graph* g);
/* exl3_use_side_stream / exl3_sync_side_stream (src/ffi.rs:198-199): the side stream handle, and a host sync on it */
EXL3_API exl3_stream exl3_side_stream(exl3_ctx* ctx);
EXL3_API int  exl3_sync_side_stream(exl3_ctx* ctx);
/* exl3_empty_cache (src/ffi.rs:200): nothing is cached by this library; kept for surface compatibility (no-op). */
EXL3_API void exl3_empty_cache(void);
/* exl3_cuda_free_mib (src/ffi.rs:202, csrc/exl3_shim.cpp:308-312): free device memory in MiB, -1 on error */
EXL3_API int64_t exl3_cuda_free_mib(void);
/* exl3_shim_set_mma_attn (src/ffi.rs:201) selects the kernel family for sequences with more than 16 packed rows, for A/B
 * runs: 1 = tcgen05/TMEM attention (default), 0 = the mma.sync kernels. */
EXL3_API void exl3_set_mma_attn(exl3_ctx* ctx, int on);

/* ------------------------------------------------------------------------------- step-level entry points
 * The decode step of the reference is host code that builds `ids / block_table / seqlens`, copies them to the device
 * and walks the layers issuing one shim call per op (src/generator.rs:1541-1581 decode_round, :1329-1352
 * prefill_round, :1667-1704 spec_verify_round; src/model.rs:1171-1194 forward_paged_batched;
 * src/modules.rs:634-789,932-940,1020-1035).  Here one call runs the whole step over a PACKED ragged batch: decode
 * rows (1 token), verify rows (a few tokens) and prefill chunks (up to a page) of different sequences share every
 * GEMM, and the per-row descriptors are built on the device.  The result equals running the reference's calls
 * sequence by sequence. */

typedef struct {
    const void* trellis;   /* [k/16, n/16, 16*K] int16 */
    const void* suh;       /* [k] fp16 */
    const void* svh;       /* [n] fp16 */
    int k, n, K, cb;       /* cb: 0 3INST, 1 MCG, 2 MUL1 */
} exl3_linear;

typedef struct {
    exl3_linear q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj;
    const void* attn_norm; /* [hidden] fp16 */
    const void* mlp_norm;  /* [hidden] fp16 */
    const void* q_norm;    /* [hd] fp16 or NULL */
    const void* k_norm;    /* [hd] fp16 or NULL */
    void* k_cache;         /* fp16 pool [pages,256,nkv,hd]              (kv_bits == 0) */
    void* v_cache;
    void* qk; void* sk;    /* quantised pools (kv_bits > 0), see exl3_bighead_attn_paged_q */
    void* qv; void* sv;
} exl3_layer;

typedef struct {
    int n_layers, hidden, nq, nkv, hd, inter, vocab;
    int kv_bits;           /* 0 = fp16 KV pools, 2..8 = quantised pools */
    int pages;             /* pages in every layer's pool */
    float norm_eps;
    float attn_factor;
    int rope_mode;         /* EXL3_ROPE_* */
    int n_freq;
    const float* inv_freq; /* [n_freq] fp32, device */
    const void* embed;     /* [vocab, hidden] fp16 */
    const void* final_norm;/* [hidden] fp16 */
    exl3_linear lm_head;
    const exl3_layer* layers;   /* HOST array of n_layers entries (device pointers inside) */
} exl3_model;

typedef struct {
    const int64_t* ids;         /* [rows] packed token ids, sequence after sequence */
    const int32_t* q_lens;      /* [bsz] rows of each sequence in this step (0 allowed) */
    int32_t* cache_seqlens;     /* [bsz] tokens already cached; advanced by q_lens at the end of the step when `advance` */
    const int32_t* block_table; /* [bsz, pages_per_seq] */
    int bsz, rows, max_q_len, pages_per_seq, advance;
    int all_rows;               /* 0: sample the last row of every sequence; 1: sample every packed row (speculative verify) */
} exl3_batch;

/* exl3_shim_hgemm (src/ffi.rs:66, csrc/exl3_shim.cpp:93 -> kernels/hgemm.cu:19-78): C[m,n] = A[m,k] . B[k,n],
 * fp16 inputs, fp32 accumulation, C fp16 or fp32.  k % 64 == 0, n % 8 == 0. */
EXL3_API int exl3_hgemm(exl3_ctx* ctx, exl3_stream stream, const void* a, const void* b, void* c, int m, int k, int n,
               int c_fp32);

/* The same activations A [m,k] through `count` (1..3) EXL3 tensors, C[i] [m, w[i]->n]: what the reference issues as
 * separate exl3_shim_gemm calls for q/k/v (src/modules.rs:646-648) and gate/up (src/modules.rs:933-934).  Results are
 * those of `count` exl3_gemm calls; tensors that agree in k, bits and codebook share one tensor-core launch. */
EXL3_API int exl3_gemm_fanout(exl3_ctx* ctx, exl3_stream stream, const void* A, int count, const exl3_linear* const* w,
                              void* const* C, int m, int c_fp32);

/* One linear layer as the reference loads it (Linear::load, src/modules.rs:97-165): features padded up to multiples of
 * 128, an EXL3 tensor (w.trellis) or a dense fp16 weight [k, n] (`dense`, w.trellis NULL, w.k / w.n still give the padded
 * sizes), an optional fp16 bias [n], the unpadded sizes, and the output policy. */
typedef struct {
    exl3_linear w;
    const void* dense;      /* fp16 [w.k, w.n] row-major, or NULL */
    const void* bias;       /* fp16 [w.n] or NULL */
    int in_unpadded, out_unpadded;
    int trim_padded_out;    /* 1: y has out_unpadded columns, 0: w.n */
    float softcap;          /* 0 = none, else y = tanh(y / softcap) * softcap */
} exl3_linear_layer;

/* Linear::forward (src/modules.rs:183-252).  x [rows, in_last] fp16 with in_last <= w.k (a narrower input is
 * zero-extended), y [rows, out_unpadded or w.n] fp16.  Bias, trim and soft-cap round to fp16 after each step like the
 * tensor ops they replace.  The reference's choice between its fused kernel and reconstruct + dense GEMM above 144 rows
 * is not reproduced: the product is exl3_gemm (or exl3_hgemm for a dense weight) at every row count. */
EXL3_API int exl3_linear_forward(exl3_ctx* ctx, exl3_stream stream, const exl3_linear_layer* layer, const void* x, int in_last,
                                 void* y, int rows);

/* ---- on-disk EXL3 checkpoints (src/safetensors.rs, Linear::load src/modules.rs:97-165)
 * A safetensors file: 8-byte little-endian header size, a JSON header {name: {dtype, shape, data_offsets}}, the data.
 * exl3_checkpoint_open parses and validates the header the way the reference does before any field can size a read
 * (header size 1..100 MiB and inside the file; shapes non-negative integers; offsets ordered and inside the file; span =
 * product(shape) * element size for the known dtypes).  On failure *out still receives an object whose
 * exl3_checkpoint_error says why; close it in either case.  Host-only: no device is needed until a tensor is read. */
typedef struct exl3_checkpoint exl3_checkpoint;
EXL3_API int  exl3_checkpoint_open(const char* path, exl3_checkpoint** out);
EXL3_API void exl3_checkpoint_close(exl3_checkpoint* ck);
EXL3_API const char* exl3_checkpoint_error(const exl3_checkpoint* ck);
EXL3_API int  exl3_checkpoint_count(const exl3_checkpoint* ck);
EXL3_API const char* exl3_checkpoint_name(const exl3_checkpoint* ck, int index);      /* header order */
EXL3_API int  exl3_checkpoint_has(const exl3_checkpoint* ck, const char* name);
EXL3_API int  exl3_checkpoint_info(const exl3_checkpoint* ck, const char* name, char* dtype, int dtype_cap, int64_t* shape,
                                   int shape_cap, int* ndim, uint64_t* bytes);
/* the tensor's bytes as stored, into device memory of at least `capacity` bytes (positional reads through a pinned
 * staging buffer; returns when the data is on the device) */
EXL3_API int  exl3_checkpoint_read(exl3_checkpoint* ck, const char* name, void* dst_device, size_t capacity, exl3_stream stream);
/* Linear::load: fills `out` from <key>.trellis/.suh/.svh (+ .mcg / .mul1 marker tensors, + .bias) or from <key>.weight
 * [out, in] (+ .bias), trying alt_key (may be NULL) when key has neither; features are padded to multiples of 128 like
 * the reference pads them.  The layer owns one device allocation; release it with exl3_linear_free. */
EXL3_API int  exl3_linear_load(exl3_checkpoint* ck, exl3_stream stream, const char* key, const char* alt_key, int in_features,
                               int out_features, int trim_padded_out, float softcap, exl3_linear_layer* out);
EXL3_API void exl3_linear_free(exl3_linear_layer* layer);

/* Model::load for the dense transformer family of exl3_step_forward (src/model.rs:262-420): reads, from one or more
 * opened files, <prefix>.embed_tokens.weight, per layer <prefix>.layers.<i>.input_layernorm.weight,
 * .post_attention_layernorm.weight, .self_attn.{q,k,v,o}_proj, .self_attn.{q,k}_norm.weight (optional),
 * .mlp.{gate,up,down}_proj, then <prefix>.norm.weight and lm_head; NEOX rotary table from rope_theta; KV planes from
 * `pool` (which must outlive the model).  Projections must be EXL3 tensors without bias and with features that are
 * multiples of 128.  On failure *out still receives an object whose exl3_model_error says why; free it in either case. */
typedef struct exl3_loaded_model exl3_loaded_model;
EXL3_API int  exl3_model_load(exl3_checkpoint* const* shards, int n_shards, exl3_stream stream, const char* prefix, int n_layers,
                              int hidden, int nq, int nkv, int hd, int inter, int vocab, float norm_eps, float rope_theta,
                              const exl3_pool* pool, exl3_loaded_model** out);
EXL3_API const exl3_model* exl3_model_get(const exl3_loaded_model* model);
EXL3_API const char* exl3_model_error(const exl3_loaded_model* model);
EXL3_API void exl3_model_free(exl3_loaded_model* model);

/* bytes of device scratch exl3_step_forward needs for up to `max_rows` packed rows and `max_bsz` sequences (all_rows:
 * for batches that sample every row, whose logits take max_rows * vocab floats) */
EXL3_API size_t exl3_step_scratch_bytes(const exl3_model* model, int max_rows, int max_bsz, int all_rows);

/* Device-side descriptor build (replaces the host loops of src/generator.rs:1548-1571): from q_lens/cache_seqlens it
 * writes cu_q [bsz+1], row_pos [rows] (RoPE position of every packed row) and last_row [bsz] (row whose logits are
 * sampled; -1 for empty sequences).  All outputs are device int32 arrays. */
EXL3_API int exl3_step_build_descriptors(exl3_ctx* ctx, exl3_stream stream, const int32_t* q_lens,
                                         const int32_t* cache_seqlens, int bsz, int rows, int32_t* cu_q,
                                         int32_t* row_pos, int32_t* last_row);

/* One forward step over the packed batch.  Writes the greedy token of every sequence to out_tokens [bsz] (int64,
 * device; 0 for empty sequences) and, when logits != NULL, the fp32 logits [bsz, vocab] of the sampled rows.  With
 * batch->all_rows every packed row is sampled: out_tokens [rows], logits [rows, vocab] - row r of a sequence carries the
 * model's choice after its first r + 1 tokens of this step, which is what a speculative verify round compares with the
 * draft (src/generator.rs:1649-1790). */
EXL3_API int exl3_step_forward(exl3_ctx* ctx, exl3_stream stream, const exl3_model* model, const exl3_batch* batch,
                               void* scratch, size_t scratch_bytes, int64_t* out_tokens, float* logits);

/* ------------------------------------------------------------------------------- the rest of the op surface
 * Every remaining exl3_shim_* symbol of src/ffi.rs has an entry point so that the crate links.  mgemm, softcap, gelu_mul
 * and relu2_mul are implemented; the others return EXL3_ERR_UNSUPPORTED (with a message in exl3_last_error) until built:
 * they serve other model families (mixture-of-experts routing, gated-delta-net layers, vision towers) or the sampler. */

/* exl3_shim_softcap (src/ffi.rs:123 -> kernels/softcap.cu:55-97): y = factor * tanh(x / factor), fp16 or fp32, in place allowed */
EXL3_API int exl3_softcap(exl3_ctx* ctx, exl3_stream stream, const void* x, void* y, float factor, int64_t numel, int fp32);
/* exl3_shim_gelu_mul / exl3_shim_relu2_mul (src/ffi.rs:126-127 -> kernels/activation.cu:181-330): z = act(x) * y, fp16;
 * act_limit != 0 clamps y to [-limit, limit] and act(x) to <= limit before the product */
EXL3_API int exl3_gelu_mul(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, float act_limit, int64_t numel);
EXL3_API int exl3_relu2_mul(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, float act_limit, int64_t numel);
/* exl3_shim_mgemm (src/ffi.rs:28-42, csrc/exl3_shim.cpp:57-75 -> kernels/quant/exl3_gemm.cu:386-678): EXL3 products over a
 * device table of tensors chosen by device-resident indices (the MoE decode path; no routing readback).  There are
 * bszm = max(bszm_in, bszm_out) slots.  Slot j multiplies A[j] (A [bszm_in, m, k] fp16; bszm_in = 1: every slot reads
 * A[0]) with tensor indices[j] (int64 [bszm], device; NULL: tensor j; a negative entry skips the slot and leaves its rows
 * of C untouched) into C[j] (C [bszm, m, n] fp16 or fp32).  trellis/suh/svh: device arrays of device pointers, one per
 * tensor, all tensors k x n at K bits with one codebook.  weights (fp16 [bszm], device) or NULL: slot j is scaled by
 * weights[j], and afterwards the bszm / num_tokens consecutive slots of each token are added in slot order (in C's
 * precision, unused slots skipped) into C[t] for token t.  A_had is accepted and ignored. */
EXL3_API int exl3_mgemm(exl3_ctx* ctx, exl3_stream stream, const void* A, const void* const* trellis, void* C,
                        const void* const* suh, void* A_had, const void* const* svh, const int64_t* indices,
                        const void* weights, int bszm_in, int bszm_out, int m, int k, int n, int K, int c_fp32, int mcg,
                        int mul1, int num_tokens);
/* exl3_shim_bighead_attn (src/ffi.rs:67-75 -> kernels/attention.cu:2292-2437): attention over plain tensors, q and o
 * [bsz,q_len,nq,hd], k and v [bsz,kv_len,nkv,hd], fp16; a causal query i sees keys <= kv_len - q_len + i.  hd = 128 only
 * (UNSUPPORTED otherwise); kv_chunk_size must be positive and is otherwise ignored; sm_scale 0 = 1/sqrt(hd). */
EXL3_API int exl3_bighead_attn(exl3_ctx* ctx, exl3_stream stream, const void* q, const void* k, const void* v, void* o, int bsz,
                               int q_len, int kv_len, int nq, int nkv, int hd, int kv_chunk_size, int causal, float sm_scale);
/* exl3_shim_gated_rms_norm (src/ffi.rs:118-122).  Not built. */
EXL3_API int exl3_gated_rms_norm(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* w, void* y, const void* g, float eps,
                                 float constant_bias, int w_groups, int gate_first, int gate_act, int rows, int dim);
/* exl3_shim_apply_rep_pens / exl3_shim_apply_pres_freq_pens (src/ffi.rs:128-135 -> kernels/generator/rep_pen.cu:24-245):
 * penalties over the token history past_ids (int64 [past_len], device) of ONE row of logits (rows must be 1, like the
 * reference); in_logits fp16 or fp32 [1, vocab], out_logits fp32 [1, vocab].  A history position at distance d from the
 * end weighs 1 for d <= sustain_range, then falls linearly to 0 over decay_range.  rep_p divides positive logits and
 * multiplies negative ones, blended by the largest weight of the token; pres_p (largest weight) and freq_p (sum of
 * weights) are subtracted; both must be >= 0. */
EXL3_API int exl3_apply_rep_pens(exl3_ctx* ctx, exl3_stream stream, const void* in_logits, int in_fp32, void* out_logits,
                                 const int64_t* past_ids, float rep_p, int sustain_range, int decay_range, int rows, int vocab,
                                 int past_len);
EXL3_API int exl3_apply_pres_freq_pens(exl3_ctx* ctx, exl3_stream stream, const void* in_logits, int in_fp32, void* out_logits,
                                       const int64_t* past_ids, float pres_p, float freq_p, int sustain_range, int decay_range,
                                       int rows, int vocab, int past_len);
/* exl3_shim_gumbel_sample / exl3_shim_gumbel_noise_f32 (src/ffi.rs:137-138 -> kernels/generator/sampling_basic.cu:93-129,
 * gumbel.cu:47-66): Gumbel noise -log(-log(u)) from the reference's Philox4x32-10 stream (seed `random`), added to fp32
 * logits element by element (noise), or added and followed by the row argmax over the first max_logit columns (sample;
 * 0 = all; logits fp16 or fp32 [rows, n], ids int64 [rows]; every row sees the same noise, as in the reference). */
EXL3_API int exl3_gumbel_sample(exl3_ctx* ctx, exl3_stream stream, const void* logits, int fp32, int64_t* ids, int rows, int n,
                                int max_logit, uint32_t random);
EXL3_API int exl3_gumbel_noise_f32(exl3_ctx* ctx, exl3_stream stream, const float* logits_in, float* logits_out, int64_t numel,
                                   uint32_t random);
/* exl3_shim_cache_rotate (src/ffi.rs:139 -> kernels/generator/cache.cu:11-85): for i in 0..n_order:
 * (page order[2i] or temp) <- (page order[2i+1] or temp), -1 standing for `temp` (one page of device scratch); order is
 * a device array of 2 * n_order int32; pages of page_bytes (a multiple of 16) bytes each. */
EXL3_API int exl3_cache_rotate(exl3_ctx* ctx, exl3_stream stream, void* cache, const int32_t* order, void* temp, int pages,
                               int n_order, size_t page_bytes);
/* exl3_shim_mul_sigmoid_ (src/ffi.rs:166 -> kernels/activation.cu:532-568): x *= sigmoid(y) in place, fp16, numel even.
 * exl3_shim_deinterleave_qg (src/ffi.rs:167 -> kernels/activation.cu:721-784): qg [rows, heads, 2, head_dim] fp16 ->
 * q, g [rows, heads, head_dim]; head_dim a multiple of 8. */
EXL3_API int exl3_mul_sigmoid_(exl3_ctx* ctx, exl3_stream stream, void* x, const void* y, int64_t numel);
EXL3_API int exl3_deinterleave_qg(exl3_ctx* ctx, exl3_stream stream, const void* qg, void* q, void* g, int rows, int heads, int head_dim);
/* hybrid-architecture ops (src/ffi.rs:163-191 -> kernels/gdn.cu, gdn_chunk.cu).  Not built. */
EXL3_API int exl3_gdn_fused_op_2(exl3_ctx* ctx, exl3_stream stream, const void* b, const void* a, const void* dt_bias, const void* a_log,
                                 void* beta, void* g, float beta_scale, int bsz, int seq, int heads);
EXL3_API int exl3_gdn_chunk_wy(exl3_ctx* ctx, exl3_stream stream, const void* k, const void* v, const void* beta, const void* a_log,
                               void* w, void* uv, int bsz, int heads, int chunks, int k_dim, int v_dim);
EXL3_API int exl3_gdn_chunk_fused(exl3_ctx* ctx, exl3_stream stream, const void* w, const void* q, const void* k, const void* qkt,
                                  const void* uv, const void* alog, const void* h0, void* out, void* ht, double scale, int bsz,
                                  int heads, int chunks, int k_dim, int v_dim);
EXL3_API int exl3_recurrent_gated_delta_rule(exl3_ctx* ctx, exl3_stream stream, const void* mixed_qkv, const void* g, const void* beta,
                                             void* recurrent_state, void* core_attn_out, int num_k_heads, int num_v_heads,
                                             int k_head_dim, int v_head_dim, const int32_t* slots, int history, int bsz, int seq);
EXL3_API int exl3_causal_conv1d_update(exl3_ctx* ctx, exl3_stream stream, const void* x, void* conv_state, const int32_t* slots,
                                       const void* weight, const void* bias, void* out, int activation, int history, int bsz,
                                       int seq, int dim, int width);

/* --------------------------------------------------------------------------------------- pools and page table
 * The reference keeps the paged KV pools and the page allocator on the Rust side: PagedCache::new / QuantPagedCache::new
 * (src/paged.rs:18-92) allocate one K and one V plane per layer, PageTable (src/paged.rs:330-506) hands out 256-token
 * pages from a free list, counts references per physical page and shares complete prompt-prefix pages between
 * sequences through chained content hashes (least recently released hashed pages are repurposed when the free list is
 * empty).  A host that has no tensor library gets the same objects here; the page table is host state, the planes are
 * device memory owned by the pool. */
/* k_bits = v_bits = 0: fp16 planes [pages,256,nkv,hd]; 2..8: int32 codes [pages,256,groups*bits] + fp16 scales
 * [pages,256,groups], groups = nkv*hd/32.  All planes start zeroed.  EXL3_ERR_NOMEM when the device cannot hold them.
 * n_layers = 0 creates the page table alone (no device memory, no device needed). */
EXL3_API int  exl3_pool_create(int device, int n_layers, int pages, int nkv, int hd, int k_bits, int v_bits, exl3_pool** out);
EXL3_API void exl3_pool_destroy(exl3_pool* pool);
/* device pointers of one layer: fp16 pools -> *k, *v (sk, sv NULL); quantised -> *k = codes of K, *sk = scales of K, ... */
EXL3_API int  exl3_pool_layer(const exl3_pool* pool, int layer, void** k, void** v, void** sk, void** sv);
EXL3_API int  exl3_pool_num_pages(const exl3_pool* pool);
EXL3_API void exl3_pool_kv_bits(const exl3_pool* pool, int* k_bits, int* v_bits);
/* pages that can be handed out: free + unreferenced hashed ones (PageTable::num_free) */
EXL3_API int  exl3_pool_num_free(const exl3_pool* pool);
EXL3_API int  exl3_pool_refcount(const exl3_pool* pool, int page);
/* PageTable::alloc: n fresh pages (reference count 1 each) into out_pages (host), or EXL3_ERR_NOMEM and nothing taken */
EXL3_API int  exl3_pool_alloc(exl3_pool* pool, int n, int32_t* out_pages);
/* PageTable::alloc_prefix: pages for a prompt of n_ids tokens plus gen_reserve tokens.  With sharing switched on
 * (exl3_pool_set_dedup) the complete leading pages whose chained hash is registered are shared instead of taken fresh;
 * *out_matched_tokens = tokens already resident in them.  out_block (host) receives *out_count page ids. */
EXL3_API int  exl3_pool_alloc_prefix(exl3_pool* pool, const int64_t* prompt_ids, int n_ids, int gen_reserve, int32_t* out_block,
                                     int block_capacity, int* out_count, int64_t* out_matched_tokens);
EXL3_API void exl3_pool_set_dedup(exl3_pool* pool, int on);
/* PageTable::register_page_hash: `page` now holds the complete 256-token span token_ids (host); prev_page = the page
 * before it in the sequence or -1.  Idempotent; spans of other lengths are ignored. */
EXL3_API int  exl3_pool_register_page_hash(exl3_pool* pool, int page, int prev_page, const int64_t* token_ids, int n_ids);
/* PageTable::release: drop one reference per listed page; unreferenced pages go back to the free list, or, if they
 * carry a hash, to the reclaimable queue */
EXL3_API int  exl3_pool_release(exl3_pool* pool, const int32_t* pages, int n);
/* PageTable::drain_evicted: hashed pages that were repurposed since the last call; returns how many were written */
EXL3_API int  exl3_pool_drain_evicted(exl3_pool* pool, int32_t* out_pages, int capacity);
/* PageTable::prefix_stats */
EXL3_API void exl3_pool_prefix_stats(const exl3_pool* pool, uint64_t* cached_tokens, uint64_t* prompt_tokens);

#ifdef __cplusplus
}
#endif
#endif /* EXL3_ABI_H */
