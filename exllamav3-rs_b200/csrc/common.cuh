// Shared declarations for the kernels of libexl3b200.so (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include "../../include/exl3_abi.h"

#define EXL3_PAGE 256

struct exl3_graph;

// Per-device state the ops share.  The reference keeps the equivalent in process-wide singletons
// (kernels/quant/exl3_devctx.cu:26-70); here it is explicit and owned by the caller.
struct exl3_ctx {
    int device;
    int num_sms;
    size_t ws_bytes;        // general scratch: split-K partials, attention split-KV partials, A_had
    uint8_t* ws;
    int* counters;          // arrival counters, all zero between calls
    int n_counters;
    int* status;            // device status word (0 = ok)
    cudaStream_t side_stream;
    cudaStream_t aux_stream;    // second lane inside one call: the decode-class attention pass runs beside the long-class one
    cudaEvent_t ev_fork, ev_join;
    uint64_t launches;
    int mma_attn;
    int use_tc;             // 1: tcgen05 GEMM for large M (default), 0: small-M kernel in passes (for A/B runs)
    int use_decode;         // 1: the streaming decode kernel takes calls of up to 16 rows (default), 0: they go the way of larger row counts
    int use_pair;           // 1: the tcgen05 GEMM runs on CTA pairs (cta_group::2, default), 0: one CTA per tile
    // per-stage device times of exl3_step_forward (off by default): events recorded at the stage boundaries of a step that
    // is not being captured, read back at its end
    int stage_prof;
    cudaEvent_t* prof_ev; int* prof_stage; int prof_ev_n;
    double stage_ms[EXL3_STAGES]; int stage_steps;
    int fuse_transform;     // 1: in the step runner the norm / activation kernels write the tensor-core GEMM's transformed activations (default), 0: separate launches
    // Work lists of the attention kernels kept across the layers of one exl3_step_forward call (they depend on the batch's
    // lengths only, not on the layer): slot 0 = decode class, slot 1 = long class.  plan_keep is set for the duration of a
    // step; outside of it every attention call builds its list anew.
    uint8_t* plan_slots;
    size_t plan_slot_bytes;
    int plan_keep;
    int plan_valid[2];
    char err[256];
};

static inline int exl3_fail(exl3_ctx* ctx, int code, const char* msg)
{
    if (ctx) { strncpy(ctx->err, msg, sizeof(ctx->err) - 1); ctx->err[sizeof(ctx->err) - 1] = 0; }
    return code;
}

#define EXL3_REQUIRE(cond, msg) do { if (!(cond)) return exl3_fail(ctx, EXL3_ERR_INVALID, msg); } while (0)

static inline int exl3_check_launch(exl3_ctx* ctx, const char* what)
{
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        char buf[256];
        snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
        cudaGetLastError();
        return exl3_fail(ctx, EXL3_ERR_CUDA, buf);
    }
    return EXL3_OK;
}

static inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

// Transformed activations of up to three EXL3 tensors that share an input, written by the kernel that produces the input
// (norm, activation) instead of by the GEMM's own transform launch: where each tensor's copy goes and its sign vector.
struct exl3_pre_act { const half* suh[3]; half* a_had[3]; int nseg; };
// gemm.cu: fills `pre` and returns true when exl3_gemm_fanout_pre can run these tensors at m rows (tensor-core path)
bool exl3_tc_pre_buffers(exl3_ctx* ctx, int count, const exl3_linear* const* w, int m, exl3_pre_act* pre);
int exl3_gemm_fanout_pre(exl3_ctx* ctx, exl3_stream stream, int count, const exl3_linear* const* w, void* const* C, int m, int c_fp32);
// elementwise.cu
int exl3_rms_norm_pre(exl3_ctx* ctx, exl3_stream stream, const void* x, int x_fp32, const void* w, float* r, float eps,
                      float cbias, float cscale, int rows, int dim, const exl3_pre_act* pre);
int exl3_silu_mul_pre(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, int rows, int dim, const exl3_pre_act* pre);

// Carve `bytes` out of the context scratch starting at *off (256-byte aligned); NULL when it does not fit.
static inline void* exl3_ws_take(exl3_ctx* ctx, size_t* off, size_t bytes)
{
    size_t o = (*off + 255) & ~(size_t)255;
    if (o + bytes > ctx->ws_bytes) return nullptr;
    *off = o + bytes;
    return ctx->ws + o;
}
