// Context, CUDA-graph and memory entry points of libexl3b200.so.
#include "common.cuh"
#include "async_copy.cuh"
#include <new>
#include <stdlib.h>

struct exl3_graph {
    exl3_ctx* ctx;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    bool capturing;
};

extern "C" const char* exl3_version(void) { return "exl3-b200 0.1 (sm_100a)"; }

extern "C" int exl3_ctx_create(int device, size_t workspace_bytes, exl3_ctx** out)
{
    if (!out) return EXL3_ERR_INVALID;
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    exl3_ctx* ctx = new (std::nothrow) exl3_ctx();
    if (!ctx) return EXL3_ERR_NOMEM;
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->mma_attn = 1;
    ctx->use_tc = getenv("EXL3_B200_NO_TC") ? 0 : 1;
    ctx->use_pair = getenv("EXL3_B200_NO_PAIR") ? 0 : 1;
    ctx->fuse_transform = getenv("EXL3_B200_NO_FUSED_TRANSFORM") ? 0 : 1;
    ctx->stage_prof = 0; ctx->prof_ev = nullptr; ctx->prof_stage = nullptr; ctx->prof_ev_n = 0; ctx->stage_steps = 0;
    for (int i = 0; i < EXL3_STAGES; ++i) ctx->stage_ms[i] = 0.0;
    ctx->use_decode = (getenv("EXL3_B200_NO_DECODE") || getenv("EXL3_B200_NO_TC")) ? 0 : 1;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete ctx; cudaGetLastError(); return EXL3_ERR_CUDA; }
    if (prop.major != 10) {
        // the library is built for sm_100a only; refuse other devices instead of failing at the first launch
        delete ctx;
        return EXL3_ERR_UNSUPPORTED;
    }
    ctx->num_sms = prop.multiProcessorCount;
    ctx->ws_bytes = workspace_bytes ? workspace_bytes : ((size_t)512 << 20);
    ctx->n_counters = 1 << 16;
    ctx->plan_slot_bytes = (size_t)1 << 20;
    ctx->plan_keep = 0; ctx->plan_valid[0] = ctx->plan_valid[1] = 0;
    bool ok = cudaMalloc(&ctx->ws, ctx->ws_bytes) == cudaSuccess &&
              cudaMalloc(&ctx->counters, ctx->n_counters * sizeof(int)) == cudaSuccess &&
              cudaMalloc(&ctx->status, 64) == cudaSuccess &&
              cudaMalloc(&ctx->plan_slots, 2 * ctx->plan_slot_bytes) == cudaSuccess &&
              cudaMemset(ctx->counters, 0, ctx->n_counters * sizeof(int)) == cudaSuccess &&
              cudaMemset(ctx->status, 0, 64) == cudaSuccess &&
              cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&ctx->aux_stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming) == cudaSuccess &&
              cudaDeviceSynchronize() == cudaSuccess;
    if (!ok) { cudaGetLastError(); exl3_ctx_destroy(ctx); return EXL3_ERR_NOMEM; }
    strcpy(ctx->err, "no error");
    *out = ctx;
    return EXL3_OK;
}

extern "C" void exl3_ctx_destroy(exl3_ctx* ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->side_stream) cudaStreamDestroy(ctx->side_stream);
    if (ctx->aux_stream) cudaStreamDestroy(ctx->aux_stream);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->counters) cudaFree(ctx->counters);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->plan_slots) cudaFree(ctx->plan_slots);
    for (int i = 0; i < ctx->prof_ev_n; ++i) cudaEventDestroy(ctx->prof_ev[i]);
    delete[] ctx->prof_ev;
    delete[] ctx->prof_stage;
    delete ctx;
}

extern "C" const char* exl3_last_error(const exl3_ctx* ctx) { return ctx ? ctx->err : "null context"; }

extern "C" uint64_t exl3_ctx_launch_count(const exl3_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int exl3_ctx_stage_profile(exl3_ctx* ctx, int enable)
{
    if (!ctx) return EXL3_ERR_INVALID;
    ctx->stage_prof = enable ? 1 : 0;
    return EXL3_OK;
}

extern "C" int exl3_ctx_stage_times(exl3_ctx* ctx, double* ms, int* steps, int reset)
{
    if (!ctx || !ms) return EXL3_ERR_INVALID;
    for (int i = 0; i < EXL3_STAGES; ++i) ms[i] = ctx->stage_ms[i];
    if (steps) *steps = ctx->stage_steps;
    if (reset) { for (int i = 0; i < EXL3_STAGES; ++i) ctx->stage_ms[i] = 0.0; ctx->stage_steps = 0; }
    return EXL3_OK;
}

extern "C" int exl3_ctx_poll_status(exl3_ctx* ctx, exl3_stream stream)
{
    if (!ctx) return EXL3_ERR_INVALID;
    int h = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(&h, ctx->status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaError_t e = cudaGetLastError();
        return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e));
    }
    if (h != 0) {
        // CTAs that gave up may have left arrival counters of shared column blocks half-way: back to the all-zero state
        // every GEMM launch expects
        cudaMemsetAsync(ctx->counters, 0, (size_t)ctx->n_counters * sizeof(int), st);
        cudaMemsetAsync(ctx->status, 0, sizeof(int), st);
        cudaStreamSynchronize(st);
        char buf[128];
        snprintf(buf, sizeof(buf), "a bounded device-side wait ran out (status word %d)", h);
        return exl3_fail(ctx, EXL3_ERR_DEVICE_WAIT, buf);
    }
    return EXL3_OK;
}

// Self-test of the bounded-wait path every kernel of the library uses: one thread waits, with the library's own helper and
// a small poll limit, on an mbarrier that nothing ever arrives on; the wait gives up, the kernel records status 1 in the
// context's status word and returns normally (no trap, no fault).  exl3_ctx_poll_status then reports
// EXL3_ERR_DEVICE_WAIT and the context stays usable.
namespace {
__global__ void selftest_wait_kernel(int* status, uint32_t polls)
{
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        exl3::mbar_init(&bar, 1);
        exl3::mbar_fence_init();
        if (!exl3::mbar_wait(&bar, 0, polls)) atomicExch(status, 1);
    }
}
}  // namespace

extern "C" int exl3_selftest_bounded_wait(exl3_ctx* ctx, exl3_stream stream, uint32_t polls)
{
    if (!ctx) return EXL3_ERR_INVALID;
    if (polls == 0 || polls > (1u << 20)) return exl3_fail(ctx, EXL3_ERR_INVALID, "selftest_bounded_wait: polls must be 1..2^20");
    selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->status, polls);
    ctx->launches++;
    return exl3_check_launch(ctx, "selftest_bounded_wait");
}

extern "C" void exl3_set_mma_attn(exl3_ctx* ctx, int on) { if (ctx) ctx->mma_attn = on ? 1 : 0; }

extern "C" void exl3_empty_cache(void) {}

extern "C" int64_t exl3_cuda_free_mib(void)
{
    size_t f = 0, t = 0;
    if (cudaMemGetInfo(&f, &t) != cudaSuccess) { cudaGetLastError(); return -1; }
    return (int64_t)(f >> 20);
}

extern "C" exl3_stream exl3_side_stream(exl3_ctx* ctx) { return ctx ? (exl3_stream)ctx->side_stream : nullptr; }

extern "C" int exl3_sync_side_stream(exl3_ctx* ctx)
{
    if (!ctx) return EXL3_ERR_INVALID;
    return cudaStreamSynchronize(ctx->side_stream) == cudaSuccess ? EXL3_OK : exl3_fail(ctx, EXL3_ERR_CUDA, "side stream sync failed");
}

extern "C" exl3_graph* exl3_graph_new(exl3_ctx* ctx)
{
    if (!ctx) return nullptr;
    exl3_graph* g = new (std::nothrow) exl3_graph();
    if (!g) return nullptr;
    g->ctx = ctx; g->graph = nullptr; g->exec = nullptr; g->capturing = false;
    return g;
}

extern "C" void exl3_graph_free(exl3_graph* g)
{
    if (!g) return;
    if (g->capturing) { cudaGraph_t tmp = nullptr; cudaStreamEndCapture(g->ctx->side_stream, &tmp); if (tmp) cudaGraphDestroy(tmp); }
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
}

extern "C" int exl3_graph_capture_begin(exl3_graph* g)
{
    if (!g || g->capturing) return 1;
    if (cudaStreamBeginCapture(g->ctx->side_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        exl3_fail(g->ctx, EXL3_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    g->capturing = true;
    return 0;
}

extern "C" int exl3_graph_capture_end(exl3_graph* g)
{
    if (!g || !g->capturing) return 1;
    g->capturing = false;
    if (g->exec) { cudaGraphExecDestroy(g->exec); g->exec = nullptr; }
    if (g->graph) { cudaGraphDestroy(g->graph); g->graph = nullptr; }
    if (cudaStreamEndCapture(g->ctx->side_stream, &g->graph) != cudaSuccess || !g->graph ||
        cudaGraphInstantiate(&g->exec, g->graph, 0) != cudaSuccess) {
        exl3_fail(g->ctx, EXL3_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    return 0;
}

extern "C" int exl3_graph_replay(exl3_graph* g)
{
    if (!g || !g->exec) return 1;
    if (cudaGraphLaunch(g->exec, g->ctx->side_stream) != cudaSuccess) {
        exl3_fail(g->ctx, EXL3_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    return 0;
}
