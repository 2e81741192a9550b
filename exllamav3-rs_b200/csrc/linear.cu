// exl3_linear_forward: the policy layer around the EXL3 product that the reference keeps in Linear::forward
// (src/modules.rs:183-252): zero-extend a narrow input to the padded in_features, multiply (EXL3 tensor or dense fp16
// weight), add the bias, trim the padded output columns, soft-cap.  The reference's switch between its fused kernel and
// reconstruct + cuBLAS above 144 rows has no counterpart: exl3_gemm takes every row count.
#include "common.cuh"

namespace {

// xp[row, 0:k) = x[row, 0:in_last) followed by zeros
__global__ void __launch_bounds__(256) pad_rows_kernel(const half* __restrict__ x, half* __restrict__ xp, int rows, int in_last, int k)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)rows * k) return;
    const int row = (int)(i / k), c = (int)(i - (long long)row * k);
    xp[i] = c < in_last ? x[(size_t)row * in_last + c] : __float2half(0.0f);
}

// y[row, 0:n_out) = softcap(yp[row, 0:n_out) + bias), each step rounded to fp16 like the tensor ops it replaces
// (y + b; then (y / cap).tanh() * cap, src/modules.rs:217-249)
__global__ void __launch_bounds__(256) linear_epilogue_kernel(const half* __restrict__ yp, const half* __restrict__ bias,
                                                              half* __restrict__ y, int rows, int n_pad, int n_out, float softcap)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)rows * n_out) return;
    const int row = (int)(i / n_out), c = (int)(i - (long long)row * n_out);
    half v = yp[(size_t)row * n_pad + c];
    if (bias) v = __hadd(v, bias[c]);
    if (softcap != 0.0f) {
        const half cap = __float2half_rn(softcap);
        half t = __hdiv(v, cap);
        t = __float2half_rn(tanhf(__half2float(t)));
        v = __hmul(t, cap);
    }
    y[i] = v;
}

}  // namespace

extern "C" int exl3_linear_forward(exl3_ctx* ctx, exl3_stream stream, const exl3_linear_layer* L, const void* x, int in_last,
                                   void* y, int rows)
{
    EXL3_REQUIRE(ctx && L && x && y, "linear_forward: null argument");
    const int k = L->w.k, n = L->w.n;
    EXL3_REQUIRE(rows >= 0 && in_last > 0 && in_last <= k, "linear_forward: the input is wider than in_features");
    EXL3_REQUIRE(L->out_unpadded > 0 && L->out_unpadded <= n, "linear_forward: bad out_unpadded");
    EXL3_REQUIRE((L->w.trellis != nullptr) != (L->dense != nullptr), "linear_forward: exactly one of trellis and dense weight");
    if (rows == 0) return EXL3_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool trim = L->trim_padded_out && L->out_unpadded != n;
    const int n_out = trim ? L->out_unpadded : n;
    const bool post = trim || L->bias || L->softcap != 0.0f;
    // scratch at the top of the context's workspace (the GEMM takes its own from the bottom)
    size_t need = 0;
    if (in_last < k) need += (((size_t)rows * k * 2) + 255) & ~(size_t)255;
    if (post) need += (((size_t)rows * n * 2) + 255) & ~(size_t)255;
    if (need > ctx->ws_bytes / 2) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "linear_forward: context scratch too small");
    const size_t lower = (ctx->ws_bytes - need) & ~(size_t)255;      // what stays for the GEMM, 256-byte aligned
    uint8_t* top = ctx->ws + lower;
    const half* xin = (const half*)x;
    if (in_last < k) {
        half* xp = (half*)top; top += (((size_t)rows * k * 2) + 255) & ~(size_t)255;
        const long long tot = (long long)rows * k;
        pad_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>((const half*)x, xp, rows, in_last, k);
        ctx->launches++;
        xin = xp;
    }
    half* yp = post ? (half*)top : (half*)y;
    // the GEMM must not reach into the scratch taken above: lend it the lower part only
    const size_t ws_saved = ctx->ws_bytes;
    ctx->ws_bytes = lower;
    int rc;
    if (L->w.trellis)
        rc = exl3_gemm(ctx, stream, xin, L->w.trellis, yp, L->w.suh, nullptr, L->w.svh, rows, k, n, L->w.K, 0, L->w.cb == 1, L->w.cb == 2);
    else
        rc = exl3_hgemm(ctx, stream, xin, L->dense, yp, rows, k, n, 0);
    ctx->ws_bytes = ws_saved;
    if (rc != EXL3_OK) return rc;
    if (post) {
        const long long tot = (long long)rows * n_out;
        linear_epilogue_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(yp, (const half*)L->bias, (half*)y, rows, n, n_out, L->softcap);
        ctx->launches++;
    }
    return exl3_check_launch(ctx, "linear_forward");
}
