// The rest of the reference's op surface (src/ffi.rs:28-42,67-75,118-139,166-191): every symbol the Rust crate binds has
// an entry point here, so the crate links against this library.  The element-wise ones are implemented; the ones that
// belong to other model families or to the sampler return EXL3_ERR_UNSUPPORTED with a message until they are built.
#include "common.cuh"

namespace {

__device__ __forceinline__ float tanh_fast(float x)
{
    float r; asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x)); return r;
}

// y = factor * tanh(x / factor) (kernels/softcap.cu:10-52): fp32 element-wise, or fp16 pairs computed in fp32
__global__ void __launch_bounds__(256) softcap_kernel(const void* __restrict__ x, void* __restrict__ y, long long numel, float factor, int fp32)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (fp32) {
        if (i >= numel) return;
        float v = reinterpret_cast<const float*>(x)[i];
        v /= factor; v = tanhf(v); v *= factor;
        reinterpret_cast<float*>(y)[i] = v;
    } else {
        if (2 * i >= numel) return;
        const half2 h = reinterpret_cast<const half2*>(x)[i];
        float v0 = __low2float(h), v1 = __high2float(h);
        v0 /= factor; v1 /= factor; v0 = tanhf(v0); v1 = tanhf(v1); v0 *= factor; v1 *= factor;
        reinterpret_cast<half2*>(y)[i] = __floats2half2_rn(v0, v1);
    }
}

// z = act(x) * y on fp16 pairs (kernels/activation_kernels.cuh:40-79,142-186): the activation is computed in fp32 and
// rounded to fp16, the optional clamp and the product are fp16 operations.  ACT 0: tanh-approximated GELU, 1: relu(x)^2.
template <int ACT>
__global__ void __launch_bounds__(256) act_mul_kernel(const half2* __restrict__ x, const half2* __restrict__ y, half2* __restrict__ z,
                                                      float act_limit, long long pairs)
{
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= pairs) return;
    half2 x2 = x[i], y2 = y[i];
    float a = __low2float(x2), b = __high2float(x2);
    if (ACT == 0) {
        const float c = 0.797884560803f;
        a = 0.5f * a * (1.0 + tanh_fast(c * (a + 0.044715f * a * a * a)));
        b = 0.5f * b * (1.0 + tanh_fast(c * (b + 0.044715f * b * b * b)));
    } else {
        a = fmaxf(0.0f, a); a = a * a;
        b = fmaxf(0.0f, b); b = b * b;
    }
    x2 = __halves2half2(__float2half_rn(a), __float2half_rn(b));
    if (act_limit != 0.0f) {
        y2 = __hmax2(y2, __float2half2_rn(-act_limit));
        y2 = __hmin2(y2, __float2half2_rn(act_limit));
        x2 = __hmin2(x2, __float2half2_rn(act_limit));
    }
    z[i] = __hmul2(x2, y2);
}

int not_built(exl3_ctx* ctx, const char* what)
{
    char buf[200];
    snprintf(buf, sizeof(buf), "%s is exported for link compatibility and not built in this library", what);
    return exl3_fail(ctx, EXL3_ERR_UNSUPPORTED, buf);
}

}  // namespace

extern "C" int exl3_softcap(exl3_ctx* ctx, exl3_stream stream, const void* x, void* y, float factor, int64_t numel, int fp32)
{
    EXL3_REQUIRE(ctx && x && y && numel >= 0 && factor != 0.0f, "softcap: bad argument");
    EXL3_REQUIRE(fp32 || numel % 2 == 0, "softcap: fp16 tensors need an even element count");
    if (numel == 0) return EXL3_OK;
    const long long items = fp32 ? numel : numel / 2;
    softcap_kernel<<<(unsigned)((items + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, y, numel, factor, fp32);
    ctx->launches++;
    return exl3_check_launch(ctx, "softcap");
}

extern "C" int exl3_gelu_mul(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, float act_limit, int64_t numel)
{
    EXL3_REQUIRE(ctx && x && y && z && numel >= 0 && numel % 2 == 0, "gelu_mul: bad argument");
    if (numel == 0) return EXL3_OK;
    act_mul_kernel<0><<<(unsigned)((numel / 2 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const half2*)x, (const half2*)y, (half2*)z, act_limit, numel / 2);
    ctx->launches++;
    return exl3_check_launch(ctx, "gelu_mul");
}

extern "C" int exl3_relu2_mul(exl3_ctx* ctx, exl3_stream stream, const void* x, const void* y, void* z, float act_limit, int64_t numel)
{
    EXL3_REQUIRE(ctx && x && y && z && numel >= 0 && numel % 2 == 0, "relu2_mul: bad argument");
    if (numel == 0) return EXL3_OK;
    act_mul_kernel<1><<<(unsigned)((numel / 2 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const half2*)x, (const half2*)y, (half2*)z, act_limit, numel / 2);
    ctx->launches++;
    return exl3_check_launch(ctx, "relu2_mul");
}

// ---- exported, not built

extern "C" int exl3_gated_rms_norm(exl3_ctx* ctx, exl3_stream, const void*, const void*, void*, const void*, float, float, int, int, int,
                                   int, int)
{ return not_built(ctx, "gated_rms_norm"); }

extern "C" int exl3_gdn_fused_op_2(exl3_ctx* ctx, exl3_stream, const void*, const void*, const void*, const void*, void*, void*, float,
                                   int, int, int)
{ return not_built(ctx, "gdn_fused_op_2"); }

extern "C" int exl3_gdn_chunk_wy(exl3_ctx* ctx, exl3_stream, const void*, const void*, const void*, const void*, void*, void*, int, int,
                                 int, int, int)
{ return not_built(ctx, "gdn_chunk_wy"); }

extern "C" int exl3_gdn_chunk_fused(exl3_ctx* ctx, exl3_stream, const void*, const void*, const void*, const void*, const void*, const void*,
                                    const void*, void*, void*, double, int, int, int, int, int)
{ return not_built(ctx, "gdn_chunk_fused"); }

extern "C" int exl3_recurrent_gated_delta_rule(exl3_ctx* ctx, exl3_stream, const void*, const void*, const void*, void*, void*, int, int,
                                               int, int, const int32_t*, int, int, int)
{ return not_built(ctx, "recurrent_gated_delta_rule"); }

extern "C" int exl3_causal_conv1d_update(exl3_ctx* ctx, exl3_stream, const void*, void*, const int32_t*, const void*, const void*, void*,
                                         int, int, int, int, int, int)
{ return not_built(ctx, "causal_conv1d_update"); }
