// exl3_reconstruct: packed EXL3 trellis tensor -> dense fp16 W[k,n], bit-exact with the reference
// (kernels/quant/reconstruct.cu:11-84).  Write-bound: 2 bytes out per K/8 bytes in.
#include "common.cuh"
#include "exl3_decode.cuh"

namespace {

// One CTA = 16 rows x 128 columns (8 tiles, one per warp).  Tiles are decoded in registers, staged through shared
// memory in row-major order and written with 16-byte stores (each row of the CTA tile is 256 contiguous bytes).
template <int K, int cb>
__global__ void __launch_bounds__(256) reconstruct_kernel(half* __restrict__ out, const uint32_t* __restrict__ trellis,
                                                          int tiles_n, int n)
{
    constexpr int TW = 8 * K;                       // words per tile
    __shared__ __align__(16) uint32_t s_in[8 * TW];
    __shared__ __align__(16) half s_out[16][128 + 8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kt = blockIdx.y, nt0 = blockIdx.x * 8;
    const uint32_t* src = trellis + ((size_t)kt * tiles_n + nt0) * TW;
    for (int i = threadIdx.x; i < 8 * TW / 4; i += 256)
        reinterpret_cast<uint4*>(s_in)[i] = reinterpret_cast<const uint4*>(src)[i];
    __syncthreads();

    uint32_t st[8];
    exl3::lane_states<K>(s_in + warp * TW, lane, st);
    half2 w01 = exl3::decode_pair<cb>(st[0], st[1]);
    half2 w23 = exl3::decode_pair<cb>(st[2], st[3]);
    half2 w45 = exl3::decode_pair<cb>(st[4], st[5]);
    half2 w67 = exl3::decode_pair<cb>(st[6], st[7]);
    const int r = 2 * (lane & 3), c = warp * 16 + (lane >> 2);
    s_out[r][c]         = __low2half(w01);
    s_out[r + 1][c]     = __high2half(w01);
    s_out[r + 8][c]     = __low2half(w23);
    s_out[r + 9][c]     = __high2half(w23);
    s_out[r][c + 8]     = __low2half(w45);
    s_out[r + 1][c + 8] = __high2half(w45);
    s_out[r + 8][c + 8] = __low2half(w67);
    s_out[r + 9][c + 8] = __high2half(w67);
    __syncthreads();

    const int row = threadIdx.x >> 4, chunk = threadIdx.x & 15;
    uint4 v = *reinterpret_cast<const uint4*>(&s_out[row][chunk * 8]);
    *reinterpret_cast<uint4*>(out + (size_t)(kt * 16 + row) * n + nt0 * 16 + chunk * 8) = v;
}

template <int K>
void launch_k(int cb, dim3 grid, cudaStream_t st, half* out, const uint32_t* tr, int tiles_n, int n)
{
    if (cb == 0)      reconstruct_kernel<K, 0><<<grid, 256, 0, st>>>(out, tr, tiles_n, n);
    else if (cb == 1) reconstruct_kernel<K, 1><<<grid, 256, 0, st>>>(out, tr, tiles_n, n);
    else              reconstruct_kernel<K, 2><<<grid, 256, 0, st>>>(out, tr, tiles_n, n);
}

}  // namespace

extern "C" int exl3_reconstruct(exl3_ctx* ctx, exl3_stream stream, void* unpacked, const void* trellis, int k, int n,
                                int K, int mcg, int mul1)
{
    EXL3_REQUIRE(ctx && unpacked && trellis, "reconstruct: null argument");
    EXL3_REQUIRE(k > 0 && n > 0 && k % 16 == 0 && n % 128 == 0, "reconstruct: k % 16 == 0 and n % 128 == 0 required");
    EXL3_REQUIRE(K >= 1 && K <= 8, "reconstruct: K must be 1..8");
    EXL3_REQUIRE(!(mcg && mul1), "reconstruct: both mcg and mul1 set");
    EXL3_REQUIRE(aligned16(unpacked) && aligned16(trellis), "reconstruct: pointers must be 16-byte aligned");
    const int cb = mcg ? 1 : (mul1 ? 2 : 0);
    dim3 grid(n / 128, k / 16);
    cudaStream_t st = (cudaStream_t)stream;
    half* out = (half*)unpacked;
    const uint32_t* tr = (const uint32_t*)trellis;
    switch (K) {
        case 1: launch_k<1>(cb, grid, st, out, tr, n / 16, n); break;
        case 2: launch_k<2>(cb, grid, st, out, tr, n / 16, n); break;
        case 3: launch_k<3>(cb, grid, st, out, tr, n / 16, n); break;
        case 4: launch_k<4>(cb, grid, st, out, tr, n / 16, n); break;
        case 5: launch_k<5>(cb, grid, st, out, tr, n / 16, n); break;
        case 6: launch_k<6>(cb, grid, st, out, tr, n / 16, n); break;
        case 7: launch_k<7>(cb, grid, st, out, tr, n / 16, n); break;
        default: launch_k<8>(cb, grid, st, out, tr, n / 16, n); break;
    }
    ctx->launches++;
    return exl3_check_launch(ctx, "reconstruct");
}
