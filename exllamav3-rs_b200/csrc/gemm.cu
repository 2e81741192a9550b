// exl3_gemm: host-side dispatch of the fused EXL3 trellis-decode GEMM.
#include "gemm_small.cuh"
#include "gemm_tc.cuh"
#include "gemm_decode.cuh"

namespace {

using namespace exl3;

// Input transform: a_dup[row][k] = (h, h) with h = fp16(H128(A o suh)/sqrt128), rowsum[row] = sum_k h.
// One CTA per row; warp w takes 128-blocks w, w+8, ...; the row sum is reduced in a fixed order.
// Arithmetic as kernels/quant/hadamard_inner.cuh:93-147 (fp16 pre-scale multiply, fp32 butterflies, one fp16 rounding).
__global__ void __launch_bounds__(256) gemm_prologue_kernel(const half* __restrict__ A, const half* __restrict__ suh,
                                                            uint32_t* __restrict__ a_dup, float* __restrict__ rowsum,
                                                            int k)
{
    __shared__ float sh[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    float part = 0.0f;
    for (int blk = warp; blk < k / 128; blk += 8) {
        uint2 raw = reinterpret_cast<const uint2*>(A + row * k + blk * 128)[lane];
        half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
        if (suh) {
            uint2 sr = reinterpret_cast<const uint2*>(suh + blk * 128)[lane];
            a = __hmul2(a, *reinterpret_cast<half2*>(&sr.x));
            b = __hmul2(b, *reinterpret_cast<half2*>(&sr.y));
        }
        float v0 = __low2float(a), v1 = __high2float(a), v2 = __low2float(b), v3 = __high2float(b);
        if (suh) {
            float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
            v0 = s0 + s1; v1 = d0 + d1; v2 = s0 - s1; v3 = d0 - d1;
            #pragma unroll
            for (int i = 1; i < 32; i <<= 1) {
                float p0 = __shfl_xor_sync(0xffffffffu, v0, i), p1 = __shfl_xor_sync(0xffffffffu, v1, i);
                float p2 = __shfl_xor_sync(0xffffffffu, v2, i), p3 = __shfl_xor_sync(0xffffffffu, v3, i);
                const bool up = lane & i;
                v0 = (up ? -v0 : v0) + p0; v1 = (up ? -v1 : v1) + p1;
                v2 = (up ? -v2 : v2) + p2; v3 = (up ? -v3 : v3) + p3;
            }
            v0 *= GS_R128; v1 *= GS_R128; v2 *= GS_R128; v3 *= GS_R128;
        }
        const uint32_t h0 = __half_as_ushort(__float2half_rn(v0)), h1 = __half_as_ushort(__float2half_rn(v1));
        const uint32_t h2 = __half_as_ushort(__float2half_rn(v2)), h3 = __half_as_ushort(__float2half_rn(v3));
        uint4 o = make_uint4(h0 * 0x10001u, h1 * 0x10001u, h2 * 0x10001u, h3 * 0x10001u);
        reinterpret_cast<uint4*>(a_dup + row * k + blk * 128)[lane] = o;
        part += __half2float(__ushort_as_half((unsigned short)h0)) + __half2float(__ushort_as_half((unsigned short)h1)) +
                __half2float(__ushort_as_half((unsigned short)h2)) + __half2float(__ushort_as_half((unsigned short)h3));
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) sh[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int w = 0; w < 8; ++w) s += sh[w];
        rowsum[row] = s;
    }
}

// Launch geometry of the persistent kernel: one CTA per resident slot (SMs x occupancy), never more than work units.
struct SmallPlan { int grid; int max_contrib; size_t partial_bytes; };

template <int K, int CB, int MT>
cudaError_t launch_small(GemmSmallParams& p, int num_sms, size_t partial_room, float* partial_base, cudaStream_t st,
                         SmallPlan* plan_out)
{
    constexpr int bytes = GemmSmallSmem<K, MT>::BYTES;
    static int occ[64] = {};            // per (K, CB, MT) instantiation and device; 0 = not configured yet
    auto kern = gemm_small_kernel<K, CB, MT>;
    int dev = 0;
    cudaGetDevice(&dev);
    int ctas_per_sm = (dev >= 0 && dev < 64) ? occ[dev] : 0;
    if (ctas_per_sm == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kern, 256, bytes);
        if (e != cudaSuccess) return e;
        if (ctas_per_sm < 1) ctas_per_sm = 1;
        if (dev >= 0 && dev < 64) occ[dev] = ctas_per_sm;
    }
    const int NST = p.k / 128;
    const long long total = (long long)(p.n / 128) * NST;
    long long grid = (long long)num_sms * ctas_per_sm;
    if (grid > total) grid = total;
    // every CTA may publish two partial tiles (its first and its last column block): the grid shrinks until they fit the
    // room, which never takes it below the number of tiles the room holds
    const size_t tile_bytes = (size_t)p.m * 128 * 4;
    while (grid > 1 && (size_t)grid * 2 * tile_bytes > partial_room) grid = grid / 2;
    const size_t need = grid > 1 ? (size_t)grid * 2 * tile_bytes : 0;
    if (need > partial_room) return cudaErrorMemoryAllocation;
    p.partial = partial_base;
    if (plan_out) { plan_out->grid = (int)grid; plan_out->max_contrib = 0; plan_out->partial_bytes = need; }
    kern<<<(unsigned)grid, 256, bytes, st>>>(p);
    return cudaPeekAtLastError();
}

template <int K, int CB>
cudaError_t launch_small_mt(int mt, GemmSmallParams& p, int sms, size_t room, float* base, cudaStream_t st, SmallPlan* pl)
{
    if (mt == 1) return launch_small<K, CB, 1>(p, sms, room, base, st, pl);
    if (mt == 2) return launch_small<K, CB, 2>(p, sms, room, base, st, pl);
    return launch_small<K, CB, 4>(p, sms, room, base, st, pl);
}

template <int K>
cudaError_t launch_small_cb(int cb, int mt, GemmSmallParams& p, int sms, size_t room, float* base, cudaStream_t st, SmallPlan* pl)
{
    if (cb == 0) return launch_small_mt<K, 0>(mt, p, sms, room, base, st, pl);
    if (cb == 1) return launch_small_mt<K, 1>(mt, p, sms, room, base, st, pl);
    return launch_small_mt<K, 2>(mt, p, sms, room, base, st, pl);
}

cudaError_t launch_small_k(int K, int cb, int mt, GemmSmallParams& p, int sms, size_t room, float* base, cudaStream_t st,
                           SmallPlan* pl)
{
    switch (K) {
        case 1: return launch_small_cb<1>(cb, mt, p, sms, room, base, st, pl);
        case 2: return launch_small_cb<2>(cb, mt, p, sms, room, base, st, pl);
        case 3: return launch_small_cb<3>(cb, mt, p, sms, room, base, st, pl);
        case 4: return launch_small_cb<4>(cb, mt, p, sms, room, base, st, pl);
        case 5: return launch_small_cb<5>(cb, mt, p, sms, room, base, st, pl);
        case 6: return launch_small_cb<6>(cb, mt, p, sms, room, base, st, pl);
        case 7: return launch_small_cb<7>(cb, mt, p, sms, room, base, st, pl);
        default: return launch_small_cb<8>(cb, mt, p, sms, room, base, st, pl);
    }
}

// Input transform for the tensor-core path: plain fp16 A_had[row][k] (one CTA per row, as above without duplication).
struct ProloguePlainArgs { const half* suh[TC_MAX_SEG]; half* a_had[TC_MAX_SEG]; };

__global__ void __launch_bounds__(256) gemm_prologue_plain_kernel(const half* __restrict__ A, const ProloguePlainArgs args, int k)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    const half* __restrict__ suh = args.suh[blockIdx.y];
    half* __restrict__ a_had = args.a_had[blockIdx.y];
    for (int blk = warp; blk < k / 128; blk += 8) {
        uint2 raw = reinterpret_cast<const uint2*>(A + row * k + blk * 128)[lane];
        half2 a = *reinterpret_cast<half2*>(&raw.x), b = *reinterpret_cast<half2*>(&raw.y);
        if (suh) {
            uint2 sr = reinterpret_cast<const uint2*>(suh + blk * 128)[lane];
            a = __hmul2(a, *reinterpret_cast<half2*>(&sr.x));
            b = __hmul2(b, *reinterpret_cast<half2*>(&sr.y));
            float v0 = __low2float(a), v1 = __high2float(a), v2 = __low2float(b), v3 = __high2float(b);
            float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
            v0 = s0 + s1; v1 = d0 + d1; v2 = s0 - s1; v3 = d0 - d1;
            #pragma unroll
            for (int i = 1; i < 32; i <<= 1) {
                float p0 = __shfl_xor_sync(0xffffffffu, v0, i), p1 = __shfl_xor_sync(0xffffffffu, v1, i);
                float p2 = __shfl_xor_sync(0xffffffffu, v2, i), p3 = __shfl_xor_sync(0xffffffffu, v3, i);
                const bool up = lane & i;
                v0 = (up ? -v0 : v0) + p0; v1 = (up ? -v1 : v1) + p1;
                v2 = (up ? -v2 : v2) + p2; v3 = (up ? -v3 : v3) + p3;
            }
            a = __floats2half2_rn(v0 * GS_R128, v1 * GS_R128);
            b = __floats2half2_rn(v2 * GS_R128, v3 * GS_R128);
        }
        uint2 o; o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint2*>(a_had + row * k + blk * 128)[lane] = o;
    }
}


// The same transform with the butterflies on the tensor core, for rows with an even number of 128-blocks: a warp takes
// two blocks at a time.  H128 = H8 (x) H16 on the index i = 16 a + b: X[a][b] of both blocks goes through shared memory
// into transposed MMA fragments (ldmatrix.trans), D0 = (H8 (+) H8) X contracts over a with the sign matrix as the A
// operand, D0 - kept exact as an fp16 pair hi + lo - becomes the A operand of the second product Y = D0 H16, whose
// columns are ordered so that a lane ends up with four consecutive outputs.  About a quarter of the instructions of the
// shuffle version (which needs 20 shuffles per 4 values); sums are formed in another order than
// hadamard_inner.cuh:93-147 does, so single results may differ from the shuffle version's by one fp16 step where the
// fp32 value sits on a rounding boundary.
__device__ __forceinline__ void gp_ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ uint32_t sign_pair(int i, int j0, int j1)
{
    const uint32_t lo = (__popc(i & j0) & 1) ? 0xBC00u : 0x3C00u, hi = (__popc(i & j1) & 1) ? 0xBC00u : 0x3C00u;
    return lo | (hi << 16);
}

constexpr int GP_PAIRS = 4;          // block pairs per warp: their loads are all in flight before the first is used

__global__ void __launch_bounds__(256) gemm_prologue_mma_kernel(const half* __restrict__ A, const ProloguePlainArgs args, int k,
                                                                long long pairs_total)
{
    __shared__ __align__(16) uint8_t stage[8][512];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long long pair0 = ((long long)blockIdx.x * 8 + warp) * GP_PAIRS;
    if (pair0 >= pairs_total) return;
    const int ppr = k / 256;                                   // block pairs per row
    const half* __restrict__ suh = args.suh[blockIdx.y];
    half* __restrict__ a_had = args.a_had[blockIdx.y];

    // constant operands: H8 (+) H8 as A of the first product, H16 with permuted columns as B of the second
    const uint32_t h8 = sign_pair(g, 2 * t, 2 * t + 1);
    uint32_t hb[2][2];
    #pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
        const int bp = 4 * (g >> 1) + 2 * nb + (g & 1);        // output column b' of MMA column g in column block nb
        hb[nb][0] = sign_pair(bp, 2 * t, 2 * t + 1);
        hb[nb][1] = sign_pair(bp, 2 * t + 8, 2 * t + 9);
    }

    // (x o suh) of every pair: lane = 8 consecutive values of the 256
    uint4 xs[GP_PAIRS];
    size_t base[GP_PAIRS];
    #pragma unroll
    for (int u = 0; u < GP_PAIRS; ++u) {
        const long long pair = pair0 + u < pairs_total ? pair0 + u : pairs_total - 1;       // the tail repeats the last pair
        const size_t row = (size_t)(pair / ppr);
        const int col0 = (int)(pair - (long long)row * ppr) * 256;
        base[u] = row * k + col0;
        xs[u] = reinterpret_cast<const uint4*>(A + base[u])[lane];
        const uint4 sg = reinterpret_cast<const uint4*>(suh + col0)[lane];
        half2* xh = reinterpret_cast<half2*>(&xs[u]);
        const half2* sh = reinterpret_cast<const half2*>(&sg);
        #pragma unroll
        for (int e = 0; e < 4; ++e) xh[e] = __hmul2(xh[e], sh[e]);
    }
    #pragma unroll
    for (int u = 0; u < GP_PAIRS; ++u) {
        if (pair0 + u >= pairs_total) break;                   // warp-uniform
        *reinterpret_cast<uint4*>(stage[warp] + lane * 16) = xs[u];
        __syncwarp();
        // four 8x8 matrices, transposed on the way out: (block 0, b 0..7), (block 0, b 8..15), (block 1, ...), (block 1, ...)
        uint32_t r0, r1, r2, r3;
        {
            const int mat = lane >> 3, rr = lane & 7;          // row a = rr of matrix mat
            gp_ldsm_x4_t(r0, r1, r2, r3, stage[warp] + (mat >> 1) * 256 + rr * 32 + (mat & 1) * 16);
        }
        __syncwarp();                                          // the staging buffer is free for the next pair
        float d0[2][4];
        #pragma unroll
        for (int bh = 0; bh < 2; ++bh) {
            d0[bh][0] = d0[bh][1] = d0[bh][2] = d0[bh][3] = 0.f;
            gd_mma(d0[bh], h8, 0u, 0u, h8, bh ? r1 : r0, bh ? r3 : r2);
        }
        // D0[(block, a')][b] -> A operand of the second product, as hi + lo
        uint32_t ahi[4], alo[4];
        #pragma unroll
        for (int bh = 0; bh < 2; ++bh)
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float p = d0[bh][2 * h], q = d0[bh][2 * h + 1];
                const half2 hi = __floats2half2_rn(p, q);
                const half2 lo = __floats2half2_rn(p - __low2float(hi), q - __high2float(hi));
                ahi[2 * bh + h] = *reinterpret_cast<const uint32_t*>(&hi);
                alo[2 * bh + h] = *reinterpret_cast<const uint32_t*>(&lo);
            }
        float y[2][4];
        #pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            y[nb][0] = y[nb][1] = y[nb][2] = y[nb][3] = 0.f;
            gd_mma(y[nb], ahi[0], ahi[1], ahi[2], ahi[3], hb[nb][0], hb[nb][1]);
            gd_mma(y[nb], alo[0], alo[1], alo[2], alo[3], hb[nb][0], hb[nb][1]);
        }
        // lane holds, for row a' = g of block 0 ([0], [1]) and of block 1 ([2], [3]), the outputs b' = 4t .. 4t+3
        #pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const half2 p = __floats2half2_rn(y[0][2 * blk] * GS_R128, y[0][2 * blk + 1] * GS_R128);
            const half2 q = __floats2half2_rn(y[1][2 * blk] * GS_R128, y[1][2 * blk + 1] * GS_R128);
            uint2 o; o.x = *reinterpret_cast<const uint32_t*>(&p); o.y = *reinterpret_cast<const uint32_t*>(&q);
            *reinterpret_cast<uint2*>(a_had + base[u] + blk * 128 + 16 * g + 4 * t) = o;
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

constexpr int TC_MAX_SMALL_M = 0;           // row counts up to this stay on the mma.sync small-M kernel (0: none do)

template <int K, int CB, int CTAS, int BN>
cudaError_t launch_tc(const CUtensorMap* amap, const CUtensorMap* rmap, const CUtensorMap* cmap, const GemmTcParams& p, int slabs, cudaStream_t st)
{
    constexpr int bytes = TcSmem<K, CTAS, BN>::BYTES;
    static bool configured[64] = {};
    auto kern = gemm_tc_kernel<K, CB, CTAS, BN>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(slabs * CTAS, (p.m + TC_BM * CTAS - 1) / (TC_BM * CTAS));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, amap[0], amap[1], amap[2], rmap[0], rmap[1], rmap[2], cmap[0], cmap[1], cmap[2], p);
}

template <int K, int CB>
cudaError_t launch_tc_ctas(bool pair, int bn, const CUtensorMap* amap, const CUtensorMap* rmap, const CUtensorMap* cmap, const GemmTcParams& p, int slabs, cudaStream_t st)
{
    if (pair && bn == 128) return launch_tc<K, CB, 2, 128>(amap, rmap, cmap, p, slabs, st);
    return pair ? launch_tc<K, CB, 2, 256>(amap, rmap, cmap, p, slabs, st) : launch_tc<K, CB, 1, 256>(amap, rmap, cmap, p, slabs, st);
}

template <int K>
cudaError_t launch_tc_cb(int cb, bool pair, int bn, const CUtensorMap* amap, const CUtensorMap* rmap, const CUtensorMap* cmap, const GemmTcParams& p, int slabs, cudaStream_t st)
{
    if (cb == 0) return launch_tc_ctas<K, 0>(pair, bn, amap, rmap, cmap, p, slabs, st);
    if (cb == 1) return launch_tc_ctas<K, 1>(pair, bn, amap, rmap, cmap, p, slabs, st);
    return launch_tc_ctas<K, 2>(pair, bn, amap, rmap, cmap, p, slabs, st);
}

cudaError_t launch_tc_k(int K, int cb, bool pair, int bn, const CUtensorMap* amap, const CUtensorMap* rmap, const CUtensorMap* cmap, const GemmTcParams& p, int slabs, cudaStream_t st)
{
    switch (K) {
        case 1: return launch_tc_cb<1>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        case 2: return launch_tc_cb<2>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        case 3: return launch_tc_cb<3>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        case 4: return launch_tc_cb<4>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        case 5: return launch_tc_cb<5>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        case 6: return launch_tc_cb<6>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        case 7: return launch_tc_cb<7>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
        default: return launch_tc_cb<8>(cb, pair, bn, amap, rmap, cmap, p, slabs, st);
    }
}

// Tensor-core path for rows [0, m) and `nseg` weight tensors that share the activations, k, bits and codebook:
// one launch of the input transforms (each tensor has its own suh) and one of the tcgen05 kernel.
// With `pre` the transformed activations are already in place (written into the buffers exl3_tc_pre_buffers named, by the
// kernel that produced the input), and the transform launch is skipped.
int gemm_tc_rows(exl3_ctx* ctx, cudaStream_t st, const half* A, int nseg, const void* const* trellis, void* const* C,
                 const half* const* suh, const half* const* svh, const int* n, int m, int k, int K, int c_fp32, int cb,
                 bool pre = false)
{
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_gemm: cuTensorMapEncodeTiled is not available from this driver");
    size_t off = 0;
    ProloguePlainArgs pa;
    CUtensorMap amap[TC_MAX_SEG], rmap[TC_MAX_SEG], cmap[TC_MAX_SEG];
    GemmTcParams p;
    memset(&p, 0, sizeof(p));
    // Slab width: 256 columns, or 128 when a single row block would put 256-column slabs on at most a quarter of the SMs
    // (q/k/v and o_proj of a verify batch: 28 and 20 slabs): the decode work, which bounds these launches, then runs on
    // twice as many SMs.
    int blocks256 = 0;
    bool n128 = true;
    for (int i = 0; i < nseg; ++i) { blocks256 += (n[i] + TC_BN - 1) / TC_BN; n128 = n128 && n[i] % 128 == 0; }
    const int bn = (ctx->use_pair && n128 && m <= 2 * TC_BM && blocks256 * 4 <= ctx->num_sms) ? 128 : TC_BN;
    int blocks = 0;
    for (int i = 0; i < TC_MAX_SEG; ++i) {
        const int j = i < nseg ? i : nseg - 1;              // unused slots repeat the last tensor (never selected)
        if (i < nseg) {
            pa.a_had[i] = (half*)exl3_ws_take(ctx, &off, (size_t)m * k * 2);
            if (!pa.a_had[i]) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "exl3_gemm: context scratch too small for the activations");
            pa.suh[i] = suh[i];
            blocks += (n[i] + bn - 1) / bn;                // a trailing 128-column half slab counts (CTA pairs only)
            cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
            cuuint64_t strides[1] = {(cuuint64_t)k * 2};
            cuuint32_t box[2] = {(cuuint32_t)TC_BK, 128u};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = enc(&amap[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, pa.a_had[i], dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_gemm: cuTensorMapEncodeTiled failed");
            // the trellis as a matrix of 64-bit words, one row per tile row (16 k); a CTA of a pair fetches a stage of its
            // half slab (4 tile rows x 8 tiles x 32K bytes) as one box
            cuuint64_t rdims[2] = {(cuuint64_t)(n[i] / 16) * 4 * K, (cuuint64_t)(k / 16)};
            cuuint64_t rstrides[1] = {(cuuint64_t)(n[i] / 16) * 32 * K};
            cuuint32_t rbox[2] = {(cuuint32_t)(bn / 2 / 16) * 4 * K, (cuuint32_t)(TC_BK / 16)};
            r = enc(&rmap[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(trellis[i]), rdims, rstrides, rbox, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_gemm: cuTensorMapEncodeTiled failed for the trellis");
            // the fp16 output as [m][n]: an epilogue warp stores its 32 rows x 128 columns as two boxes of 64 columns
            if (!c_fp32) {
                cuuint64_t cdims[2] = {(cuuint64_t)n[i], (cuuint64_t)m};
                cuuint64_t cstrides[1] = {(cuuint64_t)n[i] * 2};
                cuuint32_t cbox[2] = {64u, 32u};
                r = enc(&cmap[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C[i], cdims, cstrides, cbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r != CUDA_SUCCESS) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_gemm: cuTensorMapEncodeTiled failed for the output");
            } else
                cmap[i] = amap[i];                             // never dereferenced: fp32 outputs are stored by the threads
        } else {
            pa.a_had[i] = pa.a_had[j]; pa.suh[i] = pa.suh[j]; amap[i] = amap[j]; rmap[i] = rmap[j]; cmap[i] = cmap[j];
        }
        p.trellis[i] = (const uint32_t*)trellis[j]; p.C[i] = C[j]; p.svh[i] = svh[j]; p.n[i] = n[j];
        p.blk_end[i] = i < nseg ? blocks : 0x7fffffff;
    }
    bool all_signed = true;
    for (int i = 0; i < nseg; ++i) all_signed = all_signed && pa.suh[i] != nullptr;
    if (pre) {
        // nothing to launch
    } else if (k % 256 == 0 && all_signed) {
        const long long pairs = (long long)m * (k / 256);
        gemm_prologue_mma_kernel<<<dim3((unsigned)((pairs + 8 * GP_PAIRS - 1) / (8 * GP_PAIRS)), nseg), 256, 0, st>>>(A, pa, k, pairs);
    } else
        gemm_prologue_plain_kernel<<<dim3(m, nseg), 256, 0, st>>>(A, pa, k);
    if (!pre) ctx->launches++;
    p.status = ctx->status; p.m = m; p.k = k; p.c_fp32 = c_fp32;
    cudaError_t e = launch_tc_k(K, cb, ctx->use_pair != 0, bn, amap, rmap, cmap, p, blocks, st);
    ctx->launches++;
    if (e != cudaSuccess) { cudaGetLastError(); return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e)); }
    return EXL3_OK;
}

// ---- decode-regime kernel (1..16 rows)

constexpr int GD_MAX_M = 16;

template <int K, int CB, int MT>
cudaError_t launch_decode(const CUtensorMap* rmap, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    constexpr int bytes = GdSmem<K, MT>::BYTES;
    static bool configured[64] = {};
    auto kern = gemm_decode_kernel<K, CB, MT>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    // launched as a programmatic dependent of the input transform that precedes it on the stream
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GD_THREADS); cfg.dynamicSmemBytes = bytes; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, rmap[0], rmap[1], rmap[2], p);
}

template <int K, int CB>
cudaError_t launch_decode_mt(int mt, const CUtensorMap* rmap, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    return mt == 1 ? launch_decode<K, CB, 1>(rmap, p, grid, st) : launch_decode<K, CB, 2>(rmap, p, grid, st);
}

template <int K>
cudaError_t launch_decode_cb(int cb, int mt, const CUtensorMap* rmap, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    if (cb == 0) return launch_decode_mt<K, 0>(mt, rmap, p, grid, st);
    if (cb == 1) return launch_decode_mt<K, 1>(mt, rmap, p, grid, st);
    return launch_decode_mt<K, 2>(mt, rmap, p, grid, st);
}

cudaError_t launch_decode_k(int K, int cb, int mt, const CUtensorMap* rmap, const GemmDecodeParams& p, int grid, cudaStream_t st)
{
    switch (K) {
        case 1: return launch_decode_cb<1>(cb, mt, rmap, p, grid, st);
        case 2: return launch_decode_cb<2>(cb, mt, rmap, p, grid, st);
        case 3: return launch_decode_cb<3>(cb, mt, rmap, p, grid, st);
        case 4: return launch_decode_cb<4>(cb, mt, rmap, p, grid, st);
        case 5: return launch_decode_cb<5>(cb, mt, rmap, p, grid, st);
        case 6: return launch_decode_cb<6>(cb, mt, rmap, p, grid, st);
        case 7: return launch_decode_cb<7>(cb, mt, rmap, p, grid, st);
        default: return launch_decode_cb<8>(cb, mt, rmap, p, grid, st);
    }
}

// Decode path for m <= 16 rows and `nseg` weight tensors that share the activations, k, bits and codebook: one launch of
// the input transforms (fragment order, one per tensor) and one of the streaming kernel over all their column blocks.
int gemm_decode_rows(exl3_ctx* ctx, cudaStream_t st, const half* A, int nseg, const void* const* trellis, void* const* C,
                     const half* const* suh, const half* const* svh, const int* n, int m, int k, int K, int c_fp32, int cb)
{
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_gemm: cuTensorMapEncodeTiled is not available from this driver");
    const int mt = m <= 8 ? 1 : 2;
    size_t off = 0;
    GemmDecodePrologueArgs pa;
    CUtensorMap rmap[GD_MAX_SEG];
    GemmDecodeParams p;
    memset(&p, 0, sizeof(p));
    int blocks = 0;
    for (int i = 0; i < GD_MAX_SEG; ++i) {
        const int j = i < nseg ? i : nseg - 1;              // unused slots repeat the last tensor (never selected)
        if (i < nseg) {
            pa.a_frag[i] = (uint32_t*)exl3_ws_take(ctx, &off, (size_t)mt * k * 32);
            pa.rowsum[i] = (float*)exl3_ws_take(ctx, &off, (size_t)GD_PRO_SPLIT * mt * 8 * 4);
            if (!pa.a_frag[i] || !pa.rowsum[i]) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "exl3_gemm: context scratch too small for the activations");
            pa.suh[i] = suh[i];
            blocks += n[i] / 128;
            cuuint64_t rdims[2] = {(cuuint64_t)(n[i] / 16) * 4 * K, (cuuint64_t)(k / 16)};
            cuuint64_t rstrides[1] = {(cuuint64_t)(n[i] / 16) * 32 * K};
            cuuint32_t rbox[2] = {(cuuint32_t)2 * GD_SLOT_TILES * 4 * K, (cuuint32_t)GD_SLOT_ROWS};      // 8 tiles x 4 tile rows
            cuuint32_t estr[2] = {1, 1};
            CUresult r = enc(&rmap[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(trellis[i]), rdims, rstrides, rbox, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return exl3_fail(ctx, EXL3_ERR_CUDA, "exl3_gemm: cuTensorMapEncodeTiled failed for the trellis");
        } else {
            pa.a_frag[i] = pa.a_frag[j]; pa.rowsum[i] = pa.rowsum[j]; pa.suh[i] = pa.suh[j]; rmap[i] = rmap[j];
        }
        p.a_frag[i] = (const uint4*)pa.a_frag[i]; p.rowsum[i] = pa.rowsum[i];
        p.C[i] = C[j]; p.svh[i] = svh[j]; p.n[i] = n[j];
        p.blk_end[i] = i < nseg ? blocks : 0x7fffffff;
    }
    p.blk_end[GD_MAX_SEG - 1] = blocks;                     // the kernel reads the total from the last entry
    for (int i = nseg; i < GD_MAX_SEG - 1; ++i) p.blk_end[i] = blocks;
    if (blocks > ctx->n_counters) return exl3_fail(ctx, EXL3_ERR_INVALID, "exl3_gemm: n too large for the context's counters");
    // Split of the (column block, 512-k chunk) units over the CTAs: whole blocks per CTA when that costs at most one unit
    // more on the longest CTA than an even share of all units (no block is then shared between CTAs: no partial sums, no
    // arrival counters, and the block finish at the end of the CTA is local), an even share (stream-K) otherwise.
    const int KC = (k + GD_UNIT_K - 1) / GD_UNIT_K;
    const long long total = (long long)blocks * KC;
    const int sms = ctx->num_sms;
    const long long units_aligned = (long long)((blocks + sms - 1) / sms) * KC, units_even = (total + sms - 1) / sms;
    p.aligned = units_aligned <= units_even + 1 ? 1 : 0;
    const int grid = p.aligned ? (blocks < sms ? blocks : sms) : (int)(total < sms ? total : sms);
    p.partial = (float*)exl3_ws_take(ctx, &off, (size_t)grid * 2 * m * 128 * 4);
    if (!p.partial) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "exl3_gemm: context scratch too small for the partial sums");
    p.counters = ctx->counters; p.status = ctx->status; p.m = m; p.k = k; p.c_fp32 = c_fp32;
    p.rowsum_parts = GD_PRO_SPLIT;
    gemm_decode_prologue_kernel<<<dim3(8 * mt, nseg, GD_PRO_SPLIT), 256, 0, st>>>(A, pa, m, k);
    ctx->launches++;
    cudaError_t e = launch_decode_k(K, cb, mt, rmap, p, grid, st);
    ctx->launches++;
    if (e != cudaSuccess) { cudaGetLastError(); return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e)); }
    return EXL3_OK;
}

}  // namespace

// Rows are processed in passes of up to 64; each pass = input transform + one fused decode/MMA/output-transform launch.
extern "C" int exl3_gemm(exl3_ctx* ctx, exl3_stream stream, const void* A, const void* trellis, void* C,
                         const void* suh, void* A_had, const void* svh, int m, int k, int n, int K, int c_fp32,
                         int mcg, int mul1)
{
    (void)A_had;   // the transformed activations live in the context scratch in a duplicated layout
    EXL3_REQUIRE(ctx && A && trellis && C, "exl3_gemm: null argument");
    EXL3_REQUIRE(m >= 0 && k > 0 && n > 0 && k % 128 == 0 && n % 128 == 0, "exl3_gemm: k % 128 == 0 and n % 128 == 0 required");
    EXL3_REQUIRE(K >= 1 && K <= 8, "exl3_gemm: K must be 1..8");
    EXL3_REQUIRE(!(mcg && mul1), "exl3_gemm: both mcg and mul1 set");
    EXL3_REQUIRE(aligned16(A) && aligned16(trellis) && aligned16(C) && aligned16(suh) && aligned16(svh),
                 "exl3_gemm: pointers must be 16-byte aligned");
    if (m == 0) return EXL3_OK;
    const int cb = mcg ? 1 : (mul1 ? 2 : 0);
    cudaStream_t st = (cudaStream_t)stream;
    const int NB = n / 128, NST = k / 128;
    EXL3_REQUIRE(NB <= ctx->n_counters, "exl3_gemm: n too large for the context's counters");

    // tcgen05 kernel over 512-row blocks per CTA pair and 256-column slabs (with CTA pairs a last slab of 128 columns is
    // allowed: its missing half reads zero-filled codes and is never stored) (the last block may be partial: its rows past m are
    // zero-filled by TMA, and a block with at most 256 valid rows runs a single MMA per K step).  Measured on 5120 x 17408
    // at 4 bpw: the tcgen05 kernel takes 47-52 us for any m <= 256 (its decoders set the pace), the mma.sync small-M
    // kernel 54 us at m = 1, 73 us at m = 16 and 209 us at m = 64, so every row count goes to the former.  The small-M
    // kernel serves exl3_gemm_noalloc, EXL3_B200_NO_TC, and n % 256 == 128 under EXL3_B200_NO_PAIR.
    if (m <= GD_MAX_M && ctx->use_decode) {
        const half* suh1 = (const half*)suh; const half* svh1 = (const half*)svh;
        return gemm_decode_rows(ctx, st, (const half*)A, 1, &trellis, &C, &suh1, &svh1, &n, m, k, K, c_fp32, cb);
    }
    // (17..32 rows on a tensor with few column slabs and a long reduction dimension, 17408 x 5120, used to run as two
    // 16-row passes of the streaming kernel: 100 us against 126 us on 256-column slabs.  With 128-column slabs the
    // tcgen05 kernel takes 80 us, so every row count above 16 goes there.)
    int tc_rows = 0;
    if (m > TC_MAX_SMALL_M && (n % TC_BN == 0 || ctx->use_pair) && ctx->use_tc) {
        tc_rows = m;
        const half* suh1 = (const half*)suh; const half* svh1 = (const half*)svh;
        int rc = gemm_tc_rows(ctx, st, (const half*)A, 1, &trellis, &C, &suh1, &svh1, &n, tc_rows, k, K, c_fp32, cb);
        if (rc != EXL3_OK) return rc;
    }
    for (int row0 = tc_rows; row0 < m; row0 += 64) {
        const int rows = m - row0 < 64 ? m - row0 : 64;
        const int mt = rows <= 16 ? 1 : (rows <= 32 ? 2 : 4);
        size_t off = 0;
        uint32_t* a_dup = (uint32_t*)exl3_ws_take(ctx, &off, (size_t)rows * k * 4);
        float* rowsum = (float*)exl3_ws_take(ctx, &off, (size_t)rows * 4);
        if (!a_dup || !rowsum) return exl3_fail(ctx, EXL3_ERR_WORKSPACE, "exl3_gemm: context scratch too small for the activations");
        gemm_prologue_kernel<<<rows, 256, 0, st>>>((const half*)A + (size_t)row0 * k, (const half*)suh, a_dup, rowsum, k);
        ctx->launches++;
        // whatever scratch is left holds the partial sums of column blocks that several CTAs share
        size_t part_off = (off + 255) & ~(size_t)255;
        const size_t room = ctx->ws_bytes > part_off ? ctx->ws_bytes - part_off : 0;
        GemmSmallParams p;
        p.a_dup = a_dup; p.rowsum = rowsum; p.trellis = (const uint32_t*)trellis; p.partial = nullptr;
        p.counters = ctx->counters; p.svh = (const half*)svh; p.status = ctx->status;
        p.C = c_fp32 ? (void*)((float*)C + (size_t)row0 * n) : (void*)((half*)C + (size_t)row0 * n);
        p.m = rows; p.k = k; p.n = n; p.c_fp32 = c_fp32;
        cudaError_t e = launch_small_k(K, cb, mt, p, ctx->num_sms, room, (float*)(ctx->ws + part_off), st, nullptr);
        ctx->launches++;
        if (e != cudaSuccess) { cudaGetLastError(); return exl3_fail(ctx, EXL3_ERR_CUDA, cudaGetErrorString(e)); }
    }
    return EXL3_OK;
}

// exl3_gemm_fanout: the same activations through several EXL3 tensors (q/k/v, gate/up).  With many rows and tensors that
// agree in k, bits and codebook this is one tensor-core launch over all their column blocks; otherwise one exl3_gemm
// per tensor.
extern "C" int exl3_gemm_fanout(exl3_ctx* ctx, exl3_stream stream, const void* A, int count, const exl3_linear* const* w,
                                void* const* C, int m, int c_fp32)
{
    EXL3_REQUIRE(ctx && A && w && C && count >= 1 && count <= TC_MAX_SEG, "exl3_gemm_fanout: 1..3 tensors required");
    bool same = true;
    for (int i = 0; i < count; ++i) {
        EXL3_REQUIRE(w[i] && C[i] && w[i]->trellis, "exl3_gemm_fanout: null tensor");
        same = same && w[i]->k == w[0]->k && w[i]->K == w[0]->K && w[i]->cb == w[0]->cb && w[i]->n % TC_BN == 0 &&
               w[i]->k % 128 == 0 && w[i]->K >= 1 && w[i]->K <= 8 && aligned16(w[i]->trellis) && aligned16(C[i]) &&
               aligned16(w[i]->suh) && aligned16(w[i]->svh) && (w[i]->suh != nullptr) == (w[0]->suh != nullptr);
    }
    if (count > 1 && same && m <= GD_MAX_M && ctx->use_decode && aligned16(A)) {
        const void* tr[GD_MAX_SEG]; const half* suh[GD_MAX_SEG]; const half* svh[GD_MAX_SEG]; int n[GD_MAX_SEG];
        for (int i = 0; i < count; ++i) { tr[i] = w[i]->trellis; suh[i] = (const half*)w[i]->suh; svh[i] = (const half*)w[i]->svh; n[i] = w[i]->n; }
        return gemm_decode_rows(ctx, (cudaStream_t)stream, (const half*)A, count, tr, C, suh, svh, n, m, w[0]->k, w[0]->K, c_fp32, w[0]->cb);
    }
    if (count > 1 && same && m > TC_MAX_SMALL_M && ctx->use_tc && aligned16(A)) {
        const void* tr[TC_MAX_SEG]; const half* suh[TC_MAX_SEG]; const half* svh[TC_MAX_SEG]; int n[TC_MAX_SEG];
        for (int i = 0; i < count; ++i) { tr[i] = w[i]->trellis; suh[i] = (const half*)w[i]->suh; svh[i] = (const half*)w[i]->svh; n[i] = w[i]->n; }
        return gemm_tc_rows(ctx, (cudaStream_t)stream, (const half*)A, count, tr, C, suh, svh, n, m, w[0]->k, w[0]->K, c_fp32, w[0]->cb);
    }
    for (int i = 0; i < count; ++i) {
        int rc = exl3_gemm(ctx, stream, A, w[i]->trellis, C[i], w[i]->suh, nullptr, w[i]->svh, m, w[i]->k, w[i]->n, w[i]->K, c_fp32,
                           w[i]->cb == 1, w[i]->cb == 2);
        if (rc != EXL3_OK) return rc;
    }
    return EXL3_OK;
}

// The tensor-core path with the input transform done by the producer of the activations (see exl3_pre_act).  The buffers
// are the ones gemm_tc_rows carves from the start of the context scratch, so the two calls agree on them by construction.
static bool tc_pre_applies(exl3_ctx* ctx, int count, const exl3_linear* const* w, int m)
{
    if (!ctx || !w || count < 1 || count > TC_MAX_SEG || m <= GD_MAX_M || !ctx->use_tc) return false;
    for (int i = 0; i < count; ++i) {
        if (!w[i] || !w[i]->trellis || !w[i]->suh) return false;
        if (w[i]->k != w[0]->k || w[i]->K != w[0]->K || w[i]->cb != w[0]->cb) return false;
        if (w[i]->k % 128 != 0 || w[i]->n % 128 != 0 || !(w[i]->n % TC_BN == 0 || (ctx->use_pair && count == 1))) return false;
        if (w[i]->K < 1 || w[i]->K > 8 || !aligned16(w[i]->trellis) || !aligned16(w[i]->suh) || !aligned16(w[i]->svh)) return false;
    }
    return true;
}

bool exl3_tc_pre_buffers(exl3_ctx* ctx, int count, const exl3_linear* const* w, int m, exl3_pre_act* pre)
{
    if (!tc_pre_applies(ctx, count, w, m)) return false;
    size_t off = 0;
    pre->nseg = count;
    for (int i = 0; i < 3; ++i) { pre->suh[i] = nullptr; pre->a_had[i] = nullptr; }
    for (int i = 0; i < count; ++i) {
        pre->a_had[i] = (half*)exl3_ws_take(ctx, &off, (size_t)m * w[0]->k * 2);
        if (!pre->a_had[i]) return false;
        pre->suh[i] = (const half*)w[i]->suh;
    }
    return true;
}

int exl3_gemm_fanout_pre(exl3_ctx* ctx, exl3_stream stream, int count, const exl3_linear* const* w, void* const* C, int m, int c_fp32)
{
    EXL3_REQUIRE(tc_pre_applies(ctx, count, w, m) && C, "exl3_gemm (activations transformed by the producer): not applicable to these tensors");
    const void* tr[TC_MAX_SEG]; const half* suh[TC_MAX_SEG]; const half* svh[TC_MAX_SEG]; int n[TC_MAX_SEG];
    for (int i = 0; i < count; ++i) {
        EXL3_REQUIRE(C[i] && aligned16(C[i]), "exl3_gemm: bad output pointer");
        tr[i] = w[i]->trellis; suh[i] = (const half*)w[i]->suh; svh[i] = (const half*)w[i]->svh; n[i] = w[i]->n;
    }
    return gemm_tc_rows(ctx, (cudaStream_t)stream, nullptr, count, tr, C, suh, svh, n, m, w[0]->k, w[0]->K, c_fp32, w[0]->cb, true);
}

// ---------------------------------------------------------------------------------------------------------------------
// exl3_gemm_noalloc: the small-M EXL3 GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a matrix product: code that runs
// inside a memory-pool or allocator callback, a real-time decode loop whose latency budget forbids the implicit
// device synchronisation an allocation can cause, or a plug-in that was handed a fixed device-memory budget and may
// not grow it.  exl3_ctx_create allocates, so those callers cannot use exl3_gemm.  This entry point needs no context:
// the scratch the kernel uses (the transformed activations, split-K partial sums, arrival counters, status word) lives
// in the fixed array below, which is part of the library image.  Every GPU that loads the library holds these 8 MiB
// until the process exits, whether or not the entry point is ever called.
namespace {

constexpr size_t NA_BYTES      = (size_t)8 << 20;      // whole scratch
constexpr int    NA_MAX_M      = 16;                   // rows per call
constexpr int    NA_MAX_K      = 32768;
constexpr int    NA_MAX_N      = 524288;
constexpr size_t NA_OFF_CNT    = 0;                                    // int[NA_MAX_N / 128] arrival counters
constexpr size_t NA_OFF_STATUS = NA_OFF_CNT + (NA_MAX_N / 128) * 4;    // int status word (+ padding)
constexpr size_t NA_OFF_ROWSUM = NA_OFF_STATUS + 256;                  // float[NA_MAX_M]
constexpr size_t NA_OFF_ADUP   = NA_OFF_ROWSUM + 256;                  // uint32[NA_MAX_M][k]
constexpr size_t NA_ADUP_BYTES = (size_t)NA_MAX_M * NA_MAX_K * 4;
constexpr size_t NA_OFF_PART   = NA_OFF_ADUP + NA_ADUP_BYTES;          // float[n/128][owners][m][128] partial sums

static __device__ __align__(256) unsigned char g_noalloc_scratch[NA_BYTES];

// In host code the name g_noalloc_scratch is only a handle for the runtime, not a device address; the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
struct NoAllocDev { unsigned char* base; int num_sms; bool ready; };
NoAllocDev g_na_dev[64];

int noalloc_setup(int dev, NoAllocDev** out)
{
    if (dev < 0 || dev >= 64) return EXL3_ERR_UNSUPPORTED;
    NoAllocDev& d = g_na_dev[dev];
    if (!d.ready) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "exl3_gemm_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            cudaGetLastError();
            return EXL3_ERR_CUDA;
        }
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms <= 0) { cudaGetLastError(); return EXL3_ERR_CUDA; }
        d.base = (unsigned char*)p; d.num_sms = sms; d.ready = true;
    }
    *out = &d;
    return EXL3_OK;
}

}  // namespace

extern "C" int exl3_gemm_noalloc(exl3_stream stream, const void* A, const void* trellis, void* C, const void* suh,
                                 const void* svh, int m, int k, int n, int K, int c_fp32, int mcg, int mul1)
{
    if (!A || !trellis || !C) { fprintf(stderr, "exl3_gemm_noalloc: null argument\n"); return EXL3_ERR_INVALID; }
    if (m < 0 || k <= 0 || n <= 0 || k % 128 || n % 128 || K < 1 || K > 8 || (mcg && mul1) || !aligned16(A) ||
        !aligned16(trellis) || !aligned16(C) || !aligned16(suh) || !aligned16(svh)) {
        fprintf(stderr, "exl3_gemm_noalloc: bad shape or alignment (k %% 128 == 0, n %% 128 == 0, K in 1..8, 16-byte aligned pointers)\n");
        return EXL3_ERR_INVALID;
    }
    if (m > NA_MAX_M || k > NA_MAX_K || n > NA_MAX_N) {
        fprintf(stderr, "exl3_gemm_noalloc: m=%d k=%d n=%d exceeds the fixed scratch (limits: m <= %d, k <= %d, n <= %d); "
                        "use exl3_gemm with a context for larger problems\n", m, k, n, NA_MAX_M, NA_MAX_K, NA_MAX_N);
        return EXL3_ERR_WORKSPACE;
    }
    if (m == 0) return EXL3_OK;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    NoAllocDev* d = nullptr;
    int rc = noalloc_setup(dev, &d);
    if (rc != EXL3_OK) return rc;

    cudaStream_t st = (cudaStream_t)stream;
    const int cb = mcg ? 1 : (mul1 ? 2 : 0);
    // the array keeps whatever the previous call left: the counters must start at zero (the status word is sticky until
    // exl3_gemm_noalloc_poll_status reads and clears it)
    if (cudaMemsetAsync(d->base + NA_OFF_CNT, 0, NA_OFF_STATUS - NA_OFF_CNT, st) != cudaSuccess) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    uint32_t* a_dup = (uint32_t*)(d->base + NA_OFF_ADUP);
    float* rowsum = (float*)(d->base + NA_OFF_ROWSUM);
    gemm_prologue_kernel<<<m, 256, 0, st>>>((const half*)A, (const half*)suh, a_dup, rowsum, k);
    GemmSmallParams p;
    p.a_dup = a_dup; p.rowsum = rowsum; p.trellis = (const uint32_t*)trellis; p.partial = nullptr;
    p.counters = (int*)(d->base + NA_OFF_CNT); p.svh = (const half*)svh; p.status = (int*)(d->base + NA_OFF_STATUS);
    p.C = C; p.m = m; p.k = k; p.n = n; p.c_fp32 = c_fp32;
    cudaError_t e = launch_small_k(K, cb, 1, p, d->num_sms, NA_BYTES - NA_OFF_PART, (float*)(d->base + NA_OFF_PART), st, nullptr);
    if (e != cudaSuccess) {
        fprintf(stderr, "exl3_gemm_noalloc: launch failed: %s\n", cudaGetErrorString(e));
        cudaGetLastError();
        return EXL3_ERR_CUDA;
    }
    return EXL3_OK;
}

// The kernels behind exl3_gemm_noalloc report a bounded device-side wait that ran out through a status word inside the
// fixed array.  This copies the word to the host (synchronising `stream`), clears it, and returns EXL3_ERR_DEVICE_WAIT if
// it was set, EXL3_OK otherwise; like the entry point itself it allocates nothing.
extern "C" int exl3_gemm_noalloc_poll_status(exl3_stream stream)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    NoAllocDev* d = nullptr;
    int rc = noalloc_setup(dev, &d);
    if (rc != EXL3_OK) return rc;
    int h = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(&h, d->base + NA_OFF_STATUS, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) { cudaGetLastError(); return EXL3_ERR_CUDA; }
    if (h == 0) return EXL3_OK;
    cudaMemsetAsync(d->base + NA_OFF_STATUS, 0, sizeof(int), st);
    cudaStreamSynchronize(st);
    return EXL3_ERR_DEVICE_WAIT;
}

#ifdef GD_TRACE
extern "C" EXL3_API int exl3_debug_gd_trace(unsigned long long* host_out)
{
    return cudaMemcpyFromSymbol(host_out, exl3::g_gd_trace, sizeof(unsigned long long) * 148 * 16 * 8) == cudaSuccess ? 0 : -1;
}
#endif
