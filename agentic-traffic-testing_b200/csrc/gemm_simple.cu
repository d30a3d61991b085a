// out[t, n] (+)= sum_k X[t, k] * W[n, k] on the FMA pipe, for the shapes and types the tcgen05 GEMM does not take:
// fp32 operands (true 32-bit products, no reduced-precision matrix mode), or a reduction size that is not a multiple of
// its 64-element K block. bf16 operands are widened exactly; accumulation is fp32 in a fixed order, so a row's result
// does not depend on which other rows share the launch. 64 x 64 output tile per CTA, 4 x 4 per thread.
#include "common.cuh"

#include "../../include/atx_b200.h"

namespace atx {

constexpr int kSM = 64, kSN = 64, kSK = 16;

template <typename XT>
__device__ __forceinline__ float ldg_f(const XT* p);
template <>
__device__ __forceinline__ float ldg_f<float>(const float* p) {
    return __ldg(p);
}
template <>
__device__ __forceinline__ float ldg_f<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}

template <typename XT>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(const XT* __restrict__ W, long long ldw, const XT* __restrict__ X, long long ldx,
                   float* __restrict__ out, long long ldo, int T, int N, int K, int add) {
    __shared__ float sx[kSK][kSM + 1];
    __shared__ float sw[kSK][kSN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.y * kSM, n0 = blockIdx.x * kSN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // tx: n direction, ty: t direction
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kSK) {
        for (int e = threadIdx.x; e < kSM * kSK; e += 256) {
            const int r = e / kSK, kk = e - r * kSK;
            const int t = t0 + r, k = k0 + kk;
            sx[kk][r] = (t < T && k < K) ? ldg_f(X + static_cast<long long>(t) * ldx + k) : 0.f;
            const int n = n0 + r;
            sw[kk][r] = (n < N && k < K) ? ldg_f(W + static_cast<long long>(n) * ldw + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kSK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sx[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float* o = out + static_cast<long long>(t) * ldo + n;
            *o = add ? *o + acc[i][j] : acc[i][j];
        }
    }
}

}  // namespace atx

using namespace atx;

extern "C" int atx_gemm_simple(const void* W, long long ldw, const void* X, long long ldx, float* out, long long ldo,
                               int T, int N, int K, int add, int dtype, int flags, atx_stream_t stream) {
    ATX_REQUIRE(W && X && out, "atx_gemm_simple: null pointer");
    ATX_REQUIRE(T > 0 && N > 0 && K > 0 && ldw >= K && ldx >= K && ldo >= N,
                "atx_gemm_simple: bad shape T=%d N=%d K=%d ldw=%lld ldx=%lld ldo=%lld", T, N, K, ldw, ldx, ldo);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3((N + kSN - 1) / kSN, (T + kSM - 1) / kSM);
    cfg.blockDim = dim3(256);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    if (flags & ATX_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (dtype == ATX_DT_F32)
        ATX_CUDA(cudaLaunchKernelEx(&cfg, gemm_simple_kernel<float>, reinterpret_cast<const float*>(W), ldw,
                                    reinterpret_cast<const float*>(X), ldx, out, ldo, T, N, K, add));
    else
        ATX_CUDA(cudaLaunchKernelEx(&cfg, gemm_simple_kernel<__nv_bfloat16>, reinterpret_cast<const __nv_bfloat16*>(W),
                                    ldw, reinterpret_cast<const __nv_bfloat16*>(X), ldx, out, ldo, T, N, K, add));
    return ATX_OK;
}
