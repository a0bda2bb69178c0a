// Matrix product on the CUDA cores with 32-bit fused multiply-adds: C[M,N] (+)= A[M,K] * W[N,K]^T.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision mode)
// and accepts bfloat16 operands too (widened exactly), for any M, N, K. Every output element is one
// chain of fmaf over k = 0..K-1 in increasing order, whatever M is and wherever the row sits in
// the batch: results do not depend on how tokens are cut into steps (the property the reference
// states for its own kernels, src/gpu/device_kernels.inc:97-100).
#include "common.cuh"

namespace gi {

constexpr int kBM = 64, kBN = 64, kBK = 16;

template <typename TA, typename TW, typename TC, bool kAccumulate>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                 int lda, int ldw, int ldc) {
    pdl_prologue();
    __shared__ float sA[kBK][kBM + 4];
    __shared__ float sW[kBK][kBN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // Each thread loads 4 elements of each operand tile per k-step: tile row = threadIdx.x / 4,
    // k offsets (threadIdx.x % 4) * 4 .. +3.
    const int lr = threadIdx.x / 4, lk = (threadIdx.x % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += kBK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int am = m0 + lr, wn = n0 + lr;
            sA[lk + i][lr] = (am < M && k < K) ? to_float(A[static_cast<size_t>(am) * lda + k]) : 0.f;
            sW[lk + i][lr] = (wn < N && k < K) ? to_float(W[static_cast<size_t>(wn) * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kBK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = sW[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            TC* c = C + static_cast<size_t>(m) * ldc + n;
            const float v = kAccumulate ? to_float(*c) + acc[i][j] : acc[i][j];
            *c = from_float<TC>(v);
        }
    }
}

template <typename TA, typename TW>
int launch_simt(const void* A, const void* W, void* C, int c_dtype, int accumulate, int M, int N, int K, int lda,
                int ldw, int ldc, cudaStream_t st) {
    dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM);
    const TA* a = static_cast<const TA*>(A);
    const TW* w = static_cast<const TW*>(W);
    if (c_dtype == kF32) {
        float* c = static_cast<float*>(C);
        if (accumulate) launch_kernel((gemm_simt_kernel<TA, TW, float, true>), dim3(grid), dim3(256), 0, st, a, w, c, M, N, K, lda, ldw, ldc);
        else launch_kernel((gemm_simt_kernel<TA, TW, float, false>), dim3(grid), dim3(256), 0, st, a, w, c, M, N, K, lda, ldw, ldc);
    } else {
        __nv_bfloat16* c = static_cast<__nv_bfloat16*>(C);
        if (accumulate) launch_kernel((gemm_simt_kernel<TA, TW, __nv_bfloat16, true>), dim3(grid), dim3(256), 0, st, a, w, c, M, N, K, lda, ldw, ldc);
        else launch_kernel((gemm_simt_kernel<TA, TW, __nv_bfloat16, false>), dim3(grid), dim3(256), 0, st, a, w, c, M, N, K, lda, ldw, ldc);
    }
    return check_launch("gemm_simt");
}

}  // namespace gi

using namespace gi;

// C[M,N] (+)= A[M,K] * W[N,K]^T; row strides lda, ldw, ldc in elements.
static int gi_gemm_simt_impl(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                            int accumulate, int M, int N, int K, int lda, int ldw, int ldc, void* stream) {
    if (M == 0 || N == 0) return 0;
    GI_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: sizes must be positive (M=%d, N=%d, K=%d)", M, N, K);
    GI_REQUIRE((M + kBM - 1) / kBM <= 65535, "gemm: M=%d exceeds the grid limit", M);
    GI_REQUIRE(c_dtype == kF32 || c_dtype == kBF16, "gemm: unsupported output dtype code %d", c_dtype);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a_dtype == kF32 && w_dtype == kF32) return launch_simt<float, float>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, st);
    if (a_dtype == kF32 && w_dtype == kBF16) return launch_simt<float, __nv_bfloat16>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, st);
    if (a_dtype == kBF16 && w_dtype == kBF16) return launch_simt<__nv_bfloat16, __nv_bfloat16>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, st);
    GI_REQUIRE(false, "gemm: unsupported operand dtype codes (A=%d, W=%d)", a_dtype, w_dtype);
}

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int accumulate, int M, int N, int K, int lda, int ldw, int ldc, void* stream) {
    return gi::dispatch(gi_gemm_simt_impl, A, a_dtype, W, w_dtype, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, stream);
}
