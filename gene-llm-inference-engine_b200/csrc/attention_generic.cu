// Paged causal attention, general form: one block per (query row, query head), any mix of prompt
// portions and single decoded tokens, any head size that is a multiple of 16 up to 256, any page
// size, grouped key/value heads, optional sliding window.
//
// Definition (src/model/transformer.cpp:228-255, src/kernels/kernels.cpp:87-104): for the query
// at position P of its request, scores s_j = (q . k_j) * scale for j = lo..P only (causality is
// the loop bound; lo = 0, or P-window+1 with a window), softmax over them, out = sum_j p_j v_j.
// Softmax is computed online in 32-bit: each warp walks tiles of 32 keys in increasing order with
// a running max and sum, and the four warps are merged in warp order. A row's result depends only
// on that row's query and cache contents, never on the rest of the batch.
//
// This kernel is the whole attention of the 32-bit path and the fallback of the bfloat16 path.
#include "common.cuh"

namespace gi {

constexpr int kAttWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
    float acc = 0.f;
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int i = 0; i < hd / 4; ++i) {
        const float4 v = k4[i];
        acc = fmaf(q[4 * i + 0], v.x, acc);
        acc = fmaf(q[4 * i + 1], v.y, acc);
        acc = fmaf(q[4 * i + 2], v.z, acc);
        acc = fmaf(q[4 * i + 3], v.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int hd) {
    float acc = 0.f;
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int i = 0; i < hd / 8; ++i) {
        const uint4 raw = k8[i];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            acc = fmaf(q[8 * i + 2 * j], f.x, acc);
            acc = fmaf(q[8 * i + 2 * j + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(kAttWarps * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, T* __restrict__ out,
                               const int* __restrict__ row_req, const int* __restrict__ positions,
                               const int* __restrict__ block_tables, int table_stride, int H, int Hkv, int hd,
                               int page_size, float scale, int window) {
    pdl_prologue();
    __shared__ float s_q[kMaxHeadDim];
    __shared__ float s_acc[kAttWarps][kMaxHeadDim];
    __shared__ float s_m[kAttWarps], s_l[kAttWarps];

    const int h = blockIdx.x, t = blockIdx.y;
    const int g = h / (H / Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_tables + static_cast<size_t>(row_req[t]) * table_stride;

    for (int d = threadIdx.x; d < hd; d += blockDim.x)
        s_q[d] = to_float(q[(static_cast<size_t>(t) * H + h) * hd + d]);
    __syncthreads();

    constexpr int kDimsPerLane = kMaxHeadDim / 32;
    float acc[kDimsPerLane];
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int first_tile = lo / 32;
    const int last_tile = pos / 32;
    for (int tile = first_tile + warp; tile <= last_tile; tile += kAttWarps) {
        const int j = tile * 32 + lane;
        const bool valid = j >= lo && j <= pos;
        float score = -INFINITY;
        size_t row_off = 0;
        if (valid) {
            const int page = table[j / page_size];
            row_off = ((static_cast<size_t>(page) * Hkv + g) * page_size + (j % page_size)) * hd;
            score = dot_row<T>(s_q, k_cache + row_off, hd) * scale;
        }
        const float tile_max = warp_max(score);          // finite: a tile always holds a valid key
        const float m_new = fmaxf(m, tile_max);
        const float p = valid ? expf(score - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < kDimsPerLane; ++i) acc[i] *= corr;
        m = m_new;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const size_t off = __shfl_sync(0xffffffffu, static_cast<unsigned long long>(row_off), jj);
            if (pj == 0.f) continue;                      // uniform across the warp
            const T* vrow = v_cache + off;
#pragma unroll
            for (int i = 0; i < kDimsPerLane; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_float(vrow[d]), acc[i]);
            }
        }
    }

    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) s_acc[warp][d] = acc[i];
    }
    __syncthreads();

    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttWarps; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f;
    float f[kAttWarps];
#pragma unroll
    for (int w = 0; w < kAttWarps; ++w) {
        f[w] = (s_m[w] == -INFINITY) ? 0.f : expf(s_m[w] - M);
        L += s_l[w] * f[w];
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kAttWarps; ++w) o += s_acc[w][d] * f[w];
        out[(static_cast<size_t>(t) * H + h) * hd + d] = from_float<T>(o / L);
    }
}

}  // namespace gi

using namespace gi;

// 1 when the general kernel serves this head size: the model is refused when it is built, not at its first step.
extern "C" int gi_attention_generic_supported(int hd) { return hd % 16 == 0 && hd >= 16 && hd <= kMaxHeadDim; }

static int gi_attention_generic_impl(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                    const int* row_req, const int* positions, const int* block_tables,
                                    int table_stride, int T, int H, int Hkv, int hd, int page_size, float scale,
                                    int window, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && H > 0 && Hkv > 0 && page_size > 0, "attention: sizes must be positive");
    GI_REQUIRE(H % Hkv == 0, "attention: %d query heads are not a multiple of %d key/value heads", H, Hkv);
    GI_REQUIRE(hd % 16 == 0 && hd >= 16 && hd <= kMaxHeadDim,
               "attention: head size %d is not supported (multiples of 16 up to %d)", hd, kMaxHeadDim);
    GI_REQUIRE(T <= 65535, "attention: %d rows in one step exceed the grid limit 65535", T);
    dim3 grid(H, T);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == kF32) {
        launch_kernel((paged_attention_generic_kernel<float>), dim3(grid), dim3(kAttWarps * 32), 0, st, 
            static_cast<const float*>(q), static_cast<const float*>(k_cache), static_cast<const float*>(v_cache),
            static_cast<float*>(out), row_req, positions, block_tables, table_stride, H, Hkv, hd, page_size, scale,
            window);
    } else if (dtype == kBF16) {
        launch_kernel((paged_attention_generic_kernel<__nv_bfloat16>), dim3(grid), dim3(kAttWarps * 32), 0, st, 
            static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
            static_cast<const __nv_bfloat16*>(v_cache), static_cast<__nv_bfloat16*>(out), row_req, positions,
            block_tables, table_stride, H, Hkv, hd, page_size, scale, window);
    } else {
        GI_REQUIRE(false, "attention: unsupported dtype code %d", dtype);
    }
    return check_launch("attention_generic");
}

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_attention_generic(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype, const int* row_req, const int* positions, const int* block_tables, int table_stride, int T, int H, int Hkv, int hd, int page_size, float scale, int window, void* stream) {
    return gi::dispatch(gi_attention_generic_impl, q, k_cache, v_cache, out, dtype, row_req, positions, block_tables, table_stride, T, H, Hkv, hd, page_size, scale, window, stream);
}
