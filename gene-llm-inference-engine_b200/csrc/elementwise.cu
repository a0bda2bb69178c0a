// Memory-bound kernels of the step: embedding gather, RMSNorm, rotary position encoding fused with
// the key/value page store, SwiGLU, and the page copy used for copy-on-write.
//
// Numerics follow the reference's scalar definitions: RMSNorm `w * (scale * x)` with
// `scale = 1/sqrt(sum(x^2)/n + eps)` (src/kernels/kernels.cpp:72-83), rotation `a*c - b*s`,
// `a*s + b*c` (src/kernels/kernels.cpp:164-180), SiLU `g * (1/(1+exp(-g)))`
// (src/kernels/kernels.cpp:106-110). All arithmetic is 32-bit; only stores round.
#include "common.cuh"

#include <mutex>
#include <string>

namespace gi {

static thread_local std::string g_error;

int g_pdl_enabled = 1;

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
}

// ---------------------------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             const int* __restrict__ feedback, float* __restrict__ out, int D, float scale) {
    pdl_prologue();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0) tok = feedback[-tok - 1];      // the token a sampling kernel left on the device
    const TW* row = table + static_cast<size_t>(tok) * D;
    float* o = out + static_cast<size_t>(t) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = to_float(row[d]) * scale;
}

// ---------------------------------------------------------------------------------- RMSNorm
// One block per output row. Each thread sums a fixed strided subset with fmaf, lanes are combined
// by a fixed xor tree and warps in index order, so a row's result never depends on the batch.
// Rows whose length is a multiple of 4 are read once, 16 bytes at a time, and kept in registers
// between the sum and the scaling (up to 16 values per thread; longer rows are read twice).
template <typename TOut>
__device__ __forceinline__ void store4(TOut* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
}

template <typename TOut>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
               const float* __restrict__ weight, TOut* __restrict__ out, int D, float eps) {
    pdl_prologue();
    __shared__ float warp_part[32];
    __shared__ float s_scale;
    const int r = blockIdx.x;
    const float* xr = x + static_cast<size_t>(rows ? rows[r] : r) * D;
    TOut* o = out + static_cast<size_t>(r) * D;
    constexpr int kKeep = 4;                                    // float4 values a thread keeps
    const bool vec = (D % 4 == 0) && (reinterpret_cast<uintptr_t>(xr) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(o) % 16 == 0) && (reinterpret_cast<uintptr_t>(weight) % 16 == 0);
    float4 kept[kKeep];
    float ss = 0.f;
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const int n4 = D / 4;
        int i = threadIdx.x;
#pragma unroll
        for (int k = 0; k < kKeep; ++k, i += 256) {
            kept[k] = (i < n4) ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss = fmaf(kept[k].x, kept[k].x, ss); ss = fmaf(kept[k].y, kept[k].y, ss);
            ss = fmaf(kept[k].z, kept[k].z, ss); ss = fmaf(kept[k].w, kept[k].w, ss);
        }
        for (; i < n4; i += 256) {
            const float4 v = x4[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += 256) ss = fmaf(xr[d], xr[d], ss);
    }
    ss = warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) warp_part[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int w = 0; w < 8; ++w) total += warp_part[w];
        s_scale = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
    }
    __syncthreads();
    const float scale = s_scale;
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const float4* w4 = reinterpret_cast<const float4*>(weight);
        const int n4 = D / 4;
        int i = threadIdx.x;
#pragma unroll
        for (int k = 0; k < kKeep; ++k, i += 256) {
            if (i < n4) {
                const float4 w = w4[i];
                store4<TOut>(o + 4 * i, w.x * (scale * kept[k].x), w.y * (scale * kept[k].y), w.z * (scale * kept[k].z),
                             w.w * (scale * kept[k].w));
            }
        }
        for (; i < n4; i += 256) {
            const float4 v = x4[i], w = w4[i];
            store4<TOut>(o + 4 * i, w.x * (scale * v.x), w.y * (scale * v.y), w.z * (scale * v.z), w.w * (scale * v.w));
        }
    } else {
        for (int d = threadIdx.x; d < D; d += 256) o[d] = from_float<TOut>(weight[d] * (scale * xr[d]));
    }
}

// The same arithmetic in the same order for rows that every thread holds in registers (at most 4096 values, 16-byte
// accesses throughout, which the host checks): no loop, no second path, a few hundred instructions. Short kernels of a
// decode step pay for the instructions they have to fetch, so the common case has a kernel without the general one's code.
template <typename TOut>
__global__ void __launch_bounds__(256)
rmsnorm_rows_in_registers_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ weight, TOut* __restrict__ out, int D, float eps) {
    if (threadIdx.x == 0) timeline_record(kTlRmsNorm, 0);
    __shared__ float warp_part[8];
    __shared__ float s_scale;
    const int r = blockIdx.x;
    const int n4 = D / 4;
    // the weights belong to no earlier kernel: they are requested before this kernel waits for the one ahead
    pdl_launch_dependents();
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    float4 w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * 256;
        w[k] = (i < n4) ? __ldg(w4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    if (threadIdx.x == 0) timeline_record(kTlRmsNorm, 1);
    const float4* x4 = reinterpret_cast<const float4*>(x + static_cast<size_t>(rows ? rows[r] : r) * D);
    TOut* o = out + static_cast<size_t>(r) * D;
    float4 kept[4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * 256;
        kept[k] = (i < n4) ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(kept[k].x, kept[k].x, ss); ss = fmaf(kept[k].y, kept[k].y, ss);
        ss = fmaf(kept[k].z, kept[k].z, ss); ss = fmaf(kept[k].w, kept[k].w, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += warp_part[w];
        s_scale = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
    }
    __syncthreads();
    const float scale = s_scale;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < n4)
            store4<TOut>(o + 4 * i, w[k].x * (scale * kept[k].x), w[k].y * (scale * kept[k].y), w[k].z * (scale * kept[k].z),
                         w[k].w * (scale * kept[k].w));
    }
    if (threadIdx.x == 0) timeline_record(kTlRmsNorm, 6);
}

// ---------------------------------------------------------------------------------- SwiGLU
template <typename TOut>
__global__ void swiglu_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int I, size_t total) {
    if (threadIdx.x == 0) timeline_record(kTlSwiGLU, 0);
    pdl_prologue();
    if (threadIdx.x == 0) timeline_record(kTlSwiGLU, 1);
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / I;
    const int c = static_cast<int>(i % I);
    const float g = gu[t * 2 * I + c];
    const float u = gu[t * 2 * I + I + c];
    out[i] = from_float<TOut>(g * (1.0f / (1.0f + expf(-g))) * u);
    if (threadIdx.x == 0) timeline_record(kTlSwiGLU, 6);
}

// The same, four channels to a thread with 16-byte accesses (I a multiple of 4, pointers aligned): a quarter of the
// blocks (64 tokens of the Llama-3.2-1B shape: 512 blocks in one round instead of 2,048 in two).
template <typename TOut>
__global__ void swiglu4_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int I4, size_t total4) {
    if (threadIdx.x == 0) timeline_record(kTlSwiGLU, 0);
    pdl_prologue();
    if (threadIdx.x == 0) timeline_record(kTlSwiGLU, 1);
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const size_t t = i / I4;
    const int c = static_cast<int>(i % I4);
    const float4* row = reinterpret_cast<const float4*>(gu) + t * 2 * I4;
    const float4 g = row[c], u = row[I4 + c];
    store4<TOut>(out + 4 * i, g.x * (1.0f / (1.0f + expf(-g.x))) * u.x, g.y * (1.0f / (1.0f + expf(-g.y))) * u.y,
                 g.z * (1.0f / (1.0f + expf(-g.z))) * u.z, g.w * (1.0f / (1.0f + expf(-g.w))) * u.w);
    if (threadIdx.x == 0) timeline_record(kTlSwiGLU, 6);
}

// ---------------------------------------------------------------------------------- RoPE + store
__device__ __forceinline__ void store4(float* dst, const float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, const float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = raw;
}

// One block per token. Query heads are rotated and written to q_out; key heads are rotated and
// written to the token's cache row; value heads are copied there. cos/sin are rows of a table
// [max_position, rot_half] built on the host in double precision. A thread rotates one pair
// (both members read once), or four pairs with 16-byte accesses where the sizes allow; dims beyond
// the rotary size and the values are copied.
template <typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
rope_store_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                  const int* __restrict__ row_req, const int* __restrict__ block_tables,
                  int table_stride, const float* __restrict__ cos_t,
                  const float* __restrict__ sin_t, int rot_half, int interleaved,
                  TQ* __restrict__ q_out, TKV* __restrict__ k_cache, TKV* __restrict__ v_cache,
                  int H, int Hkv, int hd, int page_size, int write_kv) {
    if (threadIdx.x == 0) timeline_record(kTlRopeStore, 0);
    pdl_prologue();
    if (threadIdx.x == 0) timeline_record(kTlRopeStore, 1);
    const int t = blockIdx.x;
    const int pos = positions[t];
    const float* row = qkv + static_cast<size_t>(t) * (H + 2 * Hkv) * hd;
    const float* c = cos_t ? cos_t + static_cast<size_t>(pos) * rot_half : nullptr;
    const float* s = sin_t ? sin_t + static_cast<size_t>(pos) * rot_half : nullptr;
    const int half = c ? rot_half : 0;
    const int rot_dim = 2 * half;
    size_t kv_base = 0;
    if (write_kv) {
        const int page = block_tables[static_cast<size_t>(row_req[t]) * table_stride + pos / page_size];
        kv_base = (static_cast<size_t>(page) * Hkv * page_size + (pos % page_size)) * hd;
    }
    const int n_heads = H + (write_kv ? Hkv : 0);
    TQ* q_row = q_out + static_cast<size_t>(t) * H * hd;
    if (!interleaved && half % 4 == 0 && hd % 4 == 0) {
        // four pairs (k..k+3, k+half..k+half+3) per thread: 16-byte loads, 8- or 16-byte stores
        const int groups = half / 4;
        for (int e = threadIdx.x; e < n_heads * groups; e += blockDim.x) {
            const int head = e / groups, k = (e - head * groups) * 4;
            const float* v = row + static_cast<size_t>(head) * hd;
            const float4 a = *reinterpret_cast<const float4*>(v + k), b = *reinterpret_cast<const float4*>(v + k + half);
            const float4 ck = *reinterpret_cast<const float4*>(c + k), sk = *reinterpret_cast<const float4*>(s + k);
            const float4 oa = make_float4(a.x * ck.x - b.x * sk.x, a.y * ck.y - b.y * sk.y, a.z * ck.z - b.z * sk.z, a.w * ck.w - b.w * sk.w);
            const float4 ob = make_float4(a.x * sk.x + b.x * ck.x, a.y * sk.y + b.y * ck.y, a.z * sk.z + b.z * ck.z, a.w * sk.w + b.w * ck.w);
            if (head < H) {
                store4(q_row + head * hd + k, oa);
                store4(q_row + head * hd + k + half, ob);
            } else {
                TKV* kr = k_cache + kv_base + static_cast<size_t>(head - H) * page_size * hd;
                store4(kr + k, oa);
                store4(kr + k + half, ob);
            }
        }
        const int rest4 = (hd - rot_dim) / 4;                 // dims that are not rotated
        for (int e = threadIdx.x; e < n_heads * rest4; e += blockDim.x) {
            const int head = e / rest4, d = rot_dim + (e - head * rest4) * 4;
            const float4 v = *reinterpret_cast<const float4*>(row + static_cast<size_t>(head) * hd + d);
            if (head < H) store4(q_row + head * hd + d, v);
            else store4(k_cache + kv_base + static_cast<size_t>(head - H) * page_size * hd + d, v);
        }
        if (write_kv) {
            const float* vrow = row + static_cast<size_t>(H + Hkv) * hd;
            const int per_head = hd / 4;
            for (int e = threadIdx.x; e < Hkv * per_head; e += blockDim.x) {
                const int g = e / per_head, d = (e - g * per_head) * 4;
                store4(v_cache + kv_base + static_cast<size_t>(g) * page_size * hd + d,
                       *reinterpret_cast<const float4*>(vrow + static_cast<size_t>(g) * hd + d));
            }
        }
        return;
    }
    // rotated pairs
    for (int e = threadIdx.x; e < n_heads * half; e += blockDim.x) {
        const int head = e / half, k = e - head * half;
        const float* v = row + static_cast<size_t>(head) * hd;
        const int ia = interleaved ? 2 * k : k, ib = interleaved ? 2 * k + 1 : k + half;
        const float a = v[ia], b = v[ib], ck = c[k], sk = s[k];
        const float oa = a * ck - b * sk, ob = a * sk + b * ck;
        if (head < H) {
            q_row[head * hd + ia] = from_float<TQ>(oa);
            q_row[head * hd + ib] = from_float<TQ>(ob);
        } else {
            TKV* kr = k_cache + kv_base + static_cast<size_t>(head - H) * page_size * hd;
            kr[ia] = from_float<TKV>(oa);
            kr[ib] = from_float<TKV>(ob);
        }
    }
    // dims that are not rotated
    const int rest = hd - rot_dim;
    for (int e = threadIdx.x; e < n_heads * rest; e += blockDim.x) {
        const int head = e / rest, d = rot_dim + (e - head * rest);
        const float v = row[static_cast<size_t>(head) * hd + d];
        if (head < H) q_row[head * hd + d] = from_float<TQ>(v);
        else k_cache[kv_base + static_cast<size_t>(head - H) * page_size * hd + d] = from_float<TKV>(v);
    }
    if (write_kv) {
        const float* vrow = row + static_cast<size_t>(H + Hkv) * hd;
        for (int e = threadIdx.x; e < Hkv * hd; e += blockDim.x) {
            const int g = e / hd, d = e - g * hd;
            v_cache[kv_base + static_cast<size_t>(g) * page_size * hd + d] = from_float<TKV>(vrow[e]);
        }
    }
}

// ---------------------------------------------------------------------------------- page copy
__global__ void copy_pages_kernel(char* base, size_t array_stride, size_t page_bytes,
                                  const int* __restrict__ src, const int* __restrict__ dst) {
    pdl_prologue();
    char* arr = base + blockIdx.y * array_stride;
    const uint4* s = reinterpret_cast<const uint4*>(arr + static_cast<size_t>(src[blockIdx.x]) * page_bytes);
    uint4* d = reinterpret_cast<uint4*>(arr + static_cast<size_t>(dst[blockIdx.x]) * page_bytes);
    for (size_t i = threadIdx.x; i < page_bytes / 16; i += blockDim.x) d[i] = s[i];
}

}  // namespace gi

using namespace gi;
GI_TIMELINE_SETTER(gi_timeline_set_elementwise)

extern "C" {

const char* gi_last_error() { return g_error.c_str(); }

// Switches programmatic dependent launch on (1, the default) or off (0) for all later launches.
int gi_set_pdl(int enabled) {
    g_pdl_enabled = enabled ? 1 : 0;
    return 0;
}

// tokens[t] >= 0 is a token id; tokens[t] = -(k + 1) takes the id from feedback[k] (device memory
// that an earlier sampling kernel wrote; may be null when no entry is negative).
static int gi_embed_impl(const void* table, int table_dtype, const int* tokens, const int* feedback, float* out, int T, int D,
             float scale, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && D > 0, "embed: T and D must be positive (T=%d, D=%d)", T, D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (table_dtype == kF32) {
        launch_kernel((embed_kernel<float>), dim3(T), dim3(256), 0, st, static_cast<const float*>(table), tokens, feedback, out, D, scale);
    } else if (table_dtype == kBF16) {
        launch_kernel((embed_kernel<__nv_bfloat16>), dim3(T), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(table), tokens, feedback, out, D, scale);
    } else {
        GI_REQUIRE(false, "embed: unsupported table dtype code %d", table_dtype);
    }
    return check_launch("embed");
}

static int gi_rmsnorm_impl(const float* x, const int* rows, const float* weight, void* out, int out_dtype, int n_rows, int D,
               float eps, void* stream) {
    if (n_rows == 0) return 0;
    GI_REQUIRE(n_rows > 0 && D > 0, "rmsnorm: sizes must be positive (rows=%d, D=%d)", n_rows, D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // rows of at most 4096 values whose every access is 16 bytes wide: the lean kernel
    const size_t out_row_bytes = static_cast<size_t>(D) * (out_dtype == kF32 ? 4 : 2);
    const bool lean = D % 4 == 0 && D <= 4096 && out_row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0;
    if (out_dtype == kF32) {
        if (lean) launch_kernel((rmsnorm_rows_in_registers_kernel<float>), dim3(n_rows), dim3(256), 0, st, x, rows, weight, static_cast<float*>(out), D, eps);
        else launch_kernel((rmsnorm_kernel<float>), dim3(n_rows), dim3(256), 0, st, x, rows, weight, static_cast<float*>(out), D, eps);
    } else if (out_dtype == kBF16) {
        if (lean) launch_kernel((rmsnorm_rows_in_registers_kernel<__nv_bfloat16>), dim3(n_rows), dim3(256), 0, st, x, rows, weight, static_cast<__nv_bfloat16*>(out), D, eps);
        else launch_kernel((rmsnorm_kernel<__nv_bfloat16>), dim3(n_rows), dim3(256), 0, st, x, rows, weight, static_cast<__nv_bfloat16*>(out), D, eps);
    } else {
        GI_REQUIRE(false, "rmsnorm: unsupported output dtype code %d", out_dtype);
    }
    return check_launch("rmsnorm");
}

static int gi_swiglu_impl(const float* gate_up, void* out, int out_dtype, int T, int I, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && I > 0, "swiglu: sizes must be positive (T=%d, I=%d)", T, I);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t total = static_cast<size_t>(T) * I;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    const bool by4 = I % 4 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    const unsigned blocks4 = static_cast<unsigned>((total / 4 + 255) / 256);
    if (out_dtype == kF32) {
        if (by4) launch_kernel((swiglu4_kernel<float>), dim3(blocks4), dim3(256), 0, st, gate_up, static_cast<float*>(out), I / 4, total / 4);
        else launch_kernel((swiglu_kernel<float>), dim3(blocks), dim3(256), 0, st, gate_up, static_cast<float*>(out), I, total);
    } else if (out_dtype == kBF16) {
        if (by4) launch_kernel((swiglu4_kernel<__nv_bfloat16>), dim3(blocks4), dim3(256), 0, st, gate_up, static_cast<__nv_bfloat16*>(out), I / 4, total / 4);
        else launch_kernel((swiglu_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, st, gate_up, static_cast<__nv_bfloat16*>(out), I, total);
    } else {
        GI_REQUIRE(false, "swiglu: unsupported output dtype code %d", out_dtype);
    }
    return check_launch("swiglu");
}

// dtype: the type of q_out and of the cache (both f32 on the 32-bit path, both bf16 otherwise).
static int gi_rope_store_impl(const float* qkv, const int* positions, const int* row_req, const int* block_tables,
                  int table_stride, const float* cos_t, const float* sin_t, int rot_half, int interleaved,
                  void* q_out, void* k_cache, void* v_cache, int dtype, int T, int H, int Hkv, int hd,
                  int page_size, int write_kv, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && H > 0 && Hkv > 0 && hd > 0 && page_size > 0, "rope_store: sizes must be positive");
    GI_REQUIRE(2 * rot_half <= hd, "rope_store: rotary size %d exceeds the head size %d", 2 * rot_half, hd);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // a thread handles four pairs where it can: a quarter of the threads do for a token
    const bool vec = !interleaved && rot_half % 4 == 0 && hd % 4 == 0 && cos_t != nullptr;
    const int threads = vec ? 128 : 256;
    if (dtype == kF32) {
        launch_kernel((rope_store_kernel<float, float>), dim3(T), dim3(threads), 0, st, 
            qkv, positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved,
            static_cast<float*>(q_out), static_cast<float*>(k_cache), static_cast<float*>(v_cache), H, Hkv, hd,
            page_size, write_kv);
    } else if (dtype == kBF16) {
        launch_kernel((rope_store_kernel<__nv_bfloat16, __nv_bfloat16>), dim3(T), dim3(threads), 0, st, 
            qkv, positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved,
            static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
            static_cast<__nv_bfloat16*>(v_cache), H, Hkv, hd, page_size, write_kv);
    } else {
        GI_REQUIRE(false, "rope_store: unsupported dtype code %d", dtype);
    }
    return check_launch("rope_store");
}

static int gi_copy_pages_impl(void* base, long long array_stride_bytes, int n_arrays, long long page_bytes, const int* src,
                  const int* dst, int n_copies, void* stream) {
    if (n_copies == 0 || n_arrays == 0) return 0;
    GI_REQUIRE(page_bytes % 16 == 0, "copy_pages: a page of %lld bytes is not a multiple of 16", page_bytes);
    dim3 grid(n_copies, n_arrays);
    launch_kernel((copy_pages_kernel), dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), 
        static_cast<char*>(base), static_cast<size_t>(array_stride_bytes), static_cast<size_t>(page_bytes), src, dst);
    return check_launch("copy_pages");
}

}  // extern "C"

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_embed(const void* table, int table_dtype, const int* tokens, const int* feedback, float* out, int T, int D, float scale, void* stream) {
    return gi::dispatch(gi_embed_impl, table, table_dtype, tokens, feedback, out, T, D, scale, stream);
}

extern "C" int gi_rmsnorm(const float* x, const int* rows, const float* weight, void* out, int out_dtype, int n_rows, int D, float eps, void* stream) {
    return gi::dispatch(gi_rmsnorm_impl, x, rows, weight, out, out_dtype, n_rows, D, eps, stream);
}

extern "C" int gi_swiglu(const float* gate_up, void* out, int out_dtype, int T, int I, void* stream) {
    return gi::dispatch(gi_swiglu_impl, gate_up, out, out_dtype, T, I, stream);
}

extern "C" int gi_rope_store(const float* qkv, const int* positions, const int* row_req, const int* block_tables, int table_stride, const float* cos_t, const float* sin_t, int rot_half, int interleaved, void* q_out, void* k_cache, void* v_cache, int dtype, int T, int H, int Hkv, int hd, int page_size, int write_kv, void* stream) {
    return gi::dispatch(gi_rope_store_impl, qkv, positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved, q_out, k_cache, v_cache, dtype, T, H, Hkv, hd, page_size, write_kv, stream);
}

extern "C" int gi_copy_pages(void* base, long long array_stride_bytes, int n_arrays, long long page_bytes, const int* src, const int* dst, int n_copies, void* stream) {
    return gi::dispatch(gi_copy_pages_impl, base, array_stride_bytes, n_arrays, page_bytes, src, dst, n_copies, stream);
}
