// Shared helpers of the kernel library: error reporting, dtype codes, conversions.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a stream, returns 0
// on success and a non-zero code otherwise; `gi_last_error()` gives the message of the last failure
// on the calling thread. Nothing here allocates device memory: callers own every buffer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <tuple>
#include <vector>

namespace gi {

enum DType : int { kF32 = 0, kBF16 = 1 };

void set_error(const char* fmt, ...);

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch: every kernel of this library is launched with the attribute that
// lets it become resident while the kernel before it on the stream drains, and calls
// pdl_prologue() before it touches anything an earlier kernel wrote. The launch latency of a
// chain of small kernels (a decode step) then overlaps with execution.
extern int g_pdl_enabled;

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Timeline of a step (only in a library built with -DGI_TIMELINE; otherwise nothing is compiled in): kernels record
// (kernel id, event, block, %globaltimer) into a buffer that the host hands to every translation unit
// (gi_timeline_set_*), slot 0 of which counts the records. Events: 0 the block enters, 1 its wait for the
// kernel ahead is over, 2..5 kernel-specific, 6 the block (for kernels whose warps work alone: a warp) leaves.
#ifdef GI_TIMELINE
static __device__ unsigned long long* g_timeline = nullptr;
__device__ __forceinline__ void timeline_record(int kernel_id, int event) {
    unsigned long long* tl = g_timeline;
    if (!tl) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    const unsigned long long slot = atomicAdd(tl, 1ull);
    if (slot < tl[1]) {
        const unsigned block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        tl[2 + 2 * slot] = (static_cast<unsigned long long>(kernel_id) << 40) | (static_cast<unsigned long long>(event) << 32) | block;
        tl[3 + 2 * slot] = t;
    }
}
#define GI_TIMELINE_SETTER(name) \
    extern "C" int name(void* p) { return cudaMemcpyToSymbol(gi::g_timeline, &p, sizeof(p)) == cudaSuccess ? 0 : 1; }
#else
__device__ __forceinline__ void timeline_record(int, int) {}
#define GI_TIMELINE_SETTER(name) extern "C" int name(void*) { return 2; }
#endif
enum TimelineKernel : int {
    kTlRmsNorm = 1, kTlSwiGLU = 2, kTlAttentionDecode = 3, kTlAddRanges = 4, kTlRopeStore = 5, kTlAttentionPrefill = 6,
    kTlProduct = 100,            // + the form (TcSpecKind) of the few-token product
    kTlProductManyTokens = 200,  // + 2 * epilogue (TcEpilogue) + (1 on pairs of CTAs)
};

__device__ __forceinline__ void pdl_prologue() { pdl_launch_dependents(); pdl_wait(); }

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);      // errors surface in check_launch
}

// Launch programs. While a program is being recorded on the calling thread (gi_program_begin ..
// gi_program_end), every entry point that launches kernels runs as usual and also leaves a copy of its
// arguments in the program. gi_program_run() then repeats the whole sequence on a stream with one
// call: the host cost of a step's launches (argument checks, bindings) is paid once per shape.
// A program holds raw pointers and sizes: it is valid while the buffers it names are.
struct Program {
    std::vector<std::function<int(void*)>> calls;
};
extern thread_local Program* tl_recording;

// Runs impl(args...) and, while a program is recorded, stores a copy that takes the stream (the last
// argument of every launching entry point) from the later run.
template <typename... A>
inline int dispatch(int (*impl)(A...), A... args) {
    if (tl_recording != nullptr) {
        std::tuple<A...> tup(args...);
        tl_recording->calls.emplace_back([impl, tup](void* stream) mutable {
            std::get<sizeof...(A) - 1>(tup) = stream;
            return std::apply(impl, tup);
        });
    }
    return impl(args...);
}

}  // namespace gi

#define GI_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) {                   \
            gi::set_error(__VA_ARGS__);  \
            return 2;                    \
        }                                \
    } while (0)
