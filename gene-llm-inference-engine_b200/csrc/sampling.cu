// Sampling on the device: greedy argmax, and temperature sampling with optional top-k / top-p.
//
// Semantics of the reference sampler (src/sampler/sampler.h:3-27, src/sampler/sampler.cpp:55-129):
//   greedy: the largest logit, the lowest index among equals;
//   otherwise p_i = exp((logit_i - max) / temperature) * (float)(1 / sum), sum in double;
//   top-k keeps the k most likely tokens (probability descending, index ascending among equals),
//   top-p then keeps the shortest prefix of that order whose mass reaches top_p * (kept mass);
//   the draw returns the first kept token, in that order (index order when no filter is on),
//   whose cumulative probability exceeds u * (kept mass).
// The uniform number u of every row comes from the caller (the per-request xorshift64* stream is
// kept on the host so that a request's stream does not depend on the batch it is in).
//
// The sorted order is never materialised. A position in it (the k-th token, the place where the
// cumulative mass crosses a threshold) is found by a radix descent over the 32 bits of the
// probabilities: histograms of counts and of double-precision masses per 8-bit digit, four
// passes, then index order inside the last group of equal probabilities. One block per row.
#include "common.cuh"

namespace gi {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) total += scratch[w];
    return total;
}

// Greedy argmax in two steps: kArgmaxParts blocks per row each find the best of a slice of the
// vocabulary (lowest index among equals), then one block per row picks among the slice winners.
// One block per row would read 0.5 MB through a single SM.
constexpr int kArgmaxParts = 32;

__device__ __forceinline__ void argmax_block_reduce(float& best, int& best_i, float* s_val, int* s_idx) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w) {
            if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) { best = s_val[w]; best_i = s_idx[w]; }
        }
    }
}

// grid (kArgmaxParts, rows): the best of one slice -> part_val / part_idx [rows, kArgmaxParts]
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int V, float* __restrict__ part_val, int* __restrict__ part_idx) {
    pdl_prologue();
    __shared__ float s_val[8];
    __shared__ int s_idx[8];
    const float* row = logits + static_cast<size_t>(blockIdx.y) * V;
    const int per = (V + kArgmaxParts - 1) / kArgmaxParts;
    const int begin = blockIdx.x * per, end = min(V, begin + per);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += 256) {
        const float v = row[i];
        if (v > best || best_i == 0x7fffffff) { best = v; best_i = i; }   // increasing i: ties keep the lower index
    }
    argmax_block_reduce(best, best_i, s_val, s_idx);
    if (threadIdx.x == 0) {
        part_val[blockIdx.y * kArgmaxParts + blockIdx.x] = best;
        part_idx[blockIdx.y * kArgmaxParts + blockIdx.x] = best_i;
    }
}

// one warp per row
__global__ void __launch_bounds__(32)
argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int* __restrict__ out) {
    pdl_prologue();
    float best = part_val[blockIdx.x * kArgmaxParts + threadIdx.x];
    int best_i = part_idx[blockIdx.x * kArgmaxParts + threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
}

// The bits fixed so far of the value searched for: elements with (bits & mask) == prefix remain.
struct Descent {
    unsigned prefix;
    unsigned mask;
};

// Walks the values from the largest downwards, 8 bits per pass: in each pass the bucket is chosen in
// which the running total of weights (1 per element if kByCount, else the probability), started
// at `before`, first reaches (inclusive) or exceeds the target. On return d.prefix holds all 32
// bits of the value found and `before` the total weight of the strictly larger values.
template <bool kByCount>
__device__ void radix_descend(const float* __restrict__ probs, int V, double target, bool inclusive,
                              Descent& d, double& before, double* s_hist_w, unsigned* s_hist_c,
                              int* s_choice) {
    // kByCount: weight of an element is 1 (find the k-th element); else its probability.
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) { s_hist_w[b] = 0.0; s_hist_c[b] = 0u; }
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const unsigned bits = __float_as_uint(probs[i]);
            if ((bits & d.mask) == d.prefix) {
                const unsigned digit = (bits >> shift) & 255u;
                if (kByCount) atomicAdd(&s_hist_c[digit], 1u);
                else atomicAdd(&s_hist_w[digit], static_cast<double>(probs[i]));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            double run = before, run_before = before;
            int choice = 0;
            for (int b = 255; b >= 0; --b) {
                const double w = kByCount ? static_cast<double>(s_hist_c[b]) : s_hist_w[b];
                if (w == 0.0) continue;
                run_before = run;
                choice = b;
                const double next = run + w;
                if (inclusive ? (next >= target) : (next > target)) break;
                run = next;
            }
            // If rounding never reaches the target, the lowest non-empty bucket stays chosen and
            // the total before it is reported: the caller's walk over equal values then ends on
            // the last element.
            s_choice[0] = choice;
            s_hist_w[256] = run_before;
        }
        __syncthreads();
        before = s_hist_w[256];
        d.prefix |= static_cast<unsigned>(s_choice[0]) << shift;
        d.mask |= 255u << shift;
        __syncthreads();
    }
}

// Among elements whose probability bits equal `bits`, in index order: the 0-based rank of the
// first one at which before + (rank+1)*w reaches (inclusive) or exceeds the target; the element's
// index is returned; `n_equal` receives the group size.
__device__ int nth_equal_index(const float* __restrict__ probs, int V, unsigned bits, int rank, int* s_tmp) {
    // rank-th (0-based) index with probs == bits, by a block-wide ordered count.
    __shared__ int s_counts[kSampleThreads];
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int begin = threadIdx.x * per, end = min(V, begin + per);
    int c = 0;
    for (int i = begin; i < end; ++i) c += (__float_as_uint(probs[i]) == bits);
    s_counts[threadIdx.x] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, owner = blockDim.x - 1, inner = 0;
        for (int t = 0; t < static_cast<int>(blockDim.x); ++t) {
            if (run + s_counts[t] > rank) { owner = t; inner = rank - run; break; }
            run += s_counts[t];
        }
        s_tmp[0] = owner;
        s_tmp[1] = inner;
    }
    __syncthreads();
    const int owner = s_tmp[0], inner = s_tmp[1];
    __syncthreads();
    if (threadIdx.x == owner) {
        int seen = 0, found = -1;
        for (int i = begin; i < end; ++i) {
            if (__float_as_uint(probs[i]) == bits) {
                if (seen == inner) { found = i; break; }
                ++seen;
            }
        }
        s_tmp[2] = found;
    }
    __syncthreads();
    return s_tmp[2];
}

__device__ int count_equal(const float* __restrict__ probs, int V, unsigned bits, double* scratch) {
    double c = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) c += (__float_as_uint(probs[i]) == bits) ? 1.0 : 0.0;
    return static_cast<int>(block_sum_double(c, scratch));
}

// One block per row. probs: scratch [rows, V] floats.
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, float* __restrict__ probs_all, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
    pdl_prologue();
    __shared__ double s_red[32];
    __shared__ double s_hist_w[257];
    __shared__ unsigned s_hist_c[256];
    __shared__ int s_choice[4];
    __shared__ float s_maxes[32];

    const int r = blockIdx.x;
    const float* row = logits + static_cast<size_t>(r) * V;
    float* probs = probs_all + static_cast<size_t>(r) * V;
    const float temp = temperature[r];
    if (!(temp > 0.f)) return;          // a greedy row: out[r] keeps what the caller put there (its argmax)

    // max
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) s_maxes[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (blockDim.x >> 5); ++w) mx = fmaxf(mx, s_maxes[w]);

    // p_i = exp((l_i - max)/T), sum in double, then scaled by (float)(1/sum)
    double part = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float e = expf((row[i] - mx) / temp);
        probs[i] = e;
        part += static_cast<double>(e);
    }
    const double sum = block_sum_double(part, s_red);
    const float inv_sum = static_cast<float>(1.0 / sum);
    part = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float p = probs[i] * inv_sum;
        probs[i] = p;
        part += static_cast<double>(p);
    }
    __syncthreads();
    const double all_mass = block_sum_double(part, s_red);

    const int k = top_k[r];
    const float tp = top_p[r];
    const bool use_k = k > 0 && k < V;
    const bool use_p = tp < 1.0f;
    const double u = static_cast<double>(uniform[r]);

    if (!use_k && !use_p) {
        // index order: thread t owns a contiguous range; block scan of range masses in double
        __shared__ double s_range[kSampleThreads];
        const int per = (V + blockDim.x - 1) / blockDim.x;
        const int begin = threadIdx.x * per, end = min(V, begin + per);
        double mine = 0.0;
        for (int i = begin; i < end; ++i) mine += static_cast<double>(probs[i]);
        s_range[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            const double target = u * all_mass;
            double run = 0.0;
            int owner = -1;
            for (int t = 0; t < static_cast<int>(blockDim.x); ++t) {
                if (target < run + s_range[t]) { owner = t; break; }
                run += s_range[t];
            }
            s_choice[0] = owner;
            s_hist_w[256] = run;
        }
        __syncthreads();
        const int owner = s_choice[0];
        if (owner < 0) {
            if (threadIdx.x == 0) out[r] = V - 1;          // rounding guard: u was (almost) 1
        } else if (threadIdx.x == owner) {
            const double target = u * all_mass;
            double cum = s_hist_w[256];
            int pick = end - 1;
            for (int i = begin; i < end; ++i) {
                cum += static_cast<double>(probs[i]);
                if (target < cum) { pick = i; break; }
            }
            out[r] = pick;
        }
        return;
    }

    // ---- the kept set is a prefix of the order (probability descending, index ascending) ----
    // Its end is described by (boundary bits, number of boundary-valued elements kept).
    // Start: everything kept.
    double kept_mass = all_mass;
    unsigned bound_bits = 0u;        // smallest kept probability's bits
    int bound_take = 0;              // how many elements equal to it are kept (index order)
    bool bounded = false;

    if (use_k) {
        Descent d{0u, 0u};
        double before = 0.0;
        radix_descend<true>(probs, V, static_cast<double>(k), true, d, before, s_hist_w, s_hist_c, s_choice);
        bound_bits = d.prefix;
        bound_take = k - static_cast<int>(before);           // before = count of strictly larger elements
        bounded = true;
        // mass of the kept set
        double m = 0.0;
        for (int i = threadIdx.x; i < V; i += blockDim.x)
            if (__float_as_uint(probs[i]) > bound_bits) m += static_cast<double>(probs[i]);
        __syncthreads();
        kept_mass = block_sum_double(m, s_red) + static_cast<double>(bound_take) * static_cast<double>(__uint_as_float(bound_bits));
    }

    if (use_p) {
        // shortest prefix with cum >= top_p * kept_mass, inside the current kept set.
        const double threshold = static_cast<double>(tp) * kept_mass;
        // The descent runs over all elements; as the kept set is a prefix of the same order, the
        // crossing lies inside it unless rounding pushes it out, which is checked below.
        Descent d{0u, 0u};
        double before = 0.0;
        radix_descend<false>(probs, V, threshold, true, d, before, s_hist_w, s_hist_c, s_choice);
        unsigned nb = d.prefix;
        const double w = static_cast<double>(__uint_as_float(nb));
        int n_equal = count_equal(probs, V, nb, s_red);
        // first rank (1-based count) with before + c*w >= threshold
        int take = 1;
        if (w > 0.0) {
            double cum = before;
            take = n_equal;
            for (int c = 1; c <= n_equal; ++c) { cum += w; if (cum >= threshold) { take = c; break; } }
        }
        bool p_inside = true;
        if (bounded) {
            // the top-p end must not lie beyond the top-k end
            if (nb < bound_bits || (nb == bound_bits && take > bound_take)) p_inside = false;
        }
        if (p_inside) {
            bound_bits = nb;
            bound_take = take;
            bounded = true;
            kept_mass = before + static_cast<double>(take) * w;
        }
    }

    // ---- draw: first token in the order with u * kept_mass < cum ----
    const double target = u * kept_mass;
    Descent d{0u, 0u};
    double before = 0.0;
    radix_descend<false>(probs, V, target, false, d, before, s_hist_w, s_hist_c, s_choice);
    unsigned pick_bits = d.prefix;
    int rank = 0;
    {
        const double w = static_cast<double>(__uint_as_float(pick_bits));
        const int n_equal = count_equal(probs, V, pick_bits, s_red);
        rank = n_equal - 1;
        double cum = before;
        for (int c = 0; c < n_equal; ++c) { cum += w; if (target < cum) { rank = c; break; } }
    }
    // clamp to the kept set (rounding guard: the last kept token)
    if (bounded && (pick_bits < bound_bits || (pick_bits == bound_bits && rank >= bound_take))) {
        pick_bits = bound_bits;
        rank = bound_take - 1;
    }
    const int idx = nth_equal_index(probs, V, pick_bits, rank, s_choice);
    if (threadIdx.x == 0) out[r] = idx;
}

}  // namespace gi

using namespace gi;

// part_val / part_idx: caller's scratch of rows * 32 floats / ints.
static int gi_argmax_impl(const float* logits, int rows, int V, int* out, float* part_val, int* part_idx, void* stream) {
    if (rows == 0) return 0;
    GI_REQUIRE(rows > 0 && V > 0, "argmax: sizes must be positive (rows=%d, V=%d)", rows, V);
    GI_REQUIRE(rows <= 65535, "argmax: %d rows exceed the grid limit", rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    launch_kernel((argmax_partial_kernel), dim3(kArgmaxParts, rows), dim3(256), 0, st, logits, V, part_val, part_idx);
    if (check_launch("argmax")) return 1;
    launch_kernel((argmax_final_kernel), dim3(rows), dim3(32), 0, st, static_cast<const float*>(part_val),
                  static_cast<const int*>(part_idx), out);
    return check_launch("argmax");
}

// probs_scratch: [rows, V] floats owned by the caller. Rows with temperature[r] <= 0 are skipped:
// out[r] is left as it is (the caller writes the row's argmax there first).
static int gi_sample_impl(const float* logits, float* probs_scratch, int rows, int V, const float* temperature,
                         const int* top_k, const float* top_p, const float* uniform, int* out, void* stream) {
    if (rows == 0) return 0;
    GI_REQUIRE(rows > 0 && V > 0, "sample: sizes must be positive (rows=%d, V=%d)", rows, V);
    launch_kernel((sample_kernel), dim3(rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), 
        logits, probs_scratch, V, temperature, top_k, top_p, uniform, out);
    return check_launch("sample");
}

// ------------------------------------------------------------------------------------------------
// The allocation-free variant of gi_sample (declared and explained in no_alloc.h).
#include "no_alloc.h"

#include <mutex>

namespace gi {

// The work area of gi_sample_no_alloc. In host code this name is only a handle for the runtime's
// symbol table, not a device address: the address is looked up once per device below.
static __device__ __align__(256) float g_sample_work_area[GI_SAMPLE_NO_ALLOC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_work_area_address[kMaxDevices] = {};
static std::mutex g_work_area_mutex;

// Device address of the work area on the current device; looked up on the first call per device.
static int work_area_for_current_device(float** out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        set_error("sample_no_alloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
        return 1;
    }
    if (device < 0 || device >= kMaxDevices) {
        set_error("sample_no_alloc: device index %d is outside the supported range 0..%d", device, kMaxDevices - 1);
        return 2;
    }
    std::lock_guard<std::mutex> lock(g_work_area_mutex);
    if (g_work_area_address[device] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_sample_work_area);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("sample_no_alloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
            return 1;
        }
        g_work_area_address[device] = ptr;
    }
    *out = g_work_area_address[device];
    return 0;
}

}  // namespace gi

extern "C" int gi_sample_no_alloc(const float* logits, int rows, int vocab, const float* temperature,
                                  const int* top_k, const float* top_p, const float* uniform, int* out,
                                  void* stream) {
    if (rows == 0) return 0;
    GI_REQUIRE(rows > 0 && vocab > 0, "sample_no_alloc: sizes must be positive (rows=%d, vocab=%d)", rows, vocab);
    const long long need = static_cast<long long>(rows) * vocab;
    GI_REQUIRE(need <= GI_SAMPLE_NO_ALLOC_MAX_FLOATS,
               "sample_no_alloc: %d rows x %d vocabulary = %lld floats exceed the built-in work area of %d floats; "
               "sample fewer rows per call or use gi_sample with a scratch buffer of your own",
               rows, vocab, need, GI_SAMPLE_NO_ALLOC_MAX_FLOATS);
    float* work = nullptr;
    const int rc = work_area_for_current_device(&work);
    if (rc != 0) return rc;
    launch_kernel((sample_kernel), dim3(rows), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), 
        logits, work, vocab, temperature, top_k, top_p, uniform, out);
    return check_launch("sample_no_alloc");
}

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_argmax(const float* logits, int rows, int V, int* out, float* part_val, int* part_idx, void* stream) {
    return gi::dispatch(gi_argmax_impl, logits, rows, V, out, part_val, part_idx, stream);
}

extern "C" int gi_sample(const float* logits, float* probs_scratch, int rows, int V, const float* temperature, const int* top_k, const float* top_p, const float* uniform, int* out, void* stream) {
    return gi::dispatch(gi_sample_impl, logits, probs_scratch, rows, V, temperature, top_k, top_p, uniform, out, stream);
}
