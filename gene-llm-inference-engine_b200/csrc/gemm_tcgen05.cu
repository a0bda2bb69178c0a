// bfloat16 matrix product on the 5th-generation tensor cores: C (+)= A[M,K] * W[N,K]^T, 32-bit
// accumulation in tensor memory.
//
// One CTA computes a 128 x BLOCK_Q tile. Both operands are K-major, so each is fetched by TMA as
// [rows, 64] boxes with the 128-byte swizzle that tcgen05.mma reads directly (TILED kernels fetch
// the weights from a copy that is laid out tile by tile already: one untiled bulk copy of 32 KB
// brings two 64-wide blocks of K). Three roles:
//   warp 0      producer: one lane issues the loads of a pipeline of kStages stages;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (4 x K=16 per 64 columns of K)
//               and commits each stage back to the producer, and the finished tile to the epilogue;
//   warps 2..5  epilogue: tcgen05.ld of the accumulators (one lane = one row of the tile), then
//               store / accumulate into C in 32-bit, or round to bfloat16.
// The 128-row operand "P" and the BLOCK_Q-row operand "Q" can be either matrix: for many tokens P
// is the activations (C[p, q]); for few tokens the weights take the 128-row side and the tokens
// become the narrow side (C[q, p]), so that a decode step streams every weight once at full tile
// efficiency. The split over K (few tokens, narrow weight matrices) runs the splits of a tile as
// one thread-block cluster where they fit: splits 1.. write their partial tiles into the shared
// memory of split 0 with stores that count their bytes on its mbarrier (st.async), and split 0 adds them in split
// order. The tiles have a place of their own behind the pipeline stages where there is room (few
// tokens); otherwise they land in split 0's stages once it has told the others that its products are
// done with them. Where a cluster does not fit, partial tiles go to a workspace in global memory and the CTA
// that arrives last adds them, again in split order; results never depend on the order of arrival.
//
// Every wait on an mbarrier is bounded: when a limit is hit the kernel records a code in the
// status word, stops issuing work, drains its own copies with bounded waits, frees its tensor
// memory and returns; the host reads the status word with gi_gemm_tc_status().
#include "common.cuh"
#include "tma.cuh"

namespace gi {

constexpr int kBlockP = 128;
constexpr int kBlockK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 192;
constexpr unsigned long long kWaitCycles = 4000000000ull;   // about two seconds

enum TcError : int { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 3, kErrDrain = 4, kErrClusterWait = 6 };

// ------------------------------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// ---- thread-block cluster: shared memory of another CTA, barriers across CTAs
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// A 32-bit store into another CTA's shared memory that counts 4 bytes on a barrier of that CTA when it lands: the
// receiver's wait ends with the last store's arrival, with no acknowledgement to the sender and no arrival after it.
__device__ __forceinline__ void cluster_store_f32_counted(uint32_t remote_addr, float v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(remote_addr), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_local(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cluster_mbar_arrive(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Bounded wait: false when the limit is hit or another role has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// The same loads with an L2 policy: weights that a step reads once are marked to be evicted first, so that they
// do not push out what is read again soon (activations, the residual stream, tables, the kernels' own code).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_load_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart; version 1 (bit 46), layout type 2 = SWIZZLE_128B (bits 61..63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;                     // leading byte offset: unused with swizzle
    d |= static_cast<uint64_t>(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// TILED: the 128-row operand comes from a tile-by-tile copy of the matrix (see TcParams::p_tiles)
// and a stage holds two 64-wide blocks of K, fetched with one bulk copy of 32 KB.
template <int BLOCK_Q, bool TILED = false>
struct TcConfig {
    static constexpr int kKb = TILED ? 2 : 1;                  // 64-wide blocks of K per stage
    static constexpr int kBlockBytesP = kBlockP * kBlockK * 2;
    static constexpr int kBlockBytesQ = BLOCK_Q * kBlockK * 2;
    static constexpr int kStageBytesP = kBlockBytesP * kKb;
    static constexpr int kStageBytesQ = kBlockBytesQ * kKb;
    static constexpr int kStageBytes = kStageBytesP + kStageBytesQ;
    static constexpr int kStages = TILED ? ((BLOCK_Q >= 128) ? 3 : (BLOCK_Q >= 32) ? 4 : 5)
                                         : ((BLOCK_Q >= 256) ? 4 : (BLOCK_Q >= 128) ? 6 : 8);
    static constexpr int kTmemCols = BLOCK_Q < 32 ? 32 : BLOCK_Q;
    static constexpr int kSideBytes = 768;      // barriers and flags (the first 256), the tokens' positions (128) and page rows (256) of a rotating product of up to 32 tokens
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment */ + kSideBytes;
    // A cluster's split 0 receives the partial tiles of the other splits, [split - 1][q][128 rows], in its
    // pipeline stages once its own products are done with them (it tells the others when); behind them
    // lie the per-token arrays of the rotating epilogue.
    static constexpr int kPartialBytes = BLOCK_Q * kBlockP * 4;
    static constexpr int kTokenInfoBytes = BLOCK_Q * 12;
    // (not for 16 tokens: their partial tiles always find a place of their own, and the kernel that every
    // small decode step runs stays free of the extra code)
    static constexpr bool kStagesReceive = BLOCK_Q >= 32;
    static constexpr int kOwnPlaceLimit = 232448;
    static constexpr bool cluster_fits(int cluster_splits) {
        return kStagesReceive && (cluster_splits - 1) * kPartialBytes + kPartialBytes + kTokenInfoBytes <= kStages * kStageBytes;
    }
    // ... or, where the shared memory has room for it, in a place of their own behind the stages: then
    // nobody has to wait for split 0 (about 2 us less for a product of 16 tokens)
    static constexpr int smem_bytes(int cluster_splits) {
        return kSmemBytes + (cluster_splits > 1 ? (cluster_splits - 1) * kPartialBytes : 0);
    }
    // instruction descriptor: D f32 (bits 4..5 = 1), A and B bf16 (bits 7..9, 10..12 = 1), both
    // K-major, N >> 3 at bits 17..22, M >> 4 at bits 24..28
    static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BLOCK_Q >> 3) << 17) |
                                       (static_cast<uint32_t>(kBlockP >> 4) << 24);
};

// Rotation of query and key heads and the store of keys and values into the request's pages, done
// by the epilogue of the product that makes [q; k; v] (the rows of W are H query heads, Hkv key heads,
// Hkv value heads of hd features each): q goes to q_out [tokens, H * hd], k and v of token t to its
// page (block_tables[row_req[t]][pos / page_size]) in caches of [pages, Hkv, page_size, hd]; all
// bfloat16. cos/sin: tables [max position, rot_half] in 32-bit (null: no rotation).
struct RopeStoreParams {
    const int* positions;
    const int* row_req;
    const int* block_tables;
    int table_stride;
    const float* cos_t;
    const float* sin_t;
    int rot_half, interleaved;
    __nv_bfloat16* q_out;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int H, Hkv, hd, page_size, write_kv;
};

struct TcParams {
    void* C;
    int c_bf16;              // 0: C is float, 1: C is bfloat16
    int accumulate;          // C += product (float C only)
    int rows_p, rows_q, K;
    long long stride_p, stride_q;   // C[p * stride_p + q * stride_q]
    int k_blocks_per_split;
    int splits;
    float* workspace;        // [tile][split][BLOCK_Q][128] partial tiles when splits > 1
    unsigned* counters;      // one per tile, zero between launches
    int* status;
    int prefetch_p;          // P is a weight matrix no earlier kernel writes: its first tiles may be
                             // fetched before the kernel waits for the kernels it depends on
    const uint8_t* ahead;    // weights that a later product of the step will read, asked into L2 by this product's CTAs
    unsigned long long ahead_bytes;   //   once their own loads are on their way (null: none); a multiple of 32 KB
    int stream_p;            // P is a weight matrix that the step reads once (few tokens): its loads carry the
                             // evict-first L2 policy
    int cluster;             // the splits of a tile are one cluster (dims 1 x 1 x splits): reduce in shared memory
    const uint8_t* p_tiles;  // TILED kernels: the 128-row operand tile by tile, [row tile][K block][128][64] with the
                             // 128-byte swizzle applied and K padded to a multiple of 128 (tile_weight in ops/kernels.py)
    int tiles_kb;            // 64-wide blocks of K in a row of tiles
    int rope_on;             // the product is [q; k; v] (weights on the 128-row side): the CTA that holds a tile's sum
    RopeStoreParams rope;    //   rotates it and stores queries, keys and values instead of writing C
};

template <int BLOCK_Q>
__device__ __forceinline__ void store_row_chunk(const TcParams& p, bool c_bf16, bool accumulate, int row_p, int q0, const float* v) {
    // v[j] belongs to (row_p, q0 + j), j < 16
    if (row_p >= p.rows_p) return;
    const long long base = static_cast<long long>(row_p) * p.stride_p + static_cast<long long>(q0) * p.stride_q;
    const int n = min(16, p.rows_q - q0);
    if (c_bf16) {
        __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.C) + base;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < n) c[j * p.stride_q] = __float2bfloat16_rn(v[j]);
    } else if (accumulate) {
        // all loads first, then all stores: the sixteen read-modify-writes overlap instead of
        // waiting for one another
        float* c = static_cast<float*>(p.C) + base;
        float old[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) old[j] = (j < n) ? __ldcg(c + j * p.stride_q) : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < n) c[j * p.stride_q] = old[j] + v[j];
    } else {
        float* c = static_cast<float*>(p.C) + base;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < n) c[j * p.stride_q] = v[j];
    }
}

// The same for a chunk whose old values were read earlier (32-bit C, accumulate).
__device__ __forceinline__ void store_row_chunk_old(const TcParams& p, int row_p, int q0, const float* v, const float* old) {
    if (row_p >= p.rows_p) return;
    float* c = static_cast<float*>(p.C) + static_cast<long long>(row_p) * p.stride_p + static_cast<long long>(q0) * p.stride_q;
    const int n = min(16, p.rows_q - q0);
#pragma unroll
    for (int j = 0; j < 16; ++j)
        if (j < n) c[j * p.stride_q] = old[j] + v[j];
}

// SPEC 0: every form of the product in one kernel, chosen by TcParams at run time (about 5,000 instructions). The
// three forms that a decode step of up to 16 tokens runs have kernels of their own in which what TcParams says is
// compiled in and everything else is left out: a short kernel pays for every instruction it has to fetch, and the
// L2 cache that would serve the fetch is swept by the weights between two launches (measured on B200: the
// RMSNorm kernel cut from 19 KB to 6 KB of code made each of its launches 0.5 us shorter inside a decode step).
// A 16-byte read-only load that stays where it is written: the compiler moves an ordinary load down to its first
// use, which for values fetched "while the products run" is behind the wait for the products.
__device__ __forceinline__ float4 load_now_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

enum TcSpecKind : int {
    kSpecAny = 0,
    kSpecRopeCluster = 1,    // [q; k; v] with rotation and store, K split over a cluster with partial tiles in a place of their own
    kSpecAddCluster = 2,     // added into a 32-bit C (O and down products), K split over such a cluster
    kSpecStoreOne = 3,       // stored to a 32-bit C, K not split ([gate; up], the head)
};
template <int SPEC>
struct TcSpec {
    static constexpr bool fixed = SPEC != kSpecAny;
    static constexpr bool rope = SPEC == kSpecRopeCluster;
    static constexpr int cluster = (SPEC == kSpecRopeCluster || SPEC == kSpecAddCluster) ? 1 : 0;
    static constexpr bool one_split = SPEC == kSpecStoreOne;
    static constexpr bool accumulate = SPEC == kSpecAddCluster;
};

template <int BLOCK_Q, bool TILED, int SPEC = kSpecAny>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, const TcParams p) {
    using Cfg = TcConfig<BLOCK_Q, TILED>;
    using Spec = TcSpec<SPEC>;
    // what the specialised kernels know at compile time
    const bool rope_on = Spec::fixed ? Spec::rope : p.rope_on != 0;
    const int cluster = Spec::fixed ? Spec::cluster : p.cluster;
    const bool one_split = Spec::fixed ? Spec::one_split : p.splits == 1;
    const bool accumulate = Spec::fixed ? Spec::accumulate : p.accumulate != 0;
    const bool c_bf16 = Spec::fixed ? false : p.c_bf16 != 0;
    const bool prefetch_p = Spec::fixed ? true : p.prefetch_p != 0;
    const bool stream_p = Spec::fixed ? true : p.stream_p != 0;
    const int n_splits = (Spec::fixed && Spec::one_split) ? 1 : p.splits;
    // the kernel of every form names the form it runs: 11 rotating, 12 adding, 13 storing
    const int tl_id = kTlProduct + (Spec::fixed ? SPEC : 10 + (rope_on ? 1 : accumulate ? 2 : 3));
    if (threadIdx.x == 0) timeline_record(tl_id, 0);
    constexpr int kKb = Cfg::kKb;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Cfg::kStageBytes);
    // bars[0..kStages) full, [kStages..2kStages) empty, [2kStages] accumulator ready,
    // [2kStages + 1] the other splits' partial tiles have arrived (cluster reduce, split 0),
    // [2kStages + 2] split 0's stages are free to receive them (cluster reduce, the other splits)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 3);
    float* partials = reinterpret_cast<float*>((Cfg::kStagesReceive && cluster == 2) ? smem : smem + kStages * Cfg::kStageBytes + Cfg::kSideBytes);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;
    int* epi_abort = last_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_p = blockIdx.x, tile_q = blockIdx.y, split = blockIdx.z;
    const int total_kb = (p.K + kBlockK - 1) / kBlockK;
    const int kb_begin = split * p.k_blocks_per_split;
    const int kb_end = min(total_kb, kb_begin + p.k_blocks_per_split);
    const int n_blocks = max(0, kb_end - kb_begin);
    const int n_kb = (n_blocks + kKb - 1) / kKb;                // stages of kKb blocks (the host keeps splits whole)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[kStages + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * kStages]), 1);
        mbar_init(smem_u32(&bars[2 * kStages + 1]), 1u);     // one arrival (split 0's own) and the bytes of the partial tiles
        mbar_init(smem_u32(&bars[2 * kStages + 2]), 1);
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (cluster) cluster_sync_all();          // split 0's barrier exists before anyone arrives on it

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            int issued = 0;
            // The first stages are free: with prefetch_p their weight tiles are requested before
            // this kernel waits for its predecessors, so the weight stream never pauses between
            // the kernels of a decode step; the activation tiles follow after the wait.
            const int early = prefetch_p ? min(n_kb, kStages) : 0;
            const uint64_t stream_policy = l2_evict_first_policy();
            auto load_p = [&](int i, uint32_t full) {          // stage i of this CTA: blocks kb_begin + i * kKb ..
                const uint32_t dst = smem_u32(smem + (i % kStages) * Cfg::kStageBytes);
                if (TILED) {
                    const uint8_t* src = p.p_tiles + (static_cast<size_t>(tile_p) * p.tiles_kb + kb_begin + i * kKb) * Cfg::kBlockBytesP;
                    if (stream_p) bulk_load_hint(dst, src, Cfg::kStageBytesP, full, stream_policy);
                    else bulk_load(dst, src, Cfg::kStageBytesP, full);
                } else if (stream_p) {
                    tma_load_2d_hint(dst, &map_p, (kb_begin + i) * kBlockK, tile_p * kBlockP, full, stream_policy);
                } else {
                    tma_load_2d(dst, &map_p, (kb_begin + i) * kBlockK, tile_p * kBlockP, full);
                }
            };
            auto load_q = [&](int i, uint32_t full) {
                const uint32_t dst = smem_u32(smem + (i % kStages) * Cfg::kStageBytes + Cfg::kStageBytesP);
#pragma unroll
                for (int j = 0; j < kKb; ++j)
                    tma_load_2d(dst + j * Cfg::kBlockBytesQ, &map_q, (kb_begin + i * kKb + j) * kBlockK, tile_q * BLOCK_Q, full);
            };
            for (int i = 0; i < early; ++i) {
                const uint32_t full = smem_u32(&bars[i]);
                mbar_expect_tx(full, Cfg::kStageBytes);
                load_p(i, full);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            timeline_record(tl_id, 1);
            for (int i = 0; i < early; ++i) {
                load_q(i, smem_u32(&bars[i]));
                issued = i + 1;
            }
            for (int i = early; i < n_kb; ++i) {
                const int s = i % kStages;
                const uint32_t parity = ((i / kStages) & 1) ^ 1;
                if (!mbar_wait(smem_u32(&bars[kStages + s]), parity, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrProducerWait); }
                    break;
                }
                const uint32_t full = smem_u32(&bars[s]);
                mbar_expect_tx(full, Cfg::kStageBytes);
                load_p(i, full);
                load_q(i, full);
                issued = i + 1;
            }
            if (p.ahead != nullptr && !*abort_flag) {
                // This CTA's share of the weights to ask into L2, in pieces of 32 KB. The product that reads them keeps
                // only five stages per CTA in flight of its own before it may start; what lies in L2 by then is fetched
                // in a fraction of the time, so the stream from memory pauses less between the kernels of a step.
                const unsigned long long ctas = static_cast<unsigned long long>(gridDim.x) * gridDim.y * gridDim.z;
                const unsigned long long me = blockIdx.x + gridDim.x * (blockIdx.y + static_cast<unsigned long long>(gridDim.y) * blockIdx.z);
                for (unsigned long long i = me; i < p.ahead_bytes / 32768ull; i += ctas)
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.ahead + i * 32768ull), "r"(32768u) : "memory");
            }
            if (*abort_flag) {
                // drain: every copy this lane issued must have landed before the CTA may exit
                const int first = max(0, issued - kStages);
                for (int i = first; i < issued; ++i) {
                    const unsigned long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&bars[i % kStages]), (i / kStages) & 1)) {
                        if (clock64() - t0 > kWaitCycles) { atomicCAS(p.status, 0, kErrDrain); break; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % kStages;
                if (!mbar_wait(smem_u32(&bars[s]), (i / kStages) & 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrMmaWait); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (i == 0) timeline_record(tl_id, 2);
                const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
#pragma unroll
                for (int j = 0; j < kKb; ++j) {
                    const uint64_t desc_p = umma_desc(a_addr + j * Cfg::kBlockBytesP);
                    const uint64_t desc_q = umma_desc(a_addr + Cfg::kStageBytesP + j * Cfg::kBlockBytesQ);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in the address field
                        umma_bf16(tmem_base, desc_p + 2 * k, desc_q + 2 * k, Cfg::kIdesc, (i > 0 || j > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(&bars[kStages + s]));      // frees the stage once the MMAs have read it
            }
            if (ok) umma_commit(smem_u32(&bars[2 * kStages]));  // accumulator complete
            timeline_record(tl_id, 3);
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..5)
        asm volatile("griddepcontrol.wait;" ::: "memory");      // C and the workspace belong to earlier kernels until now
        const int lane_group = warp & 3;                        // the TMEM lanes this warp may read
        const int row_in_tile = lane_group * 32 + lane;
        const int row_p = tile_p * kBlockP + row_in_tile;
        // A tile of up to 32 columns that this CTA itself will add into C: the old values are requested
        // now, while the products run, instead of after them (at 32 tokens the tail after the last MMA was 6 us with
        // the loads in it).
        constexpr int kEarlyOld = BLOCK_Q <= 32 ? BLOCK_Q : 1;
        const bool early_old = BLOCK_Q <= 32 && accumulate && !c_bf16 && row_p < p.rows_p &&
                               (one_split || (cluster && split == 0));
        float old_c[kEarlyOld];
        if (early_old) {
            const float* c = static_cast<const float*>(p.C) + static_cast<long long>(row_p) * p.stride_p +
                             static_cast<long long>(tile_q * BLOCK_Q) * p.stride_q;
            const int n = min(kEarlyOld, p.rows_q - tile_q * BLOCK_Q);
#pragma unroll
            for (int j = 0; j < kEarlyOld; ++j) old_c[j] = (j < n) ? __ldcg(c + j * p.stride_q) : 0.f;
        }
        // Rotation and store: thread j < BLOCK_Q looks up the position and the page row of token j of the
        // tile now, while the products run.
        int tok_pos = 0;
        long long tok_base = -1;
        if (rope_on && row_in_tile < BLOCK_Q) {
            const int tok = tile_q * BLOCK_Q + row_in_tile;
            if (tok < p.rows_q) {
                tok_pos = p.rope.positions[tok];
                if (p.rope.write_kv) {
                    const int page = p.rope.block_tables[static_cast<size_t>(p.rope.row_req[tok]) * p.rope.table_stride + tok_pos / p.rope.page_size];
                    tok_base = (static_cast<long long>(page) * p.rope.Hkv * p.rope.page_size + (tok_pos % p.rope.page_size)) * p.rope.hd;
                }
            }
        }
        // Token tiles of 16 and 32: rotation and store are done four features at a time. The finished tile lies in shared
        // memory as [token][128 rows]; thread t takes token t / kTpt and kFeat neighbouring rows of it, reads them and their
        // rotation partners 16 bytes at a time and writes 8 bytes of bfloat16 at a time. Everything that does not need the
        // sums is worked out now, while the products run: the cosines and sines (16 bytes at a time), where each group of
        // four goes and how it is rotated. What follows the last MMA is one warp's instructions one after the other, about
        // 4 ns each: one thread per row walking over 32 tokens (two table look-ups, index arithmetic and a 2-byte store
        // per token) took 5 to 7 us there, this takes 1 to 2. The loads and the addresses are pinned with volatile asm,
        // since the compiler moves both down to their first use, behind the wait. Needs the half-split pairing with a
        // rotary half that is a multiple of 4; else the loop below.
        constexpr bool kRopeVec = BLOCK_Q <= 32;
        constexpr int kTpt = kRopeVec ? 128 / BLOCK_Q : 1;          // threads per token
        constexpr int kFeat = kRopeVec ? BLOCK_Q : 4;               // rows (features) per thread
        constexpr int kGroups = kFeat / 4;
        bool rope_vec = false;
        float4 rope_c4[kGroups], rope_s4[kGroups];
        __nv_bfloat16* v_dst[kGroups];              // where each group of 4 features goes (nullptr: nowhere)
        unsigned v_mode = 0;                        // 2 bits a group: 1 first members of rotated pairs, 2 second members
        int v_partner = 0;                          // distance to the rotation partners, in groups
        if (kRopeVec && rope_on) {
            const RopeStoreParams& rp = p.rope;
            const int rh = rp.cos_t ? rp.rot_half : 0;
            rope_vec = !rp.interleaved && rh % 4 == 0 && (reinterpret_cast<uintptr_t>(rp.cos_t) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(rp.sin_t) % 16 == 0);
            if (rope_vec) {
                const int v_tok = tile_q * BLOCK_Q + row_in_tile / kTpt;
                int pos = 0;
                long long v_base = -1;
                if (v_tok < p.rows_q) {
                    pos = rp.positions[v_tok];
                    if (rp.write_kv) {
                        const int page = rp.block_tables[static_cast<size_t>(rp.row_req[v_tok]) * rp.table_stride + pos / rp.page_size];
                        v_base = (static_cast<long long>(page) * rp.Hkv * rp.page_size + (pos % rp.page_size)) * rp.hd;
                    }
                }
                v_partner = rh / 4;
#pragma unroll
                for (int g = 0; g < kGroups; ++g) {
                    const int row = tile_p * kBlockP + (row_in_tile % kTpt) * kFeat + 4 * g;
                    const int head = row / rp.hd, d = row - head * rp.hd;
                    const bool is_q = head < rp.H, is_k = !is_q && head < rp.H + rp.Hkv;
                    rope_c4[g] = rope_s4[g] = make_float4(0.f, 0.f, 0.f, 0.f);
                    v_dst[g] = nullptr;
                    if (row < p.rows_p && v_tok < p.rows_q) {
                        if ((is_q || is_k) && d < 2 * rh) {
                            const size_t at = static_cast<size_t>(pos) * rh + (d < rh ? d : d - rh);
                            rope_c4[g] = load_now_f32x4(rp.cos_t + at);
                            rope_s4[g] = load_now_f32x4(rp.sin_t + at);
                            v_mode |= (d < rh ? 1u : 2u) << (2 * g);
                        }
                        if (is_q) v_dst[g] = rp.q_out + (static_cast<size_t>(v_tok) * rp.H + head) * rp.hd + d;
                        else if (v_base >= 0)
                            v_dst[g] = (is_k ? rp.k_cache : rp.v_cache) + v_base +
                                       static_cast<size_t>(is_k ? head - rp.H : head - rp.H - rp.Hkv) * rp.page_size * rp.hd + d;
                    }
                    asm volatile("" : "+l"(v_dst[g]));      // worked out here, not behind the wait
                }
                asm volatile("" : "+r"(v_mode), "+r"(v_partner));
            }
        }
        // The pipeline's stages are free once the accumulator is complete: the finished tile is laid
        // there as [token][128 rows] so that a thread can read its rotation partner's value.
        float* xch = reinterpret_cast<float*>(smem);
        bool emitted = false;
        auto emit = [&](int c, const float* v) {          // the final values of columns c * 16 .. of this thread's row
            if (rope_on) {
#pragma unroll
                for (int j = 0; j < 16; ++j) xch[(c * 16 + j) * kBlockP + row_in_tile] = v[j];
                emitted = true;
            } else {
                store_row_chunk<BLOCK_Q>(p, c_bf16, accumulate, row_p, tile_q * BLOCK_Q + c * 16, v);
            }
        };
        bool have = n_kb > 0;
        if (have && !mbar_wait(smem_u32(&bars[2 * kStages]), 0, abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrEpilogueWait); }
            have = false;
        }
        tc_fence_after();
        if (warp == 2 && lane == 0) timeline_record(tl_id, 4);
        // one decision for all 128 epilogue threads (they meet at named barriers below)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) *epi_abort = *abort_flag;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool aborted = *epi_abort != 0;
        constexpr int kChunks = (BLOCK_Q + 15) / 16;
        if (cluster) {
            // Splits 1.. hand their partial tile to split 0 (rank 0 of the cluster) with stores that count
            // their bytes on its barrier, zeros after giving up, so that split 0 never waits for a CTA that is gone;
            // split 0 waits (bounded) for all bytes before it leaves, so its memory outlives every write to it.
            // Where the tiles land in split 0's pipeline stages (cluster == 2): split 0 says when its
            // products are done with them (an arrival on every other split's "stages free" barrier,
            // sent even after giving up), and the others wait for that (bounded) before they write and
            // before they leave, so that the arrival never finds their memory gone.
            if (split == 0) {
                if (Cfg::kStagesReceive && cluster == 2 && warp == 2 && lane == 0) {
                    for (int s = 1; s < n_splits; ++s)
                        cluster_mbar_arrive(cluster_map(smem_u32(&bars[2 * kStages + 2]), static_cast<uint32_t>(s)));
                }
            }
            if (split != 0) {
                bool stages_free = !Cfg::kStagesReceive || cluster != 2 || mbar_try_wait_cluster(smem_u32(&bars[2 * kStages + 2]), 0);
                const unsigned long long t0 = clock64();
                while (!stages_free) {
                    stages_free = mbar_try_wait_cluster(smem_u32(&bars[2 * kStages + 2]), 0);
                    if (!stages_free && clock64() - t0 > kWaitCycles) { atomicCAS(p.status, 0, kErrClusterWait); break; }
                }
                // The stores count their bytes on split 0's barrier as they land. A CTA that has given up sends zeros, so
                // that the count is reached; only one that never heard from split 0 sends nothing (split 0 has then
                // given up too, or will when its wait runs out).
                if (stages_free) {
                    const uint32_t remote = cluster_map(smem_u32(partials), 0) +
                                            static_cast<uint32_t>((split - 1) * BLOCK_Q * kBlockP + row_in_tile) * 4u;
                    const uint32_t remote_bar = cluster_map(smem_u32(&bars[2 * kStages + 1]), 0);
                    const bool send = have && !aborted;
#pragma unroll 1
                    for (int c = 0; c < kChunks; ++c) {
                        uint32_t r[16];
                        if (send) {
                            tmem_ld_x16(tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + c * 16, r);
                            tmem_ld_wait();
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            cluster_store_f32_counted(remote + static_cast<uint32_t>((c * 16 + j) * kBlockP) * 4u,
                                                      send ? __uint_as_float(r[j]) : 0.f, remote_bar);
                    }
                }
            } else {
                if (warp == 2 && lane == 0)
                    mbar_arrive_expect_tx_local(smem_u32(&bars[2 * kStages + 1]),
                                                static_cast<uint32_t>(n_splits - 1) * 128u * kChunks * 16u * 4u);
                // up to 32 tokens: this CTA's own sums leave tensor memory while the others' are on their way
                constexpr int kOwnEarly = kChunks <= 2 ? kChunks : 0;
                uint32_t own[kOwnEarly > 0 ? kOwnEarly : 1][16];
                if (kOwnEarly > 0 && have && !aborted) {
#pragma unroll
                    for (int c = 0; c < kOwnEarly; ++c)
                        tmem_ld_x16(tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + c * 16, own[c]);
                    tmem_ld_wait();
                }
                bool all_here = mbar_try_wait_cluster(smem_u32(&bars[2 * kStages + 1]), 0);
                const unsigned long long t0 = clock64();
                while (!all_here) {
                    all_here = mbar_try_wait_cluster(smem_u32(&bars[2 * kStages + 1]), 0);
                    if (!all_here && clock64() - t0 > kWaitCycles) { atomicCAS(p.status, 0, kErrClusterWait); break; }
                }
                if (warp == 2 && lane == 0) timeline_record(tl_id, 7);
                if (all_here && !aborted) {
#pragma unroll (kOwnEarly > 0 ? kOwnEarly : 1)
                    for (int c = 0; c < kChunks; ++c) {
                        uint32_t r[16];
                        float v[16];
                        if (kOwnEarly > 0) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) r[j] = own[kOwnEarly > 0 ? c : 0][j];
                        } else if (have) {
                            tmem_ld_x16(tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + c * 16, r);
                            tmem_ld_wait();
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = have ? __uint_as_float(r[j]) : 0.f;
                        for (int s = 1; s < n_splits; ++s) {
                            const float* part = partials + static_cast<size_t>(s - 1) * BLOCK_Q * kBlockP;
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] += part[(c * 16 + j) * kBlockP + row_in_tile];
                        }
                        if (early_old) {
                            float oc[16];                         // this chunk's old values, picked with constant indices
#pragma unroll
                            for (int j = 0; j < 16; ++j) oc[j] = (kEarlyOld > 16 && c == 1) ? old_c[(kEarlyOld > 16 ? 16 : 0) + j] : old_c[j];
                            store_row_chunk_old(p, row_p, tile_q * BLOCK_Q + c * 16, v, oc);
                        }
                        else emit(c, v);
                    }
                }
            }
        } else if (!aborted) {
            if (one_split) {
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    uint32_t r[16];
                    float v[16];
                    if (have) {
                        tmem_ld_x16(tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + c * 16, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    }
                    if (early_old) {
                            float oc[16];                         // this chunk's old values, picked with constant indices
#pragma unroll
                            for (int j = 0; j < 16; ++j) oc[j] = (kEarlyOld > 16 && c == 1) ? old_c[(kEarlyOld > 16 ? 16 : 0) + j] : old_c[j];
                            store_row_chunk_old(p, row_p, tile_q * BLOCK_Q + c * 16, v, oc);
                        }
                    else emit(c, v);
                }
            } else {
                // partial tile -> workspace [tile][split][q][128 rows]; the last CTA of the tile sums all splits
                const int tile_id = tile_q * gridDim.x + tile_p;
                float* ws_tile = p.workspace + static_cast<size_t>(tile_id) * n_splits * BLOCK_Q * kBlockP;
                float* mine = ws_tile + static_cast<size_t>(split) * BLOCK_Q * kBlockP;
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    uint32_t r[16];
                    if (have) {
                        tmem_ld_x16(tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + c * 16, r);
                        tmem_ld_wait();
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        mine[(c * 16 + j) * kBlockP + row_in_tile] = have ? __uint_as_float(r[j]) : 0.f;
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const unsigned arrived = atomicAdd(&p.counters[tile_id], 1u);
                    *last_flag = (arrived == static_cast<unsigned>(n_splits - 1)) ? 1 : 0;
                    if (*last_flag) p.counters[tile_id] = 0;        // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
#pragma unroll 1
                    for (int c = 0; c < kChunks; ++c) {
                        // four splits' values are requested together (64 loads in flight), then added
                        // in split order: one split after the other would wait for memory 4 times as often
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                        for (int s0 = 0; s0 < n_splits; s0 += 4) {
                            float part[4][16];
#pragma unroll
                            for (int ds = 0; ds < 4; ++ds) {
                                const float* src = ws_tile + static_cast<size_t>(s0 + ds) * BLOCK_Q * kBlockP;
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    part[ds][j] = (s0 + ds < n_splits) ? __ldcg(&src[(c * 16 + j) * kBlockP + row_in_tile]) : 0.f;
                            }
#pragma unroll
                            for (int ds = 0; ds < 4; ++ds)
                                if (s0 + ds < n_splits) {
#pragma unroll
                                    for (int j = 0; j < 16; ++j) v[j] += part[ds][j];
                                }
                        }
                        emit(c, v);
                    }
                }
            }
        }
        if (warp == 2 && lane == 0) timeline_record(tl_id, 8);
        if (rope_on) {
            const RopeStoreParams& rp = p.rope;
            if (kRopeVec && rope_vec) {
                asm volatile("bar.sync 1, 128;" ::: "memory");          // the finished tile is complete
                if (emitted) {
                    const float4* x4 = reinterpret_cast<const float4*>(xch) + (row_in_tile / kTpt) * (kBlockP / 4) +
                                       (row_in_tile % kTpt) * kGroups;
#pragma unroll
                    for (int g = 0; g < kGroups; ++g) {
                        if (!v_dst[g]) continue;
                        const unsigned mode = (v_mode >> (2 * g)) & 3u;
                        float4 o = x4[g];
                        if (mode) {
                            // first member of a pair: a c - b s; second: a s + b c (b: the partner, rot_half rows away)
                            const bool first = mode == 1u;
                            const float4 b4 = x4[first ? g + v_partner : g - v_partner], c4 = rope_c4[g], s4 = rope_s4[g];
                            o.x = first ? o.x * c4.x - b4.x * s4.x : b4.x * s4.x + o.x * c4.x;
                            o.y = first ? o.y * c4.y - b4.y * s4.y : b4.y * s4.y + o.y * c4.y;
                            o.z = first ? o.z * c4.z - b4.z * s4.z : b4.z * s4.z + o.z * c4.z;
                            o.w = first ? o.w * c4.w - b4.w * s4.w : b4.w * s4.w + o.w * c4.w;
                        }
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(v_dst[g]) = packed;
                    }
                }
            } else {
                // behind the finished tile and, in a cluster, behind the partial tiles that other threads may still be reading
                int* tpos = reinterpret_cast<int*>(xch + ((Cfg::kStagesReceive && cluster == 2) ? max(1, n_splits - 1) : 1) * BLOCK_Q * kBlockP);
                long long* tbase = reinterpret_cast<long long*>(tpos + BLOCK_Q);
                if (row_in_tile < BLOCK_Q) { tpos[row_in_tile] = tok_pos; tbase[row_in_tile] = tok_base; }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (emitted && row_p < p.rows_p) {
                    // this thread's row is feature d of one head; its partner in a rotated pair lies in the same tile
                    const int hd = rp.hd, head = row_p / hd, d = row_p - head * hd;
                    const bool is_q = head < rp.H, is_k = !is_q && head < rp.H + rp.Hkv;
                    const int rh = rp.cos_t ? rp.rot_half : 0;
                    const bool rotate = (is_q || is_k) && d < 2 * rh;
                    int partner = row_in_tile, ci = 0;
                    bool first = true;                       // first member of the pair: a c - b s; second: a s + b c
                    if (rotate) {
                        if (rp.interleaved) { first = (d & 1) == 0; partner = row_in_tile ^ 1; ci = d >> 1; }
                        else { first = d < rh; partner = first ? row_in_tile + rh : row_in_tile - rh; ci = first ? d : d - rh; }
                    }
                    const int n_tok = min(BLOCK_Q, p.rows_q - tile_q * BLOCK_Q);
                    const size_t kv_head = static_cast<size_t>(is_q ? 0 : (is_k ? head - rp.H : head - rp.H - rp.Hkv)) * rp.page_size * hd + d;
                    __nv_bfloat16* cache = is_k ? rp.k_cache : rp.v_cache;
#pragma unroll 4
                    for (int j = 0; j < n_tok; ++j) {
                        float out = xch[j * kBlockP + row_in_tile];
                        if (rotate) {
                            const float other = xch[j * kBlockP + partner];
                            const size_t at = static_cast<size_t>(tpos[j]) * rh + ci;
                            const float ck = __ldg(rp.cos_t + at), sk = __ldg(rp.sin_t + at);
                            out = first ? out * ck - other * sk : other * sk + out * ck;
                        }
                        if (is_q) rp.q_out[(static_cast<size_t>(tile_q * BLOCK_Q + j) * rp.H + head) * hd + d] = __float2bfloat16_rn(out);
                        else if (tbase[j] >= 0) cache[tbase[j] + kv_head] = __float2bfloat16_rn(out);
                    }
                }
            }
        }
        if (warp == 2 && lane == 0) timeline_record(tl_id, 5);
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
    if (threadIdx.x == 0) timeline_record(tl_id, 6);
}

// ------------------------------------------------------------------------------------------ persistent kernel
// Many tokens: one CTA per SM walks over output tiles. Tensor memory holds two accumulators, so
// the epilogue of one tile (tcgen05.ld -> swizzled staging in shared memory -> TMA store or TMA
// reduce-add into the 32-bit residual stream) runs while the MMAs of the next tile are issued.
// Epilogues: store 32-bit, add to 32-bit, or SwiGLU: the tile's first half of columns are gate
// channels and the second half the matching up channels (two TMA loads per stage from the
// [gate; up] weight), and silu(gate) * up is stored as bfloat16.
enum TcEpilogue : int { kEpiStoreF32 = 0, kEpiAddF32 = 1, kEpiSwiGLU = 2, kEpiRopeStore = 3 };

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- CTA pairs (cta_group::2): two CTAs of a cluster on neighbouring SMs work on one 256-row tile. Each
// holds 128 rows of the tokens' operand and half of the rows of the weights' operand in its own shared
// memory and 128 rows of the accumulator in its own tensor memory; one thread of the pair's first CTA
// issues the MMAs for both. A CTA then fetches 32 KB instead of 48 KB per 64 columns of K, which is what
// an SM can take in (about 64 bytes a cycle) while its tensor core works through them in 512 cycles.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
// a TMA load into this CTA's shared memory whose bytes are counted on a barrier of either CTA of the pair
// (bar: a shared::cluster address). No multicast: each CTA fetches its own tiles.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) return false;
    }
}

template <int BLOCK_Q, bool PAIR = false>
struct TcPersistentConfig {
    static constexpr int kRowsQ = PAIR ? BLOCK_Q / 2 : BLOCK_Q;  // rows of the weights' tile in this CTA's shared memory
    static constexpr int kStageBytesP = kBlockP * kBlockK * 2;
    static constexpr int kStageBytesQ = kRowsQ * kBlockK * 2;
    static constexpr int kStageBytes = kStageBytesP + kStageBytesQ;
    static constexpr int kStages = PAIR ? ((BLOCK_Q >= 192) ? 6 : 8) : ((BLOCK_Q >= 192) ? 4 : 6);
    static constexpr int kStagingBytes = kBlockP * 128;          // 128 rows x 128 bytes, two of them
    static constexpr int kAccStride = (BLOCK_Q > 128) ? 256 : BLOCK_Q;   // columns between the two accumulators
    static constexpr int kTmemCols = 2 * kAccStride;                     // a power of two
    static constexpr int kSmemBytes = kStages * kStageBytes + 2 * kStagingBytes + 1024 + 256;
    // a pair's MMA covers 256 rows (M >> 4 at bits 24..28)
    static constexpr uint32_t kIdesc = PAIR ? ((TcConfig<BLOCK_Q>::kIdesc & ~(0x1Fu << 24)) | (static_cast<uint32_t>(256 >> 4) << 24))
                                            : TcConfig<BLOCK_Q>::kIdesc;
    static_assert(kSmemBytes <= 232448, "the pipeline does not fit into an SM's shared memory");
};

struct TcPersistentParams {
    int rows_p, rows_q, K;       // tokens, output columns of the accumulator tile space, reduction length
    int tiles_p, tiles_q;
    int up_row_offset;           // SwiGLU: row of the first up channel in the weight (= I)
    int* status;
    int splits;                  // K is cut into this many ranges, each an accumulator tile of its own whose result is
    int kb_per_split;            //   stored split_rows rows further down in the output (a workspace; the ranges are
    int split_rows;              //   added up, in order, by reduce_splits_kernel): few tiles still fill the GPU
    RopeStoreParams rope;        // epilogue kEpiRopeStore
};

constexpr int kPersistentThreads = 64 + 2 * 128;     // producer warp, MMA warp, two epilogue groups of four warps

template <int BLOCK_Q, int EPI, bool PAIR>
__global__ void __launch_bounds__(kPersistentThreads, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                          const __grid_constant__ CUtensorMap map_c, const TcPersistentParams p) {
    using Cfg = TcPersistentConfig<BLOCK_Q, PAIR>;
    constexpr int kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* staging = smem + kStages * Cfg::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * Cfg::kStagingBytes);
    // bars: [0,S) full, [S,2S) empty, [2S,2S+2) accumulator full, [2S+2,2S+4) accumulator empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (p.K + kBlockK - 1) / kBlockK;
    constexpr int kTl = kTlProductManyTokens + 2 * EPI + (PAIR ? 1 : 0);
    if (threadIdx.x == 0) timeline_record(kTl, 0);
    // PAIR: the two CTAs of a cluster walk over the same work items; rank r takes rows 128 r .. 128 r + 127 of a
    // 256-row tile of tokens and fetches rows r BLOCK_Q/2 .. of the weights' tile; p.tiles_p counts 256-row tiles.
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const int worker = PAIR ? blockIdx.x / 2 : blockIdx.x, n_workers = PAIR ? gridDim.x / 2 : gridDim.x;
    const int out_tiles = p.tiles_p * p.tiles_q;
    const int n_tiles = out_tiles * p.splits;
    // work item t: output tile t % out_tiles, range t / out_tiles of K
    auto kb_first = [&](int t) { return (t / out_tiles) * p.kb_per_split; };
    auto kb_count = [&](int t) { return min(total_kb, kb_first(t) + p.kb_per_split) - kb_first(t); };
    auto tile_p_of = [&](int t) { return PAIR ? 2 * ((t % out_tiles) % p.tiles_p) + static_cast<int>(rank) : (t % out_tiles) % p.tiles_p; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[kStages + s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars[2 * kStages + b]), 1);
            mbar_init(smem_u32(&bars[2 * kStages + 2 + b]), (PAIR ? 2 : 1) * (kPersistentThreads - 64));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols);
        else tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_launch_dependents();
    if (PAIR) cluster_sync_all();    // both CTAs' barriers exist before either signals the other's
    grid_dependency_wait();          // everything below reads what earlier kernels wrote
    if (threadIdx.x == 0) timeline_record(kTl, 1);
    // the first CTA's barriers as the other CTA addresses them: "stage full" counts both CTAs' bytes there, and
    // "accumulator empty" both CTAs' epilogue threads
    auto leader_bar = [&](int i) { return PAIR ? cluster_map(smem_u32(&bars[i]), 0u) : smem_u32(&bars[i]); };
    auto acc_empty_arrive = [&](int buf) {
        if (PAIR && rank != 0) cluster_mbar_arrive(leader_bar(2 * kStages + 2 + buf));
        else mbar_arrive(smem_u32(&bars[2 * kStages + 2 + buf]));
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0, issued_ok = 1;
            for (int t = worker; t < n_tiles && issued_ok; t += n_workers) {
                const int tile_p = tile_p_of(t), tile_q = (t % out_tiles) / p.tiles_p;
                const int kb0 = kb_first(t), n_kb = kb_count(t);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(smem_u32(&bars[kStages + s]), ((it / kStages) & 1) ^ 1, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrProducerWait); }
                        issued_ok = 0;
                        break;
                    }
                    uint8_t* stage = smem + s * Cfg::kStageBytes;
                    const int k0 = (kb0 + kb) * kBlockK;
                    if constexpr (PAIR) {
                        // the first CTA's barrier expects the bytes of both; each CTA fetches its own tokens and its half
                        // of the weights' rows (SwiGLU: the first CTA the gate rows, the second the up rows)
                        const uint32_t full = leader_bar(s);
                        if (rank == 0) mbar_expect_tx(smem_u32(&bars[s]), 2 * Cfg::kStageBytes);
                        tma_load_2d_pair(smem_u32(stage), &map_p, k0, tile_p * kBlockP, full);
                        const int n0 = (EPI == kEpiSwiGLU) ? tile_q * (BLOCK_Q / 2) + static_cast<int>(rank) * p.up_row_offset
                                                           : tile_q * BLOCK_Q + static_cast<int>(rank) * (BLOCK_Q / 2);
                        tma_load_2d_pair(smem_u32(stage + Cfg::kStageBytesP), &map_q, k0, n0, full);
                    } else {
                        const uint32_t full = smem_u32(&bars[s]);
                        mbar_expect_tx(full, Cfg::kStageBytes);
                        tma_load_2d(smem_u32(stage), &map_p, k0, tile_p * kBlockP, full);
                        if (EPI == kEpiSwiGLU) {
                            const int n0 = tile_q * (BLOCK_Q / 2);
                            tma_load_2d(smem_u32(stage + Cfg::kStageBytesP), &map_q, k0, n0, full);
                            tma_load_2d(smem_u32(stage + Cfg::kStageBytesP + Cfg::kStageBytesQ / 2), &map_q, k0, p.up_row_offset + n0, full);
                        } else {
                            tma_load_2d(smem_u32(stage + Cfg::kStageBytesP), &map_q, k0, tile_q * BLOCK_Q, full);
                        }
                    }
                }
            }
            if (*abort_flag && (!PAIR || rank == 0)) {
                const int first = max(0, it - kStages);
                for (int i = first; i < it; ++i) {
                    const unsigned long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&bars[i % kStages]), (i / kStages) & 1)) {
                        if (clock64() - t0 > kWaitCycles) { atomicCAS(p.status, 0, kErrDrain); break; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {           // a pair's MMAs are issued by its first CTA
            int it = 0, j = 0;
            bool ok = true;
            for (int t = worker; t < n_tiles && ok; t += n_workers, ++j) {
                const int buf = j & 1;
                const uint32_t acc_empty = smem_u32(&bars[2 * kStages + 2 + buf]);
                if (!(PAIR ? mbar_wait_cluster(acc_empty, ((j >> 1) & 1) ^ 1, abort_flag)
                           : mbar_wait(acc_empty, ((j >> 1) & 1) ^ 1, abort_flag))) {
                    if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrMmaWait); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * Cfg::kAccStride;
                const int n_kb = kb_count(t);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(smem_u32(&bars[s]), (it / kStages) & 1, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrMmaWait); }
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (it == 0) timeline_record(kTl, 2);
                    const uint32_t a_addr = smem_u32(smem + s * Cfg::kStageBytes);
                    const uint64_t desc_p = umma_desc(a_addr);
                    const uint64_t desc_q = umma_desc(a_addr + Cfg::kStageBytesP);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        if (PAIR) umma_bf16_pair(tmem_d, desc_p + 2 * k, desc_q + 2 * k, Cfg::kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
                        else umma_bf16(tmem_d, desc_p + 2 * k, desc_q + 2 * k, Cfg::kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    if (PAIR) umma_commit_pair(smem_u32(&bars[kStages + s]));      // the stage is free in both CTAs
                    else umma_commit(smem_u32(&bars[kStages + s]));
                }
                if (ok) {
                    if (PAIR) umma_commit_pair(smem_u32(&bars[2 * kStages + buf]));
                    else umma_commit(smem_u32(&bars[2 * kStages + buf]));
                }
            }
            timeline_record(kTl, 3);
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 2..9)
        // Two groups of four warps share a tile: group 0 (warps 2..5) takes the even column chunks,
        // group 1 (warps 6..9) the odd ones. Each group has its own staging buffer, named barrier
        // and leader thread that issues the group's TMA stores.
        const int group = (warp - 2) >> 2;
        const int lane_group = warp & 3;                         // the TMEM lanes this warp may read
        const int row = lane_group * 32 + lane;                  // row of the tile = TMEM lane
        const bool leader = (((warp - 2) & 3) == 0 && lane == 0);
        const uint32_t lane_addr = static_cast<uint32_t>(lane_group * 32) << 16;
        uint8_t* stg = staging + group * Cfg::kStagingBytes;
        const int bar_id = 1 + group;
        auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory"); };
        int j = 0;
        bool ok = true;
        for (int t = worker; t < n_tiles; t += n_workers, ++j) {
            const int tile_p = tile_p_of(t), tile_q = (t % out_tiles) / p.tiles_p;
            const int out_row = tile_p * kBlockP + (t / out_tiles) * p.split_rows;
            const int buf = j & 1;
            // Rotation and store: the token's position, its page row and the first cos/sin values are
            // requested now, while the tile's products still run.
            int rope_token = 0;
            size_t rope_kv_base = 0;
            const float *rope_cs = nullptr, *rope_sn = nullptr;
            float4 rope_c[4], rope_s[4];
            if constexpr (EPI == kEpiRopeStore) {
                const RopeStoreParams& rp = p.rope;
                rope_token = out_row + row;
                int pos = 0;
                if (rope_token < p.rows_p) {
                    pos = rp.positions[rope_token];
                    if (rp.write_kv) {
                        const int page = rp.block_tables[static_cast<size_t>(rp.row_req[rope_token]) * rp.table_stride + pos / rp.page_size];
                        rope_kv_base = (static_cast<size_t>(page) * rp.Hkv * rp.page_size + (pos % rp.page_size)) * rp.hd;
                    }
                }
                if (rp.cos_t) {
                    rope_cs = rp.cos_t + static_cast<size_t>(pos) * (rp.hd >> 1);
                    rope_sn = rp.sin_t + static_cast<size_t>(pos) * (rp.hd >> 1);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        rope_c[q4] = __ldg(reinterpret_cast<const float4*>(rope_cs) + q4);
                        rope_s[q4] = __ldg(reinterpret_cast<const float4*>(rope_sn) + q4);
                    }
                }
            }
            if (ok && !mbar_wait(smem_u32(&bars[2 * kStages + buf]), (j >> 1) & 1, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicCAS(p.status, 0, kErrEpilogueWait); }
            }
            group_sync();
            if (*abort_flag) ok = false;                          // read after the barrier: one decision for the group
            group_sync();
            if (!ok) break;
            tc_fence_after();
            if (j == 0 && warp == 2 && lane == 0) timeline_record(kTl, 4);
            const uint32_t tmem_d = tmem_base + buf * Cfg::kAccStride + lane_addr;
            if constexpr (EPI == kEpiRopeStore) {
                // A thread holds one token's row of the tile: whole heads (BLOCK_Q is a multiple of the head
                // size), so both members of a rotated pair (d, d + hd/2) are its own. 16 pairs at a time:
                // their cos/sin are read once and serve all heads of the tile that this group takes.
                const RopeStoreParams& rp = p.rope;
                const int hd = rp.hd, half = hd >> 1;
                const int heads_per_tile = BLOCK_Q / hd;
                if (group >= heads_per_tile) {
                    tc_fence_before();
                    acc_empty_arrive(buf);
                }
                const bool valid = rope_token < p.rows_p;
                for (int j = 0; j < half; j += 16) {
                    if (j > 0 && rope_cs != nullptr) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            rope_c[q4] = __ldg(reinterpret_cast<const float4*>(rope_cs + j) + q4);
                            rope_s[q4] = __ldg(reinterpret_cast<const float4*>(rope_sn + j) + q4);
                        }
                    }
                    const bool last_j = j + 16 >= half;
                    for (int hh = group; hh < heads_per_tile; hh += 2) {
                        const int head = tile_q * heads_per_tile + hh;
                        __nv_bfloat16* dst = nullptr;
                        if (valid) {
                            if (head < rp.H) dst = rp.q_out + (static_cast<size_t>(rope_token) * rp.H + head) * hd;
                            else if (!rp.write_kv) dst = nullptr;
                            else if (head < rp.H + rp.Hkv) dst = rp.k_cache + rope_kv_base + static_cast<size_t>(head - rp.H) * rp.page_size * hd;
                            else if (head < rp.H + 2 * rp.Hkv) dst = rp.v_cache + rope_kv_base + static_cast<size_t>(head - rp.H - rp.Hkv) * rp.page_size * hd;
                        }
                        const bool rotate = rope_cs != nullptr && head < rp.H + rp.Hkv;
                        uint32_t lo[16], hi[16];
                        tmem_ld_x16(tmem_d + hh * hd + j, lo);
                        tmem_ld_x16(tmem_d + hh * hd + half + j, hi);
                        tmem_ld_wait();
                        if (last_j && hh + 2 >= heads_per_tile) { tc_fence_before(); acc_empty_arrive(buf); }
                        if (dst == nullptr) continue;
                        uint32_t oa[8], ob[8];
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            const float cc[4] = {rope_c[q4].x, rope_c[q4].y, rope_c[q4].z, rope_c[q4].w};
                            const float ss[4] = {rope_s[q4].x, rope_s[q4].y, rope_s[q4].z, rope_s[q4].w};
                            float ra[4], rb[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float a = __uint_as_float(lo[q4 * 4 + e]), b = __uint_as_float(hi[q4 * 4 + e]);
                                ra[e] = rotate ? a * cc[e] - b * ss[e] : a;
                                rb[e] = rotate ? a * ss[e] + b * cc[e] : b;
                            }
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                __nv_bfloat162 pa = __floats2bfloat162_rn(ra[2 * e], ra[2 * e + 1]);
                                __nv_bfloat162 pb = __floats2bfloat162_rn(rb[2 * e], rb[2 * e + 1]);
                                oa[q4 * 2 + e] = *reinterpret_cast<uint32_t*>(&pa);
                                ob[q4 * 2 + e] = *reinterpret_cast<uint32_t*>(&pb);
                            }
                        }
                        uint4* da = reinterpret_cast<uint4*>(dst + j);
                        uint4* db = reinterpret_cast<uint4*>(dst + half + j);
                        da[0] = make_uint4(oa[0], oa[1], oa[2], oa[3]);
                        da[1] = make_uint4(oa[4], oa[5], oa[6], oa[7]);
                        db[0] = make_uint4(ob[0], ob[1], ob[2], ob[3]);
                        db[1] = make_uint4(ob[4], ob[5], ob[6], ob[7]);
                    }
                }
                continue;
            }
            constexpr int kChunks = (EPI == kEpiSwiGLU) ? BLOCK_Q / 128 : BLOCK_Q / 32;   // TMA stores per tile
            if (group >= kChunks) {                               // a tile with a single chunk: this group has nothing to read
                tc_fence_before();
                acc_empty_arrive(buf);
            }
            for (int c = group; c < kChunks; c += 2) {
                if (leader) bulk_wait_read0();                    // the group's last store has read the staging buffer
                group_sync();
                uint32_t r[32];
                const bool last = c + 2 >= kChunks;               // this group's last chunk of the tile
                if (EPI == kEpiSwiGLU) {
                    // 64 output channels per store, in two halves of 32: gate at column ch, up at BLOCK_Q/2 + ch
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int ch = c * 64 + half * 32;
                        uint32_t u[32];
                        tmem_ld_x16(tmem_d + ch, r);
                        tmem_ld_x16(tmem_d + ch + 16, r + 16);
                        tmem_ld_x16(tmem_d + BLOCK_Q / 2 + ch, u);
                        tmem_ld_x16(tmem_d + BLOCK_Q / 2 + ch + 16, u + 16);
                        tmem_ld_wait();
                        if (last && half == 1) { tc_fence_before(); acc_empty_arrive(buf); }
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {          // 8 channels = 16 bytes of bfloat16 per step
                            uint32_t packed[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float g0 = __uint_as_float(r[q4 * 8 + 2 * e]), g1 = __uint_as_float(r[q4 * 8 + 2 * e + 1]);
                                const float u0 = __uint_as_float(u[q4 * 8 + 2 * e]), u1 = __uint_as_float(u[q4 * 8 + 2 * e + 1]);
                                const float h0 = g0 * (1.0f / (1.0f + expf(-g0))) * u0;
                                const float h1 = g1 * (1.0f / (1.0f + expf(-g1))) * u1;
                                __nv_bfloat162 hb = __floats2bfloat162_rn(h0, h1);
                                packed[e] = *reinterpret_cast<uint32_t*>(&hb);
                            }
                            const int chunk16 = half * 4 + q4;
                            *reinterpret_cast<uint4*>(stg + row * 128 + ((chunk16 ^ (row & 7)) * 16)) =
                                make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        }
                    }
                } else {
                    tmem_ld_x16(tmem_d + c * 32, r);
                    tmem_ld_x16(tmem_d + c * 32 + 16, r + 16);
                    tmem_ld_wait();
                    if (last) { tc_fence_before(); acc_empty_arrive(buf); }
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        *reinterpret_cast<uint4*>(stg + row * 128 + ((q4 ^ (row & 7)) * 16)) =
                            make_uint4(r[q4 * 4], r[q4 * 4 + 1], r[q4 * 4 + 2], r[q4 * 4 + 3]);
                }
                fence_async_smem();
                group_sync();
                if (leader) {
                    const int col = (EPI == kEpiSwiGLU) ? tile_q * (BLOCK_Q / 2) + c * 64 : tile_q * BLOCK_Q + c * 32;
                    if (EPI == kEpiAddF32) tma_reduce_add_2d(&map_c, smem_u32(stg), col, out_row);
                    else tma_store_2d(&map_c, smem_u32(stg), col, out_row);
                    bulk_commit();
                }
            }
        }
        if (leader) bulk_wait_all();
        if (warp == 2 && lane == 0) timeline_record(kTl, 5);
        tc_fence_before();
    }
    __syncthreads();
    if (threadIdx.x == 0) timeline_record(kTl, 6);
    if (PAIR) cluster_sync_all();    // neither CTA leaves (or frees tensor memory) while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
        else tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------ host side
// A [rows, K] row-major bf16 matrix viewed as boxes of [box_rows, 64] with 128-byte swizzle; reads
// beyond rows or K give zeros.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, long long ld, int box_rows) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) { set_error("gemm_tc: cuTensorMapEncodeTiled is not available from the driver"); return 1; }
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("gemm_tc: cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r)); return 1; }
    return 0;
}

// The output matrix [rows, cols] (row stride ld elements) as boxes of 128 rows x 128 bytes with the
// 128-byte swizzle the epilogue writes its staging in; stores beyond rows or cols are clipped.
static int make_out_map(CUtensorMap* map, void* base, int rows, int cols, long long ld, bool bf16) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (!fn) { set_error("gemm_tc: cuTensorMapEncodeTiled is not available from the driver"); return 1; }
    const int elt = bf16 ? 2 : 4;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elt};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elt), static_cast<cuuint32_t>(kBlockP)};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides,
                    box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("gemm_tc: cuTensorMapEncodeTiled (output) failed with code %d", static_cast<int>(r)); return 1; }
    return 0;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 1;
    }
    return n;
}

template <int BLOCK_Q, int EPI>
static int launch_persistent(const CUtensorMap& mp, const CUtensorMap& mq, const CUtensorMap& mc,
                             const TcPersistentParams& p, cudaStream_t st) {
    using Cfg = TcPersistentConfig<BLOCK_Q>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BLOCK_Q, EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) { set_error("gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::kSmemBytes, cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    const int tiles = p.tiles_p * p.tiles_q * p.splits;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    launch_kernel((gemm_tc_persistent_kernel<BLOCK_Q, EPI, false>), dim3(grid), dim3(kPersistentThreads), Cfg::kSmemBytes, st, mp, mq, mc, p);
    return check_launch("gemm_tc_persistent");
}

// The same product by pairs of CTAs (clusters of two, cta_group::2); p.tiles_p counts 256-row tiles. The grid holds
// as many pairs as the device keeps resident at once (asked once per kernel), at most one per work item.
template <int BLOCK_Q, int EPI>
static int pair_capacity() {
    using Cfg = TcPersistentConfig<BLOCK_Q, true>;
    static int cached = -1;
    if (cached >= 0) return cached;
    int n = 0;
    if (cudaFuncSetAttribute(gemm_tc_persistent_kernel<BLOCK_Q, EPI, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * sm_count());
        cfg.blockDim = dim3(kPersistentThreads);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_persistent_kernel<BLOCK_Q, EPI, true>, &cfg) != cudaSuccess) n = 0;
    }
    cudaGetLastError();
    cached = n;
    return n;
}

template <int BLOCK_Q, int EPI>
static int launch_persistent_pair(const CUtensorMap& mp, const CUtensorMap& mq, const CUtensorMap& mc,
                                  const TcPersistentParams& p, cudaStream_t st) {
    using Cfg = TcPersistentConfig<BLOCK_Q, true>;
    const int capacity = pair_capacity<BLOCK_Q, EPI>();
    if (capacity < 1) { set_error("gemm_tc: the device holds no pair of CTAs of the paired product"); return 1; }
    const int items = p.tiles_p * p.tiles_q * p.splits;
    const int pairs = items < capacity ? items : capacity;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kPersistentThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_persistent_kernel<BLOCK_Q, EPI, true>, mp, mq, mc, p);
    if (e != cudaSuccess) { set_error("gemm_tc: launch of the paired product failed: %s", cudaGetErrorString(e)); return 1; }
    return check_launch("gemm_tc_persistent (pairs)");
}

static int g_cluster_reduce = 1;
static int g_stream_weights = 1;
constexpr int kMaxSmemPerBlock = 232448;       // 227 KB
constexpr int kMaxClusterSplits = 8;           // the portable cluster size

// How many clusters of `splits` CTAs of this kernel the device holds at once (0: none, or the
// partial tiles do not fit into shared memory). Asked once per size.
template <int BLOCK_Q, bool TILED>
static int cluster_capacity(int splits) {
    using Cfg = TcConfig<BLOCK_Q, TILED>;
    static int cached[kMaxClusterSplits + 1] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    const bool own_place = Cfg::smem_bytes(splits) <= Cfg::kOwnPlaceLimit;
    if (splits < 2 || splits > kMaxClusterSplits || !(own_place || Cfg::cluster_fits(splits))) return 0;
    if (cached[splits] >= 0) return cached[splits];
    int n = 0;
    if (cudaFuncSetAttribute(gemm_tc_kernel<BLOCK_Q, TILED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemPerBlock) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, splits);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = own_place ? Cfg::smem_bytes(splits) : Cfg::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = splits;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BLOCK_Q, TILED>, &cfg) != cudaSuccess) n = 0;
    }
    cudaGetLastError();
    cached[splits] = n;
    return n;
}

// Launches the kernel of one form (p.cluster decided): plainly, or as clusters of the splits of a tile.
template <int BLOCK_Q, bool TILED, int SPEC>
static int launch_tc_form(const CUtensorMap& mp, const CUtensorMap& mq, const TcParams& p, dim3 grid, cudaStream_t st) {
    using Cfg = TcConfig<BLOCK_Q, TILED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BLOCK_Q, TILED, SPEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemPerBlock);
        if (e != cudaSuccess) { set_error("gemm_tc: cannot reserve %d bytes of shared memory: %s", kMaxSmemPerBlock, cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    if (!p.cluster) {
        launch_kernel((gemm_tc_kernel<BLOCK_Q, TILED, SPEC>), dim3(grid), dim3(kThreads), Cfg::kSmemBytes, st, mp, mq, p);
        return check_launch("gemm_tc");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = p.cluster == 2 ? Cfg::kSmemBytes : Cfg::smem_bytes(p.splits);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = p.splits;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BLOCK_Q, TILED, SPEC>, mp, mq, p);
    if (e != cudaSuccess) { set_error("gemm_tc: cluster launch failed: %s", cudaGetErrorString(e)); return 1; }
    return check_launch("gemm_tc");
}

static int g_specialised = 1;

template <int BLOCK_Q, bool TILED>
static int launch_tc(const CUtensorMap& mp, const CUtensorMap& mq, TcParams p, dim3 grid, cudaStream_t st) {
    using Cfg = TcConfig<BLOCK_Q, TILED>;
    // all clusters of the launch resident at once, or the workspace path: a second wave of clusters
    // would cost more than the reduce through global memory
    const long long tiles = static_cast<long long>(grid.x) * grid.y;
    p.cluster = (p.splits > 1 && g_cluster_reduce && tiles <= cluster_capacity<BLOCK_Q, TILED>(p.splits)) ? 1 : 0;
    // the partial tiles count their bytes on one mbarrier, whose byte count ends at 2^20 - 1
    if (p.cluster && static_cast<long long>(p.splits - 1) * kBlockP * ((BLOCK_Q + 15) / 16 * 16) * 4 > 1048575ll) p.cluster = 0;
    if (p.cluster && Cfg::smem_bytes(p.splits) > Cfg::kOwnPlaceLimit) p.cluster = 2;    // partial tiles in split 0's stages
    // the forms of a decode step of up to 16 tokens over tiled weights: kernels with nothing else in them
    if constexpr (BLOCK_Q == 16 && TILED) {
        if (g_specialised && p.prefetch_p && p.stream_p && !p.c_bf16) {
            if (p.rope_on && p.cluster == TcSpec<kSpecRopeCluster>::cluster && !p.accumulate) return launch_tc_form<BLOCK_Q, TILED, kSpecRopeCluster>(mp, mq, p, grid, st);
            if (!p.rope_on && p.cluster == TcSpec<kSpecAddCluster>::cluster && p.accumulate) return launch_tc_form<BLOCK_Q, TILED, kSpecAddCluster>(mp, mq, p, grid, st);
            if (!p.rope_on && p.splits == 1 && !p.accumulate) return launch_tc_form<BLOCK_Q, TILED, kSpecStoreOne>(mp, mq, p, grid, st);
        }
    }
    return launch_tc_form<BLOCK_Q, TILED, kSpecAny>(mp, mq, p, grid, st);
}


}  // namespace gi

using namespace gi;
GI_TIMELINE_SETTER(gi_timeline_set_gemm)

// C[M,N] (+)= A[M,K] * W[N,K]^T, A and W bfloat16 row-major with row strides lda, ldw (elements),
// C float (optionally accumulated into) or bfloat16 with row stride ldc.
//   swap = 0: tokens on the 128-row side (tile 128 x block_q over [M, N]);
//   swap = 1: weights on the 128-row side, block_q >= tokens on the narrow side.
//   splits > 1 (swap only): K is cut into `splits` ranges; workspace must hold
//   tiles * splits * 128 * block_q floats and counters one zeroed word per tile.
//   w_tiles (swap only, may be null): W once more in the tile-by-tile layout of TcParams::p_tiles;
//   the weights are then fetched with bulk copies, two 64-wide blocks of K to a stage.
//   ahead, ahead_bytes (products of at most 32 tokens, may be null): memory that a later kernel of the step will
//   stream (the start of the next large weight matrix), asked into L2 by this product's CTAs.
// Switches the cluster reduce of split products on or off (on by default); returns the old value.
extern "C" int gi_gemm_tc_set_cluster(int on) {
    const int old = g_cluster_reduce;
    g_cluster_reduce = on ? 1 : 0;
    return old;
}

// Switches the evict-first L2 policy on the weight loads of few-token products on or off (on by default);
// returns the old value.
extern "C" int gi_gemm_tc_set_stream_weights(int on) {
    const int old = g_stream_weights;
    g_stream_weights = on ? 1 : 0;
    return old;
}

// Switches the kernels of single forms (TcSpecKind) on or off (on by default; off: the kernel of every form runs
// them); returns the old value.
extern "C" int gi_gemm_tc_set_specialised(int on) {
    const int old = g_specialised;
    g_specialised = on ? 1 : 0;
    return old;
}

// Clusters of `splits` CTAs the device holds at once for the kernel of this block_q (0: the
// workspace path is used). A negative count asks the same for -splits with the partial tiles in a
// place of their own only.
extern "C" int gi_gemm_tc_cluster_capacity(int block_q, int splits, int tiled) {
    if (splits < 0) {       // -splits: only if the partial tiles have a place of their own (nobody waits for split 0)
        splits = -splits;
        bool own = false;
        switch (block_q) {
            case 16: own = tiled ? TcConfig<16, true>::smem_bytes(splits) <= TcConfig<16, true>::kOwnPlaceLimit : TcConfig<16, false>::smem_bytes(splits) <= TcConfig<16, false>::kOwnPlaceLimit; break;
            case 32: own = tiled ? TcConfig<32, true>::smem_bytes(splits) <= TcConfig<32, true>::kOwnPlaceLimit : TcConfig<32, false>::smem_bytes(splits) <= TcConfig<32, false>::kOwnPlaceLimit; break;
            case 64: own = tiled ? TcConfig<64, true>::smem_bytes(splits) <= TcConfig<64, true>::kOwnPlaceLimit : TcConfig<64, false>::smem_bytes(splits) <= TcConfig<64, false>::kOwnPlaceLimit; break;
            case 128: own = tiled ? TcConfig<128, true>::smem_bytes(splits) <= TcConfig<128, true>::kOwnPlaceLimit : TcConfig<128, false>::smem_bytes(splits) <= TcConfig<128, false>::kOwnPlaceLimit; break;
            default: break;
        }
        if (!own) return 0;
    }
    switch (block_q) {
        case 16: return tiled ? cluster_capacity<16, true>(splits) : cluster_capacity<16, false>(splits);
        case 32: return tiled ? cluster_capacity<32, true>(splits) : cluster_capacity<32, false>(splits);
        case 64: return tiled ? cluster_capacity<64, true>(splits) : cluster_capacity<64, false>(splits);
        case 128: return tiled ? cluster_capacity<128, true>(splits) : cluster_capacity<128, false>(splits);
        default: return 0;
    }
}

static int run_gemm_tc(const void* A, const void* W, void* C, int c_dtype, int accumulate, int M, int N, int K,
                       long long lda, long long ldw, long long ldc, int swap, int block_q, int splits,
                       void* workspace, long long workspace_floats, void* counters, int n_counters, void* status,
                       const void* w_tiles, const RopeStoreParams* rope, const void* ahead, long long ahead_bytes, void* stream) {
    if (M == 0 || N == 0) return 0;
    GI_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: sizes must be positive (M=%d, N=%d, K=%d)", M, N, K);
    GI_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the row strides (%lld, %lld) must be multiples of 8 (16-byte rows for TMA)", K, lda, ldw);
    GI_REQUIRE((reinterpret_cast<uintptr_t>(A) % 16 == 0) && (reinterpret_cast<uintptr_t>(W) % 16 == 0),
               "gemm_tc: operands must be 16-byte aligned");
    GI_REQUIRE(c_dtype == kF32 || c_dtype == kBF16, "gemm_tc: unsupported output dtype code %d", c_dtype);
    GI_REQUIRE(!(accumulate && c_dtype != kF32), "gemm_tc: accumulation needs a 32-bit output");
    GI_REQUIRE(block_q == 16 || block_q == 32 || block_q == 64 || block_q == 128 || block_q == 256,
               "gemm_tc: block_q=%d is not one of 16, 32, 64, 128, 256", block_q);
    GI_REQUIRE(splits >= 1, "gemm_tc: splits must be >= 1");
    GI_REQUIRE(status != nullptr, "gemm_tc: a status word is required");

    TcParams p = {};
    if (rope) {
        GI_REQUIRE(swap && block_q <= 128 && !accumulate, "gemm_tc rope: needs the weights on the 128-row side");
        p.rope_on = 1;
        p.rope = *rope;
    }
    p.C = C;
    p.c_bf16 = c_dtype == kBF16;
    p.accumulate = accumulate;
    p.K = K;
    p.splits = splits;
    p.workspace = static_cast<float*>(workspace);
    p.counters = static_cast<unsigned*>(counters);
    p.status = static_cast<int*>(status);
    const int total_kb = (K + kBlockK - 1) / kBlockK;
    p.k_blocks_per_split = (total_kb + splits - 1) / splits;
    const bool tiled = swap && w_tiles != nullptr && block_q <= 128;
    p.p_tiles = tiled ? static_cast<const uint8_t*>(w_tiles) : nullptr;
    p.tiles_kb = (total_kb + 1) / 2 * 2;
    if (tiled) {
        GI_REQUIRE(reinterpret_cast<uintptr_t>(w_tiles) % 16 == 0, "gemm_tc: the tiled weights must be 16-byte aligned");
        p.k_blocks_per_split = (p.k_blocks_per_split + 1) / 2 * 2;      // a stage's two blocks belong to one split
    }

    CUtensorMap mp, mq;
    if (ahead != nullptr && ahead_bytes >= 32768 && swap && block_q <= 32) {
        GI_REQUIRE(reinterpret_cast<uintptr_t>(ahead) % 16 == 0, "gemm_tc: the weights to ask into L2 must be 16-byte aligned");
        p.ahead = static_cast<const uint8_t*>(ahead);
        p.ahead_bytes = static_cast<unsigned long long>(ahead_bytes) / 32768ull * 32768ull;
    }
    p.prefetch_p = swap ? 1 : 0;
    // measured on B200 (Llama-3.2-1B shape, a decode step): 3.5 % faster at 1 and 8 tokens, 0.8 % slower at 64
    p.stream_p = (swap && block_q <= 32 && g_stream_weights) ? 1 : 0;
    if (swap) {
        p.rows_p = N; p.rows_q = M; p.stride_p = 1; p.stride_q = ldc;
        if (make_map(&mp, W, N, K, ldw, kBlockP) || make_map(&mq, A, M, K, lda, block_q)) return 1;
    } else {
        p.rows_p = M; p.rows_q = N; p.stride_p = ldc; p.stride_q = 1;
        if (make_map(&mp, A, M, K, lda, kBlockP) || make_map(&mq, W, N, K, ldw, block_q)) return 1;
    }
    dim3 grid((p.rows_p + kBlockP - 1) / kBlockP, (p.rows_q + block_q - 1) / block_q, splits);
    GI_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm_tc: grid too large");
    if (splits > 1) {
        const long long tiles = static_cast<long long>(grid.x) * grid.y;
        GI_REQUIRE(workspace != nullptr && counters != nullptr, "gemm_tc: a split over K needs a workspace and counters");
        GI_REQUIRE(tiles * splits * kBlockP * block_q <= workspace_floats,
                   "gemm_tc: the workspace of %lld floats is too small for %lld tiles x %d splits", workspace_floats, tiles, splits);
        GI_REQUIRE(tiles <= n_counters, "gemm_tc: %lld tiles need more than the %d counters given", tiles, n_counters);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (block_q) {
        case 16: return tiled ? launch_tc<16, true>(mp, mq, p, grid, st) : launch_tc<16, false>(mp, mq, p, grid, st);
        case 32: return tiled ? launch_tc<32, true>(mp, mq, p, grid, st) : launch_tc<32, false>(mp, mq, p, grid, st);
        case 64: return tiled ? launch_tc<64, true>(mp, mq, p, grid, st) : launch_tc<64, false>(mp, mq, p, grid, st);
        case 128: return tiled ? launch_tc<128, true>(mp, mq, p, grid, st) : launch_tc<128, false>(mp, mq, p, grid, st);
        default: return launch_tc<256, false>(mp, mq, p, grid, st);
    }
}

static int gi_gemm_tc_impl(const void* A, const void* W, void* C, int c_dtype, int accumulate, int M, int N, int K,
                          long long lda, long long ldw, long long ldc, int swap, int block_q, int splits,
                          void* workspace, long long workspace_floats, void* counters, int n_counters, void* status,
                          const void* w_tiles, const void* ahead, long long ahead_bytes, void* stream) {
    return run_gemm_tc(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, swap, block_q, splits, workspace,
                       workspace_floats, counters, n_counters, status, w_tiles, nullptr, ahead, ahead_bytes, stream);
}

// The [q; k; v] product of few tokens (at most block_q <= 128, weights on the 128-row side) with rotation
// and page store done by the CTA that holds a tile's sum (RopeStoreParams). The head size must divide 128
// so that both members of a rotated pair lie in one tile; any rotary size and pairing.
static int gi_gemm_tc_rope_impl(const void* A, const void* W, int M, int K, long long lda, long long ldw, int block_q,
                               int splits, void* workspace, long long workspace_floats, void* counters, int n_counters,
                               void* status, const void* w_tiles, const int* positions, const int* row_req,
                               const int* block_tables, int table_stride, const float* cos_t, const float* sin_t,
                               int rot_half, int interleaved, void* q_out, void* k_cache, void* v_cache, int H, int Hkv,
                               int hd, int page_size, int write_kv, void* stream) {
    GI_REQUIRE(H > 0 && Hkv > 0 && hd > 0 && page_size > 0, "gemm_tc rope: sizes must be positive");
    GI_REQUIRE(kBlockP % hd == 0, "gemm_tc rope: the head size %d does not divide %d", hd, kBlockP);
    GI_REQUIRE(block_q <= 128, "gemm_tc rope: block_q=%d (at most 128 tokens to a tile)", block_q);
    GI_REQUIRE(cos_t == nullptr || (sin_t != nullptr && rot_half > 0 && 2 * rot_half <= hd),
               "gemm_tc rope: rotary size %d does not fit the head size %d", 2 * rot_half, hd);
    RopeStoreParams rope{positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved,
                         static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                         static_cast<__nv_bfloat16*>(v_cache), H, Hkv, hd, page_size, write_kv};
    const int N = (H + 2 * Hkv) * hd;
    return run_gemm_tc(A, W, nullptr, kF32, 0, M, N, K, lda, ldw, N, 1, block_q, splits, workspace, workspace_floats,
                       counters, n_counters, status, w_tiles, &rope, nullptr, 0, stream);
}

// Reads the status word (synchronises the stream): 0 = no bounded wait ever gave up.
extern "C" int gi_gemm_tc_status(const void* status, void* stream, int* out) {
    cudaError_t e = cudaMemcpyAsync(out, status, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_error("gemm_tc_status: %s", cudaGetErrorString(e)); return 1; }
    return 0;
}

// C[m, n] (+)= ws[0][m][n] + ws[1][m][n] + ... in this order: the ranges of K of a split product.
__global__ void reduce_splits_kernel(const float* __restrict__ ws, float* __restrict__ C, int M, int N4, long long ldc,
                                     long long split_stride, int splits, int accumulate) {
    if (threadIdx.x == 0) timeline_record(kTlAddRanges, 0);
    pdl_prologue();
    if (threadIdx.x == 0) timeline_record(kTlAddRanges, 1);
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<long long>(M) * N4) return;
    const int m = static_cast<int>(i / N4), n4 = static_cast<int>(i % N4);
    float4* c = reinterpret_cast<float4*>(C + static_cast<long long>(m) * ldc) + n4;
    const float4* w = reinterpret_cast<const float4*>(ws + static_cast<long long>(m) * N4 * 4) + n4;
    float4 part[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
        part[s] = s < splits ? __ldcg(w + static_cast<long long>(s) * split_stride / 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 v = accumulate ? *c : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; ++s)
        if (s < splits) { v.x += part[s].x; v.y += part[s].y; v.z += part[s].z; v.w += part[s].w; }
    *c = v;
    if (threadIdx.x == 0) timeline_record(kTlAddRanges, 6);
}

// Many tokens, one persistent CTA per SM. epilogue 0: C[M,N] = A W^T (32-bit); 1: C += A W^T (32-bit);
// 2: W is [2N, K] = [gate; up] and C[M,N] = silu(A Wgate^T) * (A Wup^T) as bfloat16.
// block_q: 256 or 128 accumulator columns per tile.
// splits > 1 (epilogues 0 and 1, N a multiple of 4, at most 8): K is cut into ranges whose tiles are work
// items of their own; their results go to `workspace` (splits x ceil(M / 128) x 128 x N floats) and a
// second kernel adds them up in order into C. Few output tiles (a few hundred tokens) then still fill the GPU.
// pair: the product runs on pairs of CTAs that share 256-row tiles of tokens (block_q 256 only).
static int gi_gemm_tc_persistent_impl(const void* A, const void* W, void* C, int epilogue, int M, int N, int K,
                                     long long lda, long long ldw, long long ldc, int block_q, void* status,
                                     int splits, void* workspace, long long workspace_floats, int pair, void* stream) {
    if (M == 0 || N == 0) return 0;
    GI_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: sizes must be positive (M=%d, N=%d, K=%d)", M, N, K);
    GI_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the row strides (%lld, %lld) must be multiples of 8 (16-byte rows for TMA)", K, lda, ldw);
    GI_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tc: unknown epilogue %d", epilogue);
    const bool bf16_out = epilogue == kEpiSwiGLU;
    GI_REQUIRE((ldc * (bf16_out ? 2 : 4)) % 16 == 0, "gemm_tc: the output row stride %lld is not a multiple of 16 bytes", ldc);
    GI_REQUIRE((reinterpret_cast<uintptr_t>(A) % 16 == 0) && (reinterpret_cast<uintptr_t>(W) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(C) % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    GI_REQUIRE(block_q == 128 || block_q == 256, "gemm_tc: block_q=%d is not 128 or 256", block_q);
    GI_REQUIRE(!pair || block_q == 256, "gemm_tc: pairs of CTAs work on tiles of 256 columns only");
    GI_REQUIRE(status != nullptr, "gemm_tc: a status word is required");
    TcPersistentParams p = {};
    p.rows_p = M; p.rows_q = N; p.K = K;
    p.tiles_p = pair ? (M + 2 * kBlockP - 1) / (2 * kBlockP) : (M + kBlockP - 1) / kBlockP;
    const int rows_per_tile_p = pair ? 2 * kBlockP : kBlockP;
    p.up_row_offset = N;
    p.status = static_cast<int*>(status);
    const int total_kb = (K + kBlockK - 1) / kBlockK;
    p.splits = 1; p.kb_per_split = total_kb; p.split_rows = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CUtensorMap mp, mq, mc;
    if (make_map(&mp, A, M, K, lda, kBlockP)) return 1;
    const bool split = splits > 1;
    if (split) {
        GI_REQUIRE(epilogue != kEpiSwiGLU && N % 4 == 0 && splits <= 8, "gemm_tc: a split over K needs a 32-bit output, N %% 4 == 0 and at most 8 ranges");
        p.kb_per_split = (total_kb + splits - 1) / splits;
        splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;             // every range holds at least one block
        p.splits = splits;
        p.split_rows = p.tiles_p * rows_per_tile_p;
        const long long need = static_cast<long long>(splits) * p.split_rows * N;
        GI_REQUIRE(workspace != nullptr && need <= workspace_floats, "gemm_tc: the workspace of %lld floats is too small for %lld", workspace_floats, need);
        if (make_out_map(&mc, workspace, splits * p.split_rows, N, N, false)) return 1;
    } else if (make_out_map(&mc, C, M, N, ldc, bf16_out)) {
        return 1;
    }
    const int run_epilogue = split ? static_cast<int>(kEpiStoreF32) : epilogue;
    auto finish = [&](int rc) -> int {
        if (rc != 0 || !split) return rc;
        const long long n = static_cast<long long>(M) * (N / 4);
        launch_kernel((reduce_splits_kernel), dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, st,
                      static_cast<const float*>(workspace), static_cast<float*>(C), M, N / 4, ldc,
                      static_cast<long long>(p.split_rows) * N, splits, epilogue == kEpiAddF32 ? 1 : 0);
        return check_launch("gemm_tc reduce");
    };
    if (epilogue == kEpiSwiGLU) {
        p.tiles_q = (N + block_q / 2 - 1) / (block_q / 2);
        if (make_map(&mq, W, 2 * N, K, ldw, block_q / 2)) return 1;
        if (pair) return launch_persistent_pair<256, kEpiSwiGLU>(mp, mq, mc, p, st);
        if (block_q == 256) return launch_persistent<256, kEpiSwiGLU>(mp, mq, mc, p, st);
        return launch_persistent<128, kEpiSwiGLU>(mp, mq, mc, p, st);
    }
    p.tiles_q = (N + block_q - 1) / block_q;
    if (make_map(&mq, W, N, K, ldw, pair ? block_q / 2 : block_q)) return 1;
    if (pair) {
        if (run_epilogue == kEpiAddF32) return launch_persistent_pair<256, kEpiAddF32>(mp, mq, mc, p, st);
        return finish(launch_persistent_pair<256, kEpiStoreF32>(mp, mq, mc, p, st));
    }
    if (block_q == 256) {
        if (run_epilogue == kEpiAddF32) return launch_persistent<256, kEpiAddF32>(mp, mq, mc, p, st);
        return finish(launch_persistent<256, kEpiStoreF32>(mp, mq, mc, p, st));
    }
    if (run_epilogue == kEpiAddF32) return launch_persistent<128, kEpiAddF32>(mp, mq, mc, p, st);
    return finish(launch_persistent<128, kEpiStoreF32>(mp, mq, mc, p, st));
}

// The [q; k; v] product of many tokens with rotation and page store in its epilogue (RopeStoreParams):
// A [M, K] bfloat16 activations, W [(H + 2 Hkv) * hd, K]; nothing else is written. Head sizes 32, 64, 128
// with the whole head rotated (rot_half = hd / 2) in the half-split pairing, or no rotation at all.
static int gi_gemm_tc_persistent_rope_impl(const void* A, const void* W, int M, int K, long long lda, long long ldw,
                                          const int* positions, const int* row_req, const int* block_tables,
                                          int table_stride, const float* cos_t, const float* sin_t, int rot_half,
                                          int interleaved, void* q_out, void* k_cache, void* v_cache, int H, int Hkv,
                                          int hd, int page_size, int write_kv, void* status, int pair, void* stream) {
    if (M == 0) return 0;
    GI_REQUIRE(M > 0 && K > 0 && H > 0 && Hkv > 0 && page_size > 0, "gemm_tc rope: sizes must be positive");
    GI_REQUIRE(hd == 32 || hd == 64 || hd == 128, "gemm_tc rope: head size %d is not 32, 64 or 128", hd);
    GI_REQUIRE(cos_t == nullptr || (sin_t != nullptr && !interleaved && rot_half * 2 == hd),
               "gemm_tc rope: only whole heads in the half-split pairing are rotated here (rot_half=%d, hd=%d, interleaved=%d)",
               rot_half, hd, interleaved);
    GI_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the row strides (%lld, %lld) must be multiples of 8 (16-byte rows for TMA)", K, lda, ldw);
    GI_REQUIRE((reinterpret_cast<uintptr_t>(A) % 16 == 0) && (reinterpret_cast<uintptr_t>(W) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(q_out) % 16 == 0) && (reinterpret_cast<uintptr_t>(k_cache) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(v_cache) % 16 == 0) &&
               (cos_t == nullptr || (reinterpret_cast<uintptr_t>(cos_t) % 16 == 0 && reinterpret_cast<uintptr_t>(sin_t) % 16 == 0)),
               "gemm_tc rope: operands must be 16-byte aligned");
    GI_REQUIRE(status != nullptr, "gemm_tc: a status word is required");
    const int N = (H + 2 * Hkv) * hd;
    TcPersistentParams p = {};
    p.rows_p = M; p.rows_q = N; p.K = K;
    p.tiles_p = pair ? (M + 2 * kBlockP - 1) / (2 * kBlockP) : (M + kBlockP - 1) / kBlockP;
    // 256 or 192 accumulator columns per tile: whichever needs fewer column-rounds of the GPU (rounds of
    // tiles over the SMs x tile width); with 3072 outputs and 2048 tokens 192 tiles of 256 are 2 rounds
    // of 256, 256 tiles of 192 are 2 rounds of 192
    const int workers = pair ? sm_count() / 2 : sm_count();
    auto rounds_cost = [&](int bq) {
        const long long tiles = static_cast<long long>(p.tiles_p) * ((N + bq - 1) / bq);
        return (tiles + workers - 1) / workers * bq;
    };
    const int block_q = (192 % hd == 0 && rounds_cost(192) < rounds_cost(256)) ? 192 : 256;
    p.tiles_q = (N + block_q - 1) / block_q;
    p.up_row_offset = 0;
    p.status = static_cast<int*>(status);
    p.splits = 1; p.kb_per_split = (K + kBlockK - 1) / kBlockK; p.split_rows = 0;
    p.rope = RopeStoreParams{positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved,
                             static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                             static_cast<__nv_bfloat16*>(v_cache), H, Hkv, hd, page_size, write_kv};
    CUtensorMap mp, mq;
    if (make_map(&mp, A, M, K, lda, kBlockP) || make_map(&mq, W, N, K, ldw, pair ? block_q / 2 : block_q)) return 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pair) {
        if (block_q == 192) return launch_persistent_pair<192, kEpiRopeStore>(mp, mq, mp /* no TMA store */, p, st);
        return launch_persistent_pair<256, kEpiRopeStore>(mp, mq, mp /* no TMA store */, p, st);
    }
    if (block_q == 192) return launch_persistent<192, kEpiRopeStore>(mp, mq, mp /* no TMA store */, p, st);
    return launch_persistent<256, kEpiRopeStore>(mp, mq, mp /* no TMA store */, p, st);
}

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_gemm_tc(const void* A, const void* W, void* C, int c_dtype, int accumulate, int M, int N, int K, long long lda, long long ldw, long long ldc, int swap, int block_q, int splits, void* workspace, long long workspace_floats, void* counters, int n_counters, void* status, const void* w_tiles, const void* ahead, long long ahead_bytes, void* stream) {
    return gi::dispatch(gi_gemm_tc_impl, A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, swap, block_q, splits, workspace, workspace_floats, counters, n_counters, status, w_tiles, ahead, ahead_bytes, stream);
}

extern "C" int gi_gemm_tc_rope(const void* A, const void* W, int M, int K, long long lda, long long ldw, int block_q, int splits, void* workspace, long long workspace_floats, void* counters, int n_counters, void* status, const void* w_tiles, const int* positions, const int* row_req, const int* block_tables, int table_stride, const float* cos_t, const float* sin_t, int rot_half, int interleaved, void* q_out, void* k_cache, void* v_cache, int H, int Hkv, int hd, int page_size, int write_kv, void* stream) {
    return gi::dispatch(gi_gemm_tc_rope_impl, A, W, M, K, lda, ldw, block_q, splits, workspace, workspace_floats, counters, n_counters, status, w_tiles, positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved, q_out, k_cache, v_cache, H, Hkv, hd, page_size, write_kv, stream);
}

extern "C" int gi_gemm_tc_persistent(const void* A, const void* W, void* C, int epilogue, int M, int N, int K, long long lda, long long ldw, long long ldc, int block_q, void* status, int splits, void* workspace, long long workspace_floats, int pair, void* stream) {
    return gi::dispatch(gi_gemm_tc_persistent_impl, A, W, C, epilogue, M, N, K, lda, ldw, ldc, block_q, status, splits, workspace, workspace_floats, pair, stream);
}

extern "C" int gi_gemm_tc_persistent_rope(const void* A, const void* W, int M, int K, long long lda, long long ldw, const int* positions, const int* row_req, const int* block_tables, int table_stride, const float* cos_t, const float* sin_t, int rot_half, int interleaved, void* q_out, void* k_cache, void* v_cache, int H, int Hkv, int hd, int page_size, int write_kv, void* status, int pair, void* stream) {
    return gi::dispatch(gi_gemm_tc_persistent_rope_impl, A, W, M, K, lda, ldw, positions, row_req, block_tables, table_stride, cos_t, sin_t, rot_half, interleaved, q_out, k_cache, v_cache, H, Hkv, hd, page_size, write_kv, status, pair, stream);
}
