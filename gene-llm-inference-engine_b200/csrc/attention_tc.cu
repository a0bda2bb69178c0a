// Prefill attention on the 5th-generation tensor cores (tcgen05), bfloat16, head sizes 64 and 128.
//
// One CTA takes 128 query rows (tokens x the query heads of one key/value group) and walks the keys
// in tiles of KEYS (128 at head size 64, 64 at head size 128) over the request's pages:
//   warp 0      TMA producer: one box per page and head, each lane requesting its own box; keys and
//               values have two-place rings and barriers of their own (a key tile is free once its S
//               product is done, a value tile only after P V), and keys run one tile ahead of values;
//   warp 1      allocates tensor memory and issues the MMAs: S = Q K^T (both operands K-major in
//               shared memory, S in tensor memory) and O += P V (P from shared memory, V as an
//               MN-major operand straight from the page layout [keys, head_dim]); S of the next tile
//               is issued as soon as the softmax warps have the current scores in registers, before
//               P V of the current tile;
//   warps 2..5  softmax: thread r owns row r of the tile, which is lane r of tensor memory, so row
//               maximum and row sum need no exchange between threads. They read S with tcgen05.ld,
//               scale O by the correction factor in tensor memory, write P = exp2(S - m) as bfloat16
//               into a swizzled K-major tile for the second MMA, and at the end normalise O.
// Scores, maxima, sums and the output accumulator are 32-bit; P is rounded to bfloat16 as the
// operand of P V. Two CTAs fit on an SM (at head size 128 thanks to the shorter key tiles), so one
// CTA's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded; on expiry a code goes to the status word and the CTA winds down.
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"

namespace gi {

namespace atc {

constexpr int kRows = 128;        // query rows per CTA
constexpr int kThreads = 192;
constexpr int kStages = 2;
constexpr unsigned long long kWaitCycles = 4000000000ull;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// try_wait with a suspend-time hint: the thread may sleep in hardware up to about that many
// nanoseconds instead of burning issue slots that the other CTA on the SM could use.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two 32-bit floats in one 64-bit register: sm_100 multiplies and adds them with one instruction, and takes the
// maximum of three values with one. The pass over a tile's scores needs 3 instructions a score with them where it
// needed 4.5 (8,192 tokens at head size 64: 486 -> 456 us).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
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
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// MN-major operand (the contraction index runs over rows of 128 bytes, 64 elements of the other
// index are contiguous in a row), 128-byte swizzle: groups of 8 rows 1024 bytes apart (stride
// offset); the leading offset (distance between 64-element blocks of the other index) is unused
// because each MMA here covers exactly one such block.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// The same with several 64-element blocks of the contiguous index in one MMA: the leading offset is
// the distance between them.
__device__ __forceinline__ uint64_t desc_mn_major_blocks(uint32_t addr, uint32_t block_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((block_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

template <int HD, int KEYS>
struct Cfg {
    static constexpr int kBlocks = HD / 64;                        // 64-wide blocks of the head dimension
    static constexpr int kQBytes = kRows * HD * 2;
    static constexpr int kTileBytes = KEYS * HD * 2;               // one K or V tile
    static constexpr int kPBytes = kRows * KEYS * 2;
    static constexpr int kSmemBytes = kQBytes + kStages * 2 * kTileBytes + kPBytes + 256;   // two CTAs fit in an SM's 228 KB
    static constexpr int kTmemCols = (KEYS + HD <= 128) ? 128 : 256;     // S: KEYS columns, O: HD columns (a power of two)
    // D f32, A and B bf16, M = 128
    static constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(KEYS >> 3) << 17) | (8u << 24);
    static constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* B is MN-major */ |
                                         (static_cast<uint32_t>(HD >> 3) << 17) | (8u << 24);
};

template <int HD, int KEYS>
__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ work, const int* __restrict__ positions,
                            const int* __restrict__ block_tables, int table_stride, int H, int Hkv, int page_size,
                            float scale_log2, int window, int* status) {
    using C = Cfg<HD, KEYS>;
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {                                  // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicCAS(status, 0, 12);
        return;
    }
    uint8_t* q_smem = smem;
    uint8_t* kv_smem = q_smem + C::kQBytes;                        // stage s: K at s * 2 * tile, V after it
    uint8_t* p_smem = kv_smem + kStages * 2 * C::kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + C::kPBytes);
    // Keys and values have rings and barriers of their own: a key tile is free again when its S product is
    // done (early in the tile's softmax), a value tile only after P V, so the keys of tile i + 1 are
    // requested more than a tile's time before their product is issued.
    constexpr int kKFull = 0, kVFull = 2, kKEmpty = 4, kVEmpty = 6, kSFull = 8, kPFull = 9, kODone = 10, kSRead = 11;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = H / Hkv;
    const int g = blockIdx.x;          // heads vary fastest: the longest work items of every head start first

    if (threadIdx.x == 0) {
        for (int b = 0; b < 8; ++b) mbar_init(smem_u32(&bars[b]), 1);
        mbar_init(smem_u32(&bars[kSFull]), 1);
        mbar_init(smem_u32(&bars[kPFull]), 128);
        mbar_init(smem_u32(&bars[kODone]), 1);
        mbar_init(smem_u32(&bars[kSRead]), 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + KEYS;
    if (threadIdx.x == 0) timeline_record(kTlAttentionPrefill, 0);
    pdl_prologue();
    if (threadIdx.x == 0) timeline_record(kTlAttentionPrefill, 1);

    const int t0 = work[blockIdx.y * 3], n_tok = work[blockIdx.y * 3 + 1], req = work[blockIdx.y * 3 + 2];
    const int n_rows = n_tok * G;
    const int pos_first = positions[t0], pos_last = pos_first + n_tok - 1;
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int lo_last = (window > 0 && pos_last - window + 1 > 0) ? pos_last - window + 1 : 0;
    const int first_tile = lo_first / KEYS, last_tile = pos_last / KEYS;
    const int n_tiles = last_tile - first_tile + 1;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        // The whole warp looks up the tile's pages (lane b: box b), one round trip to the block table
        // per tile, started before the wait for the free stage, and each lane requests its own box: one
        // thread issuing all of a tile's copies in turn was late for the MMAs.
        const int* table = block_tables + static_cast<size_t>(req) * table_stride;
        const int box_rows = page_size < KEYS ? page_size : KEYS;
        const int boxes = KEYS / box_rows;                       // at most 16 (pages of 8)
        // one tile of keys or of values: false when a wait gave up
        auto load_tile = [&](int i, bool values) -> bool {
            const int s = i % kStages;
            const int key0 = (first_tile + i) * KEYS;
            const int kb_lane = key0 + lane * box_rows;
            const bool lane_valid = lane < boxes && kb_lane <= pos_last && kb_lane + box_rows - 1 >= lo_first;
            const int page_lane = lane_valid ? table[kb_lane / page_size] : 0;
            const unsigned valid_mask = __ballot_sync(0xffffffffu, lane_valid);
            bool ok = true;
            if (lane == 0 && i >= kStages &&
                !mbar_wait(smem_u32(&bars[(values ? kVEmpty : kKEmpty) + s]), ((i / kStages) - 1) & 1, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, 8); }
                ok = false;
            }
            if (!__shfl_sync(0xffffffffu, ok ? 1 : 0, 0)) return false;
            const uint32_t tile = smem_u32(kv_smem + s * 2 * C::kTileBytes) + (values ? C::kTileBytes : 0);
            const uint32_t bar = smem_u32(&bars[(values ? kVFull : kKFull) + s]);
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(bar, static_cast<uint32_t>(__popc(valid_mask)) * box_rows * HD * 2u);
            }
            __syncwarp();                                         // the expected bytes are set before any copy can complete
            if (lane_valid) {                                     // every lane requests its own box
                const int row = (page_lane * Hkv + g) * page_size + kb_lane % page_size;
#pragma unroll
                for (int h = 0; h < C::kBlocks; ++h) {
                    const uint32_t off = static_cast<uint32_t>(h * (KEYS * 128) + lane * box_rows * 128);
                    tma_load_2d(tile + off, values ? &map_v : &map_k, h * 64, row, bar);
                }
            }
            return true;
        };
        // keys run one tile ahead of values: K(0); K(1), V(0); K(2), V(1); ... in the order in which
        // their places become free (K(i) after S(i - 2), V(i - 1) after P V(i - 3))
        for (int n = 0; n <= n_tiles; ++n) {
            if (n < n_tiles && !load_tile(n, false)) break;
            if (n >= 1 && !load_tile(n - 1, true)) break;
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // Q is written by the softmax warps; their first arrival on "p full" (phase 0) also says Q is ready
            bool ok = mbar_wait(smem_u32(&bars[kPFull]), 0, abort_flag);
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, 9); }
            // S(i + 1) goes to the tensor cores as soon as the softmax warps have read S(i) into registers
            // ("s read": three quarters into their pass over the tile), well before P(i) is full and
            // P(i) V(i) can be issued: the softmax warps find the next scores ready when they finish a tile.
            auto issue_s = [&](int i) -> bool {
                const int s = i % kStages;
                if (!mbar_wait(smem_u32(&bars[kKFull + s]), (i / kStages) & 1, abort_flag)) return false;
                tc_fence_after();
                const uint32_t k_tile = smem_u32(kv_smem + s * 2 * C::kTileBytes);
#pragma unroll
                for (int kb = 0; kb < C::kBlocks; ++kb) {
                    const uint64_t dq = desc_k_major(smem_u32(q_smem) + kb * (kRows * 128));
                    const uint64_t dk = desc_k_major(k_tile + kb * (KEYS * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k) umma(tmem_s, dq + 2 * k, dk + 2 * k, C::kIdescS, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(&bars[kSFull]));
                umma_commit(smem_u32(&bars[kKEmpty + s]));     // the key tile may be refilled
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int i = 0; i < n_tiles && ok; ++i) {
                const int s = i % kStages;
                if (i + 1 < n_tiles) {
                    if (!mbar_wait(smem_u32(&bars[kSRead]), i & 1, abort_flag)) { ok = false; break; }
                    if (!issue_s(i + 1)) { ok = false; break; }
                }
                // wait for P(i) (and the rescaled O) and for the values
                if (!mbar_wait(smem_u32(&bars[kPFull]), (i + 1) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(smem_u32(&bars[kVFull + s]), (i / kStages) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_tile = smem_u32(kv_smem + s * 2 * C::kTileBytes) + C::kTileBytes;
#pragma unroll
                for (int kb = 0; kb < KEYS / 64; ++kb) {
                    const uint64_t dp = desc_k_major(smem_u32(p_smem) + kb * (kRows * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int kk = kb * 4 + k;                                  // 16 keys per step
                        // all HD columns of O in one MMA: the 64-wide blocks of V lie KEYS * 128 bytes apart
                        const uint64_t dv = desc_mn_major_blocks(v_tile + kk * (16 * 128), KEYS * 128);
                        umma(tmem_o, dp + 2 * k, dv, C::kIdescPV, (i > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(&bars[kVEmpty + s]));  // the value tile may be refilled
                umma_commit(smem_u32(&bars[kODone]));       // O holds the sum up to this tile; P may be overwritten
            }
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(status, 0, 10); }
        }
    } else {
        // ---------------------------------------------------------------- softmax (warps 2..5)
        const int lane_group = warp & 3;
        const int r = lane_group * 32 + lane;                    // row of the tile = lane of tensor memory
        const uint32_t lane_addr = static_cast<uint32_t>(lane_group * 32) << 16;
        const bool row_valid = r < n_rows;
        const int tok = r / G, hh = r - tok * G;
        const int row_pos = row_valid ? pos_first + tok : -1;
        const int row_lo = (window > 0 && row_pos - window + 1 > 0) ? row_pos - window + 1 : 0;
        // the query tile: K-major blocks [128 rows][64] with the 128-byte swizzle
        {
            const __nv_bfloat16* src = q + (static_cast<size_t>(t0 + tok) * H + g * G + hh) * HD;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row_valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
                *reinterpret_cast<uint4*>(q_smem + (c >> 3) * (kRows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&bars[kPFull]));                 // phase 0 of "p full": Q is in place
        }
        // Online softmax with a lazily updated reference: weights are exp2(s - m_ref) where m_ref is
        // the row's reference maximum (scaled log2 domain). As long as no score of a new tile exceeds
        // m_ref by more than 8 (weights stay below 256), m_ref is kept, the tile needs one pass over S
        // and O needs no rescaling; otherwise (decided per warp, the tensor-memory accesses being
        // warp-wide) the reference moves to the new maximum, O and the sum are scaled by
        // exp2(old - new) and the tile is done again. The final division by the sum makes the result
        // independent of which references were used.
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        auto tile_pass = [&](int key0, auto edge_tag, float m_use, float& mx, float& sum, int p_free_parity, bool last_pass) {
            // one pass over the tile's scores: running maximum of the raw scores, weights, their sum,
            // and the weights as bfloat16 into the K-major P tile; loads of the next 32 columns are
            // in flight while the current ones are processed. The masking of tiles that some row
            // does not see whole is compiled into a pass of its own.
            constexpr bool kEdge = decltype(edge_tag)::value;
            const uint64_t scale2 = pack2(scale_log2, scale_log2), neg_m2 = pack2(-m_use, -m_use);
            uint64_t sum2 = pack2(0.f, 0.f);
            uint32_t buf[2][32];
            tmem_ld32(tmem_s + lane_addr, buf[0]);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < KEYS / 32; ++c) {
                if (c + 1 < KEYS / 32) tmem_ld32(tmem_s + lane_addr + (c + 1) * 32, buf[(c + 1) & 1]);
                const uint32_t* sv = buf[c & 1];
                if (c + 1 == KEYS / 32) {
                    // All scores of the tile are in registers. If this pass is the tile's last one (the
                    // reference maximum stays: known once the last 32 scores are looked at, before their
                    // weights are made), the tensor cores may write the next tile's scores over them.
                    if (!last_pass) {
                        float mx_all = mx;
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float v0 = __uint_as_float(sv[j]), v1 = __uint_as_float(sv[j + 1]);
                            if (kEdge) {
                                const int key = key0 + c * 32 + j;
                                if (!(key >= row_lo && key <= row_pos)) v0 = -INFINITY;
                                if (!(key + 1 >= row_lo && key + 1 <= row_pos)) v1 = -INFINITY;
                            }
                            mx_all = max3(mx_all, v0, v1);
                        }
                        last_pass = !__any_sync(0xffffffffu, mx_all * scale_log2 > m_ref + 8.0f);
                    }
                    if (last_pass) {
                        tc_fence_before();
                        mbar_arrive(smem_u32(&bars[kSRead]));
                    }
                }
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float v0 = __uint_as_float(sv[j]), v1 = __uint_as_float(sv[j + 1]);
                    if (kEdge) {
                        const int key = key0 + c * 32 + j;
                        if (!(key >= row_lo && key <= row_pos)) v0 = -INFINITY;
                        if (!(key + 1 >= row_lo && key + 1 <= row_pos)) v1 = -INFINITY;
                    }
                    mx = max3(mx, v0, v1);
                    const uint64_t x2 = fma2(pack2(v0, v1), scale2, neg_m2);
                    float x0, x1;
                    unpack2(x2, x0, x1);
                    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                    sum2 = add2(sum2, pack2(p0, p1));
                    __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                    packed[j >> 1] = *reinterpret_cast<uint32_t*>(&pb);
                }
                if (c == 0 && p_free_parity >= 0) {
                    // P of the tile before is still being read by its MMAs (they were issued after this
                    // tile's S): the first store waits for them; O may be touched from here on, too
                    if (!mbar_wait(smem_u32(&bars[kODone]), static_cast<uint32_t>(p_free_parity), abort_flag)) ok = false;
                    tc_fence_after();
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c & 1) * 4 + q4;                 // 16-byte chunk inside the 64-key block c / 2
                    *reinterpret_cast<uint4*>(p_smem + (c >> 1) * (kRows * 128) + r * 128 + ((chunk ^ (r & 7)) << 4)) =
                        make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
                }
                if (c + 1 < KEYS / 32) tmem_ld_wait();
            }
            float s0, s1;
            unpack2(sum2, s0, s1);
            sum += s0 + s1;
        };
        auto tile_pass_any = [&](int key0, bool edge, float m_use, float& mx, float& sum, int p_free_parity, bool last_pass) {
            if (edge) tile_pass(key0, std::true_type{}, m_use, mx, sum, p_free_parity, last_pass);
            else tile_pass(key0, std::false_type{}, m_use, mx, sum, p_free_parity, last_pass);
        };
        for (int i = 0; i < n_tiles; ++i) {
            const int key0 = (first_tile + i) * KEYS;
            if (!mbar_wait(smem_u32(&bars[kSFull]), i & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const bool edge = key0 < lo_last || key0 + KEYS - 1 > pos_first;      // some row masks some key of this tile
            float mx = -INFINITY, sum = 0.f;
            tile_pass_any(key0, edge, (m_ref == -INFINITY) ? 0.f : m_ref, mx, sum, i > 0 ? ((i - 1) & 1) : -1, false);
            if (!ok) break;
            const float m_tile = mx * scale_log2;
            const bool move = m_tile > m_ref + 8.0f;                     // also true for the first visible key (m_ref = -inf)
            if (__any_sync(0xffffffffu, move)) {
                const float m_new = fmaxf(m_ref, m_tile);
                const float corr = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
                if (i > 0) {
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t ov[32];
                        tmem_ld32(tmem_o + lane_addr + c * 32, ov);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * corr);
                        tmem_st32(tmem_o + lane_addr + c * 32, ov);
                    }
                    tmem_st_wait();
                }
                l *= corr;
                m_ref = m_new;
                mx = -INFINITY;
                sum = 0.f;
                tile_pass_any(key0, edge, (m_ref == -INFINITY) ? 0.f : m_ref, mx, sum, -1, true);
            }
            l += sum;
            if (key0 < lo_first || key0 + KEYS - 1 > pos_last) {
                // value rows outside every query's range were not fetched or never written; they meet
                // weights of exactly 0 in the MMA and must be finite: row r of the tile is this thread's
                // (after the tile has arrived: the copy must not land on top of the zeros)
                if (!mbar_wait(smem_u32(&bars[kVFull + i % kStages]), (i / kStages) & 1, abort_flag)) { ok = false; break; }
                const int key = key0 + r;
                if (r < KEYS && (key < lo_first || key > pos_last)) {
                    uint8_t* v_tile = kv_smem + (i % kStages) * 2 * C::kTileBytes + C::kTileBytes;
#pragma unroll
                    for (int c = 0; c < HD / 8; ++c)
                        *reinterpret_cast<uint4*>(v_tile + (c >> 3) * (KEYS * 128) + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(smem_u32(&bars[kPFull]));
        }
        if (ok && mbar_wait(smem_u32(&bars[kODone]), (n_tiles - 1) & 1, abort_flag)) {
            tc_fence_after();
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = out + (static_cast<size_t>(t0 + tok) * H + g * G + hh) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t ov[32];
                tmem_ld32(tmem_o + lane_addr + c * 32, ov);
                tmem_ld_wait();
                if (row_valid) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(ov[q4 * 8 + 2 * e]) * inv,
                                                                     __uint_as_float(ov[q4 * 8 + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        } else if (!*abort_flag) {
            *abort_flag = 1;
            atomicCAS(status, 0, 11);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
        if (lane == 0) timeline_record(kTlAttentionPrefill, 6);
    }
}

template <int HD, int KEYS>
static int launch(const void* q, const void* kc, const void* vc, void* out, const int* work, int n_work,
                  const int* positions, const int* tables, int table_stride, int H, int Hkv, int page_size, float scale,
                  int window, long long n_pages, int* status, cudaStream_t st) {
    using C = Cfg<HD, KEYS>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, KEYS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) { set_error("attention_prefill_tc: %s", cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    const int box_rows = page_size < KEYS ? page_size : KEYS;
    CUtensorMap mk, mv;
    const unsigned long long rows_total = static_cast<unsigned long long>(n_pages) * Hkv * page_size;
    if (make_tensor_map_2d(&mk, kc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, HD, HD, box_rows, 64,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "attention_prefill_tc")) return 1;
    if (make_tensor_map_2d(&mv, vc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, HD, HD, box_rows, 64,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "attention_prefill_tc")) return 1;
    dim3 grid(Hkv, n_work);
    launch_kernel((attention_prefill_tc_kernel<HD, KEYS>), dim3(grid), dim3(kThreads), C::kSmemBytes, st, mk, mv,
                  static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), work, positions, tables,
                  table_stride, H, Hkv, page_size, scale * kLog2e, window, status);
    return check_launch("attention_prefill_tc");
}

}  // namespace atc
}  // namespace gi

using namespace gi;
GI_TIMELINE_SETTER(gi_timeline_set_attention_tc)

// Whether the tcgen05 prefill kernel serves this shape: head size 64 or 128, at most 128 query
// heads per key/value head, pages that TMA boxes can tile.
extern "C" int gi_attention_prefill_tc_supported(int hd, int H, int Hkv, int page_size) {
    return (hd == 64 || hd == 128) && Hkv > 0 && H % Hkv == 0 && H / Hkv <= 128 && page_size % 8 == 0 &&
           (128 % page_size == 0 || page_size % 128 == 0);
}

// Prompt portions: work[3*i..] = (first step row of the tile, tokens in the tile (at most
// 128 / group size), request index).
static int gi_attention_prefill_tc_impl(const void* q, const void* k_cache, const void* v_cache, void* out, const int* work,
                                       int n_work, const int* positions, const int* block_tables, int table_stride, int H,
                                       int Hkv, int hd, int page_size, float scale, int window, long long n_pages,
                                       void* status, void* stream) {
    if (n_work == 0) return 0;
    GI_REQUIRE(gi_attention_prefill_tc_supported(hd, H, Hkv, page_size), "attention_prefill_tc: shape not supported");
    GI_REQUIRE(status != nullptr, "attention_prefill_tc: a status word is required");
    GI_REQUIRE(n_work <= 65535, "attention_prefill_tc: %d work items exceed the grid limit 65535", n_work);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define GI_ATC_LAUNCH(HD_, KEYS_)                                                                                          \
    atc::launch<HD_, KEYS_>(q, k_cache, v_cache, out, work, n_work, positions, block_tables, table_stride, H, Hkv, page_size, \
                            scale, window, n_pages, static_cast<int*>(status), st)
    // Keys per tile: 128 at head size 64; 64 at head size 128, where a CTA with 128-key tiles needs 192 KB of shared memory
    // and has an SM to itself, while two CTAs with 64-key tiles (112 KB each) overlap one's softmax with the other's
    // MMAs as at head size 64: 642 against 511 TFLOP/s at 8,192 tokens, 374 against 338 at 2,048 (24:8 heads).
    // (64-key tiles at head size 64, three CTAs to an SM: slower, 531 against 558 TFLOP/s.)
    if (hd == 64) return GI_ATC_LAUNCH(64, 128);
    return GI_ATC_LAUNCH(128, 64);
#undef GI_ATC_LAUNCH
}

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* work, int n_work, const int* positions, const int* block_tables, int table_stride, int H, int Hkv, int hd, int page_size, float scale, int window, long long n_pages, void* status, void* stream) {
    return gi::dispatch(gi_attention_prefill_tc_impl, q, k_cache, v_cache, out, work, n_work, positions, block_tables, table_stride, H, Hkv, hd, page_size, scale, window, n_pages, status, stream);
}
