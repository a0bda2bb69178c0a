// Paged causal attention in bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit accumulators
// and 32-bit online softmax). The kernels share their warp-level code (warp_tile_step):
//
//   attention_decode_tma   single decoded tokens deep in a context (the kernel decoding uses). The
//                          context is cut into chunks of kChunkKeys positions, a fixed length, so that
//                          a row's arithmetic does not depend on the batch; an item is one chunk of one
//                          (token, key/value head), with the query heads that share the key/value head
//                          packed as rows of the 16-row tile. One persistent CTA per SM; each of its
//                          warps walks its own items with its own ring of 32-key tiles that TMA fills
//                          (a box per page and head, each lane requesting its own). Partial (max, sum,
//                          output) per chunk go to a workspace and attention_combine merges them in
//                          chunk order.
//   attention_decode       the same for page sizes that TMA boxes cannot tile: one CTA per chunk, four
//                          warps a quarter each, cp.async.
//   attention_prefill_tma  portions of prompts at head sizes the tcgen05 kernel (attention_tc.cu) is
//                          not built for: 128 query rows = (tokens x heads of one key/value group) per
//                          CTA, eight consumer warps of 16 rows and a TMA producer warp, 64-key tiles.
//   attention_prefill      the same with 64 rows, four warps and cp.async, for other page sizes.
//
// Keys and values come from pages [pages, Hkv, page_size, head_dim] through the request's block
// table. Rows of a tile that lie outside every query's range are zero-filled (on load, or in shared
// memory after a TMA box brought a whole page), so stale or unwritten page contents (tests fill
// them with NaN) can never reach a result.
// Head sizes 16, 32, 64 and 128 are built; other sizes use the general kernel.
#include "common.cuh"
#include "tma.cuh"

namespace gi {

constexpr int kAttThreads = 128;
constexpr int kTileKeys = 64;
constexpr int kChunkKeys = 256;          // decode: keys per item
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;       // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Tiles are stored as rows of HD bfloat16 with their 16-byte chunks permuted so that the eight
// rows an ldmatrix reads fall into eight different bank groups.
template <int HD>
__device__ __forceinline__ int swizzled_chunk(int row, int chunk) {
    constexpr int cpr = HD / 8;                       // 16-byte chunks per row
    if (cpr >= 8) return chunk ^ (row & 7);
    if (cpr == 4) return chunk ^ ((row >> 1) & 3);
    return chunk ^ ((row >> 2) & 1);                  // cpr == 2
}
template <int HD>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + static_cast<uint32_t>((row * (HD / 8) + swizzled_chunk<HD>(row, chunk)) * 16);
}

// Tiles written by TMA: the same permutation for head sizes up to 64 (TMA's 128/64/32-byte
// swizzles are exactly the ones above); a head size of 128 is stored as two half tiles of
// [TILE][64], because a swizzled TMA box is at most 128 bytes wide.
template <int HD, int TILE, bool TMA>
__device__ __forceinline__ uint32_t kv_addr(uint32_t base, int row, int chunk) {
    if (TMA && HD == 128)
        return base + static_cast<uint32_t>((chunk >> 3) * (TILE * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
    return tile_addr<HD>(base, row, chunk);
}

// Loads keys [key0, key0 + n_rows) of one key/value head into a tile; rows outside [lo, hi] (the
// union of what the tile's queries may read) are zero-filled and their pages are not touched.
template <int HD>
__device__ __forceinline__ void load_tile_async(uint32_t tile, const __nv_bfloat16* __restrict__ cache,
                                                const int* __restrict__ table, int g, int Hkv, int page_size,
                                                int key0, int n_rows, int lo, int hi, int tid, int n_threads) {
    constexpr int cpr = HD / 8;
    for (int i = tid; i < n_rows * cpr; i += n_threads) {
        const int row = i / cpr, chunk = i % cpr;
        const int key = key0 + row;
        const bool valid = key >= lo && key <= hi;
        const __nv_bfloat16* src = cache;
        if (valid) {
            const int page = table[key / page_size];
            src = cache + ((static_cast<size_t>(page) * Hkv + g) * page_size + (key % page_size)) * HD + chunk * 8;
        }
        cp_async16(tile_addr<HD>(tile, row, chunk), src, valid);
    }
}

// Byte offsets of this lane's ldmatrix rows inside a tile, for every k-step of Q K^T and every
// n-tile of P V. The swizzle depends only on the low bits of the row, which the 8- and 16-row
// strides of the loops below leave alone, so the offsets are computed once per kernel.
template <int HD, int TILE, bool TMA>
struct LaneOffsets {
    static constexpr uint32_t kRowStride = (TMA && HD == 128) ? 128 : HD * 2;
    uint32_t k[HD / 16];
    uint32_t v[HD / 8];
    __device__ __forceinline__ void init(int lane) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) k[kk] = kv_addr<HD, TILE, TMA>(0, lane & 7, kk * 2 + ((lane >> 3) & 1));
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) v[n] = kv_addr<HD, TILE, TMA>(0, (lane & 7) + ((lane >> 3) & 1) * 8, n);
    }
};

// One warp: S = Q K^T for 16 query rows x TILE keys, online softmax update, O += P V.
// q_frag: A fragments of the 16 x HD query tile. Row limits (lo, pos) are those of the two rows
// this lane holds (lane/4 and lane/4 + 8) and are applied only when kMasked (a tile at the edge
// of some row's range). o: HD/8 n-tiles x 4 accumulators. m (in the scaled log2 domain), l: per row.
template <int HD, int TILE, bool TMA, bool kMasked, bool kUpper = true>
__device__ __forceinline__ void warp_tile_step(const uint32_t (*q_frag)[4], uint32_t k_tile, uint32_t v_tile, int key0,
                                               const int* row_lo, const int* row_pos, float scale_log2,
                                               float (*o)[4], float* m, float* l, int lane,
                                               const LaneOffsets<HD, TILE, TMA>& off) {
    // kUpper false: rows 8..15 of the tile are padding (a decode tile holds at most 8 query heads);
    // their softmax and rescaling are skipped and their weights enter P V as zeros.
    constexpr int kK = HD / 16;                 // k-steps of Q K^T
    constexpr int kN = TILE / 8;                // n-tiles of S
    constexpr int kR = kUpper ? 2 : 1;          // row halves this lane works on
    constexpr uint32_t RS = LaneOffsets<HD, TILE, TMA>::kRowStride;
    float s[kN][4];
#pragma unroll
    for (int j = 0; j < kN; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int j = 0; j < kN; ++j) {
#pragma unroll
        for (int kk = 0; kk < kK; ++kk) {
            uint32_t b0, b1;
            // B fragment of K^T: keys j*8 + lane%8 (rows), head dims kk*16 + {0, 8} (two 8x8 matrices)
            ldmatrix_x2(k_tile + j * 8 * RS + off.k[kk], b0, b1);
            mma_bf16(s[j], q_frag[kk], b0, b1);
        }
    }
    // mask (edge tiles only) and row maxima of the raw scores
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kN; ++j) {
#pragma unroll
        for (int e = 0; e < 2 * kR; ++e) {
            const int r = e >> 1;
            if (kMasked) {
                const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                if (!(key >= row_lo[r] && key <= row_pos[r])) s[j][e] = -INFINITY;
            }
            mx[r] = fmaxf(mx[r], s[j][e]);
        }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < kR; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r] * scale_log2);            // scale > 0: the maximum commutes with it
        corr[r] = (m[r] == -INFINITY) ? 0.f : exp2f(m[r] - m_new);
        m[r] = m_new;
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;                   // a row that has seen no key yet: all weights 0
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < kN; ++j) {
#pragma unroll
        for (int e = 0; e < 2 * kR; ++e) {
            const int r = e >> 1;
            const float p = exp2f(fmaf(s[j][e], scale_log2, -m_use[r]));  // masked scores (-inf) give 0
            s[j][e] = p;
            sum[r] += p;
        }
    }
#pragma unroll
    for (int r = 0; r < kR; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l[r] = l[r] * corr[r] + sum[r];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        if (kUpper) { o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
    }
    // O += P V: P as A fragments (16 keys per k-step), V^T through transposed ldmatrix
#pragma unroll
    for (int t = 0; t < TILE / 16; ++t) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * t][0], s[2 * t][1]);
        a[1] = kUpper ? pack_bf16(s[2 * t][2], s[2 * t][3]) : 0u;
        a[2] = pack_bf16(s[2 * t + 1][0], s[2 * t + 1][1]);
        a[3] = kUpper ? pack_bf16(s[2 * t + 1][2], s[2 * t + 1][3]) : 0u;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            uint32_t b0, b1;
            // keys t*16 + {0..7, 8..15} (rows of V), head dims n*8..n*8+7, transposed on load
            ldmatrix_x2_trans(v_tile + t * 16 * RS + off.v[n], b0, b1);
            mma_bf16(o[n], a, b0, b1);
        }
    }
}

// Loads the A fragments of a 16-row query tile stored (swizzled) in shared memory.
template <int HD>
__device__ __forceinline__ void load_q_frags(uint32_t q_tile, int row0, uint32_t (*q_frag)[4], int lane) {
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = row0 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(tile_addr<HD>(q_tile, row, kk * 2 + (lane >> 4)), q_frag[kk][0], q_frag[kk][1], q_frag[kk][2], q_frag[kk][3]);
    }
}

// ------------------------------------------------------------------------------------------ decode
// grid (chunks, Hkv, decode requests). rows: one per query head of the group (G <= 16).
// part_o [row_index][H][chunks][HD], part_ml [row_index][H][chunks][2] with row_index = blockIdx.z.
template <int HD>
__global__ void __launch_bounds__(kAttThreads)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ rows,
                        const int* __restrict__ row_req, const int* __restrict__ positions,
                        const int* __restrict__ block_tables, int table_stride, int H, int Hkv, int page_size,
                        float scale_log2, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int max_chunks) {
    pdl_prologue();
    extern __shared__ __align__(128) uint8_t smem[];
    const int G = H / Hkv;
    const int chunk = blockIdx.x, g = blockIdx.y, idx = blockIdx.z;
    const int t = rows[idx];
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int c0 = chunk * kChunkKeys;
    float* my_o = part_o + ((static_cast<size_t>(idx) * H + g * G) * max_chunks + chunk) * HD;
    float* my_ml = part_ml + ((static_cast<size_t>(idx) * H + g * G) * max_chunks + chunk) * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (c0 > pos || c0 + kChunkKeys <= lo) {
        // nothing of this chunk is visible: an empty partial (m = -inf, l = 0)
        if (threadIdx.x < G) {
            my_ml[static_cast<size_t>(threadIdx.x) * max_chunks * 2] = -INFINITY;
            my_ml[static_cast<size_t>(threadIdx.x) * max_chunks * 2 + 1] = 0.f;
        }
        return;
    }
    const int* table = block_tables + static_cast<size_t>(row_req[t]) * table_stride;

    // shared memory: Q tile [16][HD], then per warp a K tile and a V tile [64][HD]
    constexpr int kTileBytes = kTileKeys * HD * 2;
    const uint32_t q_tile = smem_addr(smem);
    const uint32_t k_tile = q_tile + 16 * HD * 2 + warp * 2 * kTileBytes;
    const uint32_t v_tile = k_tile + kTileBytes;
    const int key0 = c0 + warp * kTileKeys;

    // every warp loads its own keys and values; all warps share the query tile
    load_tile_async<HD>(k_tile, k_cache, table, g, Hkv, page_size, key0, kTileKeys, lo, pos, lane, 32);
    load_tile_async<HD>(v_tile, v_cache, table, g, Hkv, page_size, key0, kTileKeys, lo, pos, lane, 32);
    cp_async_commit();
    {
        constexpr int cpr = HD / 8;
        const uint4* src = reinterpret_cast<const uint4*>(q + (static_cast<size_t>(t) * H + g * G) * HD);
        for (int i = threadIdx.x; i < 16 * cpr; i += kAttThreads) {
            const int row = i / cpr, c = i % cpr;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < G) v = src[row * cpr + c];
            *reinterpret_cast<uint4*>(smem + (row * cpr + swizzled_chunk<HD>(row, c)) * 16) = v;
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    uint32_t q_frag[HD / 16][4];
    load_q_frags<HD>(q_tile, 0, q_frag, lane);
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int r0 = lane >> 2;
    int row_lo[2], row_pos[2];
    row_lo[0] = lo; row_pos[0] = (r0 < G) ? pos : -1;            // rows beyond the group see nothing
    row_lo[1] = lo; row_pos[1] = (r0 + 8 < G) ? pos : -1;
    LaneOffsets<HD, kTileKeys, false> off;
    off.init(lane);
    if (key0 <= pos && key0 + kTileKeys > lo)
        warp_tile_step<HD, kTileKeys, false, true>(q_frag, k_tile, v_tile, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
    __syncthreads();                                               // tiles are read; reuse the memory

    // merge the four warps in warp order through shared memory: [warp][16 rows][HD + 2]
    float* red = reinterpret_cast<float*>(smem);
    constexpr int kRow = HD + 2;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const int d = n * 8 + (lane & 3) * 2;
        float* a = red + (warp * 16 + r0) * kRow + d;
        float* b = red + (warp * 16 + r0 + 8) * kRow + d;
        a[0] = o[n][0]; a[1] = o[n][1]; b[0] = o[n][2]; b[1] = o[n][3];
    }
    if ((lane & 3) == 0) {
        red[(warp * 16 + r0) * kRow + HD] = m[0];
        red[(warp * 16 + r0) * kRow + HD + 1] = l[0];
        red[(warp * 16 + r0 + 8) * kRow + HD] = m[1];
        red[(warp * 16 + r0 + 8) * kRow + HD + 1] = l[1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD; i += kAttThreads) {
        const int row = i / HD, d = i % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, red[(w * 16 + row) * kRow + HD]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = red[(w * 16 + row) * kRow + HD];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            acc += red[(w * 16 + row) * kRow + d] * f;
            L += red[(w * 16 + row) * kRow + HD + 1] * f;
        }
        my_o[static_cast<size_t>(row) * max_chunks * HD + d] = acc;
        if (d == 0) {
            my_ml[static_cast<size_t>(row) * max_chunks * 2] = M;
            my_ml[static_cast<size_t>(row) * max_chunks * 2 + 1] = L;
        }
    }
}

// ------------------------------------------------------------------------------------------ decode, fed by TMA
// The same arithmetic as attention_decode_kernel per 256-key chunk, organised for bandwidth: one
// persistent CTA per SM, whose four warps are independent. A warp takes whole chunks (work item =
// request x key/value head x chunk, dealt round-robin), walks a chunk's tiles in order with the
// online softmax, and writes the chunk's partial result itself, so no warp ever waits for another.
// Each warp owns a ring of three stages (K tile + V tile) filled by TMA: one lane issues one box
// per page and head (pages [pages, Hkv, page_size, hd] are rows of a 2D tensor map), running up to
// three tiles ahead, across chunk borders. Pages wholly outside a query's range are not fetched.
template <int HD>
struct DecodeTma {
    // Eight warps with 32-key tiles where the head size allows it (two warps per scheduler hide each
    // other's fixed latencies); a head size of 128 keeps four warps for its 16 KB stages.
    static constexpr int kWarps = HD <= 64 ? 8 : 4;
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kTile = 32;
    static constexpr int kTilesPerChunk = kChunkKeys / kTile;
    static constexpr int kBoxCols = HD < 64 ? HD : 64;
    static constexpr int kHalves = HD / kBoxCols;                 // 2 for HD = 128
    static constexpr int kTileBytes = kTile * HD * 2;
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kStages = 3;
    static constexpr int kQBytes = 16 * HD * 2;
    static constexpr int kMetaRows = 512;          // requests whose (row, position, request) are staged in shared memory
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kWarps * kStages * kStageBytes + kWarps * kQBytes + kBarBytes + 3 * kMetaRows * 4 + 1024;
};

__device__ __forceinline__ void att_mbar_init(uint32_t bar) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar)); }
__device__ __forceinline__ void att_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool att_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool att_wait(uint32_t bar, uint32_t parity) {     // bounded: about two seconds
    if (att_try_wait(bar, parity)) return true;
    const unsigned long long t0 = clock64();
    while (!att_try_wait(bar, parity)) {
        if (clock64() - t0 > 4000000000ull) return false;
    }
    return true;
}
__device__ __forceinline__ void att_tma_load(uint32_t dst, const void* map, int col, int row, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(bar) : "memory");
}

// The same load marked "evict first" in L2: a decode step reads each request's keys and values once, and they
// should not push out what the step's other kernels read again soon.
__device__ __forceinline__ void att_tma_load_stream(uint32_t dst, const void* map, int col, int row, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
                 ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(bar), "l"(policy) : "memory");
}

struct DecodeItem {
    int idx, g, chunk, t, pos, req, lo, c0, tile0, tile1;
    bool visible;
};

// WIDE: a group has more than 8 query heads (both row halves of the 16-row tile are worked on); a kernel of its own,
// so that the usual one carries half as much code (short kernels pay for the instructions they fetch).
template <int HD, bool WIDE>
__global__ void __launch_bounds__(DecodeTma<HD>::kThreads, 1)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ q, const int* __restrict__ rows, int n_rows,
                            const int* __restrict__ row_req, const int* __restrict__ positions,
                            const int* __restrict__ block_tables, int table_stride, int H, int Hkv, int page_size,
                            float scale_log2, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                            int max_chunks, int n_chunks, __nv_bfloat16* __restrict__ out, int* status, int stream_kv) {
    using Cfg = DecodeTma<HD>;
    uint64_t stream_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(stream_policy));
    constexpr int kTile = Cfg::kTile, kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t stages = smem_addr(smem) + warp * kStages * Cfg::kStageBytes;
    uint8_t* q_ptr = smem + Cfg::kWarps * kStages * Cfg::kStageBytes + warp * Cfg::kQBytes;
    const uint32_t q_tile = smem_addr(q_ptr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kWarps * kStages * Cfg::kStageBytes + Cfg::kWarps * Cfg::kQBytes) + warp * kStages;
    int* meta = reinterpret_cast<int*>(smem + Cfg::kWarps * kStages * Cfg::kStageBytes + Cfg::kWarps * Cfg::kQBytes + Cfg::kBarBytes);
    const int G = H / Hkv;

    if (threadIdx.x == 0) timeline_record(kTlAttentionDecode, 0);
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) att_mbar_init(smem_addr(&bars[s]));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // Everything up to the first tiles' requests runs before the wait on the kernel ahead: the
    // step's descriptors were copied in before the step's first kernel, and of the cache only the
    // token's own position is written in this step (the tile that holds it waits, see issue()).
    pdl_launch_dependents();
    bool waited = false;
    // (step row, position, request) of every decoded token, once per CTA: the per-item look-ups
    // below would otherwise be chains of dependent global loads on each warp's critical path
    for (int i = threadIdx.x; i < n_rows && i < Cfg::kMetaRows; i += Cfg::kThreads) {
        const int t = rows[i];
        meta[i] = t;
        meta[Cfg::kMetaRows + i] = positions[t];
        meta[2 * Cfg::kMetaRows + i] = row_req[t];
    }
    __syncthreads();

    const int total = n_rows * Hkv * n_chunks;
    const int stride = gridDim.x * Cfg::kWarps;
    const int box_rows = page_size < kTile ? page_size : kTile;
    const int boxes = kTile / box_rows;

    auto item_at = [&](int w, DecodeItem& it) {
        it.chunk = w % n_chunks;
        const int rest = w / n_chunks;
        it.g = rest % Hkv;
        it.idx = rest / Hkv;
        if (it.idx < Cfg::kMetaRows) {
            it.t = meta[it.idx]; it.pos = meta[Cfg::kMetaRows + it.idx]; it.req = meta[2 * Cfg::kMetaRows + it.idx];
        } else {
            it.t = rows[it.idx]; it.pos = positions[it.t]; it.req = row_req[it.t];
        }
        it.lo = (window > 0 && it.pos - window + 1 > 0) ? it.pos - window + 1 : 0;
        it.c0 = it.chunk * kChunkKeys;
        it.visible = it.c0 <= it.pos && it.c0 + kChunkKeys > it.lo;
        it.tile0 = it.lo > it.c0 ? (it.lo - it.c0) / kTile : 0;
        const int last = (it.pos - it.c0) / kTile;
        it.tile1 = last < Cfg::kTilesPerChunk - 1 ? last : Cfg::kTilesPerChunk - 1;
    };

    // ---- producer cursor: the next tile to request
    DecodeItem pi;
    // A CTA's warps take neighbouring items (neighbouring chunks of one request lie next to each other
    // in memory); when there are fewer items than warps, each CTA takes only its share so that all SMs work.
    const int per_cta = total < static_cast<int>(gridDim.x) * Cfg::kWarps ? (total + gridDim.x - 1) / gridDim.x : Cfg::kWarps;
    const int first_item = warp < per_cta ? static_cast<int>(blockIdx.x) * per_cta + warp : total;
    int pw = first_item, ptile = 0, n_issued = 0;
    int p_pages = 0;                           // lane i: the page of the chunk's i-th page-sized run of keys
    const int pages_per_chunk = kChunkKeys / page_size > 0 ? kChunkKeys / page_size : 1;
    auto p_seek = [&]() {
        while (pw < total) {
            item_at(pw, pi);
            if (pi.visible) {
                ptile = pi.tile0;
                // the chunk's block-table entries, one per lane, requested now and used tiles later
                const int first = pi.c0 / page_size;
                const int key_of_lane = (first + lane) * page_size;
                p_pages = (lane < pages_per_chunk && key_of_lane <= pi.pos && key_of_lane + page_size - 1 >= pi.lo)
                              ? block_tables[static_cast<size_t>(pi.req) * table_stride + first + lane] : 0;
                return;
            }
            pw += stride;
        }
    };
    auto issue = [&]() {                       // requests tile (pi, ptile) into stage n_issued % kStages
        const int s = n_issued % kStages;
        const uint32_t k_tile = stages + s * Cfg::kStageBytes, v_tile = k_tile + Cfg::kTileBytes;
        const int key0 = pi.c0 + ptile * kTile;
        if (!waited && key0 + kTile > pi.pos) { pdl_wait(); waited = true; if (lane == 0) timeline_record(kTlAttentionDecode, 1); }      // the key written in this step
        // lane b requests box b of this tile (keys and values): the copies of a tile are issued side by
        // side instead of one after the other by a single lane
        const int kb = key0 + (lane < boxes ? lane : 0) * box_rows;
        const bool box_valid = lane < boxes && kb <= pi.pos && kb + box_rows - 1 >= pi.lo;
        const int box_page = __shfl_sync(0xffffffffu, p_pages, ((kb - pi.c0) / page_size) & 31);
        const unsigned valid_mask = __ballot_sync(0xffffffffu, box_valid);
        const uint32_t bar = smem_addr(&bars[s]);
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the stage was read and maybe zeroed by ordinary accesses
            att_expect_tx(bar, static_cast<uint32_t>(__popc(valid_mask)) * 2u * box_rows * HD * 2u);
        }
        __syncwarp();
        if (box_valid) {
            const int row = (box_page * Hkv + pi.g) * page_size + kb % page_size;
#pragma unroll
            for (int h = 0; h < Cfg::kHalves; ++h) {
                const uint32_t off = static_cast<uint32_t>(h * (kTile * 128) + lane * box_rows * (Cfg::kBoxCols * 2));
                if (stream_kv) {
                    att_tma_load_stream(k_tile + off, &map_k, h * 64, row, bar, stream_policy);
                    att_tma_load_stream(v_tile + off, &map_v, h * 64, row, bar, stream_policy);
                } else {
                    att_tma_load(k_tile + off, &map_k, h * 64, row, bar);
                    att_tma_load(v_tile + off, &map_v, h * 64, row, bar);
                }
            }
        }
        ++n_issued;
        if (++ptile > pi.tile1) { pw += stride; p_seek(); }
    };

    p_seek();
    while (pw < total && n_issued < kStages) issue();
    if (!waited) { pdl_wait(); waited = true; if (lane == 0 && first_item < total) timeline_record(kTlAttentionDecode, 1); }

    // ---- consumer
    DecodeItem ci;
    int n_done = 0;
    uint32_t q_frag[HD / 16][4];
    float o[HD / 8][4];
    float m[2], l[2];
    int row_lo[2], row_pos[2];
    const int r0 = lane >> 2;
    bool failed = false;
    LaneOffsets<HD, kTile, true> off;
    off.init(lane);
    for (int cw = first_item; cw < total && !failed; cw += stride) {
        item_at(cw, ci);
        float* my_o = part_o + ((static_cast<size_t>(ci.idx) * H + ci.g * G) * max_chunks + ci.chunk) * HD;
        float* my_ml = part_ml + ((static_cast<size_t>(ci.idx) * H + ci.g * G) * max_chunks + ci.chunk) * 2;
        if (!ci.visible) {
            if (lane < G) {
                my_ml[static_cast<size_t>(lane) * max_chunks * 2] = -INFINITY;
                my_ml[static_cast<size_t>(lane) * max_chunks * 2 + 1] = 0.f;
            }
            continue;
        }
        {   // the query tile of this item: rows 0..G-1 are the heads of the group, the rest zero
            constexpr int cpr = HD / 8;
            const uint4* src = reinterpret_cast<const uint4*>(q + (static_cast<size_t>(ci.t) * H + ci.g * G) * HD);
            __syncwarp();
            for (int i = lane; i < 16 * cpr; i += 32) {
                const int row = i / cpr, c = i % cpr;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (row < G) v = src[row * cpr + c];
                *reinterpret_cast<uint4*>(q_ptr + (row * cpr + swizzled_chunk<HD>(row, c)) * 16) = v;
            }
            __syncwarp();
            load_q_frags<HD>(q_tile, 0, q_frag, lane);
        }
        if (lane == 0) timeline_record(kTlAttentionDecode, 2);
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
        row_lo[0] = row_lo[1] = ci.lo;
        row_pos[0] = (r0 < G) ? ci.pos : -1;
        row_pos[1] = (r0 + 8 < G) ? ci.pos : -1;
        for (int tile = ci.tile0; tile <= ci.tile1; ++tile, ++n_done) {
            const int s = n_done % kStages;
            if (!att_wait(smem_addr(&bars[s]), (n_done / kStages) & 1)) {
                if (lane == 0) atomicCAS(status, 0, 5);
                failed = true;
                break;
            }
            const uint32_t k_tile = stages + s * Cfg::kStageBytes, v_tile = k_tile + Cfg::kTileBytes;
            const int key0 = ci.c0 + tile * kTile;
            if (key0 < ci.lo || key0 + kTile - 1 > ci.pos) {
                // an edge tile: value rows outside the range were not fetched or hold unwritten
                // positions; they are multiplied by weights of exactly 0, so they must be finite
                constexpr int cpr = HD / 8;
                for (int i = lane; i < kTile * cpr; i += 32) {
                    const int row = i / cpr, c = i % cpr;
                    const int key = key0 + row;
                    if (key < ci.lo || key > ci.pos)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(kv_addr<HD, kTile, true>(v_tile, row, c)), "r"(0) : "memory");
                }
                __syncwarp();
                warp_tile_step<HD, kTile, true, true, WIDE>(q_frag, k_tile, v_tile, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
            } else {
                warp_tile_step<HD, kTile, true, false, WIDE>(q_frag, k_tile, v_tile, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
            }
            __syncwarp();                                   // every lane is done reading the stage
            if (lane == 0 && tile == ci.tile0) timeline_record(kTlAttentionDecode, 3);
            if (pw < total) issue();
        }
        if (lane == 0) timeline_record(kTlAttentionDecode, 4);
        if (failed) break;
        if (ci.lo / kChunkKeys == ci.pos / kChunkKeys) {
            // all keys of this token lie in this one chunk: the result is final and is written as the
            // merge kernel would write it (which skips such tokens, or is not launched at all)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = r0 + 8 * r;
                if (row >= G) continue;
                __nv_bfloat16* dst = out + (static_cast<size_t>(ci.t) * H + ci.g * G + row) * HD + (lane & 3) * 2;
#pragma unroll
                for (int n = 0; n < HD / 8; ++n)
                    *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * r] / l[r], o[n][2 * r + 1] / l[r]);
            }
            continue;
        }
        // the chunk's partial result: unnormalised output, running maximum (log2 domain) and sum
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = r0 + 8 * r;
            if (row >= G) continue;
            float* dst = my_o + static_cast<size_t>(row) * max_chunks * HD + (lane & 3) * 2;
#pragma unroll
            for (int n = 0; n < HD / 8; ++n)
                *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
            if ((lane & 3) == 0) {
                my_ml[static_cast<size_t>(row) * max_chunks * 2] = m[r];
                my_ml[static_cast<size_t>(row) * max_chunks * 2 + 1] = l[r];
            }
        }
    }
    if (failed) {
        // wait (bounded) for the copies this warp still has in flight before its memory is released
        for (int i = n_done; i < n_issued; ++i) att_wait(smem_addr(&bars[i % kStages]), (i / kStages) & 1);
    }
    if (lane == 0) timeline_record(kTlAttentionDecode, 6);
}

// grid (H, decode requests), four warps. Warp w sums the chunks first + w, first + w + 4, ... in
// increasing order, each lane its own head dims, with every load requested before the first is
// used; the four sums are then added in warp order. The order depends on the row's own chunks only.
constexpr int kCombineWarps = 4;
constexpr int kCombineMaxDims = 4;                 // head dims per lane: the head sizes of these kernels end at 128

__global__ void __launch_bounds__(kCombineWarps * 32)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         const int* __restrict__ rows, const int* __restrict__ positions,
                         __nv_bfloat16* __restrict__ out, int H, int HD, int max_chunks, int window, int skip_single) {
    __shared__ float s_acc[kCombineWarps][kCombineMaxDims * 32];
    __shared__ float s_l[kCombineWarps];
    const int h = blockIdx.x, idx = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = rows[idx];
    const int pos = positions[t];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first = lo / kChunkKeys, last = pos / kChunkKeys;
    pdl_prologue();
    if (skip_single && first == last) return;        // the attention kernel wrote this token's result itself
    const float* ml = part_ml + (static_cast<size_t>(idx) * H + h) * max_chunks * 2;
    const float* po = part_o + (static_cast<size_t>(idx) * H + h) * max_chunks * HD;
    float M = -INFINITY;
    for (int c = first + lane; c <= last; c += 32) M = fmaxf(M, ml[c * 2]);
    M = warp_max(M);
    float acc[kCombineMaxDims];
#pragma unroll
    for (int i = 0; i < kCombineMaxDims; ++i) acc[i] = 0.f;
    float L = 0.f;
    constexpr int kBatch = 8;                       // chunks whose loads are in flight together
    for (int c0 = first + warp; c0 <= last; c0 += kCombineWarps * kBatch) {
        float v[kBatch][kCombineMaxDims], mc[kBatch], lc[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int c = c0 + j * kCombineWarps;
            const bool in = c <= last;
            mc[j] = in ? ml[c * 2] : -INFINITY;
            lc[j] = in ? ml[c * 2 + 1] : 0.f;
#pragma unroll
            for (int i = 0; i < kCombineMaxDims; ++i) {
                const int d = lane + 32 * i;
                v[j][i] = (in && d < HD) ? po[static_cast<size_t>(c) * HD + d] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const float f = (mc[j] == -INFINITY) ? 0.f : exp2f(mc[j] - M);
            L += lc[j] * f;
#pragma unroll
            for (int i = 0; i < kCombineMaxDims; ++i) acc[i] += v[j][i] * f;
        }
    }
#pragma unroll
    for (int i = 0; i < kCombineMaxDims; ++i) s_acc[warp][lane + 32 * i] = acc[i];
    if (lane == 0) s_l[warp] = L;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) total += s_l[w];
    for (int d = threadIdx.x; d < HD; d += kCombineWarps * 32) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < kCombineWarps; ++w) o += s_acc[w][d];
        out[(static_cast<size_t>(t) * H + h) * HD + d] = __float2bfloat16_rn(o / total);
    }
}

// ------------------------------------------------------------------------------------------ prefill
// Work item w = (first row of the tile in the step, number of tokens, request); grid (work, Hkv).
// A tile holds tokens_per_tile = 64 / G tokens; tile row r = token r / G, head r % G of the group.
template <int HD>
__global__ void __launch_bounds__(kAttThreads)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ work, const int* __restrict__ positions,
                         const int* __restrict__ block_tables, int table_stride, int H, int Hkv, int page_size,
                         float scale_log2, int window) {
    pdl_prologue();
    extern __shared__ __align__(128) uint8_t smem[];
    const int G = H / Hkv;
    const int g = blockIdx.x;          // heads vary fastest: the longest work items of every head start first
    const int t0 = work[blockIdx.y * 3], n_tok = work[blockIdx.y * 3 + 1], req = work[blockIdx.y * 3 + 2];
    const int n_rows = n_tok * G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_tables + static_cast<size_t>(req) * table_stride;
    const int pos_first = positions[t0], pos_last = pos_first + n_tok - 1;      // consecutive positions
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;

    constexpr int kTileBytes = kTileKeys * HD * 2;
    constexpr int cpr = HD / 8;
    const uint32_t q_tile = smem_addr(smem);
    const uint32_t kv_base = q_tile + 64 * HD * 2;          // stage s: K at kv_base + s*2*kTileBytes, V after it

    // the query tile: row r <- q[t0 + r / G][g * G + r % G]
    for (int i = threadIdx.x; i < 64 * cpr; i += kAttThreads) {
        const int row = i / cpr, c = i % cpr;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n_rows) {
            const int tok = row / G, hh = row % G;
            v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(t0 + tok) * H + g * G + hh) * HD + c * 8);
        }
        *reinterpret_cast<uint4*>(smem + (row * cpr + swizzled_chunk<HD>(row, c)) * 16) = v;
    }

    const int first_tile = lo_first / kTileKeys, last_tile = pos_last / kTileKeys;
    const int n_tiles = last_tile - first_tile + 1;
    auto issue = [&](int i) {
        const uint32_t kt = kv_base + (i & 1) * 2 * kTileBytes;
        const int key0 = (first_tile + i) * kTileKeys;
        load_tile_async<HD>(kt, k_cache, table, g, Hkv, page_size, key0, kTileKeys, lo_first, pos_last, threadIdx.x, kAttThreads);
        load_tile_async<HD>(kt + kTileBytes, v_cache, table, g, Hkv, page_size, key0, kTileKeys, lo_first, pos_last, threadIdx.x, kAttThreads);
        cp_async_commit();
    };
    issue(0);
    __syncthreads();                                    // the query tile is complete

    uint32_t q_frag[HD / 16][4];
    load_q_frags<HD>(q_tile, warp * 16, q_frag, lane);
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int row_lo[2], row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row < n_rows) {
            row_pos[r] = pos_first + row / G;
            row_lo[r] = (window > 0 && row_pos[r] - window + 1 > 0) ? row_pos[r] - window + 1 : 0;
        } else {
            row_pos[r] = -1; row_lo[r] = 0;
        }
    }
    // what this warp's rows can see at most (uniform across the warp)
    const int warp_row_first = warp * 16, warp_row_last = min(n_rows - 1, warp * 16 + 15);
    const int warp_pos_max = (warp_row_first < n_rows) ? pos_first + warp_row_last / G : -1;
    const int warp_pos_min = pos_first + warp_row_first / G;
    const int warp_lo_min = (window > 0 && warp_pos_min - window + 1 > 0) ? warp_pos_min - window + 1 : 0;
    const int warp_lo_max = (window > 0 && warp_pos_max - window + 1 > 0) ? warp_pos_max - window + 1 : 0;
    LaneOffsets<HD, kTileKeys, false> off;
    off.init(lane);

    for (int i = 0; i < n_tiles; ++i) {
        if (i + 1 < n_tiles) { issue(i + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        const uint32_t kt = kv_base + (i & 1) * 2 * kTileBytes;
        const int key0 = (first_tile + i) * kTileKeys;
        if (key0 <= warp_pos_max && key0 + kTileKeys > warp_lo_min) {
            // no mask where every key of the tile is visible to every row of the warp (rows beyond
            // the tile's tokens have zero queries and are never stored)
            if (key0 >= warp_lo_max && key0 + kTileKeys - 1 <= warp_pos_min)
                warp_tile_step<HD, kTileKeys, false, false>(q_frag, kt, kt + kTileBytes, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
            else
                warp_tile_step<HD, kTileKeys, false, true>(q_frag, kt, kt + kTileBytes, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
        }
        __syncthreads();                                // the stage may be overwritten by the next issue
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row >= n_rows) continue;
        const int tok = row / G, hh = row % G;
        const float inv = 1.0f / l[r];
        __nv_bfloat16* dst = out + (static_cast<size_t>(t0 + tok) * H + g * G + hh) * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        }
    }
}

// ------------------------------------------------------------------------------------------ prefill, fed by TMA
// 128 query rows per CTA (eight warps of 16 rows: tokens x heads of one key/value group), keys in
// tiles of 64 through a three-stage ring that a ninth warp fills by TMA, one box per page. A warp
// skips the tiles beyond its own rows' positions and masks only the tiles at the edge of some
// row's range.
template <int HD>
struct PrefillTma {
    static constexpr int kRows = 128;
    static constexpr int kWarps = 8;
    static constexpr int kThreads = (kWarps + 1) * 32;
    static constexpr int kTile = 64;
    static constexpr int kBoxCols = HD < 64 ? HD : 64;
    static constexpr int kHalves = HD / kBoxCols;
    static constexpr int kTileBytes = kTile * HD * 2;
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kStages = 3;
    static constexpr int kQBytes = kRows * HD * 2;
    static constexpr int kSmemBytes = kStages * kStageBytes + kQBytes + 128 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(PrefillTma<HD>::kThreads, (HD <= 64 ? 2 : 1))
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                             const int* __restrict__ work, const int* __restrict__ positions,
                             const int* __restrict__ block_tables, int table_stride, int H, int Hkv, int page_size,
                             float scale_log2, int window, int* status) {
    using Cfg = PrefillTma<HD>;
    constexpr int kTile = Cfg::kTile, kStages = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t stages = smem_addr(smem);
    uint8_t* q_ptr = smem + kStages * Cfg::kStageBytes;
    const uint32_t q_tile = smem_addr(q_ptr);
    uint64_t* full = reinterpret_cast<uint64_t*>(q_ptr + Cfg::kQBytes);
    uint64_t* empty = full + kStages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = H / Hkv;
    const int g = blockIdx.x;          // heads vary fastest: the longest work items of every head start first

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            att_mbar_init(smem_addr(&full[s]));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&empty[s])), "r"(Cfg::kWarps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_prologue();

    const int t0 = work[blockIdx.y * 3], n_tok = work[blockIdx.y * 3 + 1], req = work[blockIdx.y * 3 + 2];
    const int n_rows = n_tok * G;
    const int* table = block_tables + static_cast<size_t>(req) * table_stride;
    const int pos_first = positions[t0], pos_last = pos_first + n_tok - 1;
    const int lo_first = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int first_tile = lo_first / kTile, last_tile = pos_last / kTile;
    const int n_tiles = last_tile - first_tile + 1;
    const int box_rows = page_size < kTile ? page_size : kTile;
    const int boxes = kTile / box_rows;

    if (warp == Cfg::kWarps) {
        // ---------------------------------------------------------------- producer warp
        // All lanes look up the tile's pages at once (lane b: box b), before the wait for the free
        // stage; then every lane requests its own box (one lane issuing them in turn is slow).
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i % kStages;
            const int key0 = (first_tile + i) * kTile;
            const int kb_lane = key0 + lane * box_rows;
            const bool lane_valid = lane < boxes && kb_lane <= pos_last && kb_lane + box_rows - 1 >= lo_first;
            const int page_lane = lane_valid ? table[kb_lane / page_size] : 0;
            const unsigned valid_mask = __ballot_sync(0xffffffffu, lane_valid);
            bool ok = true;
            if (lane == 0 && i >= kStages && !att_wait(smem_addr(&empty[s]), ((i / kStages) - 1) & 1)) {
                atomicCAS(status, 0, 6);
                ok = false;
            }
            if (!__shfl_sync(0xffffffffu, ok ? 1 : 0, 0)) break;
            const uint32_t k_tile = stages + s * Cfg::kStageBytes, v_tile = k_tile + Cfg::kTileBytes;
            const uint32_t bar = smem_addr(&full[s]);
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                att_expect_tx(bar, static_cast<uint32_t>(__popc(valid_mask)) * 2u * box_rows * HD * 2u);
            }
            __syncwarp();                                         // the expected bytes are set before any copy can complete
            if (lane_valid) {                                     // every lane requests its own box
                const int row = (page_lane * Hkv + g) * page_size + kb_lane % page_size;
#pragma unroll
                for (int h = 0; h < Cfg::kHalves; ++h) {
                    const uint32_t off = static_cast<uint32_t>(h * (kTile * 128) + lane * box_rows * (Cfg::kBoxCols * 2));
                    att_tma_load(k_tile + off, &map_k, h * 64, row, bar);
                    att_tma_load(v_tile + off, &map_v, h * 64, row, bar);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    // this warp's 16 query rows: row r <- q[t0 + r / G][g * G + r % G]
    {
        constexpr int cpr = HD / 8;
        for (int i = lane; i < 16 * cpr; i += 32) {
            const int row = warp * 16 + i / cpr, c = i % cpr;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < n_rows) {
                const int tok = row / G, hh = row % G;
                v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(t0 + tok) * H + g * G + hh) * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(q_ptr + (row * cpr + swizzled_chunk<HD>(row, c)) * 16) = v;
        }
        __syncwarp();
    }
    uint32_t q_frag[HD / 16][4];
    load_q_frags<HD>(q_tile, warp * 16, q_frag, lane);
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int row_lo[2], row_pos[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row < n_rows) {
            row_pos[r] = pos_first + row / G;
            row_lo[r] = (window > 0 && row_pos[r] - window + 1 > 0) ? row_pos[r] - window + 1 : 0;
        } else {
            row_pos[r] = -1; row_lo[r] = 0;
        }
    }
    const int warp_row_first = warp * 16, warp_row_last = min(n_rows - 1, warp * 16 + 15);
    const bool warp_has_rows = warp_row_first < n_rows;
    const int warp_pos_max = warp_has_rows ? pos_first + warp_row_last / G : -1;
    const int warp_pos_min = pos_first + warp_row_first / G;
    const int warp_lo_min = (window > 0 && warp_pos_min - window + 1 > 0) ? warp_pos_min - window + 1 : 0;
    const int warp_lo_max = (window > 0 && warp_pos_max - window + 1 > 0) ? warp_pos_max - window + 1 : 0;
    LaneOffsets<HD, kTile, true> off;
    off.init(lane);

    for (int i = 0; i < n_tiles; ++i) {
        const int s = i % kStages;
        if (!att_wait(smem_addr(&full[s]), (i / kStages) & 1)) {
            if (lane == 0) atomicCAS(status, 0, 7);
            break;
        }
        const uint32_t k_tile = stages + s * Cfg::kStageBytes, v_tile = k_tile + Cfg::kTileBytes;
        const int key0 = (first_tile + i) * kTile;
        if (key0 <= warp_pos_max && key0 + kTile > warp_lo_min) {
            if (key0 >= warp_lo_max && key0 + kTile - 1 <= warp_pos_min) {
                warp_tile_step<HD, kTile, true, false>(q_frag, k_tile, v_tile, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
            } else {
                if (key0 < lo_first || key0 + kTile - 1 > pos_last) {
                    // value rows outside every query's range were not fetched or were never written:
                    // each warp zeroes them for itself (all warps store the same zeros)
                    constexpr int cpr = HD / 8;
                    for (int j = lane; j < kTile * cpr; j += 32) {
                        const int row = j / cpr, c = j % cpr;
                        const int key = key0 + row;
                        if (key < lo_first || key > pos_last)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(kv_addr<HD, kTile, true>(v_tile, row, c)), "r"(0) : "memory");
                    }
                    __syncwarp();
                }
                warp_tile_step<HD, kTile, true, true>(q_frag, k_tile, v_tile, key0, row_lo, row_pos, scale_log2, o, m, l, lane, off);
            }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&empty[s])) : "memory");
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row >= n_rows) continue;
        const int tok = row / G, hh = row % G;
        const float inv = 1.0f / l[r];
        __nv_bfloat16* dst = out + (static_cast<size_t>(t0 + tok) * H + g * G + hh) * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
    }
}

template <int HD>
static int launch_decode(const void* q, const void* kc, const void* vc, void* out, const int* rows, int n_rows,
                         const int* row_req, const int* positions, const int* tables, int table_stride, int H, int Hkv,
                         int page_size, float scale, int window, float* part_o, float* part_ml, int max_chunks,
                         int n_chunks, cudaStream_t st) {
    constexpr int smem = 16 * HD * 2 + 4 * 2 * kTileKeys * HD * 2;
    constexpr int red = 4 * 16 * (HD + 2) * 4;
    constexpr int bytes = smem > red ? smem : red;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) { set_error("attention_decode: %s", cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    dim3 grid(n_chunks, Hkv, n_rows);
    launch_kernel((attention_decode_kernel<HD>), dim3(grid), dim3(kAttThreads), bytes, st, 
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc),
        rows, row_req, positions, tables, table_stride, H, Hkv, page_size, scale * kLog2e, window, part_o, part_ml, max_chunks);
    if (check_launch("attention_decode")) return 1;
    dim3 grid2(H, n_rows);
    launch_kernel((attention_combine_kernel), dim3(grid2), dim3(kCombineWarps * 32), 0, st, part_o, part_ml, rows, positions,
                                                                   static_cast<__nv_bfloat16*>(out), H, HD, max_chunks, window, 0);
    return check_launch("attention_combine");
}

static int g_stream_kv = 1;

template <int HD>
static int launch_decode_tma(const void* q, const void* kc, const void* vc, void* out, const int* rows, int n_rows,
                             const int* row_req, const int* positions, const int* tables, int table_stride, int H, int Hkv,
                             int page_size, float scale, int window, float* part_o, float* part_ml, int max_chunks,
                             int n_chunks, long long n_pages, int* status, cudaStream_t st) {
    using Cfg = DecodeTma<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_decode_tma_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) { set_error("attention_decode: %s", cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    const int box_rows = page_size < Cfg::kTile ? page_size : Cfg::kTile;
    CUtensorMap mk, mv;
    const unsigned long long rows_total = static_cast<unsigned long long>(n_pages) * Hkv * page_size;
    if (make_tensor_map_2d(&mk, kc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, HD, HD, box_rows, Cfg::kBoxCols,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, "attention_decode")) return 1;
    if (make_tensor_map_2d(&mv, vc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, HD, HD, box_rows, Cfg::kBoxCols,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, "attention_decode")) return 1;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int items = n_rows * Hkv * n_chunks;
    int grid = items < sms ? items : sms;           // few items: fewer per CTA rather than fewer CTAs
    if (H / Hkv > 8)
        launch_kernel((attention_decode_tma_kernel<HD, true>), dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, st, mk, mv,
                  static_cast<const __nv_bfloat16*>(q), rows, n_rows, row_req, positions, tables, table_stride, H, Hkv,
                  page_size, scale * kLog2e, window, part_o, part_ml, max_chunks, n_chunks, static_cast<__nv_bfloat16*>(out), status,
                  (g_stream_kv && n_rows <= 32) ? 1 : 0);     // measured: 2 % faster at 8 requests, no gain at 64
    else
        launch_kernel((attention_decode_tma_kernel<HD, false>), dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, st, mk, mv,
                  static_cast<const __nv_bfloat16*>(q), rows, n_rows, row_req, positions, tables, table_stride, H, Hkv,
                  page_size, scale * kLog2e, window, part_o, part_ml, max_chunks, n_chunks, static_cast<__nv_bfloat16*>(out), status,
                  (g_stream_kv && n_rows <= 32) ? 1 : 0);     // measured: 2 % faster at 8 requests, no gain at 64
    if (check_launch("attention_decode_tma")) return 1;
    if (n_chunks == 1) return 0;                     // every token's keys lie in one chunk: nothing to merge
    dim3 grid2(H, n_rows);
    launch_kernel((attention_combine_kernel), dim3(grid2), dim3(kCombineWarps * 32), 0, st, part_o, part_ml, rows, positions,
                  static_cast<__nv_bfloat16*>(out), H, HD, max_chunks, window, 1);
    return check_launch("attention_combine");
}

template <int HD>
static int launch_prefill(const void* q, const void* kc, const void* vc, void* out, const int* work, int n_work,
                          const int* positions, const int* tables, int table_stride, int H, int Hkv, int page_size,
                          float scale, int window, cudaStream_t st) {
    constexpr int bytes = 64 * HD * 2 + 2 * 2 * kTileKeys * HD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) { set_error("attention_prefill: %s", cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    dim3 grid(Hkv, n_work);
    launch_kernel((attention_prefill_kernel<HD>), dim3(grid), dim3(kAttThreads), bytes, st, 
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc),
        static_cast<__nv_bfloat16*>(out), work, positions, tables, table_stride, H, Hkv, page_size, scale * kLog2e, window);
    return check_launch("attention_prefill");
}

template <int HD>
static int launch_prefill_tma(const void* q, const void* kc, const void* vc, void* out, const int* work, int n_work,
                              const int* positions, const int* tables, int table_stride, int H, int Hkv, int page_size,
                              float scale, int window, long long n_pages, int* status, cudaStream_t st) {
    using Cfg = PrefillTma<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) { set_error("attention_prefill: %s", cudaGetErrorString(e)); return 1; }
        configured = true;
    }
    const int box_rows = page_size < Cfg::kTile ? page_size : Cfg::kTile;
    CUtensorMap mk, mv;
    const unsigned long long rows_total = static_cast<unsigned long long>(n_pages) * Hkv * page_size;
    if (make_tensor_map_2d(&mk, kc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, HD, HD, box_rows, Cfg::kBoxCols,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "attention_prefill")) return 1;
    if (make_tensor_map_2d(&mv, vc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_total, HD, HD, box_rows, Cfg::kBoxCols,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, "attention_prefill")) return 1;
    dim3 grid(Hkv, n_work);
    launch_kernel((attention_prefill_tma_kernel<HD>), dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, st, mk, mv,
                  static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), work, positions, tables,
                  table_stride, H, Hkv, page_size, scale * kLog2e, window, status);
    return check_launch("attention_prefill_tma");
}

}  // namespace gi

using namespace gi;
GI_TIMELINE_SETTER(gi_timeline_set_attention)

// Query rows per work item of the prefill kernels for this page size and head size: 128 where the
// pages can be fetched by TMA boxes, 64 otherwise. A work item holds rows / group-size tokens.
extern "C" int gi_attention_prefill_rows(int page_size, int hd) {
    const int tile = 64;
    (void)hd;
    return (page_size % 8 == 0 && (tile % page_size == 0 || page_size % tile == 0)) ? 128 : 64;
}

extern "C" int gi_attention_fast_supported(int head_dim, int H, int Hkv) {
    return (head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128) && Hkv > 0 && H % Hkv == 0 && H / Hkv <= 16;
}

extern "C" int gi_attention_chunk_keys() { return kChunkKeys; }

// Switches the evict-first L2 policy on the key/value loads of decode attention on or off (on by default);
// returns the old value.
extern "C" int gi_attention_set_stream_kv(int on) {
    const int old = g_stream_kv;
    g_stream_kv = on ? 1 : 0;
    return old;
}

// Single decoded tokens: rows[i] is the step row of the i-th one. part_o holds
// n_rows * H * max_chunks * hd floats and part_ml n_rows * H * max_chunks * 2; n_chunks covers the
// longest context among the rows.
static int gi_attention_decode_impl(const void* q, const void* k_cache, const void* v_cache, void* out, const int* rows,
                                   int n_rows, const int* row_req, const int* positions, const int* block_tables,
                                   int table_stride, int H, int Hkv, int hd, int page_size, float scale, int window,
                                   float* part_o, float* part_ml, int max_chunks, int n_chunks, long long n_pages,
                                   void* status, void* stream) {
    if (n_rows == 0) return 0;
    GI_REQUIRE(gi_attention_fast_supported(hd, H, Hkv), "attention_decode: head size %d with %d/%d heads is not built", hd, H, Hkv);
    GI_REQUIRE(n_chunks >= 1 && n_chunks <= max_chunks, "attention_decode: %d chunks exceed the workspace's %d", n_chunks, max_chunks);
    GI_REQUIRE(n_rows <= 65535 && Hkv <= 65535, "attention_decode: grid too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Pages that TMA boxes can tile (8, 16, 32 ... rows that divide or are divided by the tile) take
    // the TMA-fed kernel; any other page size takes the cp.async kernel.
    const int tile = 32;
    const bool tma_ok = page_size % 8 == 0 && (tile % page_size == 0 || page_size % tile == 0) && status != nullptr &&
                        reinterpret_cast<uintptr_t>(k_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(v_cache) % 16 == 0;
    if (tma_ok) {
#define GI_DECODE_TMA(HD) return launch_decode_tma<HD>(q, k_cache, v_cache, out, rows, n_rows, row_req, positions, block_tables, \
        table_stride, H, Hkv, page_size, scale, window, part_o, part_ml, max_chunks, n_chunks, n_pages, static_cast<int*>(status), st)
        switch (hd) {
            case 16: GI_DECODE_TMA(16);
            case 32: GI_DECODE_TMA(32);
            case 64: GI_DECODE_TMA(64);
            default: GI_DECODE_TMA(128);
        }
#undef GI_DECODE_TMA
    }
#define GI_DECODE(HD) return launch_decode<HD>(q, k_cache, v_cache, out, rows, n_rows, row_req, positions, block_tables, \
                                               table_stride, H, Hkv, page_size, scale, window, part_o, part_ml, max_chunks, n_chunks, st)
    switch (hd) {
        case 16: GI_DECODE(16);
        case 32: GI_DECODE(32);
        case 64: GI_DECODE(64);
        default: GI_DECODE(128);
    }
#undef GI_DECODE
}

// Prompt portions: work[3*i..] = (first step row of the tile, tokens in the tile, request index).
static int gi_attention_prefill_impl(const void* q, const void* k_cache, const void* v_cache, void* out, const int* work,
                                    int n_work, const int* positions, const int* block_tables, int table_stride, int H,
                                    int Hkv, int hd, int page_size, float scale, int window, long long n_pages,
                                    void* status, void* stream) {
    if (n_work == 0) return 0;
    GI_REQUIRE(gi_attention_fast_supported(hd, H, Hkv), "attention_prefill: head size %d with %d/%d heads is not built", hd, H, Hkv);
    GI_REQUIRE(n_work <= 65535, "attention_prefill: %d work items exceed the grid limit 65535", n_work);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (gi_attention_prefill_rows(page_size, hd) == 128 && status != nullptr) {
#define GI_PREFILL_TMA(HD) return launch_prefill_tma<HD>(q, k_cache, v_cache, out, work, n_work, positions, block_tables, \
        table_stride, H, Hkv, page_size, scale, window, n_pages, static_cast<int*>(status), st)
        switch (hd) {
            case 16: GI_PREFILL_TMA(16);
            case 32: GI_PREFILL_TMA(32);
            case 64: GI_PREFILL_TMA(64);
            default: GI_PREFILL_TMA(128);
        }
#undef GI_PREFILL_TMA
    }
#define GI_PREFILL(HD) return launch_prefill<HD>(q, k_cache, v_cache, out, work, n_work, positions, block_tables, table_stride, \
                                                 H, Hkv, page_size, scale, window, st)
    switch (hd) {
        case 16: GI_PREFILL(16);
        case 32: GI_PREFILL(32);
        case 64: GI_PREFILL(64);
        default: GI_PREFILL(128);
    }
#undef GI_PREFILL
}

// The exported names: each runs its implementation above and, while a launch program is recorded, leaves a copy of
// its arguments in the program (common.cuh).
extern "C" int gi_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const int* rows, int n_rows, const int* row_req, const int* positions, const int* block_tables, int table_stride, int H, int Hkv, int hd, int page_size, float scale, int window, float* part_o, float* part_ml, int max_chunks, int n_chunks, long long n_pages, void* status, void* stream) {
    return gi::dispatch(gi_attention_decode_impl, q, k_cache, v_cache, out, rows, n_rows, row_req, positions, block_tables, table_stride, H, Hkv, hd, page_size, scale, window, part_o, part_ml, max_chunks, n_chunks, n_pages, status, stream);
}

extern "C" int gi_attention_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* work, int n_work, const int* positions, const int* block_tables, int table_stride, int H, int Hkv, int hd, int page_size, float scale, int window, long long n_pages, void* status, void* stream) {
    return gi::dispatch(gi_attention_prefill_impl, q, k_cache, v_cache, out, work, n_work, positions, block_tables, table_stride, H, Hkv, hd, page_size, scale, window, n_pages, status, stream);
}
