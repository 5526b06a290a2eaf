// Fused paged decode attention over the RotorQuant cache, sm_100a.
//
// Replaces fused_paged_rq_decode (triton/fused_paged_rq_decode.py:32-312 of the reference): the
// Triton kernel (one program per (sequence, query head), CUDA-core dot products, no split-KV)
// and the two dense 128x128 rotations its launcher runs around it.
//
// Work decomposition.  A tile is 128 (token, KV head) pairs: T = 128 / Ht consecutive tokens of one
// sequence times a "head tile" of Ht KV heads (Ht = all KV heads of this GPU when there are 1, 2, 4
// or 8 of them).  With a whole head tile in one CTA the payload of a token -- K indices, K norms,
// V indices, V norms of all its heads, 136 * H contiguous bytes of the slot -- arrives as ONE row of
// ONE TMA box per block of tokens, norms included.  (One CTA per KV head, as the first versions had
// it, needs a 64-byte K row, a 64-byte V row and two norm sectors per token and head: about 4.5
// memory requests for 136 bytes.  The SM's TMA unit was measured at 0.17 such rows per cycle, 16-byte
// cp.async copies at about 0.2, against 0.75 requests per cycle at the HBM roofline.)
// The (sequence, tile) space of the batch is one line of tiles, cut into contiguous pieces; a CTA
// streams the tiles of one piece for one (head tile, group of up to 8 query heads per KV head) and
// leaves one partial result per sequence its piece touches.  A second launch merges the partial
// results of every (sequence, query head), rounds, and applies R.
//
// The attention CTA is warp specialised.  Two threads work on every pair: thread t of the four K
// warps (which owns TMEM lane t) builds the pair's K digit planes, reads its scores and runs the
// softmax; thread t of the four V warps decompresses the pair's V row into the shared V tile at the
// same time.  Two more warps own the asynchronous engines.  Issuing a tcgen05.mma of these skinny
// shapes keeps the issuing thread busy for 100 (S^T, N = 64) to 140 cycles (O^T) whatever else runs, and
// two threads of different warps issue side by side without slowing each other, so one warp issues the
// S^T MMAs and fills the ring of staged tiles with TMA boxes, the other issues the O^T MMAs, each when the
// other warps have published its operands.  No block-wide barrier is met inside the tile loop;
// everything is ordered by mbarriers.
//
// Arithmetic (matches "reference decompress + SDPA"):
//   q_rot   = round_T(q @ R^T)            exact FMA chain per 4x4 block, computed per part
//   K, V    = round_T(centroid[idx]*norm) exactly the decompressed values: each pair gets a
//             table of its 8/16 rounded products, elements are fetched from it with PRMT
//   scores  = int8 tensor-core mma over 15-bit integer images of q_rot and K (exact for K, 2^-14
//             of the row maximum for q): S^T = K Q^T with the 128 pairs on the M side and the digit
//             planes of ALL query heads of the head tile on the N side; a pair reads the columns of
//             its own KV head.  fp32 scaling, exp2-domain softmax against a reference maximum per
//             head (exact maximum of the part's first tile; it moves later only when a score
//             exceeds it by 2^8)
//   P @ V   = tensor-core mma with P split into hi + lo parts (two T-precision terms, ~16 bits),
//             fp32 accumulate in tensor memory; the 16 pairs of one MMA k-step belong to one KV
//             head, so each k-step accumulates into that head's output columns
//   out     = round_T(round_T(o / l) @ R)  in the merge kernel
#include <cuda.h>          // CUtensorMap (types only; the encoder is looked up at run time)

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "rq_common.cuh"
#include "rq_tcgen05.cuh"

namespace rq {

constexpr int kQPerHead = 8;                 // query-head slots per KV head of a partial row / of one item
constexpr int kPairs = 128;                  // (token, KV head) pairs per tile = compute threads per CTA
constexpr int kComputeThreads = 128;
constexpr int kDecodeThreads = 320;          // K warps 0..3, V warps 4..7, two issuer warps
constexpr int kVWarp0 = 4;
constexpr int kSIssuerWarp = 8;              // issues S^T = K Q^T and the TMA copies
constexpr int kPvIssuerWarp = 9;             // issues O^T += V^T P
constexpr uint32_t kTmemCols = 256;          // columns allocated per CTA
constexpr uint32_t kColKhi = 0, kColKlo = 32, kColS = 64, kColS2 = 128, kColO = 192;
constexpr int kMaxCols = 64;                 // columns of one S accumulator and of O: head tile x 2 x query heads
constexpr int kInlinePlanSeqs = 256;         // up to this many sequences the CTAs scan seq_lens themselves
constexpr int kMaxLayers = 4;                // launch layers with their own piece weight
constexpr int kCtasPerSm = 2;
constexpr int kRingBytes = 54 * 1024;        // staged tiles (two or three stages)
constexpr int kMaxStages = 3;
constexpr int kRegions = 4;                  // K indices, K norms, V indices, V norms

struct DecodeParams {
    const void* q;
    int64_t q_stride_seq, q_stride_head;
    const uint8_t* cache;
    int64_t num_blocks;
    int block_size;
    int total_bytes;
    const int32_t* block_table;
    int64_t bt_stride;
    const int32_t* seq_lens;
    const float* cent_k;
    const float* cent_v;
    const float* rotation;
    float qk_scale;                        // sm_scale * log2(e)
    int H, Hq, G;                          // KV heads, query heads, Hq / H
    int head_groups;                       // ceil(G / 8)
    int ht, ht_shift;                      // KV heads per tile (1, 2, 4 or 8)
    int ttok, ttok_shift;                  // tokens per tile = 128 / ht
    int n_cols;                            // columns of S and of O: max(16, ht * 2 * NH)
    float* ws_o;                           // [row][ht * 8 slots][128], row = (group + sequence) * J + item
    float* ws_m;                           // [row][ht * 8]
    float* ws_l;
    void* out;
    int64_t o_stride_seq, o_stride_head;
    int32_t* prefix;                       // [num_seqs + 1] exclusive prefix of tiles per sequence (workspace)
    int num_seqs;
    int groups;                            // pieces; CTA = (group, item)
    int inline_plan;                       // the attention CTAs compute the prefix sums themselves
    int bs_shift;                          // log2(block_size) when it is a power of two, else -1
    // staging: a stage holds, per region, an array [ttok][w] of the region's bytes of every token
    int n_regions;                         // 1: the whole payload of the head tile is contiguous; else 4
    int reg_w[kRegions];                   // bytes copied per token and region (multiple of 16)
    int reg_base[kRegions];                // offset of the region's array inside a stage
    int stage_bytes, stages;
    int box_rows;                          // tokens per TMA box (0: no TMA, the issuer warp copies 4-byte words)
    int v_aligned;                         // V rows sit on 16-byte boundaries of the stage
    int layer_ctas;                        // CTAs per launch layer (SM count) when pieces are weighted, else 0
    int num_layers;
    int layer_w[kMaxLayers];               // piece weight of the CTAs of each launch layer
    unsigned long long* trace;             // development builds only
};

// Development builds (-DRQ_DECODE_TRACE) record clock64() at the phase boundaries of a few CTAs.
#ifdef RQ_DECODE_TRACE
#define RQ_TRACE(point)                                                                             \
    do {                                                                                            \
        if (trace_row != nullptr && lane == 0 && it < 64) trace_row[it * 16 + (point)] = clock64(); \
    } while (0)
#else
#define RQ_TRACE(point) \
    do {                \
    } while (0)
#endif

// ---- pieces -----------------------------------------------------------------------------------
//
// On one SM the CTAs that were launched first (lower block index) get the larger share of the
// issue slots while several run side by side, so equal pieces would finish far apart.  CTA c
// belongs to launch layer c / layer_ctas and its piece is proportional to that layer's weight.
// weight_cum(n) = sum of the weights of CTAs 0..n-1; piece g covers
// [total * cum(g J) / cum(G J), total * cum((g + 1) J) / cum(G J)).
__host__ __device__ inline int64_t weight_cum(int64_t n, int layer_ctas, int num_layers, const int* w) {
    if (layer_ctas <= 0) return n * 1024;
    int64_t acc = 0;
    for (int layer = 0; n > 0; ++layer) {
        const int64_t take = (layer + 1 < num_layers && n > layer_ctas) ? layer_ctas : n;
        acc += take * w[layer < num_layers ? layer : num_layers - 1];
        n -= take;
    }
    return acc;
}
__device__ __forceinline__ int64_t piece_begin(const DecodeParams& p, int64_t g, int64_t total, int J) {
    return total * weight_cum(g * J, p.layer_ctas, p.num_layers, p.layer_w) /
           weight_cum(static_cast<int64_t>(p.groups) * J, p.layer_ctas, p.num_layers, p.layer_w);
}

// Byte ranges of the four payload regions of head tile `h0 .. h0 + ht` inside a slot of H heads:
// start[r] (may be 4, 8 or 12 bytes past a 16-byte boundary) and the 16-byte boundary below it.
struct RegionWindow {
    int start[kRegions], x[kRegions];
};
__host__ __device__ inline RegionWindow region_window(int H, int h0) {
    RegionWindow rw;
    rw.start[0] = kHalfDim * h0;                       // K indices
    rw.start[1] = kHalfDim * H + 4 * h0;               // K norms
    rw.start[2] = (kHalfDim + 4) * H + kHalfDim * h0;  // V indices
    rw.start[3] = (2 * kHalfDim + 4) * H + 4 * h0;     // V norms
    for (int r = 0; r < kRegions; ++r) rw.x[r] = rw.start[r] & ~15;
    return rw;
}

// ---- small PTX wrappers ------------------------------------------------------

// Two fp32 -> packed T pair, `lo` in bits 0..15.
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 unpack_pair<__half>(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round_to<__half>(float v) {
    return __half2float(__float2half_rn(v));
}

__device__ __forceinline__ void store_rounded(__nv_bfloat16* dst, float v) { *dst = __float2bfloat16_rn(v); }
__device__ __forceinline__ void store_rounded(__half* dst, float v) { *dst = __float2half_rn(v); }

// Arrive on an mbarrier and announce `bytes` of asynchronous copies that will complete on it.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes)
                 : "memory");
}

// TMA: copy one 2-D box (inner coordinate x in elements, outer coordinate y) of the tensor described
// by `map` into shared memory; completion is signalled on the mbarrier.  No multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
        "r"(bar_addr)
        : "memory");
}

// 4-byte asynchronous copy global -> shared; the mbarrier receives one arrival (already counted in
// its expected arrivals) when every copy this thread has issued so far has landed.
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Barrier of the 128 compute threads only (the issuer warp never joins it).
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Programmatic dependent launch: the merge kernel may be scheduled while the attention kernel
// drains; it must not read the partial results before this wait returns.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ int ld_volatile_shared(const int* p) {
    int v;
    asm volatile("ld.volatile.shared.b32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_shared(int* p, int v) {
    asm volatile("st.volatile.shared.b32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

// ---- per-token lookup tables -------------------------------------------------
//
// Every (token, K|V) gets a table of its 2^BITS decompressed values round_T(centroid[i] * norm),
// stored as byte planes so that one PRMT fetches the bytes of four nibble indices at once.
//
// V tables hold the T (bf16/f16) bit patterns: a low-byte plane and a high-byte plane.
// K tables hold the same values as 15-bit integers I[i] = value * 2^(13 - e), e the exponent of
// the largest entry (exact unless the entries span more than 6 binades), split into two signed
// byte planes I = 256 * hi + lo, plus the scale 2^(e - 13).  Q K^T then runs on the int8 tensor
// path, which needs half the PRMTs of a 16-bit operand.
//   BITS == 3: 4 registers  {lo[0..3], lo[4..7], hi[0..3], hi[4..7]}
//   BITS == 4: 8 registers  {lo[0..3] .. lo[12..15], hi[0..3] .. hi[12..15]}
template <int BITS>
struct Table {
    static constexpr int kRegs = BITS == 3 ? 4 : 8;
    uint32_t r[kRegs];
};

// Power of two 2^k as a float, k in [-126, 127].
__device__ __forceinline__ float pow2i(int k) { return __int_as_float((k + 127) << 23); }

// Exponent e with 2^e <= v < 2^(e+1) for a finite normal v > 0.
__device__ __forceinline__ int exponent_of(float v) { return ((__float_as_int(v) >> 23) & 0xFF) - 127; }

// Bytes of the four entries selected by the four nibbles in sel[15:0] from one byte plane
// (plane = N/4 registers).
template <int BITS>
__device__ __forceinline__ uint32_t lookup_plane(const uint32_t* plane, uint32_t sel, uint32_t s7,
                                                 uint32_t m) {
    if constexpr (BITS == 3) {
        return prmt(plane[0], plane[1], sel);
    } else {
        const uint32_t a = prmt(plane[0], plane[1], s7), b = prmt(plane[2], plane[3], s7);
        return (a & ~m) | (b & m);
    }
}

// Lookup of both planes for the nibbles in sel[15:0].
template <int BITS>
__device__ __forceinline__ void lookup4(const Table<BITS>& t, uint32_t sel, uint32_t& lo,
                                        uint32_t& hi) {
    uint32_t s7 = 0, m = 0;
    if constexpr (BITS == 4) {
        s7 = sel & 0x7777u;
        const uint32_t y = prmt(sel, sel << 4, 0x5410);
        m = prmt(y, y, 0x9B8A);      // byte i = 0xFF when nibble i of sel has its top bit set
    }
    lo = lookup_plane<BITS>(&t.r[0], sel, s7, m);
    hi = lookup_plane<BITS>(&t.r[Table<BITS>::kRegs / 2], sel, s7, m);
}

// K table of one token.  `cmax` is the largest |centroid|: rounding is monotonic, so the largest
// table entry is round_T(cmax * norm) and needs no maximum over the entries.  The integer image is
// taken with the 1.5 * 2^23 trick: after v * scale + (1.5 * 2^23 + 128) the low 16 bits of the
// float hold the rounded integer + 128 in two's complement, which is the biased form the two signed
// digit planes are cut from.
template <typename T, int BITS>
__device__ __forceinline__ Table<BITS> build_int_table(const float* cb, float cmax, float norm, float& unscale) {
    constexpr int N = 1 << BITS;
    const float mx = round_to<T>(__fmul_rn(cmax, fabsf(norm)));
    const bool ok = mx >= 1.0e-30f && mx <= 3.0e38f;
    const int e = ok ? exponent_of(mx) : 0;
    const float scale = ok ? pow2i(13 - e) : 0.0f;
    unscale = ok ? pow2i(e - 13) : 0.0f;
    Table<BITS> t;
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        const float2 v01 = unpack_pair<T>(pack_pair<T>(__fmul_rn(cb[4 * i], norm), __fmul_rn(cb[4 * i + 1], norm)));
        const float2 v23 = unpack_pair<T>(pack_pair<T>(__fmul_rn(cb[4 * i + 2], norm), __fmul_rn(cb[4 * i + 3], norm)));
        const uint32_t u0 = __float_as_uint(fmaf(v01.x, scale, 12583040.0f)), u1 = __float_as_uint(fmaf(v01.y, scale, 12583040.0f));
        const uint32_t u2 = __float_as_uint(fmaf(v23.x, scale, 12583040.0f)), u3 = __float_as_uint(fmaf(v23.y, scale, 12583040.0f));
        const uint32_t a = prmt(u0, u1, 0x5140), b = prmt(u2, u3, 0x5140);
        t.r[i] = prmt(a, b, 0x5410) ^ 0x80808080u;
        t.r[N / 4 + i] = prmt(a, b, 0x7632);
    }
    return t;
}
template <typename T, int BITS>
__device__ __forceinline__ Table<BITS> build_value_table(const float* cb, float norm) {
    constexpr int N = 1 << BITS;
    Table<BITS> t;
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        const uint32_t p01 = pack_pair<T>(__fmul_rn(cb[4 * i], norm), __fmul_rn(cb[4 * i + 1], norm));
        const uint32_t p23 = pack_pair<T>(__fmul_rn(cb[4 * i + 2], norm), __fmul_rn(cb[4 * i + 3], norm));
        t.r[i] = prmt(p01, p23, 0x6420);
        t.r[N / 4 + i] = prmt(p01, p23, 0x7531);
    }
    return t;
}

// ---- shared memory of the attention CTA ---------------------------------------------------------
struct DecodeSmem {
    alignas(128) uint16_t v[kPairs * kHeadDim];        // V tile: core (pair/8)*16 + pos/8, core row pair%8
    uint16_t p[kPairs * 16];                           // P tile: core (pair/8)*2 + n/8, core row pair%8
    uint8_t q[kMaxCols * kHeadDim];                    // Q digit planes, K-major: core (n/8)*8 + pos/16
    alignas(16) float cb[2][16];
    float qf[32];                                      // per (head of the tile, query head): q unscale * sm_scale * log2(e)
    float mref[32];                                    // reference maxima, kept by the first lane of every head
    float alpha[32];                                   // rescale factors of a moved reference
    float red_m[8][kQPerHead];                         // per half warp (16 pairs of one head)
    float red_l[8][kQPerHead];
    int scan[4];
    uint64_t full[kMaxStages];                         // copy warp -> K / V warps: "the tile's rows landed"
    uint64_t empty[kMaxStages];                        // K / V warps -> copy warp: rows read (8 arrivals: one per warp)
    uint64_t kready, pvready, vready;                  // K / V warps -> issuer: operands published (128 arrivals each)
    uint64_t bar_s, bar_o, bar_vfree, bar_drain, bar_drain2;   // issuers -> K / V warps: MMAs complete
    uint32_t tmem_base;
    int grow_tile, redo_tile, dead;
    int32_t prefix[kInlinePlanSeqs + 1];
    alignas(1024) uint8_t ring[kRingBytes];            // stages of [region][token][bytes]
};

struct TmaMaps {
    CUtensorMap m[kRegions];
};

// Position on the line of tiles: walks the parts (piece x sequence) of one piece.
struct Walk {
    int seq, tile, t_end;     // current sequence, tile inside it, end of the part
    int64_t x;                // linear position of (seq, tile)
};

// First sequence s with prefix[s + 1] > x (x < prefix[n]).
__device__ __forceinline__ int find_seq(const int32_t* prefix, int n, int64_t x) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid + 1] > x) hi = mid;
        else lo = mid + 1;
    }
    return lo;
}

// NH = query heads computed per KV head: 4 when the GQA group has at most 4 heads, else 8.
template <typename T, int KB, int VB, int NH>
__global__ void __launch_bounds__(kDecodeThreads, kCtasPerSm)
decode_attn_kernel(const DecodeParams p, const __grid_constant__ TmaMaps maps) {
    extern __shared__ uint8_t smem_raw[];
    DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    constexpr int NK = 1 << KB, NV = 1 << VB;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int J = (p.H >> p.ht_shift) * p.head_groups;
    const int64_t group = blockIdx.x / J;
    const int item = static_cast<int>(blockIdx.x % J);
    const int S = p.stages;

    // ---- set-up: barriers, tensor memory, codebooks, tile prefix sums, a zero P tile ----
    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&sm.full[s], p.box_rows > 0 ? 1 : 32);
            mbar_init(&sm.empty[s], 8);
        }
        mbar_init(&sm.kready, kComputeThreads);
        mbar_init(&sm.pvready, kComputeThreads);
        mbar_init(&sm.vready, kComputeThreads);
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_init(&sm.bar_vfree, 1);
        mbar_init(&sm.bar_drain, 1);
        mbar_init(&sm.bar_drain2, 1);
        sm.grow_tile = -1;
        sm.redo_tile = -1;
        sm.dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // P columns a pair never writes (the other KV head's half of its 16 columns) must read as zero
    for (int i = tid; i < kPairs * 16 * 2 / 16; i += kDecodeThreads)
        reinterpret_cast<uint4*>(sm.p)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_proxy();
    if (warp == 0) tmem_alloc(&sm.tmem_base, kTmemCols);
    if (warp == kSIssuerWarp) {
        const int kv = lane >> 4, i = lane & 15;
        const int n = kv ? NV : NK;
        sm.cb[kv][i] = i < n ? __ldg((kv ? p.cent_v : p.cent_k) + i) : 0.0f;
    }
    const int32_t* prefix = p.prefix;
    if (p.inline_plan) {
        // two consecutive sequences per compute thread, warp scan, four warp totals
        int a = 0, b = 0;
        if (tid < kComputeThreads) {
            const int s0 = 2 * tid;
            if (s0 < p.num_seqs) a = (max(__ldg(p.seq_lens + s0), 0) + p.ttok - 1) >> p.ttok_shift;
            if (s0 + 1 < p.num_seqs) b = (max(__ldg(p.seq_lens + s0 + 1), 0) + p.ttok - 1) >> p.ttok_shift;
        }
        int incl = a + b;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31 && warp < 4) sm.scan[warp] = incl;
        tc_fence_before();
        __syncthreads();
        if (tid < kComputeThreads) {
            int before = incl - (a + b);
            for (int w = 0; w < warp; ++w) before += sm.scan[w];
            const int s0 = 2 * tid;
            if (s0 <= p.num_seqs) sm.prefix[s0] = before;
            if (s0 + 1 <= p.num_seqs) sm.prefix[s0 + 1] = before + a;
            if (s0 + 2 == p.num_seqs) sm.prefix[s0 + 2] = before + a + b;
        }
        prefix = sm.prefix;
    } else {
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    if (p.inline_plan && blockIdx.x == 0)          // the merge launch reads the prefix sums from the workspace
        for (int i = tid; i <= p.num_seqs; i += kDecodeThreads) p.prefix[i] = sm.prefix[i];

    const uint32_t tmem = sm.tmem_base;
    const int64_t total = prefix[p.num_seqs];
    const int64_t x0 = piece_begin(p, group, total, J);
    const int64_t x_end = piece_begin(p, group + 1, total, J);
    const bool has_work = group < p.groups && x0 < x_end;

    const int hg = item % p.head_groups;
    const int h0 = (item / p.head_groups) << p.ht_shift;            // first KV head of this CTA's head tile
    const int heads_here = min(kQPerHead, p.G - hg * kQPerHead);     // query heads per KV head handled here
    const int last_blk = static_cast<int>(p.num_blocks) - 1;
    const RegionWindow rw = region_window(p.H, h0);

    auto start_walk = [&](Walk& w) {
        w.x = x0;
        w.seq = find_seq(prefix, p.num_seqs, x0);
        const int pre = prefix[w.seq];
        w.tile = static_cast<int>(x0 - pre);
        const int64_t reach = w.tile + (x_end - x0);
        const int n_s = prefix[w.seq + 1] - pre;
        w.t_end = reach < n_s ? static_cast<int>(reach) : n_s;
    };
    // returns true when the new position is the first tile of a part
    auto advance = [&](Walk& w) -> bool {
        ++w.x;
        ++w.tile;
        if (w.tile < w.t_end || w.x >= x_end) return false;
        do { ++w.seq; } while (w.seq < p.num_seqs - 1 && prefix[w.seq + 1] - prefix[w.seq] <= 0);
        const int n_s = prefix[w.seq + 1] - prefix[w.seq];
        const int64_t left = x_end - w.x;
        w.tile = 0;
        w.t_end = left < n_s ? static_cast<int>(left) : n_s;
        return true;
    };

    bool dead = false;
#ifdef RQ_DECODE_TRACE
    // CTAs 0, 100 and 200: [cta][warp][tile][16 points]
    unsigned long long* trace_row = nullptr;
    if (p.trace != nullptr && blockIdx.x % 100 == 0 && blockIdx.x / 100 < 3 && (warp < kVWarp0 || warp == kSIssuerWarp))
        trace_row = p.trace + ((blockIdx.x / 100) * 5 + (warp == kSIssuerWarp ? 4 : warp)) * 64 * 16;
#endif

    if (has_work && warp == kSIssuerWarp) {
        // ============ S issuer + copy warp: S^T = K Q^T of every tile, and the rows of the tiles ahead ============
        const uint32_t ncols = static_cast<uint32_t>(p.n_cols);
        const uint32_t idesc_s = (2u << 4) | (1u << 7) | (1u << 10) | ((ncols >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t q_addr = smem_u32(sm.q);
        const uint32_t ring_addr = smem_u32(sm.ring);

        // ---- producer: the rows of one tile into ring stage (n % S) ----
        // Lane b keeps the block-table entry of box b of the tile to be produced next, loaded right
        // after the previous tile was issued.
        Walk pw;
        start_walk(pw);
        int produced = 0;
        int p_seq_len = max(__ldg(p.seq_lens + pw.seq), 0);
        int p_blk = 0;
        auto prefetch_blk = [&]() {
            if (p.box_rows > 0 && pw.x < x_end) {
                const int t = (pw.tile << p.ttok_shift) + lane * p.box_rows;
                p_blk = (lane * p.box_rows < p.ttok && t < p_seq_len)
                            ? __ldg(p.block_table + pw.seq * p.bt_stride + (t >> p.bs_shift)) : 0;
            }
        };
        prefetch_blk();
        auto produce = [&]() {
            const int stage = produced % S;
            const uint32_t bar = smem_u32(&sm.full[stage]);
            const uint32_t dst0 = ring_addr + static_cast<uint32_t>(stage * p.stage_bytes);
            const int tok0 = pw.tile << p.ttok_shift;
            const int n_valid = min(p.ttok, p_seq_len - tok0);
            if (p.box_rows > 0) {
                const int n_box = (n_valid + p.box_rows - 1) / p.box_rows;       // at most 16: one per lane
                int row_bytes = 0;
                for (int r = 0; r < p.n_regions; ++r) row_bytes += p.reg_w[r];
                if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_box * p.box_rows * row_bytes));
                __syncwarp();
                if (lane < n_box) {
                    const int t = tok0 + lane * p.box_rows;
                    const int blk = p_blk < 0 ? 0 : (p_blk > last_blk ? last_blk : p_blk);
                    const int slot = (blk << p.bs_shift) + (t & (p.block_size - 1));
#pragma unroll
                    for (int r = 0; r < kRegions; ++r)
                        if (r < p.n_regions)
                            tma_load_2d(dst0 + p.reg_base[r] + lane * p.box_rows * p.reg_w[r], &maps.m[r],
                                        (p.n_regions == 1 ? 0 : rw.x[r]) >> 3, slot, bar);
                }
            } else {
                // any block size: 4-byte copies of every region's window, token by token
                const int32_t* bt_row = p.block_table + pw.seq * p.bt_stride;
                for (int r = 0; r < p.n_regions; ++r) {
                    const int words = p.reg_w[r] >> 2;
                    const int src_x = p.n_regions == 1 ? 0 : rw.x[r];
                    for (int i = lane; i < n_valid * words; i += 32) {
                        const int tt = i / words, wd = i - tt * words;
                        const int t = tok0 + tt;
                        const int bi = p.bs_shift >= 0 ? (t >> p.bs_shift) : (t / p.block_size);
                        const int off = p.bs_shift >= 0 ? (t & (p.block_size - 1)) : (t % p.block_size);
                        int blk = __ldg(bt_row + bi);
                        blk = blk < 0 ? 0 : (blk > last_blk ? last_blk : blk);
                        const uint8_t* slot = p.cache + (static_cast<int64_t>(blk) * p.block_size + off) * p.total_bytes;
                        cp_async4(dst0 + p.reg_base[r] + tt * p.reg_w[r] + 4 * wd, slot + src_x + 4 * wd);
                    }
                }
                cp_async_arrive(&sm.full[stage]);
            }
            __syncwarp();
            ++produced;
            if (advance(pw)) p_seq_len = max(__ldg(p.seq_lens + pw.seq), 0);
            prefetch_blk();
        };
        // Tile n >= S may be copied once the K and the V warps have read the rows of tile n - S out of its
        // stage.  Tiles the next iteration cannot do without are waited for; further ahead, a stage that
        // is not free yet is simply tried again later.
        auto produce_ahead = [&](int it_now) {
            while (pw.x < x_end && !dead) {
                const int n = produced;
                if (n >= S) {
                    const uint32_t parity = ((n / S) - 1) & 1;
                    if (n <= it_now + 1) {
                        if (!mbar_wait(&sm.empty[n % S], parity)) { dead = true; return; }
                    } else if (!mbar_test(&sm.empty[n % S], parity)) {
                        return;
                    }
                }
                produce();
            }
        };
        produce_ahead(-1);

        Walk cw;
        start_walk(cw);
        int it = 0;
#pragma unroll 1
        for (; cw.x < x_end && !dead; ++it) {
            // the digit planes of the tile are in tensor memory, the query planes in shared memory
            RQ_TRACE(0);
            if (!mbar_wait(&sm.kready, it & 1)) { dead = true; break; }
            RQ_TRACE(1);
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    tc_mma_i8_ta(tmem + kColS, tmem + kColKhi + 8 * s, smem_desc(q_addr + 256 * s, 128, 1024),
                                 idesc_s, s > 0 ? 1u : 0u);
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    tc_mma_i8_ta(tmem + kColS2, tmem + kColKlo + 8 * s, smem_desc(q_addr + 256 * s, 128, 1024),
                                 idesc_s, s > 0 ? 1u : 0u);
                tc_commit(&sm.bar_s);
            }
            __syncwarp();
            RQ_TRACE(2);
            produce_ahead(it);
            RQ_TRACE(5);
            advance(cw);
        }
        if (dead) {
            st_volatile_shared(&sm.dead, 1);
            // copies still in flight: a bounded wait each, so that none lands after the CTA is gone
            if (p.box_rows > 0)
                for (int c = max(0, produced - S); c < produced; ++c) mbar_wait(&sm.full[c % S], (c / S) & 1);
            if (lane == 0) tc_commit(&sm.bar_drain);
            __syncwarp();
            mbar_wait(&sm.bar_drain, 0);
        }
        cp_async_wait_all();
    } else if (has_work && warp == kPvIssuerWarp) {
        // ============ P V issuer: O^T += V^T [P hi | P lo], one k-step of 16 pairs (one KV head) at a time ============
        const uint32_t idesc_o = (1u << 4) | (TcFormat<T>::kFmt << 7) | (TcFormat<T>::kFmt << 10) | (1u << 15) |
                                 (1u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);
        Walk cw;
        start_walk(cw);
        bool first_in_part = true;
        uint32_t ph_pv = 0;
        int it = 0;
        const int cols_per_head = 2 * NH;
#pragma unroll 1
        for (; cw.x < x_end; ++it) {
            if (!mbar_wait(&sm.pvready, ph_pv)) { dead = true; break; }
            ph_pv ^= 1u;
            if (ld_volatile_shared(&sm.grow_tile) == it) {
                // a score outgrew the reference maximum: hand the tile back; the K warps move the
                // maxima, rescale, rewrite P and publish again
                if (lane == 0) {
                    st_volatile_shared(&sm.redo_tile, it);
                    mbar_arrive(&sm.bar_o);
                }
                __syncwarp();
                if (!mbar_wait(&sm.pvready, ph_pv)) { dead = true; break; }
                ph_pv ^= 1u;
            }
            if (!mbar_wait(&sm.vready, it & 1)) { dead = true; break; }
            tc_fence_after();
            if (lane == 0) {
                int prev_blk = -1;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    // output columns of the KV head of pairs 16 s .. 16 s + 15, as a block of 16
                    const int blk16 = (((16 * s) >> p.ttok_shift) * cols_per_head) >> 4;
                    const uint32_t acc = (first_in_part && blk16 != prev_blk) ? 0u : 1u;
                    prev_blk = blk16;
                    tc_mma_f16(tmem + kColO + 16 * blk16, smem_desc(v_addr + 4096 * s, 2048, 128),
                               smem_desc(p_addr + 512 * s, 256, 128), idesc_o, acc);
                }
                tc_commit(&sm.bar_o);
                tc_commit(&sm.bar_vfree);
            }
            __syncwarp();
            first_in_part = advance(cw);
        }
        if (dead) {
            st_volatile_shared(&sm.dead, 1);
            if (lane == 0) tc_commit(&sm.bar_drain2);
            __syncwarp();
            mbar_wait(&sm.bar_drain2, 0);
        }
    } else if (has_work && warp < kVWarp0) {
        // =========================== K warps: digit planes, scores, softmax ===========================
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's lane quarter
        const int hh = tid >> p.ttok_shift, tt = tid & (p.ttok - 1);      // this pair: KV head of the tile, token
        const int half = tid >> 4;                                         // 16 pairs of one head
        const int halves_per_head = p.ttok >> 4, first_half = (half / halves_per_head) * halves_per_head;
        const int col16 = (hh * 2 * NH) & ~15, sub = (hh * 2 * NH) & 15;   // this head's columns: block of 16, offset
        // P: this pair's row of 16 columns; with 4 query heads its 8 values fill one 8-column core
        uint8_t* const p_dst = reinterpret_cast<uint8_t*>(sm.p) + (tid >> 3) * (2 * 128) + (tid & 7) * 16 +
                               (NH == 4 ? (sub >> 3) * 128 : 0);
        // where this pair's bytes sit inside a stage
        int f_off[kRegions];
#pragma unroll
        for (int r = 0; r < kRegions; ++r) {
            const int unit = (r & 1) ? 4 : kHalfDim;
            f_off[r] = p.n_regions == 1 ? tt * p.reg_w[0] + rw.start[r] + unit * hh
                                        : p.reg_base[r] + tt * p.reg_w[r] + (rw.start[r] - rw.x[r]) + unit * hh;
        }
        float cmax_k = 0.0f;
#pragma unroll
        for (int i = 0; i < NK; ++i) cmax_k = fmaxf(cmax_k, fabsf(sm.cb[0][i]));

        uint32_t ph_o = 0;
        int it = 0;                                // tiles streamed by this CTA so far
        int stage = 0;                             // it % S, and the parity of that stage's "landed" barrier
        uint32_t ph_full = 0;
        int64_t x = x0;
        int seq = find_seq(prefix, p.num_seqs, x0);

#pragma unroll 1
        while (x < x_end && seq < p.num_seqs && !dead) {
            const int pre = prefix[seq], n_s = prefix[seq + 1] - pre;
            if (n_s <= 0 || x >= static_cast<int64_t>(pre) + n_s) { ++seq; continue; }
            const int t_begin = static_cast<int>(x - pre);
            const int64_t reach = t_begin + (x_end - x);
            const int t_end = reach < n_s ? static_cast<int>(reach) : n_s;
            const int seq_len = max(__ldg(p.seq_lens + seq), 0);

            // ---- queries of this part: rotate, round, quantise to signed digit planes (B operand) ----
            // rows of head j of the tile: 2 NH j + g (high digits of query head g), 2 NH j + NH + g (low digits)
#pragma unroll 1
            for (int jq = warp; jq < (NH << p.ht_shift); jq += 4) {
                const int j = jq / NH, g = jq % NH;
                float r[4] = {0.f, 0.f, 0.f, 0.f};
                if (g < heads_here) {
                    const int qh = (h0 + j) * p.G + hg * kQPerHead + g;
                    const T* qp = static_cast<const T*>(p.q) + seq * p.q_stride_seq +
                                  static_cast<int64_t>(qh) * p.q_stride_head + 4 * lane;
                    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(qp));
                    const float2 x01 = unpack_pair<T>(raw.x), x23 = unpack_pair<T>(raw.y);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 rr = __ldg(reinterpret_cast<const float4*>(
                            p.rotation + (4 * lane + k) * kHeadDim + 4 * lane));
                        float acc = __fmul_rn(x01.x, rr.x);
                        acc = __fmaf_rn(x01.y, rr.y, acc);
                        acc = __fmaf_rn(x23.x, rr.z, acc);
                        acc = __fmaf_rn(x23.y, rr.w, acc);
                        r[k] = round_to<T>(acc);
                    }
                }
                float mx = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const bool ok = mx >= 1.0e-30f && mx <= 3.0e38f;
                const int e = ok ? exponent_of(mx) : 0;
                const float scale = ok ? pow2i(13 - e) : 0.0f;
                int qu[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) qu[k] = __float2int_rn(fmaf(r[k], scale, 128.0f));
                // position x of a row holds head-dim x ^ 1 (the nibble order of the cache)
                const uint32_t a = prmt(qu[1], qu[0], 0x5140), b = prmt(qu[3], qu[2], 0x5140);
                const int row_hi = 2 * NH * j + g, row_lo = row_hi + NH;
                const uint32_t in_row = (lane >> 2) * 128 + 4 * (lane & 3);
                *reinterpret_cast<uint32_t*>(&sm.q[(row_hi >> 3) * 1024 + (row_hi & 7) * 16 + in_row]) = prmt(a, b, 0x7632);
                *reinterpret_cast<uint32_t*>(&sm.q[(row_lo >> 3) * 1024 + (row_lo & 7) * 16 + in_row]) =
                    prmt(a, b, 0x5410) ^ 0x80808080u;
                if (lane == 0) sm.qf[NH * j + g] = (ok ? pow2i(e - 13) : 0.0f) * p.qk_scale;
            }
            fence_async_proxy();
            compute_sync();

            float m_ref[NH], l_acc[NH], l_pend[NH], sc[NH], qfk[NH];
#pragma unroll
            for (int g = 0; g < NH; ++g) {
                m_ref[g] = -INFINITY; l_acc[g] = 0.0f; l_pend[g] = 0.0f; sc[g] = 0.0f;
                qfk[g] = sm.qf[NH * hh + g];
            }
            bool pending = false;                    // a P V of this part has been requested and not yet awaited

            // probabilities of the tile whose scores are in sc[], against the current reference maxima
            auto emit_p = [&]() {
#pragma unroll
                for (int g = 0; g < NH; ++g) l_pend[g] = ex2_approx(sc[g] - m_ref[g]);
                uint32_t ph[NH / 2], pl[NH / 2];
#pragma unroll
                for (int j = 0; j < NH / 2; ++j) {
                    ph[j] = pack_pair<T>(l_pend[2 * j], l_pend[2 * j + 1]);
                    const float2 back = unpack_pair<T>(ph[j]);
                    pl[j] = pack_pair<T>(l_pend[2 * j] - back.x, l_pend[2 * j + 1] - back.y);
                }
                if constexpr (NH == 4) {
                    *reinterpret_cast<uint4*>(p_dst) = make_uint4(ph[0], ph[1], pl[0], pl[1]);
                } else {
                    *reinterpret_cast<uint4*>(p_dst) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                    *reinterpret_cast<uint4*>(p_dst + 128) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                }
                fence_async_proxy();
            };
            // maximum of sc[] over the pairs of this thread's KV head -> m_new[]
            auto head_max = [&](float (&m_new)[NH]) {
#pragma unroll
                for (int g = 0; g < NH; ++g) {
                    float m = sc[g];
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                    if ((lane & 15) == 0) sm.red_m[half][g] = m;
                }
                compute_sync();
#pragma unroll
                for (int g = 0; g < NH; ++g) {
                    float m = sm.red_m[first_half][g];
                    for (int i = 1; i < halves_per_head; ++i) m = fmaxf(m, sm.red_m[first_half + i][g]);
                    m_new[g] = m;
                }
                compute_sync();                      // red_m may be rewritten from here on
            };
            // Wait for the P V of tile `it - 1`; if the issuer handed the tile back because a score
            // outgrew the reference, move the maxima, rescale the sums, publish P again and wait again.
            auto settle_pending = [&]() {
                if (!mbar_wait(&sm.bar_o, ph_o)) { dead = true; return; }
                ph_o ^= 1u;
                tc_fence_after();
                if (ld_volatile_shared(&sm.redo_tile) == it - 1) {
                    float m_new[NH];
                    head_max(m_new);
#pragma unroll
                    for (int g = 0; g < NH; ++g) {
                        m_new[g] = fmaxf(m_new[g], m_ref[g]);
                        const float a = ex2_approx(m_ref[g] - m_new[g]);
                        l_acc[g] *= a;
                        m_ref[g] = m_new[g];
                        if (tt == 0) { sm.alpha[NH * hh + g] = a; sm.mref[NH * hh + g] = m_new[g]; }
                    }
                    compute_sync();
                    // O^T: lane = head-dim, column 2 NH j + g (+ NH: the lo part) = query head g of head j
                    for (int c0 = 0; c0 < p.n_cols; c0 += 16) {
                        uint32_t o[16];
                        tmem_ld16_nowait(lane_base + kColO + c0, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int col = c0 + c, j = col / (2 * NH), g = col % NH;
                            const float a = j < p.ht ? sm.alpha[NH * j + g] : 1.0f;
                            o[c] = __float_as_uint(__uint_as_float(o[c]) * a);
                        }
                        tmem_st16_nowait(lane_base + kColO + c0, o);
                    }
                    tmem_wait_st();
                    emit_p();
                    tc_fence_before();
                    mbar_arrive(&sm.pvready);
                    if (!mbar_wait(&sm.bar_o, ph_o)) { dead = true; return; }
                    ph_o ^= 1u;
                    tc_fence_after();
                }
#pragma unroll
                for (int g = 0; g < NH; ++g) l_acc[g] += l_pend[g];
                pending = false;
            };

#pragma unroll 1
            for (int tile = t_begin; tile < t_end; ++tile, ++it) {
                const bool valid = (tile << p.ttok_shift) + tt < seq_len;
                const uint8_t* stg = sm.ring + stage * p.stage_bytes;
                const int this_stage = stage;
                RQ_TRACE(0);
                if (!mbar_wait(&sm.full[stage], ph_full)) { dead = true; break; }
                if (++stage == S) { stage = 0; ph_full ^= 1u; }
                RQ_TRACE(1);

                // ---- K table, digit planes -> tensor memory ----
                float k_unscale;
                {
                    // a zero norm makes every table entry zero: pairs past the end contribute nothing
                    const float nk = valid ? *reinterpret_cast<const float*>(stg + f_off[1]) : 0.0f;
                    float cbk[NK];
#pragma unroll
                    for (int i = 0; i < NK; i += 4) {
                        const float4 c4 = *reinterpret_cast<const float4*>(&sm.cb[0][i]);
                        cbk[i] = c4.x; cbk[i + 1] = c4.y; cbk[i + 2] = c4.z; cbk[i + 3] = c4.w;
                    }
                    const Table<KB> tk = build_int_table<T, KB>(cbk, cmax_k, nk, k_unscale);
                    const uint8_t* krow = stg + f_off[0];
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const uint4 w0 = *reinterpret_cast<const uint4*>(krow + 32 * hf);
                        const uint4 w1 = *reinterpret_cast<const uint4*>(krow + 32 * hf + 16);
                        const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                        uint32_t hi[16], lo[16];
#pragma unroll
                        for (int w = 0; w < 8; ++w) {
                            lookup4<KB>(tk, words[w], lo[2 * w], hi[2 * w]);
                            lookup4<KB>(tk, words[w] >> 16, lo[2 * w + 1], hi[2 * w + 1]);
                        }
                        tmem_st16_nowait(lane_base + kColKhi + 16 * hf, hi);
                        tmem_st16_nowait(lane_base + kColKlo + 16 * hf, lo);
                    }
                }
                RQ_TRACE(2);
                __syncwarp();                        // every lane holds its K row and norm in registers:
                if (lane == 0) mbar_arrive(&sm.empty[this_stage]);   // this warp is done with the stage
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&sm.kready);
                RQ_TRACE(3);

                // ---- the previous tile's P V must be complete before P is rewritten (and may hand the tile back) ----
                if (pending) {
                    settle_pending();
                    if (dead) break;
                }
                RQ_TRACE(4);
                uint32_t d1[16], d2[16];                     // this pair's sums: 16 columns of each accumulator
                RQ_TRACE(5);
                if (!mbar_wait(&sm.bar_s, it & 1)) { dead = true; break; }
                RQ_TRACE(6);
                tc_fence_after();
                tmem_ld16_nowait(lane_base + kColS + col16, d1);
                tmem_ld16_nowait(lane_base + kColS2 + col16, d2);

                // ---- scores, reference maxima, probabilities ----
                const float tok_bias = valid ? 0.0f : -INFINITY;
                RQ_TRACE(7);
                {
                    tmem_wait_ld();
                    RQ_TRACE(8);
                    tmem_ld16_landed(d1);
                    tmem_ld16_landed(d2);
#pragma unroll
                    for (int g = 0; g < NH; ++g) {
                        // columns of this head: sub + g = Q high digits of query head g, sub + NH + g = low digits
                        int hh_, hl_, lh_, ll_;
                        if constexpr (NH == 4) {
                            hh_ = static_cast<int>(sub ? d1[8 + g] : d1[g]);
                            hl_ = static_cast<int>(sub ? d1[12 + g] : d1[4 + g]);
                            lh_ = static_cast<int>(sub ? d2[8 + g] : d2[g]);
                            ll_ = static_cast<int>(sub ? d2[12 + g] : d2[4 + g]);
                        } else {
                            hh_ = static_cast<int>(d1[g]); hl_ = static_cast<int>(d1[8 + g]);
                            lh_ = static_cast<int>(d2[g]); ll_ = static_cast<int>(d2[8 + g]);
                        }
                        const int t1 = hh_ * 256 + (hl_ + lh_);
                        const float f = fmaf(static_cast<float>(t1), 256.0f, static_cast<float>(ll_));
                        // query heads beyond the group have factor 0: they behave like heads with all-zero scores
                        // and their columns are never written out; pairs past the end get -inf (probability 0)
                        sc[g] = fmaf(f, qfk[g] * k_unscale, tok_bias);
                    }
                }
                if (tile == t_begin) {
                    // first tile of the part: the reference maxima are the exact maxima of this tile
                    float m_new[NH];
                    head_max(m_new);
#pragma unroll
                    for (int g = 0; g < NH; ++g) {
                        m_ref[g] = m_new[g];
                        if (tt == 0) sm.mref[NH * hh + g] = m_new[g];
                    }
                } else {
                    bool grow = false;
#pragma unroll
                    for (int g = 0; g < NH; ++g) grow |= sc[g] > m_ref[g] + 8.0f;
                    // rare: ask the issuer to hand the tile back instead of issuing its P V
                    if (grow) st_volatile_shared(&sm.grow_tile, it);
                }
                emit_p();
                tc_fence_before();
                mbar_arrive(&sm.pvready);
                RQ_TRACE(9);
                pending = true;
            }
            if (dead) break;

            // ---- partial result of this part -> workspace row (group + sequence) * J + item ----
            if (pending) {
                settle_pending();
                if (dead) break;
            }
#pragma unroll
            for (int g = 0; g < NH; ++g) {
                float v = l_acc[g];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if ((lane & 15) == 0) sm.red_l[half][g] = v;
            }
            compute_sync();
            const int64_t row = (group + seq) * J + item;
            const int slots = p.ht * kQPerHead;
            if (tid < p.ht * NH) {
                const int j = tid / NH, g = tid % NH;
                if (g < heads_here) {
                    float l = 0.0f;
                    for (int i = 0; i < halves_per_head; ++i) l += sm.red_l[j * halves_per_head + i][g];
                    p.ws_m[row * slots + j * kQPerHead + g] = sm.mref[NH * j + g];
                    p.ws_l[row * slots + j * kQPerHead + g] = l;
                }
            }
            for (int c0 = 0; c0 < p.ht * 2 * NH; c0 += 16) {
                uint32_t o[16];
                tmem_ld16_nowait(lane_base + kColO + c0, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    // columns come in groups of 2 NH per head: NH hi parts, then NH lo parts
                    if ((c % (2 * NH)) < NH) {
                        const int j = (c0 + c) / (2 * NH), g = c % NH;
                        if (g < heads_here && j < p.ht)      // lane (position) x holds head-dim x ^ 1
                            p.ws_o[((row * slots + j * kQPerHead + g) << 7) + (tid ^ 1)] =
                                __uint_as_float(o[c]) + __uint_as_float(o[c + NH]);
                    }
                }
            }
            tc_fence_before();
            compute_sync();                          // red_l, the query planes and O^T are free for the next part

            x += t_end - t_begin;
            if (t_end == n_s) ++seq;
        }
        if (dead) st_volatile_shared(&sm.dead, 1);
    } else if (has_work) {
        // =========================== V warps: V rows -> shared V tile ===========================
        const int pair = tid - 32 * kVWarp0;
        uint8_t* const v_dst = reinterpret_cast<uint8_t*>(sm.v) + (pair >> 3) * (16 * 128) + (pair & 7) * 16;
        const int hh = pair >> p.ttok_shift, tt = pair & (p.ttok - 1);
        const int unit_v = kHalfDim;
        const int v_off = p.n_regions == 1 ? tt * p.reg_w[0] + rw.start[2] + unit_v * hh
                                           : p.reg_base[2] + tt * p.reg_w[2] + (rw.start[2] - rw.x[2]) + unit_v * hh;
        const int vn_off = p.n_regions == 1 ? tt * p.reg_w[0] + rw.start[3] + 4 * hh
                                            : p.reg_base[3] + tt * p.reg_w[3] + (rw.start[3] - rw.x[3]) + 4 * hh;
        Walk vw;
        start_walk(vw);
        int seq_len = max(__ldg(p.seq_lens + vw.seq), 0);
        int stage = 0;
        uint32_t ph_full = 0;
#pragma unroll 1
        for (int it = 0; vw.x < x_end; ++it) {
            const bool valid = (vw.tile << p.ttok_shift) + tt < seq_len;
            const uint8_t* stg = sm.ring + stage * p.stage_bytes;
            const int this_stage = stage;
            if (!mbar_wait(&sm.full[stage], ph_full)) { dead = true; break; }
            if (++stage == S) { stage = 0; ph_full ^= 1u; }
            float cbv[NV];
#pragma unroll
            for (int i = 0; i < NV; i += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(&sm.cb[1][i]);
                cbv[i] = c4.x; cbv[i + 1] = c4.y; cbv[i + 2] = c4.z; cbv[i + 3] = c4.w;
            }
            Table<VB> tb = build_value_table<T, VB>(cbv, *reinterpret_cast<const float*>(stg + vn_off));
            if (!valid) {
                // rows past the end of the sequence may hold bytes that are not index nibbles; with an
                // all-zero table every PRMT result is zero whatever the selector (a -0.0 entry would
                // turn a selector with its top bit set into a sign mask, i.e. a NaN pattern in fp16)
#pragma unroll
                for (int r = 0; r < Table<VB>::kRegs; ++r) tb.r[r] = 0u;
            }
            const uint8_t* vrow = stg + v_off;
            uint32_t words[16];
            if (p.v_aligned) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 w4 = *reinterpret_cast<const uint4*>(vrow + 16 * c);
                    words[4 * c] = w4.x; words[4 * c + 1] = w4.y; words[4 * c + 2] = w4.z; words[4 * c + 3] = w4.w;
                }
            } else {
#pragma unroll
                for (int w = 0; w < 16; ++w) words[w] = *reinterpret_cast<const uint32_t*>(vrow + 4 * w);
            }
            __syncwarp();                            // every lane holds its V row and norm in registers:
            if (lane == 0) mbar_arrive(&sm.empty[this_stage]);  // this warp is done with the stage
            // the V tile is free once the previous tile's P V has read it
            if (it > 0 && !mbar_wait(&sm.bar_vfree, (it - 1) & 1)) { dead = true; break; }
#pragma unroll
            for (int w = 0; w < 16; ++w) {                 // 8 head-dims = one 32-bit index word per chunk
                uint32_t lo0, hi0, lo1, hi1;
                lookup4<VB>(tb, words[w], lo0, hi0);
                lookup4<VB>(tb, words[w] >> 16, lo1, hi1);
                *reinterpret_cast<uint4*>(v_dst + w * 128) =
                    make_uint4(prmt(lo0, hi0, 0x5140), prmt(lo0, hi0, 0x7362),
                               prmt(lo1, hi1, 0x5140), prmt(lo1, hi1, 0x7362));
            }
            fence_async_proxy();
            mbar_arrive(&sm.vready);
            if (advance(vw)) seq_len = max(__ldg(p.seq_lens + vw.seq), 0);
        }
        if (dead) st_volatile_shared(&sm.dead, 1);
    }

    if (tid == 0) grid_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (has_work && ld_volatile_shared(&sm.dead) != 0) {
        // A bounded wait expired somewhere in this CTA: every part of its piece is marked invalid
        // (NaN row sum), which the merge turns into NaN outputs.
        int64_t x = x0;
        int seq = find_seq(prefix, p.num_seqs, x0);
        const int slots = p.ht * kQPerHead;
        while (x < x_end && seq < p.num_seqs) {
            const int pre = prefix[seq], n_s = prefix[seq + 1] - pre;
            if (n_s <= 0 || x >= static_cast<int64_t>(pre) + n_s) { ++seq; continue; }
            const int64_t left = x_end - x, in_seq = static_cast<int64_t>(pre) + n_s - x;
            const int64_t row = (group + seq) * J + item;
            if (tid < slots) {
                p.ws_m[row * slots + tid] = 0.0f;
                p.ws_l[row * slots + tid] = __int_as_float(0x7fc00000);
            }
            x += left < in_seq ? left : in_seq;
            ++seq;
        }
    }
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// Tiles of every sequence as an exclusive prefix sum, for batches too large for the attention CTAs
// to scan themselves: prefix[s] = sum_{s' < s} ceil(len[s'] / tile_tokens), prefix[num_seqs] = total.
__global__ void decode_plan_kernel(const int32_t* __restrict__ seq_lens, int num_seqs, int tile_tokens,
                                   int32_t* __restrict__ prefix) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < num_seqs; base += blockDim.x) {
        const int s = base + threadIdx.x;
        const int n = s < num_seqs ? (max(__ldg(seq_lens + s), 0) + tile_tokens - 1) / tile_tokens : 0;
        int incl = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if ((threadIdx.x & 31) >= o) incl += v;
        }
        if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = incl;
        __syncthreads();
        int before = carry;
        for (int w = 0; w < (threadIdx.x >> 5); ++w) before += warp_sums[w];
        if (s < num_seqs) prefix[s] = before + incl - n;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) prefix[num_seqs] = carry;
}

// Merge: one warp per (sequence, query head), lane l owns head-dims 4l..4l+3 (one 4x4 block of R).
// The parts of a (sequence, head) are the groups whose pieces overlap the sequence's tile range;
// part (group, sequence) of item j lives at row (group + sequence) * J + j, and inside the row the
// query head sits in slot (KV head within its tile) * 8 + (query head within its group of 8).  Lanes
// gather the running maxima and row sums of up to 32 parts at a time; then the warp sums the
// weighted partial outputs.
constexpr int kMergeWarps = 4;
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32)
decode_merge_kernel(const DecodeParams p) {
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int64_t wq = static_cast<int64_t>(blockIdx.x) * kMergeWarps + (threadIdx.x >> 5);
    if (wq >= static_cast<int64_t>(p.num_seqs) * p.Hq) return;
    const int seq = static_cast<int>(wq / p.Hq), qh = static_cast<int>(wq % p.Hq);
    const int J = (p.H >> p.ht_shift) * p.head_groups;
    const int kvh = qh / p.G, hl = qh % p.G;
    const int item = (kvh >> p.ht_shift) * p.head_groups + hl / kQPerHead;
    const int slots = p.ht * kQPerHead;
    const int slot = (kvh & (p.ht - 1)) * kQPerHead + hl % kQPerHead;
    const int64_t a = p.prefix[seq], n = p.prefix[seq + 1] - a, total = p.prefix[p.num_seqs];

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l_all = 0.0f;
    if (n > 0) {
        // group holding tile t: the first g whose piece ends beyond t (32 candidates per round)
        auto group_of = [&](int64_t t) -> int {
            int lo = 0, hi = p.groups - 1;
            while (lo < hi) {
                const int step = (hi - lo + 30) / 31;                 // candidate 31 is always `hi`
                const int c = min(lo + lane * step, hi);
                const unsigned beyond = __ballot_sync(0xffffffffu, piece_begin(p, c + 1, total, J) > t);
                const int f = __ffs(beyond) - 1;
                const int new_hi = min(lo + f * step, hi);
                lo = f == 0 ? lo : min(lo + (f - 1) * step, hi) + 1;
                hi = new_hi;
            }
            return lo;
        };
        const int g_first = group_of(a), g_last = group_of(a + n - 1);
        float m_all = -INFINITY;
        for (int g0 = g_first; g0 <= g_last; g0 += 32) {             // normally one round
            const int gi = g0 + lane;
            // groups whose piece is empty (only when there are more groups than tiles) wrote nothing
            const bool live = gi <= g_last && piece_begin(p, gi, total, J) < piece_begin(p, gi + 1, total, J);
            const int64_t r = ((static_cast<int64_t>(gi) + seq) * J + item) * slots + slot;
            const float m = live ? p.ws_m[r] : -INFINITY;
            const float l = live ? p.ws_l[r] : 0.0f;
            float m_round = m;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m_round = fmaxf(m_round, __shfl_xor_sync(0xffffffffu, m_round, o));
            const float m_new = fmaxf(m_all, m_round);
            const float w = live ? exp2f(m - m_new) : 0.0f;
            float l_round = w * l;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l_round += __shfl_xor_sync(0xffffffffu, l_round, o);
            const float rescale = exp2f(m_all - m_new);                  // 0 in the first round
            acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
            l_all = l_all * rescale + l_round;
            m_all = m_new;
            const int n_here = min(32, g_last - g0 + 1);
#pragma unroll 4
            for (int k = 0; k < n_here; ++k) {
                const float wk = __shfl_sync(0xffffffffu, w, k);
                if (wk != 0.0f) {
                    const float4 o = *reinterpret_cast<const float4*>(
                        p.ws_o + ((((static_cast<int64_t>(g0 + k) + seq) * J + item) * slots + slot) << 7) + 4 * lane);
                    acc.x += wk * o.x; acc.y += wk * o.y; acc.z += wk * o.z; acc.w += wk * o.w;
                }
            }
        }
    }
    // an empty sequence yields zeros
    const float o[4] = {n > 0 ? round_to<T>(acc.x / l_all) : 0.0f, n > 0 ? round_to<T>(acc.y / l_all) : 0.0f,
                        n > 0 ? round_to<T>(acc.z / l_all) : 0.0f, n > 0 ? round_to<T>(acc.w / l_all) : 0.0f};
    // out[j] = sum_k o[k] R[k][j] over the 4x4 block of j, ascending k, fused multiply-adds
    float r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float4 rr = __ldg(reinterpret_cast<const float4*>(p.rotation + (4 * lane + k) * kHeadDim + 4 * lane));
        if (k == 0) {
            r[0] = __fmul_rn(o[0], rr.x); r[1] = __fmul_rn(o[0], rr.y); r[2] = __fmul_rn(o[0], rr.z); r[3] = __fmul_rn(o[0], rr.w);
        } else {
            r[0] = __fmaf_rn(o[k], rr.x, r[0]); r[1] = __fmaf_rn(o[k], rr.y, r[1]);
            r[2] = __fmaf_rn(o[k], rr.z, r[2]); r[3] = __fmaf_rn(o[k], rr.w, r[3]);
        }
    }
    T* dst = static_cast<T*>(p.out) + seq * p.o_stride_seq + static_cast<int64_t>(qh) * p.o_stride_head + 4 * lane;
    const uint2 packed = make_uint2(pack_pair<T>(r[0], r[1]), pack_pair<T>(r[2], r[3]));
    if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
        *reinterpret_cast<uint2*>(dst) = packed;
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) store_rounded(dst + j, r[j]);
    }
}

// ---- host side -------------------------------------------------------------------------------

static int env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return (e != nullptr && e[0] != '\0') ? std::atoi(e) : fallback;
}

#ifdef RQ_DECODE_TRACE
static unsigned long long* g_trace_buffer = nullptr;
#endif

// SM count of the current device (148 on a B200), looked up once per device.
static int sm_count() {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Tile geometry and scratch of one decode call.  A tile holds `ht` KV heads x 128 / ht tokens; the
// (sequence, tile) space is cut into `groups` pieces and each piece is walked by J CTAs, one per
// (head tile, group of 8 query heads per KV head).
struct DecodePlan {
    int nh;                // query heads computed per KV head and item: 4 or 8
    int ht, ht_shift;      // KV heads per tile
    int J;                 // items
    int groups;            // pieces
    size_t rows;           // partial-result rows: (group + sequence) * J + item, ht * 8 slots each
    size_t prefix_bytes;
    size_t bytes;
};
// The head tile: the largest of 1, 2, 4, 8 that divides the KV heads and whose query heads fit the
// 64 accumulator columns (2 digit planes x nh query heads per KV head).  `forced` > 0 asks for that
// many pieces per sequence.
static DecodePlan plan_decode(int num_seqs, int H, int G, int max_seq_len, int forced) {
    DecodePlan pl;
    pl.nh = G <= 4 ? 4 : 8;
    pl.ht = 1;
    pl.ht_shift = 0;
    for (int c = 2, s = 1; c <= 8; c <<= 1, ++s)
        if (H % c == 0 && c * 2 * pl.nh <= kMaxCols) { pl.ht = c; pl.ht_shift = s; }
    const int head_groups = (G + kQPerHead - 1) / kQPerHead;
    pl.J = (H / pl.ht) * head_groups;
    const int ttok = kPairs / pl.ht;
    const long long max_tiles = max_seq_len > 0 ? (max_seq_len + ttok - 1) / ttok : 1;
    const long long work = 1LL * num_seqs * max_tiles;
    long long groups = forced > 0 ? 1LL * forced * num_seqs : work;
    long long cap = (forced > 0 ? 4LL : 1LL) * sm_count() * kCtasPerSm / pl.J;
    if (cap < 1) cap = 1;
    if (groups > cap) groups = cap;
    if (groups < 1) groups = 1;
    pl.groups = static_cast<int>(groups);
    pl.rows = static_cast<size_t>((groups + num_seqs) * pl.J);
    pl.prefix_bytes = (static_cast<size_t>(num_seqs + 1) * sizeof(int32_t) + 255) / 256 * 256;
    pl.bytes = pl.prefix_bytes + pl.rows * pl.ht * kQPerHead * (kHeadDim + 2) * sizeof(float);
    return pl;
}

// ---- tensor maps of the cache ------------------------------------------------------------------
//
// The cache is described as a 2-D tensor of 8-byte elements (num_slots rows of total_bytes / 8): one
// map per staged region, box = (region width, tokens per box), no swizzle.  cuTensorMapEncodeTiled is
// a driver entry point; it is looked up through the runtime so that the library does not link against
// the driver.  Maps are remembered per (cache pointer, shape, box): a serving loop calls with the same
// cache every step.

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

struct MapKey {
    const void* cache;
    int64_t num_slots;
    int total_bytes, box_bytes, box_rows;
    bool operator==(const MapKey& o) const {
        return cache == o.cache && num_slots == o.num_slots && total_bytes == o.total_bytes &&
               box_bytes == o.box_bytes && box_rows == o.box_rows;
    }
};

static bool encode_cache_map(CUtensorMap* map, const uint8_t* cache, int64_t num_slots, int total_bytes,
                             int box_bytes, int box_rows) {
    constexpr int kSlots = 16;
    struct Entry { MapKey key; CUtensorMap map; bool used; };
    static thread_local Entry cache_maps[kSlots] = {};
    static thread_local int next = 0;
    const MapKey key{cache, num_slots, total_bytes, box_bytes, box_rows};
    for (int i = 0; i < kSlots; ++i)
        if (cache_maps[i].used && cache_maps[i].key == key) {
            std::memcpy(map, &cache_maps[i].map, sizeof(CUtensorMap));
            return true;
        }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(total_bytes / 8), static_cast<cuuint64_t>(num_slots)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(total_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes / 8), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(cache), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    Entry& e = cache_maps[next];
    next = (next + 1) % kSlots;
    e.key = key;
    std::memcpy(&e.map, map, sizeof(CUtensorMap));
    e.used = true;
    return true;
}

// Environment switches, read once per process:
//   RQ_DECODE_NO_TMA=1            the issuer warp copies the rows with 4-byte cp.async (the path of odd block sizes)
//   RQ_DECODE_NO_PDL=1            launch the merge without programmatic dependent launch
//   RQ_DECODE_EQUAL_PIECES=1      no launch-layer weights
//   RQ_DECODE_LAYER_WEIGHTS=a,b   weights of the launch layers (defaults below)
struct DecodeEnv {
    bool no_tma, no_pdl, equal_pieces;
    int weights[kMaxLayers];
    int n_weights;
};
static const DecodeEnv& decode_env() {
    static const DecodeEnv env = [] {
        DecodeEnv e{};
        e.no_tma = env_int("RQ_DECODE_NO_TMA", 0) != 0;
        e.no_pdl = env_int("RQ_DECODE_NO_PDL", 0) != 0;
        e.equal_pieces = env_int("RQ_DECODE_EQUAL_PIECES", 0) != 0;
        e.n_weights = 0;
        if (const char* w = std::getenv("RQ_DECODE_LAYER_WEIGHTS")) {
            std::string s(w);
            size_t pos = 0;
            while (pos < s.size() && e.n_weights < kMaxLayers) {
                const size_t comma = s.find(',', pos);
                const int v = std::atoi(s.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos).c_str());
                if (v > 0) e.weights[e.n_weights++] = v;
                if (comma == std::string::npos) break;
                pos = comma + 1;
            }
        }
        return e;
    }();
    return env;
}

// Staging layout of a stage for this geometry: one region when the head tile is the whole slot payload,
// else the four regions, each widened to 16-byte boundaries.
static void plan_staging(DecodeParams& p) {
    const int ttok = p.ttok;
    // Row pitch of an index region: widened by 16-byte steps (the copy reads that much more of the slot)
    // until consecutive tokens' 16-byte chunks fall into different shared-memory banks, i.e. the pitch
    // in words is an odd multiple of 4 modulo 32.
    auto conflict_free = [&](int w, int x_max) {
        while (((w / 4) % 32) % 8 != 4 && x_max + w + 16 <= p.total_bytes) w += 16;
        return w;
    };
    if (p.ht == p.H) {
        p.n_regions = 1;
        p.reg_w[0] = conflict_free((136 * p.H + 15) / 16 * 16, 0);
        p.reg_base[0] = 0;
        for (int r = 1; r < kRegions; ++r) { p.reg_w[r] = 0; p.reg_base[r] = 0; }
        p.stage_bytes = ttok * p.reg_w[0];
    } else {
        p.n_regions = kRegions;
        int base = 0;
        for (int r = 0; r < kRegions; ++r) {
            const int len = ((r & 1) ? 4 : kHalfDim) * p.ht;
            int off_max = 0, x_max = 0;
            for (int h0 = 0; h0 < p.H; h0 += p.ht) {
                const RegionWindow rw = region_window(p.H, h0);
                off_max = std::max(off_max, rw.start[r] - rw.x[r]);
                x_max = std::max(x_max, rw.x[r]);
            }
            p.reg_w[r] = (off_max + len + 15) / 16 * 16;
            if ((r & 1) == 0) p.reg_w[r] = conflict_free(p.reg_w[r], x_max);
            p.reg_base[r] = base;
            base += ttok * p.reg_w[r];
        }
        p.stage_bytes = base;
    }
    p.stages = std::min(kMaxStages, kRingBytes / p.stage_bytes);
    p.v_aligned = p.H % 4 == 0 ? 1 : 0;
}

template <typename T, int KB, int VB>
static int launch_decode(DecodeParams& p, int nh, cudaStream_t st) {
    if (!p.inline_plan) {
        decode_plan_kernel<<<1, 1024, 0, st>>>(p.seq_lens, p.num_seqs, p.ttok, p.prefix);
        if (int e = check_cuda(cudaGetLastError(), "rq_decode plan launch")) return e;
    }
    alignas(64) TmaMaps maps{};
    const int64_t num_slots = p.num_blocks * p.block_size;
    if (p.box_rows > 0) {
        bool ok = true;
        for (int r = 0; r < p.n_regions && ok; ++r)
            ok = encode_cache_map(&maps.m[r], p.cache, num_slots, p.total_bytes, p.reg_w[r], p.box_rows);
        if (!ok) p.box_rows = 0;                                           // no tensor maps: word copies
    }
    {
        const size_t smem = sizeof(DecodeSmem) + 1024;                       // + hand alignment
        const long long ctas = 1LL * p.groups * (p.H >> p.ht_shift) * p.head_groups;
        auto launch = [&](auto kernel) -> int {
            if (int e = ensure_smem(kernel, smem)) return e;
            kernel<<<static_cast<unsigned>(ctas), kDecodeThreads, smem, st>>>(p, maps);
            return check_cuda(cudaGetLastError(), "rq_decode attention launch");
        };
        if (int e = nh == 4 ? launch(decode_attn_kernel<T, KB, VB, 4>) : launch(decode_attn_kernel<T, KB, VB, 8>)) return e;
    }

    const long long warps = 1LL * p.num_seqs * p.Hq;
    const unsigned grid = static_cast<unsigned>((warps + kMergeWarps - 1) / kMergeWarps);
    if (decode_env().no_pdl) {
        decode_merge_kernel<T><<<grid, kMergeWarps * 32, 0, st>>>(p);
        return check_cuda(cudaGetLastError(), "rq_decode merge launch");
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, decode_merge_kernel<T>, p), "rq_decode merge launch");
}

template <typename T>
static int dispatch_bits(DecodeParams& p, int nh, int kb, int vb, cudaStream_t st) {
    if (kb == 3 && vb == 3) return launch_decode<T, 3, 3>(p, nh, st);
    if (kb == 4 && vb == 3) return launch_decode<T, 4, 3>(p, nh, st);
    if (kb == 3 && vb == 4) return launch_decode<T, 3, 4>(p, nh, st);
    return launch_decode<T, 4, 4>(p, nh, st);
}

}  // namespace rq

using namespace rq;

extern "C" size_t rq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                            int head_dim, int max_seq_len, int num_splits) {
    if (num_seqs <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim != kHeadDim) return 0;
    if (num_q_heads % num_kv_heads != 0) return 0;
    return plan_decode(num_seqs, num_kv_heads, num_q_heads / num_kv_heads, max_seq_len, num_splits).bytes;
}

extern "C" int rq_decode(const void* q, void* out, int dtype, int64_t q_stride_seq,
                         int64_t q_stride_head, int64_t o_stride_seq, int64_t o_stride_head,
                         int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                         const uint8_t* kv_cache, int64_t num_blocks, int block_size,
                         int total_bytes, const int32_t* block_table, int64_t block_table_stride,
                         const int32_t* seq_lens, const float* centroids_k, int n_centroids_k,
                         const float* centroids_v, int n_centroids_v, const float* rotation,
                         float sm_scale, int max_seq_len, void* workspace, size_t workspace_bytes,
                         int num_splits, void* stream) {
    if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_blocks < 0 || block_size <= 0 ||
        max_seq_len < 0 || num_splits < 0)
        return fail(RQ_ERR_INVALID_ARG, "rq_decode: negative or zero size");
    if (head_dim != kHeadDim)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: head_dim %d (only 128)", head_dim);
    if (dtype != RQ_DTYPE_F16 && dtype != RQ_DTYPE_BF16)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: query dtype must be f16 or bf16");
    if (num_q_heads % num_kv_heads != 0)
        return fail(RQ_ERR_INVALID_ARG, "rq_decode: %d query heads not a multiple of %d KV heads",
                    num_q_heads, num_kv_heads);
    if (total_bytes != num_kv_heads * kSlotPerHead)
        return fail(RQ_ERR_INVALID_ARG, "rq_decode: total_bytes %d != %d heads * 256", total_bytes,
                    num_kv_heads);
    if ((n_centroids_k != 8 && n_centroids_k != 16) || (n_centroids_v != 8 && n_centroids_v != 16))
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: codebooks must have 8 or 16 centroids");
    if (num_seqs == 0) return RQ_OK;
    if (num_seqs > 65535)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: more than 65535 sequences in one call");
    if (!q || !out || !kv_cache || !block_table || !seq_lens || !centroids_k || !centroids_v || !rotation)
        return fail(RQ_ERR_INVALID_ARG, "rq_decode: null pointer");
    if (!aligned(q, 8) || (q_stride_seq * 2) % 8 != 0 || (q_stride_head * 2) % 8 != 0)
        return fail(RQ_ERR_ALIGNMENT, "rq_decode: query rows must be 8-byte aligned");
    if (!aligned(kv_cache, 16) || !aligned(rotation, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_decode: kv_cache and rotation must be 16-byte aligned");

    const int G = num_q_heads / num_kv_heads;
    const int head_groups = (G + kQPerHead - 1) / kQPerHead;
    const DecodePlan pl = plan_decode(num_seqs, num_kv_heads, G, max_seq_len, num_splits);
    if (static_cast<long long>(pl.J) > 65535)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: too many KV heads");
    const size_t need = pl.bytes;
    if (!workspace || workspace_bytes < need)
        return fail(RQ_ERR_WORKSPACE, "rq_decode: workspace of %zu bytes needed, %zu given", need,
                    workspace_bytes);
    if (!aligned(workspace, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_decode: workspace must be 16-byte aligned");
    int bs_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
        if ((1 << sft) == block_size) bs_shift = sft;

    DecodeParams p{};
    p.q = q; p.q_stride_seq = q_stride_seq; p.q_stride_head = q_stride_head;
    p.cache = kv_cache; p.num_blocks = num_blocks; p.block_size = block_size;
    p.total_bytes = total_bytes; p.block_table = block_table; p.bt_stride = block_table_stride;
    p.seq_lens = seq_lens; p.cent_k = centroids_k; p.cent_v = centroids_v; p.rotation = rotation;
    p.qk_scale = sm_scale * 1.4426950408889634f;
    p.H = num_kv_heads; p.Hq = num_q_heads; p.G = G; p.head_groups = head_groups;
    p.ht = pl.ht; p.ht_shift = pl.ht_shift;
    p.ttok = kPairs / pl.ht;
    p.ttok_shift = 7 - pl.ht_shift;
    p.n_cols = std::max(16, pl.ht * 2 * pl.nh);
    p.prefix = static_cast<int32_t*>(workspace);
    const size_t slots = pl.rows * pl.ht * kQPerHead;
    p.ws_o = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.prefix_bytes);
    p.ws_m = p.ws_o + slots * kHeadDim;
    p.ws_l = p.ws_m + slots;
    p.num_seqs = num_seqs; p.groups = pl.groups;
    p.inline_plan = num_seqs <= kInlinePlanSeqs ? 1 : 0;
    p.bs_shift = bs_shift;
    plan_staging(p);
    // TMA boxes: power-of-two blocks of 8 tokens or more, slot numbers that fit a 32-bit coordinate
    const DecodeEnv& env = decode_env();
    p.box_rows = (!env.no_tma && bs_shift >= 3 && num_blocks * block_size <= INT32_MAX) ? std::min(block_size, p.ttok) : 0;
    // Launch-layer weights: only when (nearly) every SM holds its full set of CTAs.  RQ_DECODE_LAYER_WEIGHTS
    // overrides the defaults.
    const int sms = sm_count();
    const long long ctas = 1LL * pl.groups * pl.J;
    p.layer_ctas = 0;
    p.num_layers = kCtasPerSm;
    static const int kDefaultWeights[kMaxLayers] = {1024, 1024, 1024, 1024};
    for (int i = 0; i < kMaxLayers; ++i)
        p.layer_w[i] = env.n_weights > 0 ? env.weights[i < env.n_weights ? i : env.n_weights - 1] : kDefaultWeights[i];
    if (!env.equal_pieces && ctas > 1LL * (kCtasPerSm - 1) * sms) p.layer_ctas = sms;
    p.out = out; p.o_stride_seq = o_stride_seq; p.o_stride_head = o_stride_head;
#ifdef RQ_DECODE_TRACE
    p.trace = g_trace_buffer;
#endif

    const int kb = n_centroids_k == 8 ? 3 : 4, vb = n_centroids_v == 8 ? 3 : 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RQ_DTYPE_BF16) return dispatch_bits<__nv_bfloat16>(p, pl.nh, kb, vb, st);
    return dispatch_bits<__half>(p, pl.nh, kb, vb, st);
}

#ifdef RQ_DECODE_TRACE
// Development builds only: device buffer of 3 x 5 x 64 x 16 clock values (see RQ_TRACE).
extern "C" int rq_debug_set_trace(void* device_buffer) {
    rq::g_trace_buffer = static_cast<unsigned long long*>(device_buffer);
    return RQ_OK;
}
#endif

// ---- decode with library-owned scratch ------------------------------------------------------
//
// Some callers have no way to hand rq_decode a workspace: a serving process that gave all free
// HBM to its KV-cache pool at start-up and must not allocate afterwards, or a host runtime whose
// request path is forbidden to call an allocator.  For them the library keeps one fixed scratch
// area per GPU in its own image.  It exists on every GPU that loads the library, for the life
// of the process, whether or not this entry point is ever called.
static __device__ __align__(256) unsigned char g_decode_scratch[RQ_DECODE_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_decode_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address is looked up
// once per device with cudaGetSymbolAddress (with that device current) and remembered.
int static_scratch_address(void** out) {
    static std::mutex mu;
    static void* cached[64] = {nullptr};
    int dev = 0;
    if (int e = rq::check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
    if (dev < 0 || dev >= 64)
        return rq::fail(RQ_ERR_UNSUPPORTED, "rq_decode_static_scratch: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        if (int e = rq::check_cuda(cudaGetSymbolAddress(&ptr, g_decode_scratch),
                                   "cudaGetSymbolAddress(decode scratch)"))
            return e;
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return RQ_OK;
}
}  // namespace

extern "C" int rq_decode_static_scratch(const void* q, void* out, int dtype, int64_t q_stride_seq,
                                        int64_t q_stride_head, int64_t o_stride_seq,
                                        int64_t o_stride_head, int num_seqs, int num_q_heads,
                                        int num_kv_heads, int head_dim, const uint8_t* kv_cache,
                                        int64_t num_blocks, int block_size, int total_bytes,
                                        const int32_t* block_table, int64_t block_table_stride,
                                        const int32_t* seq_lens, const float* centroids_k,
                                        int n_centroids_k, const float* centroids_v,
                                        int n_centroids_v, const float* rotation, float sm_scale,
                                        int max_seq_len, int num_splits, void* stream) {
    // the same argument checks as rq_decode, before anything is sized from the arguments
    if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_seq_len < 0 || num_splits < 0)
        return rq::fail(RQ_ERR_INVALID_ARG, "rq_decode_static_scratch: negative or zero size");
    if (head_dim != rq::kHeadDim)
        return rq::fail(RQ_ERR_UNSUPPORTED, "rq_decode_static_scratch: head_dim %d (only 128)", head_dim);
    if (num_q_heads % num_kv_heads != 0)
        return rq::fail(RQ_ERR_INVALID_ARG, "rq_decode_static_scratch: %d query heads not a multiple of %d KV heads",
                        num_q_heads, num_kv_heads);
    if (num_seqs == 0) return RQ_OK;
    const size_t need = rq_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim,
                                                  max_seq_len, num_splits);
    if (need > static_cast<size_t>(RQ_DECODE_STATIC_SCRATCH_BYTES))
        return rq::fail(RQ_ERR_WORKSPACE,
                        "rq_decode_static_scratch: this call needs %zu scratch bytes, the built-in area "
                        "holds %zu; use rq_decode with a caller-provided workspace",
                        need, static_cast<size_t>(RQ_DECODE_STATIC_SCRATCH_BYTES));
    void* scratch = nullptr;
    if (int e = static_scratch_address(&scratch)) return e;
    return rq_decode(q, out, dtype, q_stride_seq, q_stride_head, o_stride_seq, o_stride_head, num_seqs,
                     num_q_heads, num_kv_heads, head_dim, kv_cache, num_blocks, block_size, total_bytes,
                     block_table, block_table_stride, seq_lens, centroids_k, n_centroids_k, centroids_v,
                     n_centroids_v, rotation, sm_scale, max_seq_len, scratch,
                     static_cast<size_t>(RQ_DECODE_STATIC_SCRATCH_BYTES), num_splits, stream);
}
