// Fused paged decode attention over the RotorQuant cache, sm_100a.
//
// Replaces fused_paged_rq_decode (triton/fused_paged_rq_decode.py:32-312 of the reference): the
// Triton kernel (one program per (sequence, query head), CUDA-core dot products, no split-KV)
// and the two dense 128x128 rotations its launcher runs around it.
//
// Work decomposition.  Three launches: a one-CTA prefix sum of the tiles per sequence, an attention
// kernel that streams equal shares of the (sequence, tile) space per KV head and leaves partial
// results, and a merge kernel that combines them, rounds, and applies R.  The 136 payload bytes of
// a (token, KV head) are read from HBM exactly once for all query heads of the GQA group.  Two
// attention kernels share that frame:
//   decode_umma_kernel    (default) one thread per token, tcgen05 MMAs with TMEM accumulators, the
//                         K tile as a TMEM A operand, TMA-staged index rows;
//   decode_stream_kernel  (RQ_DECODE_PATH=stream) one warp per 16-token tile, mma.sync.
//
// Arithmetic (matches "reference decompress + SDPA"):
//   q_rot   = round_T(q @ R^T)            exact FMA chain per 4x4 block, computed in the prologue
//   K, V    = round_T(centroid[idx]*norm) exactly the decompressed values: each token gets a
//             table of its 8/16 rounded products, elements are fetched from it with PRMT
//   scores  = int8 tensor-core mma over 15-bit integer images of q_rot and K (exact for K, 2^-14
//             of the row maximum for q), fp32 scaling, exp2-domain online softmax
//   P @ V   = tensor-core mma with P split into hi + lo parts (two T-precision terms, ~16 bits),
//             fp32 accumulate
//   out     = round_T(round_T(o / l) @ R)  in the merge kernel
// Both kernels are bound by the dequantisation instructions (one byte permute per V value, half
// of one per K value), not by tensor throughput; the tcgen05 kernel wins by putting the 128 tokens
// of a tile on the M side (M = tokens for S^T, M = head-dims for O^T), which removes the per-warp
// MMA, ldmatrix and fragment bookkeeping of the mma.sync formulation.
#include <cuda.h>          // CUtensorMap (types only; the encoder is looked up at run time)

#include <cstdlib>
#include <mutex>
#include <string>

#include "rq_common.cuh"
#include "rq_tcgen05.cuh"

namespace rq {

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kTile = 16;                 // tokens per tile (one mma k-step of P@V)
constexpr int kStages = 3;                // cp.async ring depth per warp
constexpr int kVPitch = 80;               // bytes per token row of V indices in smem (64 + pad)
constexpr int kHeadsPerCta = 8;           // query heads handled per CTA (mma N of P@V)

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
    float* ws_o;                           // [row][8 heads][128], row = (group + sequence) * J + item
    float* ws_m;                           // [row][8 heads]
    float* ws_l;
    // merge
    void* out;
    int64_t o_stride_seq, o_stride_head;
    // streaming kernel
    const int32_t* tile_prefix;           // [num_seqs + 1] exclusive prefix of tiles per sequence
    const int2* seq_groups;               // [num_seqs] first and last group overlapping the sequence
    int num_seqs;
    int stream_warps;                     // warps of the streaming grid (multiple of 8)
    int stream_groups;                    // groups of J workers; each owns one piece of the tile space
    const int32_t* group_cum;             // [groups + 1] running sum of the groups' weights (piece boundaries)
    int weight_layers;                    // CTAs per weight layer (SM count) when the pieces are weighted, else 0
    int bs_shift;                         // log2(block_size) when it is a power of two, else -1
};

// The line of all tiles is cut into one piece per group, in proportion to the groups' weights:
// piece g = [piece_begin(g), piece_begin(g + 1)).
__device__ __forceinline__ int64_t piece_begin(const int32_t* __restrict__ cum, int groups, int64_t g, int64_t total) {
    return total * __ldg(cum + g) / __ldg(cum + groups);
}

// ---- small PTX wrappers ------------------------------------------------------

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1,
                                                        uint32_t a2, uint32_t a3, uint32_t b0,
                                                        uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1,
                                                 uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

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

// Half of a token's tables, built by one lane; lanes l and l ^ 16 hold the two halves of a token.
// NH = entries in this half (4 or 8); planes come out as NH/4 registers each.
template <typename T, int NH>
__device__ __forceinline__ void build_half_value_table(const float* __restrict__ cb_half, float norm,
                                                       uint32_t* lo, uint32_t* hi) {
    uint32_t pairs[NH / 2];
#pragma unroll
    for (int i = 0; i < NH / 2; ++i)
        pairs[i] = pack_pair<T>(__fmul_rn(cb_half[2 * i], norm), __fmul_rn(cb_half[2 * i + 1], norm));
#pragma unroll
    for (int i = 0; i < NH / 4; ++i) {
        lo[i] = prmt(pairs[2 * i], pairs[2 * i + 1], 0x6420);
        hi[i] = prmt(pairs[2 * i], pairs[2 * i + 1], 0x7531);
    }
}

template <typename T, int NH>
__device__ __forceinline__ void build_half_int_table(const float* __restrict__ cb_half, float norm,
                                                     uint32_t* lo, uint32_t* hi, float& unscale) {
    float v[NH];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < NH; ++i) {
        v[i] = round_to<T>(__fmul_rn(cb_half[i], norm));
        mx = fmaxf(mx, fabsf(v[i]));
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));      // maximum over the whole table
    const bool ok = mx >= 1.0e-30f && mx <= 3.0e38f;
    const int e = ok ? exponent_of(mx) : 0;
    const float scale = ok ? pow2i(13 - e) : 0.0f;
    unscale = ok ? pow2i(e - 13) : 0.0f;
    int u[NH];
#pragma unroll
    for (int i = 0; i < NH; ++i) u[i] = __float2int_rn(fmaf(v[i], scale, 128.0f));
#pragma unroll
    for (int i = 0; i < NH / 4; ++i) {
        const uint32_t a = prmt(u[4 * i], u[4 * i + 1], 0x5140);
        const uint32_t b = prmt(u[4 * i + 2], u[4 * i + 3], 0x5140);
        lo[i] = prmt(a, b, 0x5410) ^ 0x80808080u;
        hi[i] = prmt(a, b, 0x7632);
    }
}

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

template <int BITS>
__device__ __forceinline__ void store_table(uint32_t* dst, const Table<BITS>& t) {
#pragma unroll
    for (int r4 = 0; r4 < Table<BITS>::kRegs / 4; ++r4)
        *reinterpret_cast<uint4*>(dst + 4 * r4) =
            make_uint4(t.r[4 * r4], t.r[4 * r4 + 1], t.r[4 * r4 + 2], t.r[4 * r4 + 3]);
}
template <int BITS>
__device__ __forceinline__ Table<BITS> load_table(const uint32_t* src) {
    Table<BITS> t;
#pragma unroll
    for (int r4 = 0; r4 < Table<BITS>::kRegs / 4; ++r4) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + 4 * r4);
        t.r[4 * r4] = v.x; t.r[4 * r4 + 1] = v.y; t.r[4 * r4 + 2] = v.z; t.r[4 * r4 + 3] = v.w;
    }
    return t;
}

// int8 tensor-core MMA, D(16x8,s32) += A(16x32,s8) * B(32x8,s8).
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same with a zero accumulator input: starts a chain without clearing registers first.
__device__ __forceinline__ void mma_s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

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

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- the streaming kernel ---------------------------------------------------------------------
//
// Work is the linear space of (sequence, 16-token tile).  It is cut into equal contiguous pieces,
// one per GROUP of J warps (J = KV heads x head groups; warp j of a group streams item j of the
// piece), on a fixed-size grid of two 8-warp CTAs per SM.  Every warp streams the same number of
// tiles whatever the batch looks like: no wave quantisation, no idle tail, and the per-sequence
// set-up is paid once per piece.  The warps of a group read the same tokens at about the same
// time, so neighbouring heads share the 128-byte lines that DRAM delivers (a warp-per-head order
// that spreads the heads in time was measured to double DRAM traffic).  Warps never synchronise
// with each other.  A piece that crosses into the next sequence yields one partial result per
// part; part (group, sequence) of item j is stored at workspace row (group + sequence) * J + j,
// unique because group and sequence only grow along the space.
//
// Each warp owns a 3-stage ring of tiles in shared memory.  Two ways to fill it:
//   TMA   (KV heads a multiple of 4, power-of-two block size >= 16): one lane issues four
//         cp.async.bulk.tensor boxes per tile -- 16 tokens x 64 B of K indices, the same of V
//         indices (64-byte swizzle: conflict-free reads of dense rows), and 16 tokens x 16 B
//         around the K norm and the V norm of the head -- completing on one mbarrier per stage.
//         Address arithmetic per tile: one block-table entry and one slot number.
//   cp.async (any layout): every lane copies 16-, 8- or 4-byte pieces with its own addresses.

// Ring stage of the cp.async path.
struct __align__(16) Stage {
    uint8_t k[kTile][kHalfDim];        // K indices of 16 tokens
    uint8_t v[kTile][kVPitch];         // V indices, padded rows (conflict-free 16-byte reads)
    float norms[2 * kTile];            // [0..15] K norms, [16..31] V norms
};

constexpr int kNormBox = 16;           // bytes per token of a norm box (4 heads)
constexpr uint32_t kTmaTileBytes = 2 * kTile * kHalfDim + 2 * kTile * kNormBox;

template <bool TMA>
struct StreamWarpSmem;

template <>
struct __align__(256) StreamWarpSmem<false> {
    uint16_t vt[kTile][kHeadDim];      // V transposition tile; also Q set-up scratch and output stage
    Stage stage[kStages];
    uint32_t tbl_k[kTile][8];
    uint32_t tbl_v[kTile][8];
    float k_unscale[kTile];
};

template <>
struct __align__(512) StreamWarpSmem<true> {
    uint8_t v[kStages][kTile * kHalfDim];    // 64-byte swizzled: chunk c of row r at c ^ ((r >> 1) & 3)
    uint8_t k[kStages][kTile * kHalfDim];    // same swizzle
    uint8_t kn[kStages][kTile * kNormBox];   // K norms of heads 4*(head/4) .. +3 per token
    uint8_t vn[kStages][kTile * kNormBox];
    uint16_t vt[kTile][kHeadDim];
    uint32_t tbl_k[kTile][8];
    uint32_t tbl_v[kTile][8];
    float k_unscale[kTile];
    uint64_t bar[kStages];                   // "tile landed" barriers
};
static_assert(sizeof(StreamWarpSmem<true>::vt) >= 2 * kHeadsPerCta * kHeadDim, "vt holds the query byte planes");
static_assert(sizeof(StreamWarpSmem<true>::vt) >= sizeof(float) * kHeadsPerCta * kHeadDim, "vt stages the partial output");
static_assert(offsetof(StreamWarpSmem<true>, vt) % 256 == 0, "vt rows must be 256-byte aligned");
static_assert(offsetof(StreamWarpSmem<true>, kn) % 128 == 0 && offsetof(StreamWarpSmem<true>, vn) % 128 == 0,
              "TMA destinations are 128-byte aligned");

// What one lane reads of a tile, whichever way the tile reached shared memory.
struct TileView {
    const uint8_t* k0;       // this lane's 16 K index bytes of token g (token g + 8: + 8 * 64)
    const uint8_t* va;       // this lane's V index bytes 0..15 of its half row of token tv
    const uint8_t* vb;       // bytes 16..31 of the same half row
    float norm_k, norm_v;    // norms of token (lane & 15)
};

// One 16-token tile: tables, S = Q K^T (int8), online softmax, V transposition, O += P V.
template <typename T, int KB, int VB>
__device__ __forceinline__ void stream_tile(uint32_t (*tbl_k)[8], uint32_t (*tbl_v)[8],
                                            float* k_unscale, const float (&cbk)[(1 << KB) / 2],
                                            const float (&cbv)[(1 << VB) / 2], const TileView& tvw,
                                            int n_valid, int lane, int g, int tig,
                                            const uint32_t (&qa)[4][4], float q_factor, float& m_run,
                                            float& l_run, float (&o_acc)[8][4], int tv,
                                            uint32_t vt_store_base, uint32_t lm_base) {
    // ---- per-token tables: lane builds one half (lane >> 4) of the K and of the V table of
    //      token (lane & 15), so both half-warps run the same instructions ----
    {
        const int i = lane & 15, hb = lane >> 4;
        const bool valid = i < n_valid;
        const float norm_k = valid ? tvw.norm_k : 0.0f;
        const float norm_v = valid ? tvw.norm_v : 0.0f;
        constexpr int NKH = (1 << KB) / 2, NVH = (1 << VB) / 2;
        float unscale;
        uint32_t lo[NKH / 4], hi[NKH / 4];
        build_half_int_table<T, NKH>(cbk, norm_k, lo, hi, unscale);
        uint32_t vlo[NVH / 4], vhi[NVH / 4];
        build_half_value_table<T, NVH>(cbv, norm_v, vlo, vhi);
        if (!valid) {
            // rows past the end of the sequence may hold bytes that are not index nibbles; with an
            // all-zero table every PRMT result is zero whatever the selector (a -0.0 entry would
            // turn a selector with its top bit set into a sign mask, i.e. a NaN pattern in fp16)
#pragma unroll
            for (int r = 0; r < NVH / 4; ++r) { vlo[r] = 0u; vhi[r] = 0u; }
        }
#pragma unroll
        for (int r = 0; r < NKH / 4; ++r) {
            tbl_k[i][hb * (NKH / 4) + r] = lo[r];
            tbl_k[i][2 * (NKH / 4) + hb * (NKH / 4) + r] = hi[r];
        }
#pragma unroll
        for (int r = 0; r < NVH / 4; ++r) {
            tbl_v[i][hb * (NVH / 4) + r] = vlo[r];
            tbl_v[i][2 * (NVH / 4) + hb * (NVH / 4) + r] = vhi[r];
        }
        if (hb == 0) k_unscale[i] = unscale;
    }
    __syncwarp();

    // ---- decompress V into the transposition buffer: lane = (token tv, half row) ----
    auto dequant_v = [&]() {
        const Table<VB> tb = load_table<VB>(tbl_v[tv]);
        const uint4 va = *reinterpret_cast<const uint4*>(tvw.va);
        const uint4 vb = *reinterpret_cast<const uint4*>(tvw.vb);
        const uint32_t words[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            uint32_t lo0, hi0, lo1, hi1;
            lookup4<VB>(tb, words[w], lo0, hi0);
            lookup4<VB>(tb, words[w] >> 16, lo1, hi1);
            // chunk (8*vhalf + w) ^ (tv & 7): vt rows are 256-byte aligned, so XOR the address
            st_shared_v4(vt_store_base ^ (16u * w), prmt(lo0, hi0, 0x5140), prmt(lo0, hi0, 0x7362),
                         prmt(lo1, hi1, 0x5140), prmt(lo1, hi1, 0x7362));
        }
    };

    // ---- S = Q K^T on the int8 path: rows = heads (g), columns = tokens ----
    // acc_h = [Qhi; Qlo] . Khi, acc_l = [Qhi; Qlo] . Klo: entries 0,1 are the Qhi rows, entries
    // 2,3 the Qlo rows of the same head and the same two tokens.  The two token groups (nt) run
    // as independent accumulation chains.
    float sc[4];
    {
        int acc_h[2][4], acc_l[2][4];
        uint32_t words[2][4];
        Table<KB> tk[2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const uint4 kw = *reinterpret_cast<const uint4*>(tvw.k0 + nt * 8 * kHalfDim);
            words[nt][0] = kw.x; words[nt][1] = kw.y; words[nt][2] = kw.z; words[nt][3] = kw.w;
            tk[nt] = load_table<KB>(tbl_k[g + 8 * nt]);
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                uint32_t lo0, hi0, lo1, hi1;
                lookup4<KB>(tk[nt], words[nt][w], lo0, hi0);            // nibbles 0..3 -> k-slots 4tig..
                lookup4<KB>(tk[nt], words[nt][w] >> 16, lo1, hi1);      // nibbles 4..7 -> k-slots 16+4tig..
                if (w == 0) {
                    mma_s8_first(acc_h[nt], qa[w][0], qa[w][1], qa[w][2], qa[w][3], hi0, hi1);
                    mma_s8_first(acc_l[nt], qa[w][0], qa[w][1], qa[w][2], qa[w][3], lo0, lo1);
                } else {
                    mma_s8(acc_h[nt], qa[w][0], qa[w][1], qa[w][2], qa[w][3], hi0, hi1);
                    mma_s8(acc_l[nt], qa[w][0], qa[w][1], qa[w][2], qa[w][3], lo0, lo1);
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float2 ku = *reinterpret_cast<const float2*>(&k_unscale[8 * nt + 2 * tig]);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int t1 = acc_h[nt][c] * 256 + (acc_h[nt][c + 2] + acc_l[nt][c]);
                const float f = fmaf(static_cast<float>(t1), 256.0f, static_cast<float>(acc_l[nt][c + 2]));
                sc[2 * nt + c] = f * (q_factor * (c ? ku.y : ku.x));
            }
        }
    }
    if (n_valid < kTile) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int tok = 8 * (x >> 1) + 2 * tig + (x & 1);
            if (tok >= n_valid) sc[x] = -INFINITY;
        }
    }

    // ---- online softmax for head g over this thread's 4 columns ----
    float m_new = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 1));
    m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 2));
    // The running reference m_run only moves when the tile maximum exceeds it by more than 8
    // (probabilities then stay below 2^8, harmless in fp32), which makes rescaling rare.
    // Every tile holds at least one valid token, so m_new is finite; m_run starts at -inf.
    const bool grew = m_new > m_run + 8.0f;
    if (__any_sync(0xffffffffu, grew)) {
        const float m_upd = grew ? m_new : m_run;
        const float alpha = ex2_approx(m_run - m_upd);      // 0 on the first tile, 1 if unchanged
        l_run *= alpha;
        // accumulator columns are heads 2tig, 2tig+1: fetch their factors from rows g'
        const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * tig) * 4);
        const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * tig + 1) * 4);
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            o_acc[mt][0] *= a0; o_acc[mt][1] *= a1;
            o_acc[mt][2] *= a0; o_acc[mt][3] *= a1;
        }
        m_run = m_upd;
    }
    float pr[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        pr[c] = ex2_approx(sc[c] - m_run);
        l_run += pr[c];
    }
    // P as mma B operand (k = tokens 2tig,2tig+1 | 2tig+8,2tig+9; n = head g), hi + lo parts
    const uint32_t ph0 = pack_pair<T>(pr[0], pr[1]), ph1 = pack_pair<T>(pr[2], pr[3]);
    const float2 h0 = unpack_pair<T>(ph0), h1 = unpack_pair<T>(ph1);
    const uint32_t pl0 = pack_pair<T>(pr[0] - h0.x, pr[1] - h0.y);
    const uint32_t pl1 = pack_pair<T>(pr[2] - h1.x, pr[3] - h1.y);

    dequant_v();
    __syncwarp();

    // ---- O^T += V^T P^T : rows = 16 head-dim positions per m-tile, columns = heads ----
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, lm_base ^ (32u * mt));
        mma16816<T>(o_acc[mt], a[0], a[1], a[2], a[3], ph0, ph1);
        mma16816<T>(o_acc[mt], a[0], a[1], a[2], a[3], pl0, pl1);
    }
}

// Tiles of every sequence as an exclusive prefix sum: prefix[s] = sum_{s' < s} ceil(len[s'] / tile_tokens).
// First the piece boundaries of the groups (see piece_begin), then the prefix sums, then, for the merge,
// the first and last group whose piece overlaps each sequence.
__global__ void decode_plan_kernel(const int32_t* __restrict__ seq_lens, int num_seqs, int tile_tokens,
                                   int32_t* __restrict__ prefix, int groups, int2* __restrict__ seq_groups,
                                   int32_t* __restrict__ group_cum, int workers_per_group, int weight_layers) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    // Weights of the groups.  On one SM the CTAs that were launched first (lower block index) get
    // the larger share of the issue slots while four of them run side by side, so that equal pieces
    // would finish up to 40 % apart; worker c belongs to layer c / weight_layers and gets a piece
    // in proportion to the speed measured for that layer.  weight_layers == 0: equal pieces.
    for (int g = threadIdx.x; g <= groups; g += blockDim.x) {
        int64_t acc = 0;                                        // sum of the weights of the workers before group g
        const int64_t before = static_cast<int64_t>(g) * workers_per_group;
        if (weight_layers > 0) {
            const int w[4] = {1290, 1090, 950, 766};
            int64_t left = before;
            for (int layer = 0; left > 0; ++layer) {
                const int64_t n = left < weight_layers ? left : weight_layers;
                acc += n * w[layer < 3 ? layer : 3];
                left -= n;
            }
        } else {
            acc = before * 1024;
        }
        group_cum[g] = static_cast<int32_t>(acc);
    }
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
    __syncthreads();
    const int64_t total = carry;
    // group holding tile t: the first g whose piece ends beyond t
    auto group_of = [&](int64_t t) -> int {
        int lo = 0, hi = groups - 1;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (total * group_cum[mid + 1] / group_cum[groups] > t) hi = mid;
            else lo = mid + 1;
        }
        return lo;
    };
    for (int s = threadIdx.x; s < num_seqs; s += blockDim.x) {
        const int64_t a = prefix[s];
        const int64_t n = (max(__ldg(seq_lens + s), 0) + tile_tokens - 1) / tile_tokens;
        int2 r = make_int2(0, -1);                                      // empty sequence: no groups
        if (n > 0) {
            r.x = group_of(a);
            r.y = group_of(a + n - 1);
        }
        seq_groups[s] = r;
    }
}

template <typename T, int KB, int VB, bool TMA>
__global__ void __launch_bounds__(kDecodeThreads, 2)
decode_stream_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_idx,
                     const __grid_constant__ CUtensorMap map_norm) {
    extern __shared__ uint8_t smem_raw[];
    using Smem = StreamWarpSmem<TMA>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the dynamic area is aligned by hand: swizzled TMA tiles want 512-byte alignment
    uint8_t* smem_base = smem_raw + ((512u - (smem_u32(smem_raw) & 511u)) & 511u);
    Smem& ws = reinterpret_cast<Smem*>(smem_base)[warp];
    const int g = lane >> 2, tig = lane & 3;

    // ---- this warp's piece: warp = (group, item); a group of J consecutive warps walks one
    //      range of the (sequence, tile) space, one warp per (KV head, head group) ----
    const int J = p.H * p.head_groups;                         // items per sequence
    const int64_t total = __ldg(p.tile_prefix + p.num_seqs);   // tiles of all sequences
    const int64_t wq = static_cast<int64_t>(blockIdx.x) * kDecodeWarps + warp;
    const int64_t group = wq / J;
    const int item = static_cast<int>(wq % J);
    if (group >= p.stream_groups) return;
    int64_t x = piece_begin(p.group_cum, p.stream_groups, group, total);
    const int64_t x_end = piece_begin(p.group_cum, p.stream_groups, group + 1, total);
    if (x >= x_end) return;

    // this lane's half of the codebooks (the half-table it builds for every token)
    constexpr int NKH = (1 << KB) / 2, NVH = (1 << VB) / 2;
    float cbk[NKH], cbv[NVH];
#pragma unroll
    for (int i = 0; i < NKH; ++i) cbk[i] = __ldg(p.cent_k + (lane >> 4) * NKH + i);
#pragma unroll
    for (int i = 0; i < NVH; ++i) cbv[i] = __ldg(p.cent_v + (lane >> 4) * NVH + i);

    const SlotLayout lay = slot_layout(p.H);
    const bool fast_bt = p.bs_shift >= 4;                      // power-of-two block size >= 16
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);
    const uint32_t tb = static_cast<uint32_t>(p.total_bytes);
    const int tv = lane & 15, vhalf = lane >> 4;
    const int lm_tok = (lane & 7) + ((lane & 16) ? 8 : 0);
    const int lm_chunk = (lane >> 3) & 1;
    const uint32_t vt_store_base = smem_u32(&ws.vt[tv][0]) + 128u * vhalf + 16u * (tv & 7);
    const uint32_t lm_base = smem_u32(&ws.vt[lm_tok][0]) + 16u * (lm_chunk ^ (lm_tok & 7));

    uint32_t par_bits = 0;                                     // TMA: phase parity of each stage barrier
    bool dead = false;                                         // TMA: a bounded wait expired
    if constexpr (TMA) {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) mbar_init(&ws.bar[s], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
    }

    // sequence holding position x: first s with prefix[s + 1] > x
    int seq = 0;
    for (int base = 0; base < p.num_seqs; base += 32) {
        const int s = base + lane;
        const int64_t end = s < p.num_seqs ? __ldg(p.tile_prefix + s + 1) : INT64_MAX;
        const unsigned hit = __ballot_sync(0xffffffffu, end > x);
        if (hit) { seq = base + __ffs(hit) - 1; break; }
    }

#pragma unroll 1
    while (x < x_end && seq < p.num_seqs) {
        // ---- the part of this piece inside one sequence ----
        const int pre = __ldg(p.tile_prefix + seq), n_s = __ldg(p.tile_prefix + seq + 1) - pre;
        if (n_s <= 0 || x >= static_cast<int64_t>(pre) + n_s) { ++seq; continue; }
        const int t_begin = static_cast<int>(x - pre);
        const int64_t reach = t_begin + (x_end - x);
        const int t_end = reach < n_s ? static_cast<int>(reach) : n_s;
        const int kvh = item / p.head_groups, hg = item % p.head_groups;
        const int heads_here = min(kHeadsPerCta, p.G - hg * kHeadsPerCta);
        const int first_qh = kvh * p.G + hg * kHeadsPerCta;
        const int seq_len = max(__ldg(p.seq_lens + seq), 0);
        const int32_t* bt_row = p.block_table + seq * p.bt_stride;

        // ---- ring filling ----
        int pf_tile = t_begin, pf_stage = 0;
        [[maybe_unused]] int pf_blk = 0;                           // TMA: block of tile pf_tile
        [[maybe_unused]] const uint8_t* pf_base = nullptr;         // cp.async: first slot of tile pf_tile
        const int last_blk = static_cast<int>(p.num_blocks) - 1;
        auto block_of = [&](int tile) -> int {                     // fast paths: block holding the tile
            const int blk = __ldg(bt_row + ((tile * kTile) >> p.bs_shift));
            return blk < 0 ? 0 : (blk > last_blk ? last_blk : blk);
        };
        // cp.async path: per-lane source and destination offsets
        [[maybe_unused]] const uint32_t src_k = (lane >> 2) * tb + kvh * kHalfDim + 16 * (lane & 3);
        [[maybe_unused]] const uint32_t dst_k = (lane >> 2) * kHalfDim + 16 * (lane & 3);
        [[maybe_unused]] const uint32_t dst_v16 = sizeof(Stage::k) + (lane >> 2) * kVPitch + 16 * (lane & 3);
        [[maybe_unused]] const uint32_t src_n = (lane & 15) * tb + ((lane >> 4) ? lay.v_norm : lay.k_norm) + 4 * kvh;
        [[maybe_unused]] const uint32_t dst_n = sizeof(Stage::k) + sizeof(Stage::v) + 4 * lane;
        // TMA path: byte coordinates of the four boxes inside a slot
        [[maybe_unused]] const int x_k = kvh * kHalfDim, x_v = lay.v_idx + kvh * kHalfDim;
        [[maybe_unused]] const int x_kn = lay.k_norm + kNormBox * (kvh >> 2);
        [[maybe_unused]] const int x_vn = lay.v_norm + kNormBox * (kvh >> 2);

        auto issue_next = [&]() {
            if constexpr (TMA) {
                if (pf_tile < t_end) {
                    const int slot = (pf_blk << p.bs_shift) + ((pf_tile * kTile) & (p.block_size - 1));
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&ws.bar[0]) + 8u * pf_stage;
                        mbar_expect_tx(bar, kTmaTileBytes);
                        tma_load_2d(smem_u32(&ws.k[0][0]) + 1024u * pf_stage, &map_idx, x_k, slot, bar);
                        tma_load_2d(smem_u32(&ws.kn[0][0]) + 256u * pf_stage, &map_norm, x_kn, slot, bar);
                        tma_load_2d(smem_u32(&ws.vn[0][0]) + 256u * pf_stage, &map_norm, x_vn, slot, bar);
                        tma_load_2d(smem_u32(&ws.v[0][0]) + 1024u * pf_stage, &map_idx, x_v, slot, bar);
                    }
                    ++pf_tile;
                    pf_stage = pf_stage + 1 == kStages ? 0 : pf_stage + 1;
                    if (pf_tile < t_end) pf_blk = block_of(pf_tile);
                }
            } else {
                if (pf_tile < t_end) {
                    uint8_t* stg = reinterpret_cast<uint8_t*>(&ws.stage[pf_stage]);
                    if (fast_bt) {
                        const uint8_t* base = pf_base;
                        cp_async16(stg + dst_k, base + src_k);
                        cp_async16(stg + dst_k + 8 * kHalfDim, base + src_k + 8 * tb);
                        if (v_align == 16) {
                            cp_async16(stg + dst_v16, base + src_k + lay.v_idx);
                            cp_async16(stg + dst_v16 + 8 * kVPitch, base + src_k + 8 * tb + lay.v_idx);
                        } else if (v_align == 8) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int c = lane + 32 * j, i = c >> 3, part = c & 7;
                                cp_async8(stg + sizeof(Stage::k) + i * kVPitch + 8 * part,
                                          base + i * tb + lay.v_idx + kvh * kHalfDim + 8 * part);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int c = lane + 32 * j, i = c >> 4, part = c & 15;
                                cp_async4(stg + sizeof(Stage::k) + i * kVPitch + 4 * part,
                                          base + i * tb + lay.v_idx + kvh * kHalfDim + 4 * part);
                            }
                        }
                        cp_async4(stg + dst_n, base + src_n);
                    } else {
                        auto token_ptr = [&](int i) -> const uint8_t* {
                            const int t = min(pf_tile * kTile + i, seq_len - 1);
                            int64_t blk = __ldg(bt_row + t / p.block_size);
                            blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
                            return p.cache + (blk * p.block_size + (t % p.block_size)) * p.total_bytes;
                        };
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int c = lane + 32 * j, i = c >> 2, part = c & 3;
                            cp_async16(stg + i * kHalfDim + 16 * part,
                                       token_ptr(i) + lay.k_idx + kvh * kHalfDim + 16 * part);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int c = lane + 32 * j, i = c >> 4, part = c & 15;
                            cp_async4(stg + sizeof(Stage::k) + i * kVPitch + 4 * part,
                                      token_ptr(i) + lay.v_idx + kvh * kHalfDim + 4 * part);
                        }
                        cp_async4(stg + dst_n, token_ptr(lane & 15) +
                                                   ((lane >> 4) ? lay.v_norm : lay.k_norm) + 4 * kvh);
                    }
                    ++pf_tile;
                    pf_stage = pf_stage + 1 == kStages ? 0 : pf_stage + 1;
                    if (fast_bt && pf_tile < t_end) {
                        const int64_t slot = (static_cast<int64_t>(block_of(pf_tile)) << p.bs_shift) +
                                             ((pf_tile * kTile) & (p.block_size - 1));
                        pf_base = p.cache + slot * p.total_bytes;
                    }
                }
                cp_async_commit();
            }
        };
        // first tiles in flight before the query set-up; the block-table entry of the tile after
        // the one being issued is read one step ahead so that its latency is off the issue path
        if constexpr (TMA) {
            pf_blk = block_of(t_begin);
        } else if (fast_bt) {
            const int64_t slot = (static_cast<int64_t>(block_of(t_begin)) << p.bs_shift) +
                                 ((t_begin * kTile) & (p.block_size - 1));
            pf_base = p.cache + slot * p.total_bytes;
        }
        if (!dead) {
#pragma unroll 1
            for (int s = 0; s < kStages - 1; ++s) issue_next();
        }

        // ---- queries of this item: rotate, round, quantise to signed byte planes (scratch: vt) ----
        uint8_t* q_hi = reinterpret_cast<uint8_t*>(&ws.vt[0][0]);     // [8][128]
        uint8_t* q_lo = q_hi + kHeadsPerCta * kHeadDim;
        float my_unscale = 0.0f;                                       // lane g keeps the factor of head g
#pragma unroll 1
        for (int h = 0; h < kHeadsPerCta; ++h) {
            float r[4] = {0.f, 0.f, 0.f, 0.f};
            if (h < heads_here) {
                const T* qp = static_cast<const T*>(p.q) + seq * p.q_stride_seq +
                              static_cast<int64_t>(first_qh + h) * p.q_stride_head + 4 * lane;
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(qp));
                const float2 x01 = unpack_pair<T>(raw.x), x23 = unpack_pair<T>(raw.y);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 rr = __ldg(reinterpret_cast<const float4*>(
                        p.rotation + (4 * lane + j) * kHeadDim + 4 * lane));
                    float acc = __fmul_rn(x01.x, rr.x);
                    acc = __fmaf_rn(x01.y, rr.y, acc);
                    acc = __fmaf_rn(x23.x, rr.z, acc);
                    acc = __fmaf_rn(x23.y, rr.w, acc);
                    r[j] = round_to<T>(acc);
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
            for (int j = 0; j < 4; ++j) qu[j] = __float2int_rn(fmaf(r[j], scale, 128.0f));
            const uint32_t a = prmt(qu[1], qu[0], 0x5140), b = prmt(qu[3], qu[2], 0x5140);
            *reinterpret_cast<uint32_t*>(q_lo + h * kHeadDim + 4 * lane) = prmt(a, b, 0x5410) ^ 0x80808080u;
            *reinterpret_cast<uint32_t*>(q_hi + h * kHeadDim + 4 * lane) = prmt(a, b, 0x7632);
            if (g == h) my_unscale = ok ? pow2i(e - 13) : 0.0f;
        }
        __syncwarp();
        uint32_t qa[4][4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const int off = g * kHeadDim + 32 * tig + 8 * w;
            qa[w][0] = *reinterpret_cast<const uint32_t*>(q_hi + off);
            qa[w][1] = *reinterpret_cast<const uint32_t*>(q_lo + off);
            qa[w][2] = *reinterpret_cast<const uint32_t*>(q_hi + off + 4);
            qa[w][3] = *reinterpret_cast<const uint32_t*>(q_lo + off + 4);
        }
        const float q_factor = my_unscale * p.qk_scale;
        __syncwarp();                                  // vt is free for the tile loop

        float m_run = -INFINITY, l_run = 0.0f;
        float o_acc[8][4];
#pragma unroll
        for (int mt = 0; mt < 8; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) o_acc[mt][c] = 0.0f;

        // this lane's read offsets inside a stage
        [[maybe_unused]] const int sw_k = (g >> 1) & 3, sw_v = (tv >> 1) & 3;
        [[maybe_unused]] const uint32_t tk_off = g * kHalfDim + 16 * (tig ^ sw_k);
        [[maybe_unused]] const uint32_t tva_off = tv * kHalfDim + 16 * ((2 * vhalf) ^ sw_v);
        [[maybe_unused]] const uint32_t tn_off = kNormBox * (lane & 15) + 4 * (kvh & 3);

        int cur_stage = 0;
#pragma unroll 1
        for (int tile = t_begin; tile < t_end && !dead; ++tile) {
            issue_next();
            TileView view;
            if constexpr (TMA) {
                if (!mbar_wait(&ws.bar[cur_stage], (par_bits >> cur_stage) & 1u)) {
                    // A copy that never landed: give the tiles in flight one more bounded wait
                    // each and stop streaming; this and all later parts of the warp are marked
                    // invalid (NaN row sum), which the merge turns into NaN outputs.
#pragma unroll 1
                    for (int s = 0; s < kStages; ++s) mbar_wait(&ws.bar[s], (par_bits >> s) & 1u);
                    dead = true;
                    break;
                }
                par_bits ^= 1u << cur_stage;
                view.k0 = ws.k[cur_stage] + tk_off;
                view.va = ws.v[cur_stage] + tva_off;
                view.vb = ws.v[cur_stage] + (tva_off ^ 16u);
                view.norm_k = *reinterpret_cast<const float*>(ws.kn[cur_stage] + tn_off);
                view.norm_v = *reinterpret_cast<const float*>(ws.vn[cur_stage] + tn_off);
            } else {
                cp_async_wait<kStages - 1>();
                __syncwarp();
                const Stage& st = ws.stage[cur_stage];
                view.k0 = &st.k[g][16 * tig];
                view.va = &st.v[tv][32 * vhalf];
                view.vb = view.va + 16;
                view.norm_k = st.norms[lane & 15];
                view.norm_v = st.norms[kTile + (lane & 15)];
            }
            cur_stage = cur_stage + 1 == kStages ? 0 : cur_stage + 1;
            stream_tile<T, KB, VB>(ws.tbl_k, ws.tbl_v, ws.k_unscale, cbk, cbv, view,
                                   min(kTile, seq_len - tile * kTile), lane, g, tig, qa, q_factor,
                                   m_run, l_run, o_acc, tv, vt_store_base, lm_base);
            __syncwarp();      // the stage, the tables and vt may be overwritten from here on
        }
        if constexpr (TMA) {
            if (dead) l_run = __int_as_float(0x7fc00000);
        } else {
            cp_async_wait<0>();
        }

        // ---- partial result of this part -> workspace row (warp + item) ----
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        float* o_s = reinterpret_cast<float*>(&ws.vt[0][0]);          // [8 heads][128]
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const int d = 16 * mt + (g ^ 1);
            o_s[(2 * tig) * kHeadDim + d] = o_acc[mt][0];
            o_s[(2 * tig + 1) * kHeadDim + d] = o_acc[mt][1];
            o_s[(2 * tig) * kHeadDim + d + 8] = o_acc[mt][2];
            o_s[(2 * tig + 1) * kHeadDim + d + 8] = o_acc[mt][3];
        }
        __syncwarp();
        const int64_t row = (group + seq) * J + item;
#pragma unroll 1
        for (int h = 0; h < heads_here; ++h) {
            const float4 v = *reinterpret_cast<const float4*>(&o_s[h * kHeadDim + 4 * lane]);
            *reinterpret_cast<float4*>(p.ws_o + (row * kHeadsPerCta + h) * kHeadDim + 4 * lane) = v;
        }
        if (tig == 0 && g < heads_here) {
            p.ws_m[row * kHeadsPerCta + g] = m_run;
            p.ws_l[row * kHeadsPerCta + g] = l_run;
        }
        __syncwarp();

        x += t_end - t_begin;
        if (t_end == n_s) ++seq;
    }
}

// ---- the tensor-memory kernel -------------------------------------------------------------------
//
// One CTA of 128 threads streams 128-token tiles of one (KV head, head group) item; thread t owns
// token t of the tile and TMEM lane t.  Per tile:
//   1. the thread builds the K and V tables of its token and turns the 128 K indices into the two
//      signed digit planes of the 15-bit integer image (32 registers each), which it stores into
//      its TMEM lane: the K tile never touches shared memory;
//   2. S^T = K Q^T on the tcgen05 int8 path with the K planes as the TMEM A operand and the query
//      digit planes (rows 0..7 high digits of the 8 heads, rows 8..15 low digits) as a 2 KB shared
//      B operand: two accumulators of 16 columns (K high x [Q high | Q low], K low x [..]);
//   3. meanwhile the thread decompresses the V row of its token into the shared V tile, in the
//      core-matrix order of an MN-major operand (the tensor core does the transposition);
//   4. each thread reads the 32 sums of its token, forms the G scores, exponentiates against a
//      CTA-wide lazy reference maximum per head (it moves only when a score exceeds it by 2^8,
//      found with one block vote), and writes its probabilities, split into hi + lo parts of T
//      precision, as 16 values of the shared P tile;
//   5. O^T += V^T [P hi | P lo] on the tcgen05 16-bit path: 128 head-dim lanes x 16 columns.
// Index bytes and norms go straight from global memory into registers, one tile ahead; the four
// 16-byte loads of a thread cover whole 32-byte sectors, which the L1 keeps between the loads.
// Pieces, partial-result rows and the merge are those of the streaming kernel with 128-token tiles
// and one CTA per (group, item).

constexpr int kUTile = 128;                  // tokens per tile
constexpr int kUThreads = 128;
constexpr int kUCtasPerSm = 4;
constexpr uint32_t kUTmemCols = 128;         // columns allocated per CTA
constexpr uint32_t kUColKhi = 0, kUColKlo = 32, kUColS = 64, kUColO = 96;

struct __align__(512) UmmaSmem {
    uint8_t stage[4][2][32 * kHalfDim];      // per warp: K | V index rows of its 32 tokens of the next tile
                                             // (TMA, 64-byte swizzle: chunk c of row r at c ^ ((r >> 1) & 3))
    uint16_t v[kUTile * kHeadDim];           // V tile: core (token/8)*16 + pos/8, core row token%8
    uint16_t p[kUTile * 16];                 // P tile: core (token/8)*2 + n/8, core row token%8
    uint8_t q[16 * kHeadDim];                // Q digit planes, K-major: core (n/8)*8 + pos/16
    float cb[2][16];
    float qf[kHeadsPerCta];                  // q unscale * sm_scale * log2(e) per head
    float red[4][kHeadsPerCta];              // cross-warp reductions
    uint64_t bar_s, bar_o;
    uint64_t bar_in[4];                      // per warp: "staged rows landed"
    uint32_t tmem_base;
};

// Full tables of one token, built by one thread.
template <typename T, int BITS>
__device__ __forceinline__ Table<BITS> build_int_table(const float* cb, float norm, float& unscale) {
    constexpr int N = 1 << BITS;
    float v[N];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        v[i] = round_to<T>(__fmul_rn(cb[i], norm));
        mx = fmaxf(mx, fabsf(v[i]));
    }
    const bool ok = mx >= 1.0e-30f && mx <= 3.0e38f;
    const int e = ok ? exponent_of(mx) : 0;
    const float scale = ok ? pow2i(13 - e) : 0.0f;
    unscale = ok ? pow2i(e - 13) : 0.0f;
    Table<BITS> t;
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        const int u0 = __float2int_rn(fmaf(v[4 * i], scale, 128.0f)), u1 = __float2int_rn(fmaf(v[4 * i + 1], scale, 128.0f));
        const int u2 = __float2int_rn(fmaf(v[4 * i + 2], scale, 128.0f)), u3 = __float2int_rn(fmaf(v[4 * i + 3], scale, 128.0f));
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

// NH = query heads computed per item: 4 when the GQA group has at most 4 heads, else 8.
// MODE = how the index rows reach the CTA: 0 direct global loads by every thread, 1 TMA boxes for K and
// V rows, 2 TMA boxes for the K rows and 4-byte cp.async for V rows that are not 16-byte aligned.
template <typename T, int KB, int VB, int MODE, int NH>
__global__ void __launch_bounds__(kUThreads, kUCtasPerSm)
decode_umma_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_idx) {
    constexpr bool TMA = MODE != 0;
    constexpr bool v_by_tma = MODE == 1;
    extern __shared__ uint8_t smem_raw[];
    // aligned by hand: the swizzled TMA rows want 512-byte alignment
    UmmaSmem& sm = *reinterpret_cast<UmmaSmem*>(smem_raw + ((512u - (smem_u32(smem_raw) & 511u)) & 511u));
    constexpr int NK = 1 << KB, NV = 1 << VB;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- this CTA's piece: CTA = (group, item) ----
    const int J = p.H * p.head_groups;
    const int64_t total = __ldg(p.tile_prefix + p.num_seqs);
    const int64_t group = blockIdx.x / J;
    const int item = static_cast<int>(blockIdx.x % J);
    if (group >= p.stream_groups) return;
    int64_t x = piece_begin(p.group_cum, p.stream_groups, group, total);
    const int64_t x_end = piece_begin(p.group_cum, p.stream_groups, group + 1, total);
    if (x >= x_end) return;

    if (tid == 0) {
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
#pragma unroll
        for (int w = 0; w < 4; ++w) mbar_init(&sm.bar_in[w], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    if (warp == 0) tmem_alloc(&sm.tmem_base, kUTmemCols);
    if (tid < 32) {
        const int kv = tid >> 4, i = tid & 15;
        const int n = kv ? NV : NK;
        sm.cb[kv][i] = i < n ? __ldg((kv ? p.cent_v : p.cent_k) + i) : 0.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's lane quarter

    const SlotLayout lay = slot_layout(p.H);
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);
    // S^T: s32 accumulator, int8 operands, N = 16, M = 128;  O^T: f32 accumulator, T operands, both MN-major
    const uint32_t idesc_s = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t idesc_o = (1u << 4) | (TcFormat<T>::kFmt << 7) | (TcFormat<T>::kFmt << 10) | (1u << 15) |
                             (1u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t q_addr = smem_u32(sm.q), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);
    uint8_t* const v_dst = reinterpret_cast<uint8_t*>(sm.v) + (tid >> 3) * (16 * 128) + (tid & 7) * 16;
    uint8_t* const p_dst = reinterpret_cast<uint8_t*>(sm.p) + (tid >> 3) * (2 * 128) + (tid & 7) * 16;

    // sequence holding position x: first s with prefix[s + 1] > x
    int seq = 0;
    for (int base = 0; base < p.num_seqs; base += 32) {
        const int s = base + lane;
        const int64_t end = s < p.num_seqs ? __ldg(p.tile_prefix + s + 1) : INT64_MAX;
        const unsigned hit = __ballot_sync(0xffffffffu, end > x);
        if (hit) { seq = base + __ffs(hit) - 1; break; }
    }

    uint32_t ph_s = 0, ph_o = 0;              // phase parities of the two barriers
    [[maybe_unused]] uint32_t ph_in = 0;      // ... and of this warp's staging barrier
    bool dead = false;                        // a bounded wait expired (same value in all threads)
    // staged rows of this thread's token: 16-byte chunk c sits at chunk c ^ ((lane >> 1) & 3)
    [[maybe_unused]] const uint8_t* const stage_k = sm.stage[warp][0] + lane * kHalfDim;
    [[maybe_unused]] const uint8_t* const stage_v = sm.stage[warp][1] + lane * kHalfDim;
    [[maybe_unused]] const uint32_t stage_sw = 16u * ((lane >> 1) & 3);

#pragma unroll 1
    while (x < x_end && seq < p.num_seqs) {
        const int pre = __ldg(p.tile_prefix + seq), n_s = __ldg(p.tile_prefix + seq + 1) - pre;
        if (n_s <= 0 || x >= static_cast<int64_t>(pre) + n_s) { ++seq; continue; }
        const int t_begin = static_cast<int>(x - pre);
        const int64_t reach = t_begin + (x_end - x);
        const int t_end = reach < n_s ? static_cast<int>(reach) : n_s;
        const int kvh = item / p.head_groups, hg = item % p.head_groups;
        const int heads_here = min(kHeadsPerCta, p.G - hg * kHeadsPerCta);
        const int first_qh = kvh * p.G + hg * kHeadsPerCta;
        const int seq_len = max(__ldg(p.seq_lens + seq), 0);
        const int32_t* bt_row = p.block_table + seq * p.bt_stride;
        const int last_blk = static_cast<int>(p.num_blocks) - 1;

        // Index words and norms of this thread's token, fetched one tile ahead.  Past the end of the
        // sequence nothing is fetched and the norm is 0, which zeroes the value of every table entry;
        // the words then keep their last contents, which must still be index words (a nibble with
        // its top bit set would make PRMT return a sign mask instead of a table byte), hence the
        // clearing here.
        uint32_t kw[16], vw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { kw[i] = 0u; vw[i] = 0u; }
        float nk = 0.0f, nv = 0.0f;
        bool failed_in = false;

        // ---- where this thread's token of a tile lives ----
        // cp.async-free direct path: pointer to the token's K index row (nullptr past the end).
        [[maybe_unused]] auto slot_of = [&](int tile) -> const uint8_t* {
            const int tok = tile * kUTile + tid;
            if (tok >= seq_len) return nullptr;
            const int bi = p.bs_shift >= 0 ? (tok >> p.bs_shift) : (tok / p.block_size);
            const int off = p.bs_shift >= 0 ? (tok & (p.block_size - 1)) : (tok % p.block_size);
            int blk = __ldg(bt_row + bi);
            blk = blk < 0 ? 0 : (blk > last_blk ? last_blk : blk);
            return p.cache + (static_cast<int64_t>(blk) * p.block_size + off) * p.total_bytes + kvh * kHalfDim;
        };
        [[maybe_unused]] auto fetch_direct = [&](int which, const uint8_t* slot, uint32_t (&w)[16], float& norm) {
            norm = 0.0f;               // a zero norm makes every table entry zero: stale index words are harmless
            if (slot != nullptr) {
                if (which) load_idx64(slot + lay.v_idx, v_align, w);
                else load_idx64(slot + lay.k_idx, 16, w);
                norm = __ldg(reinterpret_cast<const float*>(slot + (which ? lay.v_norm : lay.k_norm) -
                                                            kvh * (kHalfDim - 4)));
            }
        };
        // TMA path.  A warp stages the index rows of its 32 tokens of the NEXT tile in shared memory
        // (two 16-token boxes per region; a 16-token group never straddles a block).  Lane l keeps
        // the block-table entry of its group (l / 16) for the tile after that, loaded a tile early,
        // and the slot number of its own token in the staged tile (-1 past the end).
        [[maybe_unused]] int pf_blk = 0, staged_slot = -1;
        [[maybe_unused]] auto load_blk = [&](int tile) -> int {
            const int t = tile * kUTile + 32 * warp + (lane & 16);
            return (tile < t_end && t < seq_len) ? __ldg(bt_row + (t >> p.bs_shift)) : 0;
        };
        [[maybe_unused]] auto issue_tile = [&](int tile, int blk) {      // completes one phase of bar_in[warp]
            const int t = tile * kUTile + 32 * warp + (lane & 16);
            blk = blk < 0 ? 0 : (blk > last_blk ? last_blk : blk);
            const int gslot = (blk << p.bs_shift) + (t & (p.block_size - 1));
            const int s0 = __shfl_sync(0xffffffffu, gslot, 0), s1 = __shfl_sync(0xffffffffu, gslot, 16);
            const bool on0 = tile * kUTile + 32 * warp < seq_len, on1 = tile * kUTile + 32 * warp + 16 < seq_len;
            staged_slot = (t + (lane & 15) < seq_len) ? gslot + (lane & 15) : -1;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&sm.bar_in[warp]);
                if (on0) {
                    const uint32_t group_bytes = v_by_tma ? 2048u : 1024u;
                    mbar_expect_tx(bar, on1 ? 2 * group_bytes : group_bytes);
                    tma_load_2d(smem_u32(sm.stage[warp][0]), &map_idx, kvh * kHalfDim, s0, bar);
                    if (v_by_tma) tma_load_2d(smem_u32(sm.stage[warp][1]), &map_idx, lay.v_idx + kvh * kHalfDim, s0, bar);
                    if (on1) {
                        tma_load_2d(smem_u32(sm.stage[warp][0]) + 1024u, &map_idx, kvh * kHalfDim, s1, bar);
                        if (v_by_tma)
                            tma_load_2d(smem_u32(sm.stage[warp][1]) + 1024u, &map_idx, lay.v_idx + kvh * kHalfDim, s1, bar);
                    }
                } else {
                    mbar_arrive(&sm.bar_in[warp]);
                }
            }
            if constexpr (!v_by_tma) {
                // V rows that do not start on 16-byte boundaries (1 or 2 KV heads on this GPU): the warp
                // copies them with 4-byte cp.async, two rows per instruction, into the same swizzled order
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int row = 2 * i + (lane >> 4), word = lane & 15;
                    if (tile * kUTile + 32 * warp + row < seq_len) {
                        const int slot = (i < 8 ? s0 : s1) + (row & 15);
                        cp_async4(sm.stage[warp][1] + row * kHalfDim + (((word >> 2) ^ ((row >> 1) & 3)) << 4) + ((word & 3) << 2),
                                  p.cache + static_cast<int64_t>(slot) * p.total_bytes + lay.v_idx + kvh * kHalfDim + 4 * word);
                    }
                }
                cp_async_commit();
            }
        };
        // the staged V rows are complete (the K rows are covered by the barrier)
        [[maybe_unused]] auto v_rows_landed = [&]() {
            if constexpr (!v_by_tma) {
                cp_async_wait<0>();
                __syncwarp();
            }
        };
        [[maybe_unused]] auto fetch_staged = [&](int which, uint32_t (&w)[16], float& norm) {
            norm = 0.0f;
            if (staged_slot >= 0) {
                const uint8_t* rows = which ? stage_v : stage_k;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 x4 = *reinterpret_cast<const uint4*>(rows + ((16u * c) ^ stage_sw));
                    w[4 * c] = x4.x; w[4 * c + 1] = x4.y; w[4 * c + 2] = x4.z; w[4 * c + 3] = x4.w;
                }
                norm = __ldg(reinterpret_cast<const float*>(
                    p.cache + static_cast<int64_t>(staged_slot) * p.total_bytes + (which ? lay.v_norm : lay.k_norm) + 4 * kvh));
            }
        };
        // the first tile's rows are requested before the query set-up, which hides most of their latency
        if (!dead) {
            if constexpr (TMA) {
                issue_tile(t_begin, load_blk(t_begin));
                pf_blk = load_blk(t_begin + 1);
            } else {
                const uint8_t* first = slot_of(t_begin);
                fetch_direct(0, first, kw, nk);
                fetch_direct(1, first, vw, nv);
            }
        }

        // ---- queries of this item: rotate, round, quantise to signed digit planes (B operand) ----
#pragma unroll 1
        for (int round = 0; round < NH / 4; ++round) {
            const int h = 4 * round + warp;
            float r[4] = {0.f, 0.f, 0.f, 0.f};
            if (h < heads_here) {
                const T* qp = static_cast<const T*>(p.q) + seq * p.q_stride_seq +
                              static_cast<int64_t>(first_qh + h) * p.q_stride_head + 4 * lane;
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(qp));
                const float2 x01 = unpack_pair<T>(raw.x), x23 = unpack_pair<T>(raw.y);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 rr = __ldg(reinterpret_cast<const float4*>(
                        p.rotation + (4 * lane + j) * kHeadDim + 4 * lane));
                    float acc = __fmul_rn(x01.x, rr.x);
                    acc = __fmaf_rn(x01.y, rr.y, acc);
                    acc = __fmaf_rn(x23.x, rr.z, acc);
                    acc = __fmaf_rn(x23.y, rr.w, acc);
                    r[j] = round_to<T>(acc);
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
            for (int j = 0; j < 4; ++j) qu[j] = __float2int_rn(fmaf(r[j], scale, 128.0f));
            // position x of a row holds head-dim x ^ 1 (the nibble order of the cache)
            const uint32_t a = prmt(qu[1], qu[0], 0x5140), b = prmt(qu[3], qu[2], 0x5140);
            const uint32_t off = (lane >> 2) * 128 + (h & 7) * 16 + 4 * (lane & 3);
            *reinterpret_cast<uint32_t*>(&sm.q[off]) = prmt(a, b, 0x7632);                       // row h: high digits
            *reinterpret_cast<uint32_t*>(&sm.q[1024 + off]) = prmt(a, b, 0x5410) ^ 0x80808080u;  // row 8 + h: low digits
            if (lane == 0) sm.qf[h] = (ok ? pow2i(e - 13) : 0.0f) * p.qk_scale;
        }
        fence_async_proxy();
        __syncthreads();

        if constexpr (TMA) {
            if (!dead) {
                failed_in |= !mbar_wait(&sm.bar_in[warp], ph_in);
                ph_in ^= 1u;
                v_rows_landed();
                fetch_staged(0, kw, nk);
                fetch_staged(1, vw, nv);
                __syncwarp();
                if (t_begin + 1 < t_end) issue_tile(t_begin + 1, pf_blk);
                pf_blk = load_blk(t_begin + 2);
            }
        }

        float m_ref[NH], l_acc[NH];
#pragma unroll
        for (int h = 0; h < NH; ++h) { m_ref[h] = -INFINITY; l_acc[h] = 0.0f; }
        bool pv_pending = false;

#pragma unroll 1
        for (int tile = t_begin; tile < t_end && !dead; ++tile) {
            [[maybe_unused]] const uint8_t* next_slot = nullptr;
            if constexpr (!TMA) next_slot = tile + 1 < t_end ? slot_of(tile + 1) : nullptr;
            const bool valid = tile * kUTile + tid < seq_len;
            bool failed = failed_in;
            failed_in = false;

            // ---- 1, 2: K table, digit planes -> TMEM, S^T = K Q^T ----
            float k_unscale;
            {
                const Table<KB> tk = build_int_table<T, KB>(sm.cb[0], nk, k_unscale);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int w = 0; w < 8; ++w) {
                        const uint32_t word = kw[8 * half + w];
                        lookup4<KB>(tk, word, lo[2 * w], hi[2 * w]);
                        lookup4<KB>(tk, word >> 16, lo[2 * w + 1], hi[2 * w + 1]);
                    }
                    tmem_st16_nowait(lane_base + kUColKhi + 16 * half, hi);
                    tmem_st16_nowait(lane_base + kUColKlo + 16 * half, lo);
                }
            }
            if constexpr (TMA) {
                if (tile + 1 < t_end) {                  // the staged rows of the next tile
                    failed |= !mbar_wait(&sm.bar_in[warp], ph_in);
                    ph_in ^= 1u;
                    fetch_staged(0, kw, nk);
                }
            } else {
                fetch_direct(0, next_slot, kw, nk);
            }
            tmem_wait_st();                              // the digit planes are in TMEM
            tc_fence_before();
            __syncthreads();
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    tc_mma_i8_ta(tmem + kUColS, tmem + kUColKhi + 8 * s, smem_desc(q_addr + 256 * s, 128, 1024),
                                 idesc_s, s > 0 ? 1u : 0u);
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    tc_mma_i8_ta(tmem + kUColS + 16, tmem + kUColKlo + 8 * s, smem_desc(q_addr + 256 * s, 128, 1024),
                                 idesc_s, s > 0 ? 1u : 0u);
                tc_commit(&sm.bar_s);
            }

            // ---- 3: V row -> shared tile (the previous tile's P V must have read it) ----
            if (pv_pending) {
                failed |= !mbar_wait(&sm.bar_o, ph_o);
                ph_o ^= 1u;
                tc_fence_after();
            }
            uint32_t d[32];                              // the 32 sums of this token (see step 4)
            {
                const Table<VB> tb = build_value_table<T, VB>(sm.cb[1], nv);
#pragma unroll
                for (int c = 0; c < 16; ++c) {       // 8 head-dims = one 32-bit index word per chunk
                    if (c == 8) {
                        // S^T is normally complete by now: request this token's sums so that the TMEM
                        // read runs under the second half of the V row
                        failed |= !mbar_wait(&sm.bar_s, ph_s);
                        ph_s ^= 1u;
                        tc_fence_after();
                        tmem_ld32_nowait(lane_base + kUColS, d);
                    }
                    uint32_t lo0, hi0, lo1, hi1;
                    lookup4<VB>(tb, vw[c], lo0, hi0);
                    lookup4<VB>(tb, vw[c] >> 16, lo1, hi1);
                    *reinterpret_cast<uint4*>(v_dst + c * 128) =
                        make_uint4(prmt(lo0, hi0, 0x5140), prmt(lo0, hi0, 0x7362),
                                   prmt(lo1, hi1, 0x5140), prmt(lo1, hi1, 0x7362));
                }
            }
            if constexpr (TMA) {
                v_rows_landed();
                if (tile + 1 < t_end) fetch_staged(1, vw, nv);
                __syncwarp();                            // the staging rows are free again
                if (tile + 2 < t_end) issue_tile(tile + 2, pf_blk);
                pf_blk = load_blk(tile + 3);
            } else {
                fetch_direct(1, next_slot, vw, nv);
            }

            // ---- 4: scores, lazy reference maximum, probabilities ----
            float sc[NH];
            const float tok_bias = valid ? 0.0f : -INFINITY;
            {
                tmem_wait_ld();
                tmem_ld32_landed(d);
                const float4 qf0 = *reinterpret_cast<const float4*>(&sm.qf[0]);
                const float4 qf1 = *reinterpret_cast<const float4*>(&sm.qf[4]);
                const float qf[8] = {qf0.x, qf0.y, qf0.z, qf0.w, qf1.x, qf1.y, qf1.z, qf1.w};
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    // d[h] = Khi.Qhi, d[8+h] = Khi.Qlo, d[16+h] = Klo.Qhi, d[24+h] = Klo.Qlo
                    const int t1 = static_cast<int>(d[h]) * 256 + (static_cast<int>(d[8 + h]) + static_cast<int>(d[16 + h]));
                    const float f = fmaf(static_cast<float>(t1), 256.0f, static_cast<float>(static_cast<int>(d[24 + h])));
                    // heads beyond the group have factor 0: they behave like heads with all-zero scores and
                    // their columns are never written out; tokens past the end get -inf (probability 0)
                    sc[h] = fmaf(f, qf[h] * k_unscale, tok_bias);
                }
            }
            bool grow = false;
#pragma unroll
            for (int h = 0; h < NH; ++h) grow |= sc[h] > m_ref[h] + 8.0f;
            // The probabilities are written on the assumption that no reference maximum moves; the
            // block votes at the barrier that the P V issue needs anyway, and in the rare other case
            // the maxima are moved and the probabilities written again.
            float pr[NH];
            auto emit_p = [&]() {
#pragma unroll
                for (int h = 0; h < NH; ++h) pr[h] = ex2_approx(sc[h] - m_ref[h]);
                uint32_t ph[4] = {0u, 0u, 0u, 0u}, pl[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int j = 0; j < NH / 2; ++j) {
                    ph[j] = pack_pair<T>(pr[2 * j], pr[2 * j + 1]);
                    const float2 back = unpack_pair<T>(ph[j]);
                    pl[j] = pack_pair<T>(pr[2 * j] - back.x, pr[2 * j + 1] - back.y);
                }
                *reinterpret_cast<uint4*>(p_dst) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                *reinterpret_cast<uint4*>(p_dst + 128) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                fence_async_proxy();
                tc_fence_before();
            };
            emit_p();
            if (__syncthreads_or(grow || failed)) {
                if (__syncthreads_or(failed)) { dead = true; break; }
                // move the reference maxima: CTA-wide maximum per head, rescale sums and O^T
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    float m = sc[h];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                    if (lane == 0) sm.red[warp][h] = m;
                }
                __syncthreads();
                float alpha[kHeadsPerCta];
#pragma unroll
                for (int h = NH; h < kHeadsPerCta; ++h) alpha[h] = 1.0f;
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const float m_tile = fmaxf(fmaxf(sm.red[0][h], sm.red[1][h]), fmaxf(sm.red[2][h], sm.red[3][h]));
                    const float m_new = fmaxf(m_ref[h], m_tile);
                    alpha[h] = (m_new == -INFINITY) ? 1.0f : ex2_approx(m_ref[h] - m_new);   // 0 on the first tile
                    l_acc[h] *= alpha[h];
                    m_ref[h] = m_new;
                }
                if (tile > t_begin) {                // O^T holds a sum: lane = head-dim, column = head (hi | lo)
                    uint32_t o[16];
                    tmem_ld16_nowait(lane_base + kUColO, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha[c & 7]);
                    tmem_st16_nowait(lane_base + kUColO, o);
                    tmem_wait_st();
                }
                emit_p();
                __syncthreads();
            }
#pragma unroll
            for (int h = 0; h < NH; ++h) l_acc[h] += pr[h];

            // ---- 5: O^T += V^T [P hi | P lo] ----
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    tc_mma_f16(tmem + kUColO, smem_desc(v_addr + 4096 * s, 2048, 128),
                               smem_desc(p_addr + 512 * s, 256, 128), idesc_o, (tile > t_begin || s > 0) ? 1u : 0u);
                tc_commit(&sm.bar_o);
            }
            pv_pending = true;
        }

        // ---- partial result of this part -> workspace row (group + sequence) * J + item ----
        if (pv_pending) {
            const bool failed = !mbar_wait(&sm.bar_o, ph_o);
            ph_o ^= 1u;
            tc_fence_after();
            if (__syncthreads_or(failed)) dead = true;
        }
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            float v = l_acc[h];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) sm.red[warp][h] = v;
        }
        __syncthreads();
        const int64_t row = (group + seq) * J + item;
        if (tid < heads_here) {
            float m = m_ref[0];
#pragma unroll
            for (int h = 1; h < NH; ++h) m = tid == h ? m_ref[h] : m;
            const float l = (sm.red[0][tid] + sm.red[1][tid]) + (sm.red[2][tid] + sm.red[3][tid]);
            p.ws_m[row * kHeadsPerCta + tid] = m;
            p.ws_l[row * kHeadsPerCta + tid] = dead ? __int_as_float(0x7fc00000) : l;
        }
        if (!dead) {
            uint32_t o[16];
            tmem_ld16_nowait(lane_base + kUColO, o);
            tmem_wait_ld();
#pragma unroll
            for (int h = 0; h < NH; ++h)               // lane (position) x holds head-dim x ^ 1
                if (h < heads_here)
                    p.ws_o[(row * kHeadsPerCta + h) * kHeadDim + (tid ^ 1)] =
                        __uint_as_float(o[h]) + __uint_as_float(o[8 + h]);
        }
        tc_fence_before();
        __syncthreads();

        x += t_end - t_begin;
        if (t_end == n_s) ++seq;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kUTmemCols);
}

// Merge for the streaming kernel: the parts of a (sequence, head) are the groups whose pieces
// overlap the sequence's tile range; part (group, sequence) of item j lives at row
// (group + sequence) * J + j.  Warp 0 gathers the running maxima and row sums of up to 32 parts
// at a time with one load per lane; then every thread sums its head-dim over the parts.
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
decode_stream_merge_kernel(const DecodeParams p) {
    __shared__ float o_s[kHeadDim];
    __shared__ float w_s[32];
    __shared__ float l_s, m_s;
    const int seq = blockIdx.x / p.Hq, qh = blockIdx.x % p.Hq;
    const int d = threadIdx.x, lane = d & 31;
    const int J = p.H * p.head_groups;
    const int kvh = qh / p.G, hl = qh % p.G;
    const int item = kvh * p.head_groups + hl / kHeadsPerCta, h = hl % kHeadsPerCta;
    const int2 gr = __ldg(p.seq_groups + seq);
    const int64_t total = __ldg(p.tile_prefix + p.num_seqs);
    const bool n_s = gr.y >= gr.x;                                     // the sequence has tiles
    float acc = 0.0f;
    float l_all = 0.0f;
    if (n_s) {                                                         // uniform for the CTA
        const int64_t g_first = gr.x, g_last = gr.y;
        float m_all = -INFINITY;
        for (int64_t g0 = g_first; g0 <= g_last; g0 += 32) {           // normally one round
            const int64_t gi = g0 + lane;
            // groups whose piece is empty (only when there are more groups than tiles) wrote nothing
            const bool live = gi <= g_last && piece_begin(p.group_cum, p.stream_groups, gi, total) <
                                                  piece_begin(p.group_cum, p.stream_groups, gi + 1, total);
            const int64_t r = ((gi + seq) * J + item) * kHeadsPerCta + h;
            if (d < 32) {
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
                w_s[lane] = w;
                if (lane == 0) { m_s = m_new; l_s = l_round; }
            }
            __syncthreads();
            const float rescale = exp2f(m_all - m_s);                  // 0 in the first round
            acc *= rescale;
            l_all = l_all * rescale + l_s;
            m_all = m_s;
            const int64_t left = g_last - g0 + 1;
            const int n_here = left < 32 ? static_cast<int>(left) : 32;
            for (int k = 0; k < n_here; ++k) {
                const float w = w_s[k];
                if (w != 0.0f) acc += w * p.ws_o[(((g0 + k + seq) * J + item) * kHeadsPerCta + h) * kHeadDim + d];
            }
            __syncthreads();
        }
    }
    const float o = n_s ? acc / l_all : 0.0f;          // an empty sequence yields zeros
    o_s[d] = round_to<T>(o);
    __syncthreads();
    // out[j] = sum_k o[k] R[k][j] over the 4x4 block of j, ascending k, fused multiply-adds
    const int b4 = d & ~3;
    float r = __fmul_rn(o_s[b4], __ldg(p.rotation + b4 * kHeadDim + d));
#pragma unroll
    for (int k = 1; k < 4; ++k) r = __fmaf_rn(o_s[b4 + k], __ldg(p.rotation + (b4 + k) * kHeadDim + d), r);
    T* dst = static_cast<T*>(p.out) + seq * p.o_stride_seq + static_cast<int64_t>(qh) * p.o_stride_head + d;
    store_rounded(dst, r);
}

// ---- host side -------------------------------------------------------------------------------

// Two kernels implement the decode: the tensor-memory kernel (default) and the warp-streaming
// kernel.  RQ_DECODE_PATH=stream in the environment selects the latter (for comparisons).
enum class DecodePath { kUmma, kStream };
static DecodePath decode_path() {
    static const DecodePath path = [] {
        const char* e = std::getenv("RQ_DECODE_PATH");
        return (e != nullptr && std::string(e) == "stream") ? DecodePath::kStream : DecodePath::kUmma;
    }();
    return path;
}

// Grid and scratch of one decode call.  The (sequence, tile) space is cut into `groups` equal
// pieces; each piece is walked by J workers (warps of the streaming kernel, CTAs of the
// tensor-memory kernel), one per (KV head, head group).
struct StreamPlan {
    int warps;             // streaming kernel: launched warps (multiple of 8)
    int groups;            // pieces
    size_t rows;           // partial-result rows: (group + sequence) * J + item
    size_t prefix_bytes;
    size_t bytes;
};
static void finish_plan(StreamPlan& pl, long long groups, long long J, int num_seqs) {
    pl.groups = static_cast<int>(groups);
    pl.warps = static_cast<int>((groups * J + kDecodeWarps - 1) / kDecodeWarps * kDecodeWarps);
    pl.rows = static_cast<size_t>((groups + num_seqs) * J);
    // tile prefix sums [num_seqs + 1] (int32, padded to 8 bytes), then the group range of every sequence (int2)
    // then the running weights of the groups (int32 [groups + 1])
    pl.prefix_bytes = ((static_cast<size_t>(num_seqs + 2) / 2 * 2) * sizeof(int32_t) + static_cast<size_t>(num_seqs) * sizeof(int2) +
                       static_cast<size_t>(groups + 1) * sizeof(int32_t) + 255) / 256 * 256;
    pl.bytes = pl.prefix_bytes + pl.rows * kHeadsPerCta * (kHeadDim + 2) * sizeof(float);
}
// Streaming kernel: groups get at least 8 tiles of 16 tokens each when the bound on the work
// allows; the grid never exceeds two 8-warp CTAs per SM (148 SMs).  `forced` > 0 asks for that
// many pieces per sequence.
static StreamPlan plan_stream(int num_seqs, int H, int head_groups, int max_seq_len, int forced) {
    const long long J = 1LL * H * head_groups;
    const long long max_tiles = max_seq_len > 0 ? (max_seq_len + kTile - 1) / kTile : 1;
    const long long work = 1LL * num_seqs * max_tiles;                   // tiles per item, at most
    long long groups = forced > 0 ? 1LL * forced * num_seqs : (work + 7) / 8;
    long long cap = (forced > 0 ? 4LL : 1LL) * 148 * 2 * kDecodeWarps / J;
    if (cap < 1) cap = 1;
    if (groups > cap) groups = cap;
    if (groups < 1) groups = 1;
    StreamPlan pl;
    finish_plan(pl, groups, J, num_seqs);
    return pl;
}
// Tensor-memory kernel: one 128-token tile per piece at least; at most four CTAs per SM.
static StreamPlan plan_umma(int num_seqs, int H, int head_groups, int max_seq_len, int forced) {
    const long long J = 1LL * H * head_groups;
    const long long max_tiles = max_seq_len > 0 ? (max_seq_len + kUTile - 1) / kUTile : 1;
    const long long work = 1LL * num_seqs * max_tiles;
    long long groups = forced > 0 ? 1LL * forced * num_seqs : work;
    long long cap = (forced > 0 ? 4LL : 1LL) * 148 * kUCtasPerSm / J;
    if (cap < 1) cap = 1;
    if (groups > cap) groups = cap;
    if (groups < 1) groups = 1;
    StreamPlan pl;
    finish_plan(pl, groups, J, num_seqs);
    return pl;
}
static StreamPlan plan_decode(int num_seqs, int H, int head_groups, int max_seq_len, int forced) {
    return decode_path() == DecodePath::kUmma ? plan_umma(num_seqs, H, head_groups, max_seq_len, forced)
                                              : plan_stream(num_seqs, H, head_groups, max_seq_len, forced);
}

// ---- tensor maps of the cache for the TMA path ------------------------------------------------
//
// The cache is described as a 2-D byte tensor (num_slots rows of total_bytes): one map with a
// 16 x 64 B box and 64-byte swizzle for the index regions, one with a 16 x 16 B box for the norms.
// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the
// library does not link against the driver.

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

static bool encode_cache_map(CUtensorMap* map, const uint8_t* cache, int64_t num_slots, int total_bytes,
                             int box_bytes, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(total_bytes), static_cast<cuuint64_t>(num_slots)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(total_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(kTile)};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(cache), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The TMA path needs 16-byte aligned box origins (KV heads a multiple of 4), tiles that never
// straddle a block (power-of-two block size >= 16) and slot numbers that fit an int32 coordinate.
// RQ_DECODE_NO_TMA=1 in the environment selects the cp.async path everywhere (for comparisons).
// The tensor-memory kernel only needs that for its K rows (always aligned); V rows of 1 or 2 KV heads
// go through cp.async there.
static bool tma_eligible(const DecodeParams& p, bool aligned_v_rows_needed) {
    static const bool disabled = [] {
        const char* e = std::getenv("RQ_DECODE_NO_TMA");
        return e != nullptr && e[0] != '\0' && e[0] != '0';
    }();
    return !disabled && (p.H % 4 == 0 || !aligned_v_rows_needed) && p.bs_shift >= 4 && aligned(p.cache, 16) &&
           p.num_blocks * p.block_size <= INT32_MAX && p.total_bytes == p.H * 256;
}

template <typename T, int KB, int VB, bool TMA>
static int launch_stream(const DecodeParams& p, const CUtensorMap& map_idx, const CUtensorMap& map_norm,
                         cudaStream_t st) {
    const size_t smem = kDecodeWarps * sizeof(StreamWarpSmem<TMA>) + 512;    // + hand alignment
    if (int e = ensure_smem(decode_stream_kernel<T, KB, VB, TMA>, smem)) return e;
    decode_stream_kernel<T, KB, VB, TMA>
        <<<p.stream_warps / kDecodeWarps, kDecodeThreads, smem, st>>>(p, map_idx, map_norm);
    return check_cuda(cudaGetLastError(), "rq_decode stream launch");
}

template <typename T, int KB, int VB>
static int launch_decode(const DecodeParams& p, int num_seqs, cudaStream_t st) {
    const bool umma = decode_path() == DecodePath::kUmma;
    decode_plan_kernel<<<1, 1024, 0, st>>>(p.seq_lens, num_seqs, umma ? kUTile : kTile,
                                           const_cast<int32_t*>(p.tile_prefix), p.stream_groups,
                                           const_cast<int2*>(p.seq_groups), const_cast<int32_t*>(p.group_cum),
                                           p.H * p.head_groups, p.weight_layers);
    if (int e = check_cuda(cudaGetLastError(), "rq_decode plan launch")) return e;
    alignas(64) CUtensorMap map_idx{}, map_norm{};
    bool tma = tma_eligible(p, !umma);
    const int64_t num_slots = p.num_blocks * p.block_size;
    if (tma) tma = encode_cache_map(&map_idx, p.cache, num_slots, p.total_bytes, kHalfDim, CU_TENSOR_MAP_SWIZZLE_64B);
    if (umma) {
        const size_t smem = sizeof(UmmaSmem) + 512;                              // + hand alignment
        const long long ctas = 1LL * p.stream_groups * p.H * p.head_groups;
        auto launch = [&](auto kernel) -> int {
            if (int e = ensure_smem(kernel, smem)) return e;
            kernel<<<static_cast<unsigned>(ctas), kUThreads, smem, st>>>(p, map_idx);
            return RQ_OK;
        };
        const bool few = p.G <= 4;                                               // at most 4 query heads per item
        const int mode = !tma ? 0 : (p.H % 4 == 0 ? 1 : 2);
        int e = RQ_OK;
        if (mode == 0) e = few ? launch(decode_umma_kernel<T, KB, VB, 0, 4>) : launch(decode_umma_kernel<T, KB, VB, 0, 8>);
        else if (mode == 1) e = few ? launch(decode_umma_kernel<T, KB, VB, 1, 4>) : launch(decode_umma_kernel<T, KB, VB, 1, 8>);
        else e = few ? launch(decode_umma_kernel<T, KB, VB, 2, 4>) : launch(decode_umma_kernel<T, KB, VB, 2, 8>);
        if (e) return e;
        if (int e = check_cuda(cudaGetLastError(), "rq_decode tensor-memory launch")) return e;
    } else {
        if (tma) tma = encode_cache_map(&map_norm, p.cache, num_slots, p.total_bytes, kNormBox, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (int e = tma ? launch_stream<T, KB, VB, true>(p, map_idx, map_norm, st)
                        : launch_stream<T, KB, VB, false>(p, map_idx, map_norm, st))
            return e;
    }
    decode_stream_merge_kernel<T><<<num_seqs * p.Hq, kHeadDim, 0, st>>>(p);
    return check_cuda(cudaGetLastError(), "rq_decode merge launch");
}

template <typename T>
static int dispatch_bits(const DecodeParams& p, int num_seqs, int kb, int vb, cudaStream_t st) {
    if (kb == 3 && vb == 3) return launch_decode<T, 3, 3>(p, num_seqs, st);
    if (kb == 4 && vb == 3) return launch_decode<T, 4, 3>(p, num_seqs, st);
    if (kb == 3 && vb == 4) return launch_decode<T, 3, 4>(p, num_seqs, st);
    return launch_decode<T, 4, 4>(p, num_seqs, st);
}

}  // namespace rq

using namespace rq;

extern "C" size_t rq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                            int head_dim, int max_seq_len, int num_splits) {
    if (num_seqs <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim != kHeadDim) return 0;
    const int G = num_q_heads / num_kv_heads;
    const int head_groups = (G + kHeadsPerCta - 1) / kHeadsPerCta;
    return plan_decode(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits).bytes;
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
    const int head_groups = (G + kHeadsPerCta - 1) / kHeadsPerCta;
    const StreamPlan pl = plan_decode(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits);
    const size_t need = pl.bytes;
    if (!workspace || workspace_bytes < need)
        return fail(RQ_ERR_WORKSPACE, "rq_decode: workspace of %zu bytes needed, %zu given", need,
                    workspace_bytes);
    if (!aligned(workspace, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_decode: workspace must be 16-byte aligned");
    if (static_cast<long long>(num_kv_heads) * head_groups > 65535)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: too many KV heads");

    DecodeParams p{};
    p.q = q; p.q_stride_seq = q_stride_seq; p.q_stride_head = q_stride_head;
    p.cache = kv_cache; p.num_blocks = num_blocks; p.block_size = block_size;
    p.total_bytes = total_bytes; p.block_table = block_table; p.bt_stride = block_table_stride;
    p.seq_lens = seq_lens; p.cent_k = centroids_k; p.cent_v = centroids_v; p.rotation = rotation;
    p.qk_scale = sm_scale * 1.4426950408889634f;
    p.H = num_kv_heads; p.Hq = num_q_heads; p.G = G; p.head_groups = head_groups;
    p.tile_prefix = static_cast<const int32_t*>(workspace);
    p.seq_groups = reinterpret_cast<const int2*>(static_cast<const int32_t*>(workspace) + (num_seqs + 2) / 2 * 2);
    p.group_cum = reinterpret_cast<const int32_t*>(p.seq_groups + num_seqs);
    const size_t rows = pl.rows * kHeadsPerCta;
    p.ws_o = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.prefix_bytes);
    p.ws_m = p.ws_o + rows * kHeadDim;
    p.ws_l = p.ws_m + rows;
    p.num_seqs = num_seqs; p.stream_warps = pl.warps; p.stream_groups = pl.groups;
    // weighted pieces only for the tensor-memory kernel with (nearly) four CTAs on every SM
    p.weight_layers = (decode_path() == DecodePath::kUmma && std::getenv("RQ_DECODE_EQUAL_PIECES") == nullptr &&
                       1LL * pl.groups * num_kv_heads * head_groups > 3LL * 148) ? 148 : 0;
    p.bs_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
        if ((1 << sft) == block_size) p.bs_shift = sft;
    p.out = out; p.o_stride_seq = o_stride_seq; p.o_stride_head = o_stride_head;

    const int kb = n_centroids_k == 8 ? 3 : 4, vb = n_centroids_v == 8 ? 3 : 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RQ_DTYPE_BF16) return dispatch_bits<__nv_bfloat16>(p, num_seqs, kb, vb, st);
    return dispatch_bits<__half>(p, num_seqs, kb, vb, st);
}

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
