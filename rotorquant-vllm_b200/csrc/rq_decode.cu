// Fused paged decode attention over the RotorQuant cache, sm_100a.
//
// Replaces fused_paged_rq_decode (triton/fused_paged_rq_decode.py:32-312 of the reference): the
// Triton kernel (one program per (sequence, query head), CUDA-core dot products, no split-KV)
// and the two dense 128x128 rotations its launcher runs around it.
//
// Work decomposition.  Three launches: a one-CTA prefix sum of the tiles per sequence, the
// streaming kernel (see below: every warp of a fixed grid streams an equal share of the
// (sequence, 16-token tile) space for one KV head, with a private cp.async ring, so the 136
// payload bytes of a (token, KV head) are read from HBM exactly once for all query heads of the
// GQA group), and a merge kernel that combines the partial results, rounds, and applies R.
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
// mma.sync m16n8k16 is used on purpose: M is the 4..8 query heads of one KV head, far below the
// 128-row tiles tcgen05 needs, and the kernel is bound by HBM bytes and dequantisation
// instructions, not by tensor throughput.
#include <mutex>

#include "rq_common.cuh"

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
    int num_seqs;
    int stream_warps;                     // warps of the streaming grid (multiple of 8)
    int stream_groups;                    // groups of J warps; each owns one piece of the tile space
    int bs_shift;                         // log2(block_size) when it is a power of two, else -1
};

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

// ---- shared memory ------------------------------------------------------------

struct __align__(16) Stage {
    uint8_t k[kTile][kHalfDim];        // K indices of 16 tokens
    uint8_t v[kTile][kVPitch];         // V indices, padded rows (conflict-free 16-byte reads)
    float norms[2 * kTile];            // [0..15] K norms, [16..31] V norms
};
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

struct __align__(256) StreamWarpSmem {
    uint16_t vt[kTile][kHeadDim];      // V transposition tile; also Q set-up scratch and output stage
    Stage stage[kStages];
    uint32_t tbl_k[kTile][8];
    uint32_t tbl_v[kTile][8];
    float k_unscale[kTile];
    float cb[2][16];                   // K and V codebooks (per warp: no CTA-wide barrier needed)
};
static_assert(sizeof(StreamWarpSmem::vt) >= 2 * kHeadsPerCta * kHeadDim, "vt holds the query byte planes");
static_assert(sizeof(StreamWarpSmem::vt) >= sizeof(float) * kHeadsPerCta * kHeadDim, "vt stages the partial output");

// One 16-token tile: tables, S = Q K^T (int8), online softmax, V transposition, O += P V.
template <typename T, int KB, int VB>
__device__ __forceinline__ void stream_tile(StreamWarpSmem& ws, const Stage& st, int n_valid, int lane,
                                            int g, int tig, const uint32_t (&qa)[4][4], float q_factor,
                                            float& m_run, float& l_run, float (&o_acc)[8][4], int tv,
                                            int vhalf, uint32_t vt_store_base, uint32_t lm_base) {
    // ---- per-token tables: lane builds one half (lane >> 4) of the K and of the V table of
    //      token (lane & 15), so both half-warps run the same instructions ----
    {
        const int i = lane & 15, hb = lane >> 4;
        const bool valid = i < n_valid;
        const float norm_k = valid ? st.norms[i] : 0.0f;
        const float norm_v = valid ? st.norms[kTile + i] : 0.0f;
        constexpr int NKH = (1 << KB) / 2, NVH = (1 << VB) / 2;
        float unscale;
        uint32_t lo[NKH / 4], hi[NKH / 4];
        build_half_int_table<T, NKH>(&ws.cb[0][hb * NKH], norm_k, lo, hi, unscale);
        uint32_t vlo[NVH / 4], vhi[NVH / 4];
        build_half_value_table<T, NVH>(&ws.cb[1][hb * NVH], norm_v, vlo, vhi);
#pragma unroll
        for (int r = 0; r < NKH / 4; ++r) {
            ws.tbl_k[i][hb * (NKH / 4) + r] = lo[r];
            ws.tbl_k[i][2 * (NKH / 4) + hb * (NKH / 4) + r] = hi[r];
        }
#pragma unroll
        for (int r = 0; r < NVH / 4; ++r) {
            ws.tbl_v[i][hb * (NVH / 4) + r] = vlo[r];
            ws.tbl_v[i][2 * (NVH / 4) + hb * (NVH / 4) + r] = vhi[r];
        }
        if (hb == 0) ws.k_unscale[i] = unscale;
    }
    __syncwarp();

    // ---- S = Q K^T on the int8 path: rows = heads (g), columns = tokens ----
    float sc[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
        // acc_h = [Qhi; Qlo] . Khi, acc_l = [Qhi; Qlo] . Klo: entries 0,1 are the Qhi rows,
        // entries 2,3 the Qlo rows of the same head and the same two tokens
        int acc_h[4] = {0, 0, 0, 0}, acc_l[4] = {0, 0, 0, 0};
        const int tok = g + 8 * nt;
        const uint4 kw = *reinterpret_cast<const uint4*>(&st.k[tok][16 * tig]);
        const Table<KB> tk = load_table<KB>(ws.tbl_k[tok]);
        const uint32_t words[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t lo0, hi0, lo1, hi1;
            lookup4<KB>(tk, words[w], lo0, hi0);            // nibbles 0..3 -> k-slots 4tig..
            lookup4<KB>(tk, words[w] >> 16, lo1, hi1);      // nibbles 4..7 -> k-slots 16+4tig..
            mma_s8(acc_h, qa[w][0], qa[w][1], qa[w][2], qa[w][3], hi0, hi1);
            mma_s8(acc_l, qa[w][0], qa[w][1], qa[w][2], qa[w][3], lo0, lo1);
        }
        const float2 ku = *reinterpret_cast<const float2*>(&ws.k_unscale[8 * nt + 2 * tig]);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int t1 = acc_h[c] * 256 + (acc_h[c + 2] + acc_l[c]);
            const float f = fmaf(static_cast<float>(t1), 256.0f, static_cast<float>(acc_l[c + 2]));
            sc[2 * nt + c] = f * (q_factor * (c ? ku.y : ku.x));
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

    // ---- decompress V into the transposition buffer: lane = (token tv, half row) ----
    {
        const Table<VB> tb = load_table<VB>(ws.tbl_v[tv]);
        const uint4 va = *reinterpret_cast<const uint4*>(&st.v[tv][32 * vhalf]);
        const uint4 vb = *reinterpret_cast<const uint4*>(&st.v[tv][32 * vhalf + 16]);
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
    }
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

// Tiles of every sequence as an exclusive prefix sum: prefix[s] = sum_{s' < s} ceil(len[s'] / 16).
__global__ void decode_plan_kernel(const int32_t* __restrict__ seq_lens, int num_seqs,
                                   int32_t* __restrict__ prefix) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < num_seqs; base += blockDim.x) {
        const int s = base + threadIdx.x;
        const int n = s < num_seqs ? (max(__ldg(seq_lens + s), 0) + kTile - 1) / kTile : 0;
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

template <typename T, int KB, int VB>
__global__ void __launch_bounds__(kDecodeThreads, 2)
decode_stream_kernel(const DecodeParams p) {
    extern __shared__ __align__(256) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    StreamWarpSmem& ws = reinterpret_cast<StreamWarpSmem*>(smem_raw)[warp];
    const int g = lane >> 2, tig = lane & 3;

    // ---- this warp's piece: warp = (group, item); a group of J consecutive warps walks one
    //      range of the (sequence, tile) space, one warp per (KV head, head group) ----
    const int J = p.H * p.head_groups;                         // items per sequence
    const int64_t total = __ldg(p.tile_prefix + p.num_seqs);   // tiles of all sequences
    const int64_t wq = static_cast<int64_t>(blockIdx.x) * kDecodeWarps + warp;
    const int64_t group = wq / J;
    const int item = static_cast<int>(wq % J);
    if (group >= p.stream_groups) return;
    int64_t x = group * total / p.stream_groups;
    const int64_t x_end = (group + 1) * total / p.stream_groups;
    if (x >= x_end) return;

    if (lane < 32) {
        const int kv = lane >> 4, i = lane & 15;
        const int n = kv ? (1 << VB) : (1 << KB);
        ws.cb[kv][i] = i < n ? __ldg((kv ? p.cent_v : p.cent_k) + i) : 0.0f;
    }
    const SlotLayout lay = slot_layout(p.H);
    const bool fast_bt = p.bs_shift >= 4;                      // power-of-two block size >= 16
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);
    const uint32_t tb = static_cast<uint32_t>(p.total_bytes);
    const int tv = lane & 15, vhalf = lane >> 4;
    const int lm_tok = (lane & 7) + ((lane & 16) ? 8 : 0);
    const int lm_chunk = (lane >> 3) & 1;
    const uint32_t vt_store_base = smem_u32(&ws.vt[tv][0]) + 128u * vhalf + 16u * (tv & 7);
    const uint32_t lm_base = smem_u32(&ws.vt[lm_tok][0]) + 16u * (lm_chunk ^ (lm_tok & 7));

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

        auto clamp_block = [&](int64_t blk) -> int64_t {
            return blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
        };
        auto tile_base = [&](int tile) -> const uint8_t* {     // fast path: first slot of the tile
            const int t0 = tile * kTile;
            const int64_t blk = clamp_block(__ldg(bt_row + (t0 >> p.bs_shift)));
            return p.cache + ((blk << p.bs_shift) + (t0 & (p.block_size - 1))) * p.total_bytes;
        };
        auto token_ptr = [&](int tile, int i) -> const uint8_t* {   // general path
            const int t = min(tile * kTile + i, seq_len - 1);
            const int64_t blk = clamp_block(__ldg(bt_row + t / p.block_size));
            return p.cache + (blk * p.block_size + (t % p.block_size)) * p.total_bytes;
        };
        const uint32_t src_k = (lane >> 2) * tb + kvh * kHalfDim + 16 * (lane & 3);
        const uint32_t dst_k = (lane >> 2) * kHalfDim + 16 * (lane & 3);
        const uint32_t dst_v16 = sizeof(Stage::k) + (lane >> 2) * kVPitch + 16 * (lane & 3);
        const uint32_t src_n = (lane & 15) * tb + ((lane >> 4) ? lay.v_norm : lay.k_norm) + 4 * kvh;
        const uint32_t dst_n = sizeof(Stage::k) + sizeof(Stage::v) + 4 * lane;
        auto issue = [&](int tile, int s, const uint8_t* base) {
            uint8_t* stg = reinterpret_cast<uint8_t*>(&ws.stage[s]);
            if (fast_bt) {
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
                return;
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = lane + 32 * j, i = c >> 2, part = c & 3;
                cp_async16(stg + i * kHalfDim + 16 * part,
                           token_ptr(tile, i) + lay.k_idx + kvh * kHalfDim + 16 * part);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = lane + 32 * j, i = c >> 4, part = c & 15;
                cp_async4(stg + sizeof(Stage::k) + i * kVPitch + 4 * part,
                          token_ptr(tile, i) + lay.v_idx + kvh * kHalfDim + 4 * part);
            }
            cp_async4(stg + dst_n, token_ptr(tile, lane & 15) +
                                       ((lane >> 4) ? lay.v_norm : lay.k_norm) + 4 * kvh);
        };

        // first tiles in flight before the query set-up; the block-table entry of the tile after
        // the one being issued is read one step ahead so that its latency is off the issue path
        int pf_tile = t_begin, pf_stage = 0;
        const uint8_t* pf_base = fast_bt ? tile_base(t_begin) : nullptr;
        auto issue_next = [&]() {
            if (pf_tile < t_end) {
                issue(pf_tile, pf_stage, pf_base);
                ++pf_tile;
                pf_stage = pf_stage + 1 == kStages ? 0 : pf_stage + 1;
                if (fast_bt && pf_tile < t_end) pf_base = tile_base(pf_tile);
            }
            cp_async_commit();
        };
#pragma unroll 1
        for (int s = 0; s < kStages - 1; ++s) issue_next();

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

        int cur_stage = 0;
#pragma unroll 1
        for (int tile = t_begin; tile < t_end; ++tile) {
            issue_next();
            cp_async_wait<kStages - 1>();
            __syncwarp();
            const Stage& st = ws.stage[cur_stage];
            cur_stage = cur_stage + 1 == kStages ? 0 : cur_stage + 1;
            stream_tile<T, KB, VB>(ws, st, min(kTile, seq_len - tile * kTile), lane, g, tig, qa, q_factor,
                                   m_run, l_run, o_acc, tv, vhalf, vt_store_base, lm_base);
            __syncwarp();      // the stage, the tables and vt may be overwritten from here on
        }
        cp_async_wait<0>();

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
    const int pre = __ldg(p.tile_prefix + seq), n_s = __ldg(p.tile_prefix + seq + 1) - pre;
    const int64_t total = __ldg(p.tile_prefix + p.num_seqs);
    const int64_t ng = p.stream_groups;
    float acc = 0.0f;
    float l_all = 0.0f;
    if (n_s > 0) {                                                     // uniform for the CTA
        const int64_t a = pre, b = a + n_s;                            // the sequence's tiles
        const int64_t g_first = ((a + 1) * ng - 1) / total;           // group holding tile a
        const int64_t g_last = (b * ng - 1) / total;                  // group holding tile b - 1
        float m_all = -INFINITY;
        for (int64_t g0 = g_first; g0 <= g_last; g0 += 32) {           // normally one round
            const int64_t gi = g0 + lane;
            // groups whose piece is empty (more groups than tiles) wrote nothing
            const bool live = gi <= g_last && gi * total / ng < (gi + 1) * total / ng;
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
    const float o = n_s > 0 ? acc / l_all : 0.0f;      // an empty sequence yields zeros
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

// Grid of the streaming kernel and the scratch it needs.  Warps get at least 8 tiles each when
// the bound on the work allows; the grid never exceeds two 8-warp CTAs per SM (148 SMs).
struct StreamPlan {
    int warps;             // launched warps (multiple of 8)
    int groups;            // groups of J warps
    size_t rows;           // partial-result rows: (group + sequence) * J + item
    size_t prefix_bytes;
    size_t bytes;
};
// Groups get at least 8 tiles each when the bound on the work allows; the grid never exceeds two
// 8-warp CTAs per SM (148 SMs).  `forced` > 0 asks for that many pieces per sequence.
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
    pl.groups = static_cast<int>(groups);
    pl.warps = static_cast<int>((groups * J + kDecodeWarps - 1) / kDecodeWarps * kDecodeWarps);
    pl.rows = static_cast<size_t>((groups + num_seqs) * J);
    pl.prefix_bytes = (static_cast<size_t>(num_seqs + 1) * sizeof(int32_t) + 255) / 256 * 256;
    pl.bytes = pl.prefix_bytes + pl.rows * kHeadsPerCta * (kHeadDim + 2) * sizeof(float);
    return pl;
}

template <typename T, int KB, int VB>
static int launch_decode(const DecodeParams& p, int num_seqs, cudaStream_t st) {
    const size_t smem = kDecodeWarps * sizeof(StreamWarpSmem);
    if (int e = ensure_smem(decode_stream_kernel<T, KB, VB>, smem)) return e;
    decode_plan_kernel<<<1, 1024, 0, st>>>(p.seq_lens, num_seqs, const_cast<int32_t*>(p.tile_prefix));
    if (int e = check_cuda(cudaGetLastError(), "rq_decode plan launch")) return e;
    decode_stream_kernel<T, KB, VB><<<p.stream_warps / kDecodeWarps, kDecodeThreads, smem, st>>>(p);
    if (int e = check_cuda(cudaGetLastError(), "rq_decode stream launch")) return e;
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
    return plan_stream(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits).bytes;
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
    const StreamPlan pl = plan_stream(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits);
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
    const size_t rows = pl.rows * kHeadsPerCta;
    p.ws_o = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.prefix_bytes);
    p.ws_m = p.ws_o + rows * kHeadDim;
    p.ws_l = p.ws_m + rows;
    p.num_seqs = num_seqs; p.stream_warps = pl.warps; p.stream_groups = pl.groups;
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
