// Fused paged decode attention over the RotorQuant cache, sm_100a.
//
// Replaces fused_paged_rq_decode (triton/fused_paged_rq_decode.py:32-312 of the reference): the
// Triton kernel (one program per (sequence, query head), CUDA-core dot products, no split-KV)
// and the two dense 128x128 rotations its launcher runs around it.
//
// Work decomposition.  One CTA = one (sequence, KV head, context split); its eight warps walk
// the split's 16-token tiles round robin, each with a private cp.async ring in shared memory,
// so the 136 payload bytes of a (token, KV head) are read from HBM exactly once for all query
// heads of the GQA group.  A second small kernel merges the splits, rounds, and applies R.
//
// Arithmetic (matches "reference decompress + SDPA"):
//   q_rot   = round_T(q @ R^T)            exact FMA chain per 4x4 block, computed in the prologue
//   K, V    = round_T(centroid[idx]*norm) exactly the decompressed values: each token gets a
//             table of its 8/16 rounded products, elements are fetched from it with PRMT
//   scores  = tensor-core mma (bf16/f16 inputs, fp32 accumulate), exp2-domain online softmax
//   P @ V   = tensor-core mma with P split into hi + lo parts (two T-precision terms, ~16 bits),
//             fp32 accumulate
//   out     = round_T(round_T(o / l) @ R)  in the merge kernel
// mma.sync m16n8k16 is used on purpose: M is the 4..8 query heads of one KV head, far below the
// 128-row tiles tcgen05 needs, and the kernel is bound by HBM bytes and dequantisation
// instructions, not by tensor throughput.
#include "rq_common.cuh"

namespace rq {

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kTile = 16;                 // tokens per tile (one mma k-step of P@V)
constexpr int kStages = 4;                // cp.async ring depth per warp
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
    int tiles_per_split;
    int num_splits;
    float* ws_o;                           // [seq][Hq][split][128]
    float* ws_m;                           // [seq][Hq][split]
    float* ws_l;
    // merge
    void* out;
    int64_t o_stride_seq, o_stride_head;
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
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1,
                                                 uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
    asm volatile(
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
// A table holds round_T(centroid[i] * norm) for i < 2^BITS, split into a low-byte plane and a
// high-byte plane so that one PRMT fetches the bytes of four nibble indices at once.
//   BITS == 3: 4 registers  {lo[0..3], lo[4..7], hi[0..3], hi[4..7]}
//   BITS == 4: 8 registers  {lo[0..3] .. lo[12..15], hi[0..3] .. hi[12..15]}
template <int BITS>
struct Table {
    static constexpr int kRegs = BITS == 3 ? 4 : 8;
    uint32_t r[kRegs];
};

template <typename T, int BITS>
__device__ __forceinline__ Table<BITS> build_table(const float* __restrict__ cb, float norm) {
    constexpr int N = 1 << BITS;
    uint32_t pairs[N / 2];
#pragma unroll
    for (int i = 0; i < N / 2; ++i)
        pairs[i] = pack_pair<T>(__fmul_rn(cb[2 * i], norm), __fmul_rn(cb[2 * i + 1], norm));
    Table<BITS> t;
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        t.r[i] = prmt(pairs[2 * i], pairs[2 * i + 1], 0x6420);             // low bytes
        t.r[N / 4 + i] = prmt(pairs[2 * i], pairs[2 * i + 1], 0x7531);     // high bytes
    }
    return t;
}

// Bytes of the four entries selected by the four nibbles in sel[15:0]: lo plane and hi plane.
template <int BITS>
__device__ __forceinline__ void lookup4(const Table<BITS>& t, uint32_t sel, uint32_t& lo,
                                        uint32_t& hi) {
    if constexpr (BITS == 3) {
        lo = prmt(t.r[0], t.r[1], sel);
        hi = prmt(t.r[2], t.r[3], sel);
    } else {
        const uint32_t s7 = sel & 0x7777u;
        // byte i of `m` is 0xFF when nibble i of sel has its top bit set
        const uint32_t y = prmt(sel, sel << 4, 0x5410);
        const uint32_t m = prmt(y, y, 0x9B8A);
        const uint32_t la = prmt(t.r[0], t.r[1], s7), lb = prmt(t.r[2], t.r[3], s7);
        const uint32_t ha = prmt(t.r[4], t.r[5], s7), hb = prmt(t.r[6], t.r[7], s7);
        lo = (la & ~m) | (lb & m);
        hi = (ha & ~m) | (hb & m);
    }
}

// ---- shared memory ------------------------------------------------------------

struct __align__(16) Stage {
    uint8_t k[kTile][kHalfDim];        // K indices of 16 tokens
    uint8_t v[kTile][kVPitch];         // V indices, padded rows (conflict-free 8-byte reads)
    float norms[2 * kTile];            // [0..15] K norms, [16..31] V norms
};
struct __align__(16) WarpSmem {
    Stage stage[kStages];
    uint32_t tbl_k[kTile][8];          // per-token K tables (4 or 8 registers used)
    uint32_t tbl_v[kTile][8];
};
static_assert(sizeof(WarpSmem) >= sizeof(float) * (kHeadsPerCta * kHeadDim + 2 * kHeadsPerCta),
              "the per-warp area is reused for the cross-warp merge");

struct __align__(16) DecodeSmem {
    WarpSmem warp[kDecodeWarps];
    uint16_t q[kHeadsPerCta][kHeadDim];   // rotated queries, element d stored at d ^ 1
    float cb[2][16];                      // K and V codebooks
};

// ---- the split kernel -------------------------------------------------------------

template <typename T, int KB, int VB>
__global__ void __launch_bounds__(kDecodeThreads, 2)
decode_split_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(smem_raw);

    const int split = blockIdx.x;
    const int kvh = blockIdx.y / p.head_groups;
    const int hg = blockIdx.y % p.head_groups;
    const int seq = blockIdx.z;
    const int heads_here = min(kHeadsPerCta, p.G - hg * kHeadsPerCta);
    const int first_qh = kvh * p.G + hg * kHeadsPerCta;

    int seq_len = __ldg(p.seq_lens + seq);
    seq_len = max(seq_len, 0);
    const int total_tiles = (seq_len + kTile - 1) / kTile;
    const int tile_begin = split * p.tiles_per_split;
    const int tile_end = min(total_tiles, tile_begin + p.tiles_per_split);
    if (tile_begin >= tile_end) return;        // uniform for the CTA

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;

    // ---- prologue: codebooks, q_rot = round(q @ R^T) into shared memory ----
    if (tid < 32) {
        const int kv = tid >> 4, i = tid & 15;
        const int n = kv ? (1 << VB) : (1 << KB);
        sm.cb[kv][i] = i < n ? __ldg((kv ? p.cent_v : p.cent_k) + i) : 0.0f;
    }
    {
        // 8 heads x 32 blocks of four = 256 work items, one per thread
        const int h = tid >> 5, blk = tid & 31;
        float r[4] = {0.f, 0.f, 0.f, 0.f};
        if (h < heads_here) {
            const T* qp = static_cast<const T*>(p.q) + seq * p.q_stride_seq +
                          static_cast<int64_t>(first_qh + h) * p.q_stride_head + 4 * blk;
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(qp));
            const float2 x01 = unpack_pair<T>(raw.x), x23 = unpack_pair<T>(raw.y);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 rr = __ldg(reinterpret_cast<const float4*>(
                    p.rotation + (4 * blk + j) * kHeadDim + 4 * blk));
                float acc = __fmul_rn(x01.x, rr.x);
                acc = __fmaf_rn(x01.y, rr.y, acc);
                acc = __fmaf_rn(x23.x, rr.z, acc);
                acc = __fmaf_rn(x23.y, rr.w, acc);
                r[j] = acc;
            }
        }
        // element d lives at index d ^ 1: (r1, r0, r3, r2)
        uint2 st;
        st.x = pack_pair<T>(r[1], r[0]);
        st.y = pack_pair<T>(r[3], r[2]);
        *reinterpret_cast<uint2*>(&sm.q[h][4 * blk]) = st;
    }
    __syncthreads();

    // Query fragments (mma A operand, rows = heads, upper 8 rows are zero).  For k-step
    // ks = 2w + e the thread supplies k-slots {2tig,2tig+1} and {2tig+8,2tig+9}, which this
    // kernel maps to the elements of nibbles 4e..4e+3 of word w of the thread's 16-byte chunk.
    uint32_t qa[8][2];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int off = 32 * tig + 8 * (ks >> 1) + 4 * (ks & 1);
        qa[ks][0] = *reinterpret_cast<const uint32_t*>(&sm.q[g][off]);
        qa[ks][1] = *reinterpret_cast<const uint32_t*>(&sm.q[g][off + 2]);
    }

    // ---- per-warp streaming state ----
    WarpSmem& ws = sm.warp[warp];
    const SlotLayout lay = slot_layout(p.H);
    const bool fast_bt = (p.block_size % kTile) == 0;
    const int32_t* bt_row = p.block_table + seq * p.bt_stride;
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);

    auto phys_slot0 = [&](int tile) -> int64_t {      // slot of the tile's first token (fast path)
        const int t0 = tile * kTile;
        int64_t blk = __ldg(bt_row + t0 / p.block_size);
        blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
        return blk * p.block_size + (t0 % p.block_size);
    };
    auto token_slot = [&](int tile, int i, int64_t slot0) -> int64_t {
        if (fast_bt) return slot0 + i;
        int t = tile * kTile + i;
        t = min(t, seq_len - 1);
        int64_t blk = __ldg(bt_row + t / p.block_size);
        blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
        return blk * p.block_size + (t % p.block_size);
    };

    auto issue = [&](int tile, int s, int64_t slot0) {
        Stage& st = ws.stage[s];
        const uint8_t* head_base = p.cache + kvh * kHalfDim;
        // K indices: 64 chunks of 16 bytes, two per lane
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = lane + 32 * j, i = c >> 2, part = c & 3;
            const uint8_t* src = head_base + token_slot(tile, i, slot0) * p.total_bytes + 16 * part;
            cp_async16(&st.k[i][16 * part], src + lay.k_idx);
            if (v_align == 16) cp_async16(&st.v[i][16 * part], src + lay.v_idx);
        }
        if (v_align == 8) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = lane + 32 * j, i = c >> 3, part = c & 7;
                cp_async8(&st.v[i][8 * part], head_base + token_slot(tile, i, slot0) * p.total_bytes +
                                                  lay.v_idx + 8 * part);
            }
        } else if (v_align == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = lane + 32 * j, i = c >> 4, part = c & 15;
                cp_async4(&st.v[i][4 * part], head_base + token_slot(tile, i, slot0) * p.total_bytes +
                                                  lay.v_idx + 4 * part);
            }
        }
        {   // norms: lanes 0..15 K, 16..31 V
            const int i = lane & 15, kv = lane >> 4;
            cp_async4(&st.norms[lane], p.cache + token_slot(tile, i, slot0) * p.total_bytes +
                                           (kv ? lay.v_norm : lay.k_norm) + 4 * kvh);
        }
    };

    // online-softmax state of head g (partial over this thread's token columns)
    float m_run = -INFINITY, l_run = 0.0f;
    float o_acc[8][4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) o_acc[mt][c] = 0.0f;

    const int first_tile = tile_begin + warp;
    const int n_my = first_tile < tile_end ? (tile_end - first_tile + kDecodeWarps - 1) / kDecodeWarps : 0;

    // prefetch pipeline: block-table entry of the next tile to issue is read one step ahead
    int pf_it = 0;
    int64_t pf_slot0 = (n_my > 0 && fast_bt) ? phys_slot0(first_tile) : 0;
    auto issue_next = [&]() {
        if (pf_it < n_my) {
            const int tile = first_tile + pf_it * kDecodeWarps;
            issue(tile, pf_it % kStages, pf_slot0);
            ++pf_it;
            if (pf_it < n_my && fast_bt) pf_slot0 = phys_slot0(first_tile + pf_it * kDecodeWarps);
        }
        cp_async_commit();
    };
#pragma unroll 1
    for (int s = 0; s < kStages - 1; ++s) issue_next();

#pragma unroll 1
    for (int it = 0; it < n_my; ++it) {
        issue_next();
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const Stage& st = ws.stage[it % kStages];
        const int tile = first_tile + it * kDecodeWarps;
        const int n_valid = min(kTile, seq_len - tile * kTile);

        // ---- per-token tables: lane builds token (lane & 15) of K (lanes 0-15) or V ----
        {
            const int i = lane & 15;
            const float norm = i < n_valid ? st.norms[lane] : 0.0f;
            if (lane < 16) {
                const Table<KB> t = build_table<T, KB>(sm.cb[0], norm);
#pragma unroll
                for (int r4 = 0; r4 < Table<KB>::kRegs / 4; ++r4)
                    *reinterpret_cast<uint4*>(&ws.tbl_k[i][4 * r4]) =
                        make_uint4(t.r[4 * r4], t.r[4 * r4 + 1], t.r[4 * r4 + 2], t.r[4 * r4 + 3]);
            } else {
                const Table<VB> t = build_table<T, VB>(sm.cb[1], norm);
#pragma unroll
                for (int r4 = 0; r4 < Table<VB>::kRegs / 4; ++r4)
                    *reinterpret_cast<uint4*>(&ws.tbl_v[i][4 * r4]) =
                        make_uint4(t.r[4 * r4], t.r[4 * r4 + 1], t.r[4 * r4 + 2], t.r[4 * r4 + 3]);
            }
        }
        __syncwarp();

        // ---- S = Q K^T : rows = heads (g), columns = tokens; two 8-token column tiles ----
        float s_acc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) s_acc[nt][c] = 0.0f;
            const int tok = g + 8 * nt;
            const uint4 kw = *reinterpret_cast<const uint4*>(&st.k[tok][16 * tig]);
            Table<KB> tk;
#pragma unroll
            for (int r4 = 0; r4 < Table<KB>::kRegs / 4; ++r4) {
                const uint4 tv = *reinterpret_cast<const uint4*>(&ws.tbl_k[tok][4 * r4]);
                tk.r[4 * r4] = tv.x; tk.r[4 * r4 + 1] = tv.y; tk.r[4 * r4 + 2] = tv.z; tk.r[4 * r4 + 3] = tv.w;
            }
            const uint32_t words[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    uint32_t lo, hi;
                    lookup4<KB>(tk, e ? (words[w] >> 16) : words[w], lo, hi);
                    const uint32_t b0 = prmt(lo, hi, 0x5140);     // nibbles 0,1 of this half
                    const uint32_t b1 = prmt(lo, hi, 0x7362);     // nibbles 2,3
                    mma16816<T>(s_acc[nt], qa[2 * w + e][0], 0u, qa[2 * w + e][1], 0u, b0, b1);
                }
            }
        }

        // ---- online softmax for head g over this thread's 4 columns ----
        float sc[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int tok = 8 * nt + 2 * tig + c;
                sc[2 * nt + c] = tok < n_valid ? s_acc[nt][c] * p.qk_scale : -INFINITY;
            }
        float m_new = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 1));
        m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 2));
        m_new = fmaxf(m_new, m_run);
        // every tile holds at least one valid token, so m_new is finite
        const bool grew = m_new > m_run;
        if (__any_sync(0xffffffffu, grew)) {
            const float alpha = exp2f(m_run - m_new);      // 0 on the first tile
            l_run *= alpha;
            // accumulator columns are heads 2tig, 2tig+1: fetch their factors from rows g'
            const float a0 = __shfl_sync(0xffffffffu, alpha, (2 * tig) * 4);
            const float a1 = __shfl_sync(0xffffffffu, alpha, (2 * tig + 1) * 4);
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                o_acc[mt][0] *= a0; o_acc[mt][1] *= a1;
                o_acc[mt][2] *= a0; o_acc[mt][3] *= a1;
            }
            m_run = m_new;
        }
        float pr[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            pr[c] = exp2f(sc[c] - m_run);
            l_run += pr[c];
        }
        // P as mma B operand (k = tokens 2tig,2tig+1 | 2tig+8,2tig+9; n = head g), hi + lo parts
        const uint32_t ph0 = pack_pair<T>(pr[0], pr[1]), ph1 = pack_pair<T>(pr[2], pr[3]);
        const float2 h0 = unpack_pair<T>(ph0), h1 = unpack_pair<T>(ph1);
        const uint32_t pl0 = pack_pair<T>(pr[0] - h0.x, pr[1] - h0.y);
        const uint32_t pl1 = pack_pair<T>(pr[2] - h1.x, pr[3] - h1.y);

        // ---- O^T += V^T P^T : rows = this thread's 16 head-dim slots, columns = heads ----
        {
            const int ta = 2 * tig, tb = 2 * tig + 8;      // token pairs (ta,ta+1) and (tb,tb+1)
            uint2 vw[4];
            Table<VB> tv[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int tok = (x < 2 ? ta : tb) + (x & 1);
                vw[x] = *reinterpret_cast<const uint2*>(&st.v[tok][8 * g]);
#pragma unroll
                for (int r4 = 0; r4 < Table<VB>::kRegs / 4; ++r4) {
                    const uint4 q4 = *reinterpret_cast<const uint4*>(&ws.tbl_v[tok][4 * r4]);
                    tv[x].r[4 * r4] = q4.x; tv[x].r[4 * r4 + 1] = q4.y;
                    tv[x].r[4 * r4 + 2] = q4.z; tv[x].r[4 * r4 + 3] = q4.w;
                }
            }
#pragma unroll
            for (int sg = 0; sg < 4; ++sg) {               // selector sg covers nibbles 4sg..4sg+3
                uint32_t pairreg[2][4];                     // [pair a|b][nibble] = (tok, tok+1) halves
#pragma unroll
                for (int pb = 0; pb < 2; ++pb) {
                    uint32_t lo0, hi0, lo1, hi1;
                    const uint32_t w0 = (sg < 2) ? vw[2 * pb].x : vw[2 * pb].y;
                    const uint32_t w1 = (sg < 2) ? vw[2 * pb + 1].x : vw[2 * pb + 1].y;
                    lookup4<VB>(tv[2 * pb], (sg & 1) ? (w0 >> 16) : w0, lo0, hi0);
                    lookup4<VB>(tv[2 * pb + 1], (sg & 1) ? (w1 >> 16) : w1, lo1, hi1);
                    const uint32_t pl = prmt(lo0, lo1, 0x5140), pl2 = prmt(lo0, lo1, 0x7362);
                    const uint32_t ph = prmt(hi0, hi1, 0x5140), ph2 = prmt(hi0, hi1, 0x7362);
                    pairreg[pb][0] = prmt(pl, ph, 0x5140);
                    pairreg[pb][1] = prmt(pl, ph, 0x7362);
                    pairreg[pb][2] = prmt(pl2, ph2, 0x5140);
                    pairreg[pb][3] = prmt(pl2, ph2, 0x7362);
                }
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int mt = 2 * sg + half;
                    const uint32_t a0 = pairreg[0][2 * half], a1 = pairreg[0][2 * half + 1];
                    const uint32_t a2 = pairreg[1][2 * half], a3 = pairreg[1][2 * half + 1];
                    mma16816<T>(o_acc[mt], a0, a1, a2, a3, ph0, ph1);
                    mma16816<T>(o_acc[mt], a0, a1, a2, a3, pl0, pl1);
                }
            }
        }
        __syncwarp();        // the stage and the tables may be overwritten from here on
    }
    cp_async_wait<0>();

    // ---- cross-warp merge inside the CTA (each warp parks its state in its own area) ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncwarp();
    {
        float* area = reinterpret_cast<float*>(&ws);
        float* o_s = area;                                  // [8 heads][128]
        float* m_s = area + kHeadsPerCta * kHeadDim;        // [8]
        float* l_s = m_s + kHeadsPerCta;
        if (tig == 0) { m_s[g] = m_run; l_s[g] = l_run; }
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            // rows g / g+8 of m-tile mt are nibbles 2mt / 2mt+1 = head-dim 16g+2mt+1 / 16g+2mt
            const int d = 16 * g + 2 * mt;
            *reinterpret_cast<float2*>(&o_s[(2 * tig) * kHeadDim + d]) =
                make_float2(o_acc[mt][2], o_acc[mt][0]);
            *reinterpret_cast<float2*>(&o_s[(2 * tig + 1) * kHeadDim + d]) =
                make_float2(o_acc[mt][3], o_acc[mt][1]);
        }
    }
    __syncthreads();
    {
        const int h = tid >> 5, d4 = (tid & 31) * 4;
        if (h < heads_here) {
            float m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < kDecodeWarps; ++w) {
                const float* area = reinterpret_cast<const float*>(&sm.warp[w]);
                m_all = fmaxf(m_all, area[kHeadsPerCta * kHeadDim + h]);
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float l_all = 0.0f;
#pragma unroll
            for (int w = 0; w < kDecodeWarps; ++w) {
                const float* area = reinterpret_cast<const float*>(&sm.warp[w]);
                const float mw = area[kHeadsPerCta * kHeadDim + h];
                const float wgt = (mw == -INFINITY) ? 0.0f : exp2f(mw - m_all);
                const float4 o = *reinterpret_cast<const float4*>(&area[h * kHeadDim + d4]);
                acc.x += wgt * o.x; acc.y += wgt * o.y; acc.z += wgt * o.z; acc.w += wgt * o.w;
                l_all += wgt * area[kHeadsPerCta * kHeadDim + kHeadsPerCta + h];
            }
            const int64_t row = (static_cast<int64_t>(seq) * p.Hq + first_qh + h) * p.num_splits + split;
            *reinterpret_cast<float4*>(p.ws_o + row * kHeadDim + d4) = acc;
            if ((tid & 31) == 0) { p.ws_m[row] = m_all; p.ws_l[row] = l_all; }
        }
    }
}

// ---- merge kernel: combine splits, normalise, round, rotate back by R ---------------------

template <typename T>
__global__ void __launch_bounds__(kHeadDim)
decode_merge_kernel(const DecodeParams p) {
    __shared__ float o_s[kHeadDim];
    const int seq = blockIdx.x / p.Hq, qh = blockIdx.x % p.Hq;
    const int d = threadIdx.x;
    int seq_len = max(__ldg(p.seq_lens + seq), 0);
    const int total_tiles = (seq_len + kTile - 1) / kTile;
    const int n_act = min(p.num_splits, (total_tiles + p.tiles_per_split - 1) / p.tiles_per_split);
    const int64_t row0 = (static_cast<int64_t>(seq) * p.Hq + qh) * p.num_splits;
    float m_all = -INFINITY;
    for (int s = 0; s < n_act; ++s) m_all = fmaxf(m_all, p.ws_m[row0 + s]);
    float acc = 0.0f, l_all = 0.0f;
    for (int s = 0; s < n_act; ++s) {
        const float wgt = exp2f(p.ws_m[row0 + s] - m_all);
        acc += wgt * p.ws_o[(row0 + s) * kHeadDim + d];
        l_all += wgt * p.ws_l[row0 + s];
    }
    // an empty sequence yields zeros (the reference starts l at 1 and acc at 0)
    const float o = n_act > 0 ? acc / l_all : 0.0f;
    o_s[d] = round_to<T>(o);
    __syncthreads();
    // out[j] = sum_k o[k] R[k][j] over the 4x4 block of j, ascending k, fused multiply-adds
    const int b = d & ~3;
    float r = __fmul_rn(o_s[b], __ldg(p.rotation + b * kHeadDim + d));
#pragma unroll
    for (int k = 1; k < 4; ++k) r = __fmaf_rn(o_s[b + k], __ldg(p.rotation + (b + k) * kHeadDim + d), r);
    T* dst = static_cast<T*>(p.out) + seq * p.o_stride_seq + static_cast<int64_t>(qh) * p.o_stride_head + d;
    store_rounded(dst, r);
}

// ---- host side -------------------------------------------------------------------------------

struct SplitPlan {
    int tiles_per_split;
    int num_splits;
};

// Context splits: enough CTAs for two full waves (148 SMs x 2 CTAs) when the batch alone does
// not provide them, at least 16 tiles (256 tokens) and at most 128 tiles (2048 tokens) per split.
static SplitPlan plan_splits(int num_seqs, int H, int head_groups, int max_seq_len, int forced) {
    const int max_tiles = max_seq_len > 0 ? (max_seq_len + kTile - 1) / kTile : 1;
    int splits;
    if (forced > 0) {
        splits = forced;
    } else {
        const long long base = 1LL * num_seqs * H * head_groups;
        const long long want = 2LL * 148 * 2;
        splits = static_cast<int>((want + base - 1) / base);
        const int by_min = (max_tiles + 15) / 16;       // >= 16 tiles per split
        const int by_max = (max_tiles + 127) / 128;     // <= 128 tiles per split
        if (splits > by_min) splits = by_min;
        if (splits < by_max) splits = by_max;
        if (splits < 1) splits = 1;
    }
    if (splits > max_tiles) splits = max_tiles;
    SplitPlan pl;
    pl.tiles_per_split = (max_tiles + splits - 1) / splits;
    pl.num_splits = (max_tiles + pl.tiles_per_split - 1) / pl.tiles_per_split;
    return pl;
}

static size_t workspace_bytes_for(int num_seqs, int Hq, int splits) {
    const size_t rows = static_cast<size_t>(num_seqs) * Hq * splits;
    return rows * (kHeadDim + 2) * sizeof(float);
}

template <typename T, int KB, int VB>
static int launch_decode(const DecodeParams& p, int num_seqs, cudaStream_t st) {
    const size_t smem = sizeof(DecodeSmem);
    if (int e = ensure_smem(decode_split_kernel<T, KB, VB>, smem)) return e;
    dim3 grid(p.num_splits, p.H * p.head_groups, num_seqs);
    decode_split_kernel<T, KB, VB><<<grid, kDecodeThreads, smem, st>>>(p);
    if (int e = check_cuda(cudaGetLastError(), "rq_decode split launch")) return e;
    decode_merge_kernel<T><<<num_seqs * p.Hq, kHeadDim, 0, st>>>(p);
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
    const SplitPlan pl = plan_splits(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits);
    return workspace_bytes_for(num_seqs, num_q_heads, pl.num_splits);
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
    const SplitPlan pl = plan_splits(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits);
    const size_t need = workspace_bytes_for(num_seqs, num_q_heads, pl.num_splits);
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
    p.tiles_per_split = pl.tiles_per_split; p.num_splits = pl.num_splits;
    const size_t rows = static_cast<size_t>(num_seqs) * num_q_heads * pl.num_splits;
    p.ws_o = static_cast<float*>(workspace);
    p.ws_m = p.ws_o + rows * kHeadDim;
    p.ws_l = p.ws_m + rows;
    p.out = out; p.o_stride_seq = o_stride_seq; p.o_stride_head = o_stride_head;

    const int kb = n_centroids_k == 8 ? 3 : 4, vb = n_centroids_v == 8 ? 3 : 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RQ_DTYPE_BF16) return dispatch_bits<__nv_bfloat16>(p, num_seqs, kb, vb, st);
    return dispatch_bits<__half>(p, num_seqs, kb, vb, st);
}
