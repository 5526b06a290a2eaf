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
struct __align__(256) WarpSmem {
    uint16_t vt[kTile][kHeadDim];      // decompressed V tile, 16-byte chunks XOR-swizzled by token
    Stage stage[kStages];
    uint32_t tbl_k[kTile][8];          // per-token K integer planes (4 or 8 registers used)
    uint32_t tbl_v[kTile][8];          // per-token V value planes
    float k_unscale[kTile];            // 2^(e-13) of every K table
};
static_assert(sizeof(WarpSmem) >= sizeof(float) * (kHeadsPerCta * kHeadDim + 2 * kHeadsPerCta),
              "the per-warp area is reused for the cross-warp merge");

struct __align__(256) DecodeSmem {
    WarpSmem warp[kDecodeWarps];
    uint8_t q_hi[kHeadsPerCta][kHeadDim];   // signed byte planes of the rotated queries' integer
    uint8_t q_lo[kHeadsPerCta][kHeadDim];   // image (256 * hi + lo); element d stored at index d ^ 1
    float q_unscale[kHeadsPerCta];
    float cb[2][16];                         // K and V codebooks
};

// ---- the split kernel -------------------------------------------------------------

template <typename T, int KB, int VB>
__global__ void __launch_bounds__(kDecodeThreads, 2)
decode_split_kernel(const DecodeParams p) {
    extern __shared__ __align__(256) uint8_t smem_raw[];
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

    // ---- per-warp streaming state ----
    WarpSmem& ws = sm.warp[warp];
    const SlotLayout lay = slot_layout(p.H);
    const bool fast_bt = (p.block_size % kTile) == 0;
    const int32_t* bt_row = p.block_table + seq * p.bt_stride;
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);

    auto clamp_block = [&](int64_t blk) -> int64_t {
        return blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
    };
    // fast path (block_size a multiple of 16): the 16 slots of a tile are contiguous
    auto phys_slot0 = [&](int tile) -> int64_t {
        const int t0 = tile * kTile;
        return clamp_block(__ldg(bt_row + t0 / p.block_size)) * p.block_size + (t0 % p.block_size);
    };
    auto token_slot = [&](int tile, int i) -> int64_t {      // general path: one lookup per token
        const int t = min(tile * kTile + i, seq_len - 1);
        return clamp_block(__ldg(bt_row + t / p.block_size)) * p.block_size + (t % p.block_size);
    };

    // Per-lane source offsets (bytes from the tile's first slot) and shared-memory destinations
    // (bytes from the stage) of this lane's copies; fixed for the whole kernel.
    const uint32_t tb = static_cast<uint32_t>(p.total_bytes);
    const uint32_t src_k = (lane >> 2) * tb + kvh * kHalfDim + 16 * (lane & 3);      // + 8*tb for copy 2
    const uint32_t dst_k = (lane >> 2) * kHalfDim + 16 * (lane & 3);
    const uint32_t dst_v16 = sizeof(Stage::k) + (lane >> 2) * kVPitch + 16 * (lane & 3);
    const uint32_t src_n = (lane & 15) * tb + ((lane >> 4) ? lay.v_norm : lay.k_norm) + 4 * kvh;
    const uint32_t dst_n = sizeof(Stage::k) + sizeof(Stage::v) + 4 * lane;

    auto issue = [&](int tile, int s, int64_t slot0) {
        uint8_t* stg = reinterpret_cast<uint8_t*>(&ws.stage[s]);
        if (fast_bt) {
            const uint8_t* base = p.cache + slot0 * p.total_bytes;
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
        // general path: tokens of a tile may sit in different blocks
        const uint8_t* head_base = p.cache + kvh * kHalfDim;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c = lane + 32 * j, i = c >> 2, part = c & 3;
            const uint8_t* src = head_base + token_slot(tile, i) * p.total_bytes + 16 * part;
            cp_async16(stg + i * kHalfDim + 16 * part, src + lay.k_idx);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = lane + 32 * j, i = c >> 4, part = c & 15;
            cp_async4(stg + sizeof(Stage::k) + i * kVPitch + 4 * part,
                      head_base + token_slot(tile, i) * p.total_bytes + lay.v_idx + 4 * part);
        }
        cp_async4(stg + dst_n, p.cache + token_slot(tile, lane & 15) * p.total_bytes +
                                   ((lane >> 4) ? lay.v_norm : lay.k_norm) + 4 * kvh);
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
    int pf_it = 0, pf_stage = 0;
    int64_t pf_slot0 = (n_my > 0 && fast_bt) ? phys_slot0(first_tile) : 0;
    auto issue_next = [&]() {
        if (pf_it < n_my) {
            const int tile = first_tile + pf_it * kDecodeWarps;
            issue(tile, pf_stage, pf_slot0);
            ++pf_it;
            pf_stage = pf_stage + 1 == kStages ? 0 : pf_stage + 1;
            if (pf_it < n_my && fast_bt) pf_slot0 = phys_slot0(first_tile + pf_it * kDecodeWarps);
        }
        cp_async_commit();
    };
#pragma unroll 1
    for (int s = 0; s < kStages - 1; ++s) issue_next();

    // (the first tiles are now in flight; their latency overlaps the query set-up below)
    // ---- prologue: codebooks; q_rot = round_T(q @ R^T) as int16 planes in shared memory ----
    if (tid < 32) {
        const int kv = tid >> 4, i = tid & 15;
        const int n = kv ? (1 << VB) : (1 << KB);
        sm.cb[kv][i] = i < n ? __ldg((kv ? p.cent_v : p.cent_k) + i) : 0.0f;
    }
    {
        // warp h rotates head h: lane = one 4x4 block
        const int h = warp, blk = lane;
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
                r[j] = round_to<T>(acc);
            }
        }
        float mx = fmaxf(fmaxf(fabsf(r[0]), fabsf(r[1])), fmaxf(fabsf(r[2]), fabsf(r[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const bool ok = mx >= 1.0e-30f && mx <= 3.0e38f;
        const int e = ok ? exponent_of(mx) : 0;
        const float scale = ok ? pow2i(13 - e) : 0.0f;
        int qu[4];      // integer image + 128: byte 1 = signed high digit, byte 0 ^ 0x80 = signed low digit
#pragma unroll
        for (int j = 0; j < 4; ++j) qu[j] = __float2int_rn(fmaf(r[j], scale, 128.0f));
        // element d lives at index d ^ 1: byte order (1, 0, 3, 2)
        const uint32_t a = prmt(qu[1], qu[0], 0x5140), b = prmt(qu[3], qu[2], 0x5140);
        *reinterpret_cast<uint32_t*>(&sm.q_lo[h][4 * blk]) = prmt(a, b, 0x5410) ^ 0x80808080u;
        *reinterpret_cast<uint32_t*>(&sm.q_hi[h][4 * blk]) = prmt(a, b, 0x7632);
        if (lane == 0) sm.q_unscale[h] = ok ? pow2i(e - 13) : 0.0f;
    }
    __syncthreads();

    // Query fragments (mma A operand): rows 0..7 carry the high digits of heads 0..7, rows 8..15
    // the low digits of the same heads, so one MMA yields Qhi.K and Qlo.K for a K plane.  In
    // k-step w the thread supplies k-slots 4tig..4tig+3 and 16+4tig..16+4tig+3, which this kernel
    // maps to the elements of nibbles 0..3 and 4..7 of word w of its 16-byte chunk of a K row.
    uint32_t qa[4][4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const int off = 32 * tig + 8 * w;
        qa[w][0] = *reinterpret_cast<const uint32_t*>(&sm.q_hi[g][off]);
        qa[w][1] = *reinterpret_cast<const uint32_t*>(&sm.q_lo[g][off]);
        qa[w][2] = *reinterpret_cast<const uint32_t*>(&sm.q_hi[g][off + 4]);
        qa[w][3] = *reinterpret_cast<const uint32_t*>(&sm.q_lo[g][off + 4]);
    }
    const float q_factor = sm.q_unscale[g] * p.qk_scale;


    // per-lane constants of the V transpose: this lane decompresses half a row of token tv ...
    const int tv = lane & 15, vhalf = lane >> 4;
    // ... and feeds ldmatrix with row (lane & 7) of 8x8 matrix (lane >> 3)
    const int lm_tok = (lane & 7) + ((lane & 16) ? 8 : 0);
    const int lm_chunk = (lane >> 3) & 1;
    // generic addresses whose low byte already holds the swizzle; chunk selection is one XOR
    const uint32_t vt_store_base = static_cast<uint32_t>(__cvta_generic_to_shared(&ws.vt[tv][0])) +
                                   128u * vhalf + 16u * (tv & 7);
    const uint32_t lm_base = static_cast<uint32_t>(__cvta_generic_to_shared(&ws.vt[lm_tok][0])) +
                             16u * (lm_chunk ^ (lm_tok & 7));

    int cur_stage = 0;
#pragma unroll 1
    for (int it = 0; it < n_my; ++it) {
        issue_next();
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const Stage& st = ws.stage[cur_stage];
        cur_stage = cur_stage + 1 == kStages ? 0 : cur_stage + 1;
        const int tile = first_tile + it * kDecodeWarps;
        const int n_valid = min(kTile, seq_len - tile * kTile);

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
            build_half_int_table<T, NKH>(&sm.cb[0][hb * NKH], norm_k, lo, hi, unscale);
            uint32_t vlo[NVH / 4], vhi[NVH / 4];
            build_half_value_table<T, NVH>(&sm.cb[1][hb * NVH], norm_v, vlo, vhi);
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
        __syncwarp();        // the stage, the tables and vt may be overwritten from here on
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
            // row g of m-tile mt is position g of 8-wide chunk 2mt, i.e. head-dim 16mt + (g^1);
            // row g+8 is the same position of chunk 2mt+1
            const int d = 16 * mt + (g ^ 1);
            o_s[(2 * tig) * kHeadDim + d] = o_acc[mt][0];
            o_s[(2 * tig + 1) * kHeadDim + d] = o_acc[mt][1];
            o_s[(2 * tig) * kHeadDim + d + 8] = o_acc[mt][2];
            o_s[(2 * tig + 1) * kHeadDim + d + 8] = o_acc[mt][3];
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
