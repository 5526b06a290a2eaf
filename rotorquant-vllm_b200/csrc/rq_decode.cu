// Fused paged decode attention over the RotorQuant cache, sm_100a.
//
// Replaces fused_paged_rq_decode (triton/fused_paged_rq_decode.py:32-312 of the reference): the
// Triton kernel (one program per (sequence, query head), CUDA-core dot products, no split-KV)
// and the two dense 128x128 rotations its launcher runs around it.
//
// Work decomposition.  The (sequence, 128-token tile) space of the batch is one line of tiles,
// cut into contiguous pieces; a CTA streams the tiles of one piece for one (KV head, group of up
// to 8 query heads) and leaves one partial result per sequence its piece touches.  A second
// launch merges the partial results of every (sequence, query head), rounds, and applies R.  The
// 136 payload bytes of a (token, KV head) are read from HBM exactly once for all query heads of
// the GQA group.
//
// The attention CTA is warp specialised: four compute warps (thread t owns token t of the tile
// and TMEM lane t) and one issuer warp that owns every asynchronous engine -- it fills a ring of
// index-row tiles with TMA boxes (or per-row bulk copies), and issues the tcgen05 MMAs when the
// compute warps have published their operands.  Compute warps never issue a copy or an MMA and
// meet no block-wide barrier inside the tile loop; everything is ordered by mbarriers.
//
// Arithmetic (matches "reference decompress + SDPA"):
//   q_rot   = round_T(q @ R^T)            exact FMA chain per 4x4 block, computed per part
//   K, V    = round_T(centroid[idx]*norm) exactly the decompressed values: each token gets a
//             table of its 8/16 rounded products, elements are fetched from it with PRMT
//   scores  = int8 tensor-core mma over 15-bit integer images of q_rot and K (exact for K, 2^-14
//             of the row maximum for q), fp32 scaling, exp2-domain softmax against a reference
//             maximum per head (exact maximum of the part's first tile; it moves later only when
//             a score exceeds it by 2^8)
//   P @ V   = tensor-core mma with P split into hi + lo parts (two T-precision terms, ~16 bits),
//             fp32 accumulate in tensor memory
//   out     = round_T(round_T(o / l) @ R)  in the merge kernel
#include <cuda.h>          // CUtensorMap (types only; the encoder is looked up at run time)

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "rq_common.cuh"
#include "rq_tcgen05.cuh"

namespace rq {

constexpr int kHeadsPerCta = 8;              // query heads per item (mma N of P@V is 2 x 8)
constexpr int kTileTokens = 128;             // tokens per tile = compute threads per CTA
constexpr int kComputeThreads = 128;
constexpr int kDecodeThreads = 160;          // + the issuer warp
constexpr int kIssuerWarp = 4;
constexpr uint32_t kTmemCols = 128;          // columns allocated per CTA
constexpr uint32_t kColKhi = 0, kColKlo = 32, kColS = 64, kColO = 96;
constexpr int kInlinePlanSeqs = 256;         // up to this many sequences the CTAs scan seq_lens themselves
constexpr int kMaxLayers = 4;                // launch layers with their own piece weight
constexpr int kMaxCtasPerSm = 3;

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
    void* out;
    int64_t o_stride_seq, o_stride_head;
    int32_t* prefix;                       // [num_seqs + 1] exclusive prefix of tiles per sequence (workspace)
    int num_seqs;
    int groups;                            // pieces; CTA = (group, item)
    int inline_plan;                       // the attention CTAs compute the prefix sums themselves
    int bs_shift;                          // log2(block_size) when it is a power of two, else -1
    int box_tokens;                        // tokens per TMA box (16, or 8 for block size 8)
    int layer_ctas;                        // CTAs per launch layer (SM count) when pieces are weighted, else 0
    int num_layers;
    int layer_w[kMaxLayers];               // piece weight of the CTAs of each launch layer
    unsigned long long* trace;             // development builds only
};

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

// Untiled bulk copy of `bytes` (a multiple of 16; both addresses 16-byte aligned) global -> shared.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar_addr) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar_addr)
        : "memory");
}

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
//
// MODE = how the index rows of a tile reach the ring:
//   1  TMA boxes of 16 (or 8) tokens x 64 B for K and for V rows, 64-byte swizzle (KV heads a multiple
//      of 4, so V rows start on 16-byte boundaries; power-of-two block size >= 8)
//   2  the same boxes for K; V rows, which start 4, 8 or 12 bytes past a 16-byte boundary, as boxes of
//      80 B from the boundary below, unswizzled (power-of-two block size >= 8)
//   0  one 64-byte (K) and one 80-byte (V) bulk copy per token, unswizzled: any block size
template <int MODE>
struct DecodeSmem {
    static constexpr int kStages = MODE == 1 ? 2 : 3;
    static constexpr int kVPitch = MODE == 1 ? 64 : 80;
    static constexpr int kCtasPerSm = MODE == 1 ? 3 : 2;
    alignas(1024) uint8_t ring_k[kStages][kTileTokens * kHalfDim];
    alignas(128) uint8_t ring_v[kStages][kTileTokens * kVPitch];
    alignas(128) uint16_t v[kTileTokens * kHeadDim];   // V tile: core (token/8)*16 + pos/8, core row token%8
    uint16_t p[kTileTokens * 16];                      // P tile: core (token/8)*2 + n/8, core row token%8
    uint8_t q[16 * kHeadDim];                          // Q digit planes, K-major: core (n/8)*8 + pos/16
    float cb[2][16];
    float qf[kHeadsPerCta];                            // q unscale * sm_scale * log2(e) per head
    float red_m[4][kHeadsPerCta];                      // cross-warp reductions
    float red_l[4][kHeadsPerCta];
    int scan[4];
    uint64_t full[kStages];                            // "rows of the tile landed"
    uint64_t kready, pvready;                          // compute -> issuer: operands published (128 arrivals)
    uint64_t bar_s, bar_o, bar_drain;                  // issuer -> compute: MMAs complete
    uint32_t tmem_base;
    int grow_tile, redo_tile, dead;
    int32_t prefix[kInlinePlanSeqs + 1];
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

// NH = query heads computed per item: 4 when the GQA group has at most 4 heads, else 8.
template <typename T, int KB, int VB, int MODE, int NH>
__global__ void __launch_bounds__(kDecodeThreads, DecodeSmem<MODE>::kCtasPerSm)
decode_attn_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v) {
    using Smem = DecodeSmem<MODE>;
    constexpr int S = Smem::kStages;
    constexpr int VP = Smem::kVPitch;
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    constexpr int NK = 1 << KB, NV = 1 << VB;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int J = p.H * p.head_groups;
    const int64_t group = blockIdx.x / J;
    const int item = static_cast<int>(blockIdx.x % J);

    // ---- set-up: barriers, tensor memory, codebooks, tile prefix sums ----
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(&sm.full[s], 1);
        mbar_init(&sm.kready, kComputeThreads);
        mbar_init(&sm.pvready, kComputeThreads);
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_init(&sm.bar_drain, 1);
        sm.grow_tile = -1;
        sm.redo_tile = -1;
        sm.dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    if (warp == 0) tmem_alloc(&sm.tmem_base, kTmemCols);
    if (warp == kIssuerWarp) {
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
            if (s0 < p.num_seqs) a = (max(__ldg(p.seq_lens + s0), 0) + kTileTokens - 1) / kTileTokens;
            if (s0 + 1 < p.num_seqs) b = (max(__ldg(p.seq_lens + s0 + 1), 0) + kTileTokens - 1) / kTileTokens;
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

    const SlotLayout lay = slot_layout(p.H);
    const int kvh = item / p.head_groups, hg = item % p.head_groups;
    const int heads_here = min(kHeadsPerCta, p.G - hg * kHeadsPerCta);
    const int first_qh = kvh * p.G + hg * kHeadsPerCta;
    // V rows: byte offset of the row inside the slot, rounded down to a 16-byte boundary for the copy
    const int v_row = lay.v_idx + kvh * kHalfDim;
    const int v_copy_x = MODE == 1 ? v_row : (v_row & ~15);
    const int v_off = v_row - v_copy_x;                       // 0, 4, 8 or 12
    const int last_blk = static_cast<int>(p.num_blocks) - 1;

    bool dead = false;

    if (has_work && warp == kIssuerWarp) {
        // =========================== issuer warp ===========================
        const uint32_t idesc_s = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t idesc_o = (1u << 4) | (TcFormat<T>::kFmt << 7) | (TcFormat<T>::kFmt << 10) | (1u << 15) |
                                 (1u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t q_addr = smem_u32(sm.q), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);

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

        // ---- producer: the rows of one tile into ring stage (n % S) ----
        // The sequence length and this lane's block-table entry of the tile to be produced next are
        // loaded right after the previous tile was issued, so that no load latency sits between the
        // moment a stage becomes free and the copies into it.
        Walk pw;
        start_walk(pw);
        int produced = 0;
        int p_seq_len = max(__ldg(p.seq_lens + pw.seq), 0);
        int p_blk = 0;
        auto prefetch_blk = [&]() {
            if constexpr (MODE != 0) {
                const int t = pw.tile * kTileTokens + lane * p.box_tokens;
                p_blk = (pw.x < x_end && lane * p.box_tokens < kTileTokens && t < p_seq_len)
                            ? __ldg(p.block_table + pw.seq * p.bt_stride + (t >> p.bs_shift)) : 0;
            }
        };
        prefetch_blk();
        auto produce = [&]() {
            const int stage = produced % S;
            const uint32_t bar = smem_u32(&sm.full[stage]);
            const int tok0 = pw.tile * kTileTokens;
            const int n_valid = min(kTileTokens, p_seq_len - tok0);
            const uint32_t k_dst = smem_u32(sm.ring_k[stage]), v_dst = smem_u32(sm.ring_v[stage]);
            if constexpr (MODE != 0) {
                const int bt_tok = p.box_tokens;                  // 16 or 8: at most 16 boxes, one per lane
                const int n_box = (n_valid + bt_tok - 1) / bt_tok;
                const uint32_t box_bytes = static_cast<uint32_t>(bt_tok) * (kHalfDim + VP);
                if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_box) * box_bytes);
                __syncwarp();
                if (lane < n_box) {
                    const int t = tok0 + lane * bt_tok;
                    const int blk = p_blk < 0 ? 0 : (p_blk > last_blk ? last_blk : p_blk);
                    const int slot = (blk << p.bs_shift) + (t & (p.block_size - 1));
                    tma_load_2d(k_dst + static_cast<uint32_t>(lane * bt_tok) * kHalfDim, &map_k, kvh * kHalfDim, slot, bar);
                    tma_load_2d(v_dst + static_cast<uint32_t>(lane * bt_tok) * VP, &map_v, v_copy_x, slot, bar);
                }
            } else {
                const int32_t* bt_row = p.block_table + pw.seq * p.bt_stride;
                if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_valid) * (kHalfDim + VP));
                __syncwarp();
                for (int i = lane; i < n_valid; i += 32) {
                    const int t = tok0 + i;
                    const int bi = p.bs_shift >= 0 ? (t >> p.bs_shift) : (t / p.block_size);
                    const int off = p.bs_shift >= 0 ? (t & (p.block_size - 1)) : (t % p.block_size);
                    int blk = __ldg(bt_row + bi);
                    blk = blk < 0 ? 0 : (blk > last_blk ? last_blk : blk);
                    const uint8_t* slot = p.cache + (static_cast<int64_t>(blk) * p.block_size + off) * p.total_bytes;
                    bulk_load(k_dst + static_cast<uint32_t>(i) * kHalfDim, slot + kvh * kHalfDim, kHalfDim, bar);
                    bulk_load(v_dst + static_cast<uint32_t>(i) * VP, slot + v_copy_x, VP, bar);
                }
            }
            __syncwarp();
            ++produced;
            if (advance(pw)) p_seq_len = max(__ldg(p.seq_lens + pw.seq), 0);
            prefetch_blk();
        };
#pragma unroll 1
        for (int s = 0; s < S && pw.x < x_end; ++s) produce();

        // ---- consumer of the compute warps' operands: issue the MMAs of every tile ----
        Walk cw;
        start_walk(cw);
        bool first_in_part = true;
        uint32_t ph_pv = 0;
        int it = 0;
#pragma unroll 1
        for (; cw.x < x_end; ++it) {
            // S^T = K Q^T: the digit planes of the tile are in tensor memory, the query planes in shared memory
            if (!mbar_wait(&sm.kready, it & 1)) { dead = true; break; }
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    tc_mma_i8_ta(tmem + kColS, tmem + kColKhi + 8 * s, smem_desc(q_addr + 256 * s, 128, 1024),
                                 idesc_s, s > 0 ? 1u : 0u);
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    tc_mma_i8_ta(tmem + kColS + 16, tmem + kColKlo + 8 * s, smem_desc(q_addr + 256 * s, 128, 1024),
                                 idesc_s, s > 0 ? 1u : 0u);
                tc_commit(&sm.bar_s);
            }
            __syncwarp();
            // O^T += V^T [P hi | P lo]
            if (!mbar_wait(&sm.pvready, ph_pv)) { dead = true; break; }
            ph_pv ^= 1u;
            if (ld_volatile_shared(&sm.grow_tile) == it) {
                // a score outgrew the reference maximum: hand the tile back; the compute warps move the
                // maxima, rescale, rewrite P and publish again
                if (lane == 0) {
                    st_volatile_shared(&sm.redo_tile, it);
                    mbar_arrive(&sm.bar_o);
                }
                __syncwarp();
                if (!mbar_wait(&sm.pvready, ph_pv)) { dead = true; break; }
                ph_pv ^= 1u;
            }
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    tc_mma_f16(tmem + kColO, smem_desc(v_addr + 4096 * s, 2048, 128),
                               smem_desc(p_addr + 512 * s, 256, 128), idesc_o, (!first_in_part || s > 0) ? 1u : 0u);
                tc_commit(&sm.bar_o);
            }
            __syncwarp();
            // every compute thread has read its rows of this tile's stage: refill it
            if (pw.x < x_end) produce();
            first_in_part = advance(cw);
        }
        if (dead) {
            st_volatile_shared(&sm.dead, 1);
            // copies still in flight: a bounded wait each, so that none lands after the CTA is gone
            for (int c = it; c < produced; ++c) mbar_wait(&sm.full[c % S], (c / S) & 1);
            if (lane == 0) tc_commit(&sm.bar_drain);
            __syncwarp();
            mbar_wait(&sm.bar_drain, 0);
        }
    } else if (has_work) {
        // =========================== compute warps ===========================
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's lane quarter
        uint8_t* const v_dst = reinterpret_cast<uint8_t*>(sm.v) + (tid >> 3) * (16 * 128) + (tid & 7) * 16;
        uint8_t* const p_dst = reinterpret_cast<uint8_t*>(sm.p) + (tid >> 3) * (2 * 128) + (tid & 7) * 16;
        const uint32_t k_sw = MODE != 0 ? 16u * ((tid >> 1) & 3) : 0u;      // swizzle of this token's row
        float cmax_k = 0.0f;
#pragma unroll
        for (int i = 0; i < NK; ++i) cmax_k = fmaxf(cmax_k, fabsf(sm.cb[0][i]));

        uint32_t ph_o = 0;
        int it = 0;                                // tiles streamed by this CTA so far
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
            const int32_t* bt_row = p.block_table + seq * p.bt_stride;

            // Norms of this thread's token: fetched one tile ahead, the block-table entry two tiles ahead.
            auto load_blk = [&](int tile) -> int {
                const int tok = tile * kTileTokens + tid;
                if (tile >= t_end || tok >= seq_len) return -1;
                const int bi = p.bs_shift >= 0 ? (tok >> p.bs_shift) : (tok / p.block_size);
                const int blk = __ldg(bt_row + bi);
                return blk < 0 ? 0 : (blk > last_blk ? last_blk : blk);
            };
            auto load_norms = [&](int tile, int blk, float& nk, float& nv) {
                nk = 0.0f;
                nv = 0.0f;                           // zero norms make every table entry zero
                if (blk >= 0) {
                    const int tok = tile * kTileTokens + tid;
                    const int off = p.bs_shift >= 0 ? (tok & (p.block_size - 1)) : (tok % p.block_size);
                    const uint8_t* slot = p.cache + (static_cast<int64_t>(blk) * p.block_size + off) * p.total_bytes;
                    nk = __ldg(reinterpret_cast<const float*>(slot + lay.k_norm + 4 * kvh));
                    nv = __ldg(reinterpret_cast<const float*>(slot + lay.v_norm + 4 * kvh));
                }
            };
            float nk, nv, nk_next = 0.0f, nv_next = 0.0f;
            load_norms(t_begin, load_blk(t_begin), nk, nv);
            int blk_next = load_blk(t_begin + 1);

            // ---- queries of this part: rotate, round, quantise to signed digit planes (B operand) ----
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
            compute_sync();

            float m_ref[NH], l_acc[NH], l_pend[NH], sc[NH];
#pragma unroll
            for (int h = 0; h < NH; ++h) { m_ref[h] = -INFINITY; l_acc[h] = 0.0f; l_pend[h] = 0.0f; sc[h] = 0.0f; }
            bool pending = false;                    // a P V of this part has been requested and not yet awaited

            // probabilities of the tile whose scores are in sc[], against the current reference maxima
            auto emit_p = [&]() {
                uint32_t ph[4] = {0u, 0u, 0u, 0u}, pl[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int h = 0; h < NH; ++h) l_pend[h] = ex2_approx(sc[h] - m_ref[h]);
#pragma unroll
                for (int j = 0; j < NH / 2; ++j) {
                    ph[j] = pack_pair<T>(l_pend[2 * j], l_pend[2 * j + 1]);
                    const float2 back = unpack_pair<T>(ph[j]);
                    pl[j] = pack_pair<T>(l_pend[2 * j] - back.x, l_pend[2 * j + 1] - back.y);
                }
                *reinterpret_cast<uint4*>(p_dst) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                *reinterpret_cast<uint4*>(p_dst + 128) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                fence_async_proxy();
            };
            // CTA-wide maximum of sc[] per head -> m_new[]
            auto tile_max = [&](float (&m_new)[NH]) {
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    float m = sc[h];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                    if (lane == 0) sm.red_m[warp][h] = m;
                }
                compute_sync();
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    m_new[h] = fmaxf(fmaxf(sm.red_m[0][h], sm.red_m[1][h]), fmaxf(sm.red_m[2][h], sm.red_m[3][h]));
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
                    tile_max(m_new);
                    uint32_t o[16];
                    tmem_ld16_nowait(lane_base + kColO, o);          // lane = head-dim, column = head (hi | lo)
                    float alpha[kHeadsPerCta];
#pragma unroll
                    for (int h = NH; h < kHeadsPerCta; ++h) alpha[h] = 1.0f;
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        m_new[h] = fmaxf(m_new[h], m_ref[h]);
                        alpha[h] = ex2_approx(m_ref[h] - m_new[h]);
                        l_acc[h] *= alpha[h];
                        m_ref[h] = m_new[h];
                    }
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha[c & 7]);
                    tmem_st16_nowait(lane_base + kColO, o);
                    tmem_wait_st();
                    emit_p();
                    tc_fence_before();
                    mbar_arrive(&sm.pvready);
                    if (!mbar_wait(&sm.bar_o, ph_o)) { dead = true; return; }
                    ph_o ^= 1u;
                    tc_fence_after();
                }
#pragma unroll
                for (int h = 0; h < NH; ++h) l_acc[h] += l_pend[h];
                pending = false;
            };

#pragma unroll 1
            for (int tile = t_begin; tile < t_end; ++tile, ++it) {
                const int stage = it % S;
                const bool valid = tile * kTileTokens + tid < seq_len;
                // next tile's norms are requested now and used a tile later; its block-table entry was
                // loaded a tile ago
                load_norms(tile + 1, blk_next, nk_next, nv_next);
                blk_next = load_blk(tile + 2);
                if (!mbar_wait(&sm.full[stage], (it / S) & 1)) { dead = true; break; }

                // ---- K table, digit planes -> tensor memory ----
                float k_unscale;
                {
                    const Table<KB> tk = build_int_table<T, KB>(sm.cb[0], cmax_k, nk, k_unscale);
                    const uint8_t* krow = sm.ring_k[stage] + tid * kHalfDim;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const uint4 w0 = *reinterpret_cast<const uint4*>(krow + ((32u * half) ^ k_sw));
                        const uint4 w1 = *reinterpret_cast<const uint4*>(krow + ((32u * half + 16u) ^ k_sw));
                        const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                        uint32_t hi[16], lo[16];
#pragma unroll
                        for (int w = 0; w < 8; ++w) {
                            lookup4<KB>(tk, words[w], lo[2 * w], hi[2 * w]);
                            lookup4<KB>(tk, words[w] >> 16, lo[2 * w + 1], hi[2 * w + 1]);
                        }
                        tmem_st16_nowait(lane_base + kColKhi + 16 * half, hi);
                        tmem_st16_nowait(lane_base + kColKlo + 16 * half, lo);
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&sm.kready);

                // ---- V row -> shared tile (the previous tile's P V must have read it) ----
                if (pending) {
                    settle_pending();
                    if (dead) break;
                }
                uint32_t d[32];                              // the 32 sums of this token
                {
                    Table<VB> tb = build_value_table<T, VB>(sm.cb[1], nv);
                    if (!valid) {
                        // rows past the end of the sequence may hold bytes that are not index nibbles; with an
                        // all-zero table every PRMT result is zero whatever the selector (a -0.0 entry would
                        // turn a selector with its top bit set into a sign mask, i.e. a NaN pattern in fp16)
#pragma unroll
                        for (int r = 0; r < Table<VB>::kRegs; ++r) tb.r[r] = 0u;
                    }
                    const uint8_t* vrow = sm.ring_v[stage] + tid * VP;
#pragma unroll
                    for (int quarter = 0; quarter < 4; ++quarter) {
                        if (quarter == 2) {
                            // S^T is normally complete by now: request this token's sums so that the
                            // tensor-memory read runs under the second half of the V row
                            if (!mbar_wait(&sm.bar_s, it & 1)) { dead = true; break; }
                            tc_fence_after();
                            tmem_ld32_nowait(lane_base + kColS, d);
                        }
                        uint32_t words[4];
                        if constexpr (MODE == 1) {
                            const uint4 w4 = *reinterpret_cast<const uint4*>(vrow + ((16u * quarter) ^ k_sw));
                            words[0] = w4.x; words[1] = w4.y; words[2] = w4.z; words[3] = w4.w;
                        } else {
#pragma unroll
                            for (int w = 0; w < 4; ++w)
                                words[w] = *reinterpret_cast<const uint32_t*>(vrow + v_off + 16 * quarter + 4 * w);
                        }
#pragma unroll
                        for (int w = 0; w < 4; ++w) {          // 8 head-dims = one 32-bit index word per chunk
                            uint32_t lo0, hi0, lo1, hi1;
                            lookup4<VB>(tb, words[w], lo0, hi0);
                            lookup4<VB>(tb, words[w] >> 16, lo1, hi1);
                            *reinterpret_cast<uint4*>(v_dst + (4 * quarter + w) * 128) =
                                make_uint4(prmt(lo0, hi0, 0x5140), prmt(lo0, hi0, 0x7362),
                                           prmt(lo1, hi1, 0x5140), prmt(lo1, hi1, 0x7362));
                        }
                    }
                    if (dead) break;
                }

                // ---- scores, reference maxima, probabilities ----
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
                if (tile == t_begin) {
                    // first tile of the part: the reference maxima are the exact maxima of this tile
                    float m_new[NH];
                    tile_max(m_new);
#pragma unroll
                    for (int h = 0; h < NH; ++h) m_ref[h] = m_new[h];
                } else {
                    bool grow = false;
#pragma unroll
                    for (int h = 0; h < NH; ++h) grow |= sc[h] > m_ref[h] + 8.0f;
                    // rare: ask the issuer to hand the tile back instead of issuing its P V
                    if (grow) st_volatile_shared(&sm.grow_tile, it);
                }
                emit_p();
                tc_fence_before();
                mbar_arrive(&sm.pvready);
                pending = true;
                nk = nk_next;
                nv = nv_next;
            }
            if (dead) break;

            // ---- partial result of this part -> workspace row (group + sequence) * J + item ----
            if (pending) {
                settle_pending();
                if (dead) break;
            }
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                float v = l_acc[h];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) sm.red_l[warp][h] = v;
            }
            compute_sync();
            const int64_t row = (group + seq) * J + item;
            if (tid < heads_here) {
                float m = m_ref[0];
#pragma unroll
                for (int h = 1; h < NH; ++h) m = tid == h ? m_ref[h] : m;
                const float l = (sm.red_l[0][tid] + sm.red_l[1][tid]) + (sm.red_l[2][tid] + sm.red_l[3][tid]);
                p.ws_m[row * kHeadsPerCta + tid] = m;
                p.ws_l[row * kHeadsPerCta + tid] = l;
            }
            {
                uint32_t o[16];
                tmem_ld16_nowait(lane_base + kColO, o);
                tmem_wait_ld();
#pragma unroll
                for (int h = 0; h < NH; ++h)               // lane (position) x holds head-dim x ^ 1
                    if (h < heads_here)
                        p.ws_o[(row * kHeadsPerCta + h) * kHeadDim + (tid ^ 1)] =
                            __uint_as_float(o[h]) + __uint_as_float(o[8 + h]);
            }
            tc_fence_before();
            compute_sync();                          // red_l, the query planes and O^T are free for the next part

            x += t_end - t_begin;
            if (t_end == n_s) ++seq;
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
        while (x < x_end && seq < p.num_seqs) {
            const int pre = prefix[seq], n_s = prefix[seq + 1] - pre;
            if (n_s <= 0 || x >= static_cast<int64_t>(pre) + n_s) { ++seq; continue; }
            const int64_t left = x_end - x, in_seq = static_cast<int64_t>(pre) + n_s - x;
            const int64_t row = (group + seq) * J + item;
            if (tid < kHeadsPerCta) {
                p.ws_m[row * kHeadsPerCta + tid] = 0.0f;
                p.ws_l[row * kHeadsPerCta + tid] = __int_as_float(0x7fc00000);
            }
            x += left < in_seq ? left : in_seq;
            ++seq;
        }
    }
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// Tiles of every sequence as an exclusive prefix sum, for batches too large for the attention CTAs
// to scan themselves: prefix[s] = sum_{s' < s} ceil(len[s'] / 128), prefix[num_seqs] = total.
__global__ void decode_plan_kernel(const int32_t* __restrict__ seq_lens, int num_seqs, int32_t* __restrict__ prefix) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < num_seqs; base += blockDim.x) {
        const int s = base + threadIdx.x;
        const int n = s < num_seqs ? (max(__ldg(seq_lens + s), 0) + kTileTokens - 1) / kTileTokens : 0;
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
// part (group, sequence) of item j lives at row (group + sequence) * J + j.  Lanes gather the running
// maxima and row sums of up to 32 parts at a time; then the warp sums the weighted partial outputs.
constexpr int kMergeWarps = 4;
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32)
decode_merge_kernel(const DecodeParams p) {
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int64_t wq = static_cast<int64_t>(blockIdx.x) * kMergeWarps + (threadIdx.x >> 5);
    if (wq >= static_cast<int64_t>(p.num_seqs) * p.Hq) return;
    const int seq = static_cast<int>(wq / p.Hq), qh = static_cast<int>(wq % p.Hq);
    const int J = p.H * p.head_groups;
    const int kvh = qh / p.G, hl = qh % p.G;
    const int item = kvh * p.head_groups + hl / kHeadsPerCta, h = hl % kHeadsPerCta;
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
            const int64_t r = ((static_cast<int64_t>(gi) + seq) * J + item) * kHeadsPerCta + h;
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
                        p.ws_o + (((static_cast<int64_t>(g0 + k) + seq) * J + item) * kHeadsPerCta + h) * kHeadDim + 4 * lane);
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

// Grid and scratch of one decode call.  The (sequence, tile) space is cut into `groups` pieces;
// each piece is walked by J CTAs, one per (KV head, head group).
struct DecodePlan {
    int groups;            // pieces
    size_t rows;           // partial-result rows: (group + sequence) * J + item
    size_t prefix_bytes;
    size_t bytes;
};
// One 128-token tile per piece at least; at most `ctas_per_sm` CTAs per SM.  `forced` > 0 asks for that
// many pieces per sequence.
static DecodePlan plan_decode(int num_seqs, int H, int head_groups, int max_seq_len, int forced, int ctas_per_sm) {
    const long long J = 1LL * H * head_groups;
    const long long max_tiles = max_seq_len > 0 ? (max_seq_len + kTileTokens - 1) / kTileTokens : 1;
    const long long work = 1LL * num_seqs * max_tiles;
    long long groups = forced > 0 ? 1LL * forced * num_seqs : work;
    long long cap = (forced > 0 ? 4LL : 1LL) * sm_count() * ctas_per_sm / J;
    if (cap < 1) cap = 1;
    if (groups > cap) groups = cap;
    if (groups < 1) groups = 1;
    DecodePlan pl;
    pl.groups = static_cast<int>(groups);
    pl.rows = static_cast<size_t>((groups + num_seqs) * J);
    pl.prefix_bytes = (static_cast<size_t>(num_seqs + 1) * sizeof(int32_t) + 255) / 256 * 256;
    pl.bytes = pl.prefix_bytes + pl.rows * kHeadsPerCta * (kHeadDim + 2) * sizeof(float);
    return pl;
}

// ---- tensor maps of the cache for the TMA path ------------------------------------------------
//
// The cache is described as a 2-D byte tensor (num_slots rows of total_bytes).  cuTensorMapEncodeTiled
// is a driver entry point; it is looked up through the runtime so that the library does not link
// against the driver.  Maps are remembered per (cache pointer, shape, box): a serving loop calls
// with the same cache every step.

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
    int total_bytes, box_bytes, box_tokens, swizzle;
    bool operator==(const MapKey& o) const {
        return cache == o.cache && num_slots == o.num_slots && total_bytes == o.total_bytes &&
               box_bytes == o.box_bytes && box_tokens == o.box_tokens && swizzle == o.swizzle;
    }
};

static bool encode_cache_map(CUtensorMap* map, const uint8_t* cache, int64_t num_slots, int total_bytes,
                             int box_bytes, int box_tokens, bool swizzle64) {
    constexpr int kSlots = 16;
    struct Entry { MapKey key; CUtensorMap map; bool used; };
    static thread_local Entry cache_maps[kSlots] = {};
    static thread_local int next = 0;
    const MapKey key{cache, num_slots, total_bytes, box_bytes, box_tokens, swizzle64 ? 1 : 0};
    for (int i = 0; i < kSlots; ++i)
        if (cache_maps[i].used && cache_maps[i].key == key) {
            std::memcpy(map, &cache_maps[i].map, sizeof(CUtensorMap));
            return true;
        }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(total_bytes), static_cast<cuuint64_t>(num_slots)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(total_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_tokens)};
    const cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(cache), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    Entry& e = cache_maps[next];
    next = (next + 1) % kSlots;
    e.key = key;
    std::memcpy(&e.map, map, sizeof(CUtensorMap));
    e.used = true;
    return true;
}

// Environment switches, read once per process:
//   RQ_DECODE_NO_TMA=1            per-row bulk copies everywhere (comparisons)
//   RQ_DECODE_NO_PDL=1            launch the merge without programmatic dependent launch
//   RQ_DECODE_EQUAL_PIECES=1      no launch-layer weights
//   RQ_DECODE_LAYER_WEIGHTS=a,b,c weights of the launch layers (defaults below)
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

template <typename T, int KB, int VB, int MODE>
static int launch_attn(const DecodeParams& p, const CUtensorMap& map_k, const CUtensorMap& map_v, cudaStream_t st) {
    const size_t smem = sizeof(DecodeSmem<MODE>) + 1024;                     // + hand alignment
    const long long ctas = 1LL * p.groups * p.H * p.head_groups;
    auto launch = [&](auto kernel) -> int {
        if (int e = ensure_smem(kernel, smem)) return e;
        kernel<<<static_cast<unsigned>(ctas), kDecodeThreads, smem, st>>>(p, map_k, map_v);
        return check_cuda(cudaGetLastError(), "rq_decode attention launch");
    };
    return p.G <= 4 ? launch(decode_attn_kernel<T, KB, VB, MODE, 4>) : launch(decode_attn_kernel<T, KB, VB, MODE, 8>);
}

template <typename T, int KB, int VB>
static int launch_decode(DecodeParams& p, int mode, cudaStream_t st) {
    if (!p.inline_plan) {
        decode_plan_kernel<<<1, 1024, 0, st>>>(p.seq_lens, p.num_seqs, p.prefix);
        if (int e = check_cuda(cudaGetLastError(), "rq_decode plan launch")) return e;
    }
    alignas(64) CUtensorMap map_k{}, map_v{};
    const int64_t num_slots = p.num_blocks * p.block_size;
    if (mode != 0) {
        const bool ok = encode_cache_map(&map_k, p.cache, num_slots, p.total_bytes, kHalfDim, p.box_tokens, true) &&
                        encode_cache_map(&map_v, p.cache, num_slots, p.total_bytes, mode == 1 ? kHalfDim : 80,
                                         p.box_tokens, mode == 1);
        if (!ok) mode = 0;                                                 // no tensor maps: per-row copies
    }
    int e = mode == 1   ? launch_attn<T, KB, VB, 1>(p, map_k, map_v, st)
            : mode == 2 ? launch_attn<T, KB, VB, 2>(p, map_k, map_v, st)
                        : launch_attn<T, KB, VB, 0>(p, map_k, map_v, st);
    if (e) return e;

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
static int dispatch_bits(DecodeParams& p, int mode, int kb, int vb, cudaStream_t st) {
    if (kb == 3 && vb == 3) return launch_decode<T, 3, 3>(p, mode, st);
    if (kb == 4 && vb == 3) return launch_decode<T, 4, 3>(p, mode, st);
    if (kb == 3 && vb == 4) return launch_decode<T, 3, 4>(p, mode, st);
    return launch_decode<T, 4, 4>(p, mode, st);
}

// How the rows of a tile are staged for this cache geometry (see DecodeSmem).
static int staging_mode(int num_kv_heads, int block_size, int bs_shift, const uint8_t* cache, int64_t num_blocks) {
    if (decode_env().no_tma || bs_shift < 3 || !aligned(cache, 16) || num_blocks * block_size > INT32_MAX) return 0;
    return num_kv_heads % 4 == 0 ? 1 : 2;
}

}  // namespace rq

using namespace rq;

extern "C" size_t rq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                            int head_dim, int max_seq_len, int num_splits) {
    if (num_seqs <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim != kHeadDim) return 0;
    if (num_q_heads % num_kv_heads != 0) return 0;
    const int G = num_q_heads / num_kv_heads;
    const int head_groups = (G + kHeadsPerCta - 1) / kHeadsPerCta;
    // sized for the densest launch (three CTAs per SM) whatever staging mode the call will use
    return plan_decode(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits, kMaxCtasPerSm).bytes;
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
    if (static_cast<long long>(num_kv_heads) * head_groups > 65535)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decode: too many KV heads");
    int bs_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
        if ((1 << sft) == block_size) bs_shift = sft;
    const int mode = staging_mode(num_kv_heads, block_size, bs_shift, kv_cache, num_blocks);
    const int ctas_per_sm = mode == 1 ? DecodeSmem<1>::kCtasPerSm : DecodeSmem<2>::kCtasPerSm;
    const DecodePlan pl = plan_decode(num_seqs, num_kv_heads, head_groups, max_seq_len, num_splits, ctas_per_sm);
    const size_t need = pl.bytes;
    if (!workspace || workspace_bytes < need)
        return fail(RQ_ERR_WORKSPACE, "rq_decode: workspace of %zu bytes needed, %zu given", need,
                    workspace_bytes);
    if (!aligned(workspace, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_decode: workspace must be 16-byte aligned");

    DecodeParams p{};
    p.q = q; p.q_stride_seq = q_stride_seq; p.q_stride_head = q_stride_head;
    p.cache = kv_cache; p.num_blocks = num_blocks; p.block_size = block_size;
    p.total_bytes = total_bytes; p.block_table = block_table; p.bt_stride = block_table_stride;
    p.seq_lens = seq_lens; p.cent_k = centroids_k; p.cent_v = centroids_v; p.rotation = rotation;
    p.qk_scale = sm_scale * 1.4426950408889634f;
    p.H = num_kv_heads; p.Hq = num_q_heads; p.G = G; p.head_groups = head_groups;
    p.prefix = static_cast<int32_t*>(workspace);
    const size_t rows = pl.rows * kHeadsPerCta;
    p.ws_o = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.prefix_bytes);
    p.ws_m = p.ws_o + rows * kHeadDim;
    p.ws_l = p.ws_m + rows;
    p.num_seqs = num_seqs; p.groups = pl.groups;
    p.inline_plan = num_seqs <= kInlinePlanSeqs ? 1 : 0;
    p.bs_shift = bs_shift;
    p.box_tokens = block_size >= 16 ? 16 : block_size;
    // Launch-layer weights: only when (nearly) every SM holds its full set of CTAs.  The defaults were
    // fitted on a B200 from the finish times of equal pieces (see weight_cum); RQ_DECODE_LAYER_WEIGHTS
    // overrides them.
    const DecodeEnv& env = decode_env();
    const int sms = sm_count();
    const long long ctas = 1LL * pl.groups * num_kv_heads * head_groups;
    p.layer_ctas = 0;
    p.num_layers = ctas_per_sm;
    static const int kDefault3[kMaxLayers] = {1024, 1024, 1024, 1024};
    static const int kDefault2[kMaxLayers] = {1024, 1024, 1024, 1024};
    for (int i = 0; i < kMaxLayers; ++i) {
        const int* def = ctas_per_sm == 3 ? kDefault3 : kDefault2;
        p.layer_w[i] = env.n_weights > 0 ? env.weights[i < env.n_weights ? i : env.n_weights - 1] : def[i];
    }
    if (!env.equal_pieces && ctas > 1LL * (ctas_per_sm - 1) * sms) p.layer_ctas = sms;
    p.out = out; p.o_stride_seq = o_stride_seq; p.o_stride_head = o_stride_head;

    const int kb = n_centroids_k == 8 ? 3 : 4, vb = n_centroids_v == 8 ? 3 : 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RQ_DTYPE_BF16) return dispatch_bits<__nv_bfloat16>(p, mode, kb, vb, st);
    return dispatch_bits<__half>(p, mode, kb, vb, st);
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
