// Fused paged decode attention over the RotorQuant cache, sm_100a.
//
// Replaces fused_paged_rq_decode (triton/fused_paged_rq_decode.py:32-312 of the reference): the
// Triton kernel (one program per (sequence, query head), CUDA-core dot products, no split-KV)
// and the two dense 128x128 rotations its launcher runs around it.
//
// Work decomposition.  A tile is 128 consecutive tokens of one sequence and one KV head.  The
// (sequence, tile) space of the batch is one line of tiles, cut into contiguous pieces; a CTA
// streams the tiles of one piece for one (KV head, group of up to 8 query heads) and leaves one
// partial result per sequence its piece touches.  The 136 payload bytes of a (token, KV head) are
// read from HBM exactly once for all query heads of the GQA group.  A second launch merges the
// partial results of every (sequence, query head), rounds, and applies R.  Up to 128 sequences the
// attention CTAs compute the tile prefix sums themselves; larger batches get a one-CTA plan launch.
//
// The attention CTA has 128 threads, one per token of the tile and per TMEM lane; four CTAs share
// an SM, which is what keeps the SM's issue slots busy while any one CTA waits on its tensor-core
// or memory steps.  (Warp-specialised variants with separate issuer, copy, K and V warps and two
// CTAs per SM were built and measured: every one of them was slower, because fewer threads are
// left for the byte permutes that bound the kernel.)
//
// Arithmetic (matches "reference decompress + SDPA"):
//   q_rot   = round_T(q @ R^T)            exact FMA chain per 4x4 block, computed per part
//   K, V    = round_T(centroid[idx]*norm) exactly the decompressed values: each token gets a
//             table of its 8/16 rounded products, elements are fetched from it with PRMT
//   scores  = int8 tensor-core mma over 15-bit integer images of q_rot and K (exact for K, 2^-14
//             of the row maximum for q): S^T = K Q^T with the 128 tokens on the M side, the K
//             digit planes as a TMEM A operand and the query digit planes as the shared B operand;
//             fp32 scaling, exp2-domain softmax against a reference maximum per head (it moves
//             only when a score exceeds it by 2^8)
//   P @ V   = tensor-core mma with P split into hi + lo parts (two T-precision terms, ~16 bits),
//             fp32 accumulate in tensor memory: O^T += V^T [P hi | P lo]
//   out     = round_T(round_T(o / l) @ R)  in the merge kernel
// The kernel is bound by the dequantisation instructions (one byte permute per V value, half of
// one per K value), not by tensor throughput.

#include <cuda.h>          // CUtensorMap (types only; the encoder is looked up at run time)

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "rq_common.cuh"
#include "rq_tcgen05.cuh"

namespace rq {

constexpr int kHeadsPerCta = 8;              // query-head slots of a partial row / of one item
constexpr int kQPerHead = kHeadsPerCta;
constexpr int kTokenBox = 16;                // tokens per TMA box (never straddles a block of 16 or more)
constexpr int kInlinePlanSeqs = 128;         // up to this many sequences the CTAs scan seq_lens themselves
constexpr int kMaxLayers = 4;                // launch layers with their own piece weight
constexpr int kCtasPerSm = 4;
constexpr int kMaxPeers = 8;                 // GPUs of one NVLink domain that a sharded decode writes to

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
    float* ws_o;                           // [row][8 slots][128], row = (group + sequence) * J + item
    float* ws_m;                           // [row][8]
    float* ws_l;
    void* out;
    int64_t o_stride_seq, o_stride_head;
    // head-sharded decode: the merge writes every output row into the same place of each GPU's gathered
    // buffer (plain stores over NVLink into peer memory; the local GPU's buffer is one of the entries)
    void* peer_out[kMaxPeers];
    int num_peers;                         // 0: write `out` only
    int32_t* prefix;                       // [num_seqs + 1] exclusive prefix of tiles per sequence (workspace)
    int2* seq_groups;                      // [num_seqs] first and last group whose piece holds tiles of the sequence
    int num_seqs;
    int groups;                            // pieces; CTA = (group, item), item = (KV head, head group)
    int inline_plan;                       // the attention CTAs compute the prefix sums themselves
    int bs_shift;                          // log2(block_size) when it is a power of two, else -1
    int layer_ctas;                        // CTAs per launch layer (SM count) when pieces are weighted, else 0
    int num_layers;
    int layer_w[kMaxLayers];               // piece weight of the CTAs of each launch layer
};

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
// by `map` into shared memory; completion is signalled on the mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
        "r"(bar_addr)
        : "memory");
}

// 4-byte asynchronous copy global -> shared.
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Programmatic dependent launch: the merge kernel may be scheduled while the attention kernel
// drains; it must not read the partial results before this wait returns.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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

// ---- the attention kernel ---------------------------------------------------------------------
//
// One CTA = 128 threads = 128 tokens of a tile; thread t owns token t of the tile and TMEM lane t.
// Per tile:
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
// Index rows reach the CTA as TMA boxes of 16 tokens x 64 bytes (64-byte swizzle), staged per warp
// one tile ahead; norms are read straight from global memory.  Caches whose geometry rules TMA out
// (block sizes that are not a power of two >= 16) are read with direct 16-byte loads instead, and
// V rows that do not start on 16-byte boundaries (1 or 2 KV heads) with 4-byte cp.async.

constexpr int kUTile = 128;                  // tokens per tile
constexpr int kUThreads = 128;
constexpr int kUCtasPerSm = kCtasPerSm;
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
    int32_t prefix[kInlinePlanSeqs + 1];     // tile prefix sums when the CTA plans for itself
    int32_t scan[4];
    int64_t piece[2];                        // this CTA's piece of the tile line
    uint64_t bar_s, bar_o;
    uint64_t bar_in[4];                      // per warp: "staged rows landed"
    uint32_t tmem_base;
};

// NH = query heads computed per item: 4 when the GQA group has at most 4 heads, else 8.
// MODE = how the index rows reach the CTA: 0 direct global loads by every thread, 1 TMA boxes for K and
// V rows, 2 TMA boxes for the K rows and 4-byte cp.async for V rows that are not 16-byte aligned.
template <typename T, int KB, int VB, int MODE, int NH>
__global__ void __launch_bounds__(kUThreads, kUCtasPerSm)
decode_attn_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_idx) {
    constexpr bool TMA = MODE != 0;
    constexpr bool v_by_tma = MODE == 1;
    extern __shared__ uint8_t smem_raw[];
    // aligned by hand: the swizzled TMA rows want 512-byte alignment
    UmmaSmem& sm = *reinterpret_cast<UmmaSmem*>(smem_raw + ((512u - (smem_u32(smem_raw) & 511u)) & 511u));
    constexpr int NK = 1 << KB, NV = 1 << VB;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- tiles of every sequence as an exclusive prefix sum; this CTA's piece: CTA = (group, item) ----
    const int J = p.H * p.head_groups;
    const int64_t group = blockIdx.x / J;
    const int item = static_cast<int>(blockIdx.x % J);
    const int32_t* prefix = p.prefix;
    int64_t x, x_end;
    if (p.inline_plan) {                       // one sequence per thread, warp scan, four warp totals
        const int n = tid < p.num_seqs ? (max(__ldg(p.seq_lens + tid), 0) + kUTile - 1) / kUTile : 0;
        int incl = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) sm.scan[warp] = incl;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += sm.scan[w];
        if (tid == 0) sm.prefix[0] = 0;
        if (tid < p.num_seqs) sm.prefix[tid + 1] = before + incl;
        // the two piece boundaries cost 64-bit divisions: two lanes compute them for the CTA
        if (warp == 1 && lane < 2 && group < p.groups) {
            const int64_t total = (sm.scan[0] + sm.scan[1]) + (sm.scan[2] + sm.scan[3]);
            sm.piece[lane] = piece_begin(p, group + lane, total, J);
        }
        __syncthreads();
        prefix = sm.prefix;
        x = sm.piece[0];
        x_end = sm.piece[1];
        if (blockIdx.x == 0)                   // the merge launch reads the prefix sums from the workspace
            for (int i = tid; i <= p.num_seqs; i += kUThreads) p.prefix[i] = sm.prefix[i];
    } else if (group < p.groups) {
        const int64_t total = prefix[p.num_seqs];
        x = piece_begin(p, group, total, J);
        x_end = piece_begin(p, group + 1, total, J);
    }
    if (tid == 0) grid_launch_dependents();    // the merge kernel may be scheduled; it waits for this grid's end
    if (group >= p.groups || x >= x_end) return;

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
        const int64_t end = s < p.num_seqs ? prefix[s + 1] : INT64_MAX;
        const unsigned hit = __ballot_sync(0xffffffffu, end > x);
        if (hit) { seq = base + __ffs(hit) - 1; break; }
    }

    float cmax_k = 0.0f;                      // largest |K centroid|
#pragma unroll
    for (int i = 0; i < NK; ++i) cmax_k = fmaxf(cmax_k, fabsf(sm.cb[0][i]));

    uint32_t ph_s = 0, ph_o = 0;              // phase parities of the two barriers
    [[maybe_unused]] uint32_t ph_in = 0;      // ... and of this warp's staging barrier
    bool dead = false;                        // a bounded wait expired (same value in all threads)
    // staged rows of this thread's token: 16-byte chunk c sits at chunk c ^ ((lane >> 1) & 3)
    [[maybe_unused]] const uint8_t* const stage_k = sm.stage[warp][0] + lane * kHalfDim;
    [[maybe_unused]] const uint8_t* const stage_v = sm.stage[warp][1] + lane * kHalfDim;
    [[maybe_unused]] const uint32_t stage_sw = 16u * ((lane >> 1) & 3);

#pragma unroll 1
    while (x < x_end && seq < p.num_seqs) {
        const int pre = prefix[seq], n_s = prefix[seq + 1] - pre;
        if (n_s <= 0 || x >= static_cast<int64_t>(pre) + n_s) { ++seq; continue; }
        const int t_begin = static_cast<int>(x - pre);
        const int64_t reach = t_begin + (x_end - x);
        const int t_end = reach < n_s ? static_cast<int>(reach) : n_s;
        // the merge reads which groups hold parts of a sequence: the CTAs of item 0 leave the first and the
        // last one (the groups in between all do, their pieces being contiguous)
        if (item == 0 && tid == 0) {
            if (t_begin == 0) p.seq_groups[seq].x = static_cast<int>(group);
            if (t_end == n_s) p.seq_groups[seq].y = static_cast<int>(group);
        }
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
                // (instruction i copies rows 2i and 2i + 1; all addresses are bases plus multiples of i)
                const int half = lane >> 4, word = lane & 15;
                const int rows_left = seq_len - (tile * kUTile + 32 * warp + half);     // row 2i exists when 2i < rows_left
                const int64_t two_slots = 2 * static_cast<int64_t>(p.total_bytes);
                const uint8_t* const col = p.cache + lay.v_idx + kvh * kHalfDim + 4 * word;
                const uint8_t* src0 = col + static_cast<int64_t>(s0 + half) * p.total_bytes;
                const uint8_t* src1 = col + static_cast<int64_t>(s1 + half) * p.total_bytes;
                const uint32_t dst = smem_u32(sm.stage[warp][1]) + half * kHalfDim + ((word & 3) << 2);
                uint32_t chunk[4];                       // 16-byte chunk of this word under the row's swizzle, (row >> 1) & 3 == i & 3
#pragma unroll
                for (int c = 0; c < 4; ++c) chunk[c] = dst + ((((word >> 2) ^ c)) << 4);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (2 * i < rows_left) cp_async4(chunk[i & 3] + i * 2 * kHalfDim, i < 8 ? src0 : src1);
                    if (i < 8) src0 += two_slots;
                    else src1 += two_slots;
                }
            }
        };
        // the staged V rows are complete (the K rows are covered by the barrier)
        [[maybe_unused]] auto v_rows_landed = [&]() {
            if constexpr (!v_by_tma) {
                cp_async_wait_all();
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
                float cbk[NK];
#pragma unroll
                for (int i = 0; i < NK; i += 4) {
                    const float4 c4 = *reinterpret_cast<const float4*>(&sm.cb[0][i]);
                    cbk[i] = c4.x; cbk[i + 1] = c4.y; cbk[i + 2] = c4.z; cbk[i + 3] = c4.w;
                }
                const Table<KB> tk = build_int_table<T, KB>(cbk, cmax_k, nk, k_unscale);
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
                float cbv[NV];
#pragma unroll
                for (int i = 0; i < NV; i += 4) {
                    const float4 c4 = *reinterpret_cast<const float4*>(&sm.cb[1][i]);
                    cbv[i] = c4.x; cbv[i + 1] = c4.y; cbv[i + 2] = c4.z; cbv[i + 3] = c4.w;
                }
                const Table<VB> tb = build_value_table<T, VB>(cbv, nv);
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
// query head sits in slot (query head within its group of 8).  Lanes
// gather the running maxima and row sums of up to 32 parts at a time; then the warp sums the
// weighted partial outputs.  Which groups those are was recorded per sequence by the attention CTAs.
// W = 1: a warp per row (the usual few parts per row).  W = 4: a CTA per row, warp s taking every fourth round
// of 32 parts and the four partial sums combined through shared memory -- for long sequences on few heads,
// where a row has dozens of parts and there are too few rows to hide the latency of walking them.
constexpr int kMergeWarps = 4;
template <typename T, int W>
__global__ void __launch_bounds__(kMergeWarps * 32)
decode_merge_kernel(const DecodeParams p) {
    __shared__ float part_ml[W > 1 ? W : 1][2];
    __shared__ float4 part_acc[W > 1 ? W : 1][32];
    const int lane = threadIdx.x & 31;
    const int sub = (threadIdx.x >> 5) % W;
    // the lane's 4x4 block of R does not depend on the attention launch: fetch it before waiting for that
    float4 rr[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
        rr[k] = __ldg(reinterpret_cast<const float4*>(p.rotation + (4 * lane + k) * kHeadDim + 4 * lane));
    grid_dependency_wait();
    const int64_t wq = static_cast<int64_t>(blockIdx.x) * (kMergeWarps / W) + (threadIdx.x >> 5) / W;
    if (wq >= static_cast<int64_t>(p.num_seqs) * p.Hq) return;          // (all warps of a row together)
    const int seq = static_cast<int>(wq / p.Hq), qh = static_cast<int>(wq % p.Hq);
    const int J = p.H * p.head_groups;
    const int kvh = qh / p.G, hl = qh % p.G;
    const int item = kvh * p.head_groups + hl / kQPerHead;
    constexpr int slots = kQPerHead;
    const int slot = hl % kQPerHead;
    const int64_t a = p.prefix[seq], n = p.prefix[seq + 1] - a, total = p.prefix[p.num_seqs];
    const int2 range = p.seq_groups[seq];

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l_all = 0.0f;
    if (n > 0) {
        // first and last group with tiles of this sequence, as the attention CTAs recorded them (clamped: a
        // CTA whose bounded wait expired may not have got there, and the output is NaN then anyway)
        const int g_first = min(max(range.x, 0), p.groups - 1);
        const int g_last = min(max(range.y, g_first), p.groups - 1);
        // Groups whose piece is empty wrote nothing.  No piece is empty when the smallest weighted piece
        // holds a tile, which is the normal case; only batches with fewer tiles than that check per group.
        int min_w = 1024;
        if (p.layer_ctas > 0) {
            min_w = p.layer_w[0];
            for (int i = 1; i < p.num_layers; ++i) min_w = min(min_w, p.layer_w[i]);
        }
        const bool dense = total * J * min_w >=
                           weight_cum(static_cast<int64_t>(p.groups) * J, p.layer_ctas, p.num_layers, p.layer_w);
        float m_all = -INFINITY;
        for (int g0 = g_first + 32 * sub; g0 <= g_last; g0 += 32 * W) {             // normally one round
            const int gi = g0 + lane;
            const bool live = gi <= g_last &&
                              (dense || piece_begin(p, gi, total, J) < piece_begin(p, gi + 1, total, J));
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
#pragma unroll 8
            for (int k = 0; k < n_here; ++k) {
                const float wk = __shfl_sync(0xffffffffu, w, k);
                if (wk != 0.0f) {
                    const float4 o = *reinterpret_cast<const float4*>(
                        p.ws_o + ((((static_cast<int64_t>(g0 + k) + seq) * J + item) * slots + slot) << 7) + 4 * lane);
                    acc.x += wk * o.x; acc.y += wk * o.y; acc.z += wk * o.z; acc.w += wk * o.w;
                }
            }
        }
        if constexpr (W > 1) {                                   // combine the warps' partial sums in warp 0
            if (lane == 0) { part_ml[sub][0] = m_all; part_ml[sub][1] = l_all; }
            part_acc[sub][lane] = acc;
        }
    }
    if constexpr (W > 1) {
        __syncthreads();
        if (sub != 0) return;
        if (n > 0) {
            float m = part_ml[0][0];
#pragma unroll
            for (int s2 = 1; s2 < W; ++s2) m = fmaxf(m, part_ml[s2][0]);
            acc = make_float4(0.f, 0.f, 0.f, 0.f);
            l_all = 0.0f;
#pragma unroll
            for (int s2 = 0; s2 < W; ++s2) {
                const float ms = part_ml[s2][0];
                const float ws = ms == -INFINITY ? 0.0f : exp2f(ms - m);      // a warp without parts
                const float4 a4 = part_acc[s2][lane];
                acc.x += ws * a4.x; acc.y += ws * a4.y; acc.z += ws * a4.z; acc.w += ws * a4.w;
                l_all += ws * part_ml[s2][1];
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
        if (k == 0) {
            r[0] = __fmul_rn(o[0], rr[0].x); r[1] = __fmul_rn(o[0], rr[0].y);
            r[2] = __fmul_rn(o[0], rr[0].z); r[3] = __fmul_rn(o[0], rr[0].w);
        } else {
            r[0] = __fmaf_rn(o[k], rr[k].x, r[0]); r[1] = __fmaf_rn(o[k], rr[k].y, r[1]);
            r[2] = __fmaf_rn(o[k], rr[k].z, r[2]); r[3] = __fmaf_rn(o[k], rr[k].w, r[3]);
        }
    }
    const int64_t offset = seq * p.o_stride_seq + static_cast<int64_t>(qh) * p.o_stride_head + 4 * lane;
    const uint2 packed = make_uint2(pack_pair<T>(r[0], r[1]), pack_pair<T>(r[2], r[3]));
    auto store = [&](void* base) {
        T* dst = static_cast<T*>(base) + offset;
        if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
            *reinterpret_cast<uint2*>(dst) = packed;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) store_rounded(dst + j, r[j]);
        }
    };
    if (p.num_peers == 0) {
        store(p.out);
    } else {
        // No fence here: the arrive-and-wait kernel that announces these rows is a later launch on the same
        // stream, and a grid has ended only when all its stores, peer memory included, have been performed.
        for (int g = 0; g < p.num_peers; ++g) store(p.peer_out[g]);
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

// Grid and scratch of one decode call.  The (sequence, tile) space is cut into `groups` pieces and
// each piece is walked by J CTAs, one per (KV head, group of 8 query heads).
struct DecodePlan {
    int nh;                // query heads computed per item: 4 or 8
    int J;                 // items
    int groups;            // pieces
    size_t rows;           // partial-result rows: (group + sequence) * J + item, 8 slots each
    size_t prefix_bytes;
    size_t bytes;
};
// One 128-token tile per piece at least; at most four CTAs per SM.  `forced` > 0 asks for that many
// pieces per sequence.
static DecodePlan plan_decode(int num_seqs, int H, int G, int max_seq_len, int forced) {
    DecodePlan pl;
    pl.nh = G <= 4 ? 4 : 8;
    const int head_groups = (G + kQPerHead - 1) / kQPerHead;
    pl.J = H * head_groups;
    const long long max_tiles = max_seq_len > 0 ? (max_seq_len + kUTile - 1) / kUTile : 1;
    const long long work = 1LL * num_seqs * max_tiles;
    long long groups = forced > 0 ? 1LL * forced * num_seqs : work;
    long long cap = (forced > 0 ? 4LL : 1LL) * sm_count() * kCtasPerSm / pl.J;
    if (cap < 1) cap = 1;
    if (groups > cap) groups = cap;
    if (groups < 1) groups = 1;
    pl.groups = static_cast<int>(groups);
    pl.rows = static_cast<size_t>((groups + num_seqs) * pl.J);
    // tile prefix sums [num_seqs + 1] (int32, padded to 8 bytes), then the group range of every sequence (int2)
    pl.prefix_bytes = ((static_cast<size_t>(num_seqs + 2) / 2 * 2) * sizeof(int32_t) +
                       static_cast<size_t>(num_seqs) * sizeof(int2) + 255) / 256 * 256;
    pl.bytes = pl.prefix_bytes + pl.rows * kQPerHead * (kHeadDim + 2) * sizeof(float);
    return pl;
}

// ---- tensor maps of the cache ------------------------------------------------------------------
//
// The cache is described as a 2-D byte tensor (num_slots rows of total_bytes) with a box of 16 tokens
// x 64 bytes (one index row per token) and 64-byte swizzle.  cuTensorMapEncodeTiled is
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
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(total_bytes), static_cast<cuuint64_t>(num_slots)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(total_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(cache), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
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
//   RQ_DECODE_NO_TMA=1            every thread loads its own rows (the path of odd block sizes)
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

template <typename T, int KB, int VB>
static int launch_decode(DecodeParams& p, int nh, bool tma, cudaStream_t st) {
    if (!p.inline_plan) {
        decode_plan_kernel<<<1, 1024, 0, st>>>(p.seq_lens, p.num_seqs, kUTile, p.prefix);
        if (int e = check_cuda(cudaGetLastError(), "rq_decode plan launch")) return e;
    }
    alignas(64) CUtensorMap map_idx{};
    if (tma)
        tma = encode_cache_map(&map_idx, p.cache, p.num_blocks * p.block_size, p.total_bytes, kHalfDim, kTokenBox);
    {
        const size_t smem = sizeof(UmmaSmem) + 512;                              // + hand alignment
        const long long ctas = 1LL * p.groups * p.H * p.head_groups;
        auto launch = [&](auto kernel) -> int {
            if (int e = ensure_smem(kernel, smem)) return e;
            kernel<<<static_cast<unsigned>(ctas), kUThreads, smem, st>>>(p, map_idx);
            return check_cuda(cudaGetLastError(), "rq_decode attention launch");
        };
        // rows by TMA when the geometry allows; V rows of 1 or 2 KV heads are not 16-byte aligned
        const int mode = !tma ? 0 : (p.H % 4 == 0 ? 1 : 2);
        int e = RQ_OK;
        if (mode == 0) e = nh == 4 ? launch(decode_attn_kernel<T, KB, VB, 0, 4>) : launch(decode_attn_kernel<T, KB, VB, 0, 8>);
        else if (mode == 1) e = nh == 4 ? launch(decode_attn_kernel<T, KB, VB, 1, 4>) : launch(decode_attn_kernel<T, KB, VB, 1, 8>);
        else e = nh == 4 ? launch(decode_attn_kernel<T, KB, VB, 2, 4>) : launch(decode_attn_kernel<T, KB, VB, 2, 8>);
        if (e) return e;
    }

    // rows with many parts each (long sequences on few heads): a CTA per row instead of a warp per row
    const long long rows = 1LL * p.num_seqs * p.Hq;
    const bool wide = p.groups > 8LL * p.num_seqs;
    const unsigned grid = static_cast<unsigned>(wide ? rows : (rows + kMergeWarps - 1) / kMergeWarps);
    if (decode_env().no_pdl) {
        if (wide) decode_merge_kernel<T, kMergeWarps><<<grid, kMergeWarps * 32, 0, st>>>(p);
        else decode_merge_kernel<T, 1><<<grid, kMergeWarps * 32, 0, st>>>(p);
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
    return check_cuda(wide ? cudaLaunchKernelEx(&cfg, decode_merge_kernel<T, kMergeWarps>, p)
                           : cudaLaunchKernelEx(&cfg, decode_merge_kernel<T, 1>, p), "rq_decode merge launch");
}

template <typename T>
static int dispatch_bits(DecodeParams& p, int nh, bool tma, int kb, int vb, cudaStream_t st) {
    if (kb == 3 && vb == 3) return launch_decode<T, 3, 3>(p, nh, tma, st);
    if (kb == 4 && vb == 3) return launch_decode<T, 4, 3>(p, nh, tma, st);
    if (kb == 3 && vb == 4) return launch_decode<T, 3, 4>(p, nh, tma, st);
    return launch_decode<T, 4, 4>(p, nh, tma, st);
}

}  // namespace rq

using namespace rq;

extern "C" size_t rq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                            int head_dim, int max_seq_len, int num_splits) {
    if (num_seqs <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim != kHeadDim) return 0;
    if (num_q_heads % num_kv_heads != 0) return 0;
    return plan_decode(num_seqs, num_kv_heads, num_q_heads / num_kv_heads, max_seq_len, num_splits).bytes;
}

static int decode_impl(const void* q, void* out, int dtype, int64_t q_stride_seq,
                       int64_t q_stride_head, int64_t o_stride_seq, int64_t o_stride_head,
                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                       const uint8_t* kv_cache, int64_t num_blocks, int block_size,
                       int total_bytes, const int32_t* block_table, int64_t block_table_stride,
                       const int32_t* seq_lens, const float* centroids_k, int n_centroids_k,
                       const float* centroids_v, int n_centroids_v, const float* rotation,
                       float sm_scale, int max_seq_len, void* workspace, size_t workspace_bytes,
                       int num_splits, void* const* peer_out, int num_peers, void* stream) {
    if (num_peers < 0 || num_peers > kMaxPeers || (num_peers > 0 && peer_out == nullptr))
        return fail(RQ_ERR_INVALID_ARG, "rq_decode: %d peer outputs (at most %d)", num_peers, kMaxPeers);
    for (int g = 0; g < num_peers; ++g)
        if (peer_out[g] == nullptr) return fail(RQ_ERR_INVALID_ARG, "rq_decode: null peer output %d", g);
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
    p.prefix = static_cast<int32_t*>(workspace);
    p.seq_groups = reinterpret_cast<int2*>(static_cast<int32_t*>(workspace) + (num_seqs + 2) / 2 * 2);
    const size_t slots = pl.rows * kQPerHead;
    p.ws_o = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.prefix_bytes);
    p.ws_m = p.ws_o + slots * kHeadDim;
    p.ws_l = p.ws_m + slots;
    p.num_seqs = num_seqs; p.groups = pl.groups;
    p.inline_plan = num_seqs <= kInlinePlanSeqs ? 1 : 0;
    p.bs_shift = bs_shift;
    // TMA boxes of 16 tokens: power-of-two blocks of 16 tokens or more (a box never straddles a block),
    // slot numbers that fit a 32-bit coordinate
    const DecodeEnv& env = decode_env();
    const bool tma = !env.no_tma && bs_shift >= 4 && num_blocks * block_size <= INT32_MAX;
    // Launch-layer weights: only when (nearly) every SM holds its full set of CTAs.  RQ_DECODE_LAYER_WEIGHTS
    // overrides the defaults (measured: the CTAs launched first on an SM get the larger share of the
    // issue slots while four run side by side).
    const int sms = sm_count();
    const long long ctas = 1LL * pl.groups * pl.J;
    p.layer_ctas = 0;
    p.num_layers = kCtasPerSm;
    static const int kDefaultWeights[kMaxLayers] = {1290, 1090, 950, 766};
    for (int i = 0; i < kMaxLayers; ++i)
        p.layer_w[i] = env.n_weights > 0 ? env.weights[i < env.n_weights ? i : env.n_weights - 1] : kDefaultWeights[i];
    if (!env.equal_pieces && ctas > 1LL * (kCtasPerSm - 1) * sms) p.layer_ctas = sms;
    p.out = out; p.o_stride_seq = o_stride_seq; p.o_stride_head = o_stride_head;
    p.num_peers = num_peers;
    for (int g = 0; g < num_peers; ++g) p.peer_out[g] = peer_out[g];

    const int kb = n_centroids_k == 8 ? 3 : 4, vb = n_centroids_v == 8 ? 3 : 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RQ_DTYPE_BF16) return dispatch_bits<__nv_bfloat16>(p, pl.nh, tma, kb, vb, st);
    return dispatch_bits<__half>(p, pl.nh, tma, kb, vb, st);
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
    return decode_impl(q, out, dtype, q_stride_seq, q_stride_head, o_stride_seq, o_stride_head, num_seqs,
                       num_q_heads, num_kv_heads, head_dim, kv_cache, num_blocks, block_size, total_bytes,
                       block_table, block_table_stride, seq_lens, centroids_k, n_centroids_k, centroids_v,
                       n_centroids_v, rotation, sm_scale, max_seq_len, workspace, workspace_bytes, num_splits,
                       nullptr, 0, stream);
}

// Head-sharded decode: rq_decode whose merge kernel writes every output row into `num_peers` buffers, one
// per GPU of the tensor-parallel group (the calling GPU's own gathered buffer among them), at the same
// offsets as `out`.  Followed by rq_peer_barrier it replaces "decode + all-gather of the head outputs".
extern "C" int rq_decode_sharded(const void* q, int dtype, int64_t q_stride_seq, int64_t q_stride_head,
                                 int64_t o_stride_seq, int64_t o_stride_head, int num_seqs, int num_q_heads,
                                 int num_kv_heads, int head_dim, const uint8_t* kv_cache, int64_t num_blocks,
                                 int block_size, int total_bytes, const int32_t* block_table,
                                 int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
                                 int n_centroids_k, const float* centroids_v, int n_centroids_v,
                                 const float* rotation, float sm_scale, int max_seq_len, void* workspace,
                                 size_t workspace_bytes, int num_splits, void* const* peer_out, int num_peers,
                                 void* stream) {
    if (num_peers <= 0 || peer_out == nullptr)
        return fail(RQ_ERR_INVALID_ARG, "rq_decode_sharded: at least one output buffer is needed");
    return decode_impl(q, peer_out[0], dtype, q_stride_seq, q_stride_head, o_stride_seq, o_stride_head, num_seqs,
                       num_q_heads, num_kv_heads, head_dim, kv_cache, num_blocks, block_size, total_bytes,
                       block_table, block_table_stride, seq_lens, centroids_k, n_centroids_k, centroids_v,
                       n_centroids_v, rotation, sm_scale, max_seq_len, workspace, workspace_bytes, num_splits,
                       peer_out, num_peers, stream);
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
