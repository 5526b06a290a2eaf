// Fused paged INT8 prefill attention over the RotorQuant cache on tcgen05 tensor cores, sm_100a.
//
// Replaces fused_paged_rq_int8_prefill (triton/fused_paged_rq_int8_prefill.py:43-363 of the
// reference: one sequence, 64-row Q tiles, mma.sync-class IMMA through Triton, K dequantised and
// re-quantised for every Q tile and every query head, no causal tile skipping) and the two dense
// rotations around it.  This kernel handles several sequences (cu_seqlens_q), a cached prefix
// (query rows are the last rows of the sequence), stacks the G query heads of a KV head into the
// MMA M dimension so that a K/V tile is dequantised once per GQA group, and skips KV tiles that
// are entirely masked.
//
// One CTA = 128 MMA rows = (128 / G) query tokens x G heads of one (sequence, KV head); one
// thread owns one row (= one TMEM lane).  Per 128-key tile:
//   1. every thread dequantises one key: K -> int8 codes with a per-key scale (8/16-entry code
//      table, PRMT lookup), V -> exact round_T(centroid * norm) values; both go to shared memory
//      in the tcgen05 core-matrix layout (no swizzle);
//   2. S = Q K^T   tcgen05.mma kind::i8, int32 accumulator in TMEM (4 instructions, K = 32 each);
//   3. each thread reads its row of S from TMEM, scales by q_scale[row] * k_scale[key], applies
//      the causal mask, runs the online softmax, writes P (bf16/f16) to shared memory;
//   4. O += P V    tcgen05.mma kind::f16, fp32 accumulator in TMEM (8 instructions, K = 16 each).
// The epilogue divides by the row sum, rounds, applies R, rounds and stores.
//
// INT8 scheme (the reference quantises Q per 64x128 tile and K per BLOCK_N x 128 tile with
// round-half-up-then-truncate, fused_paged_rq_int8_prefill.py:113-115,:176-178; here the scales
// are per query row and per key, round to nearest even):
//   q_i8[m][d] = rint(q_rot[m][d] * 127 / max_d |q_rot[m][d]|),  k_i8[t][d] likewise from the
//   decompressed key;  score = q_scale[m] * k_scale[t] * sum_d q_i8 k_i8.
//
// Every wait on an mbarrier is bounded; on expiry the CTA records an error, frees its TMEM and
// returns.
#include <type_traits>

#include "rq_common.cuh"
#include "rq_tcgen05.cuh"

namespace rq {

constexpr int kPfThreads = 256;       // two threads per row / key
constexpr int kPfRows = 128;          // MMA M
constexpr int kPfKeys = 128;          // keys per tile (MMA N of S, K extent of P V)
constexpr uint32_t kTmemCols = 256;   // S: columns 0..127 (int32), O: columns 128..255 (fp32)

struct PrefillParams {
    const void* q;
    void* out;
    int64_t q_stride_tok, q_stride_head, o_stride_tok, o_stride_head;
    const int32_t* cu_seqlens_q;      // nullptr: one sequence owning all rows
    int num_tokens;
    int H, Hq, G;
    int tokens_per_tile;              // 128 / G
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
    float qk_scale;                   // sm_scale * log2(e)
    int* error_flag;                  // optional device int, set non-zero when a wait expired
    uint8_t* stage;                   // staged path: scratch records (see prefill_stage_kernel)
    int stage_tiles_per_seq;
};

template <typename T> using PfType = TcFormat<T>;

template <typename T>
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pf_pack<__nv_bfloat16>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <>
__device__ __forceinline__ uint32_t pf_pack<__half>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <typename T>
__device__ __forceinline__ float2 pf_unpack(uint32_t v);
template <>
__device__ __forceinline__ float2 pf_unpack<__nv_bfloat16>(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 pf_unpack<__half>(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <typename T>
__device__ __forceinline__ float pf_round(float v) {
    return pf_unpack<T>(pf_pack<T>(v, 0.0f)).x;
}
__device__ __forceinline__ float pf_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- shared memory -------------------------------------------------------------------------
//
// Operand tiles in core-matrix order (a core matrix = 8 rows x 16 bytes, 128 contiguous bytes):
//   q, k : int8,  K-major   core index = (row / 8) * 8 + (byte / 16)     row = query row | key
//   p    : 16-bit, K-major  core index = (row / 8) * 16 + (key / 8)
//   v    : 16-bit, MN-major core index = (key / 8) * 16 + (dim / 8), core row = key % 8
// Within a 128-byte K row and within an 8-wide V chunk, position x holds head-dim x ^ 1 (the
// nibble order of the cache); q is stored the same way and the epilogue undoes it for O.
struct __align__(128) PrefillSmem {
    uint8_t q[kPfRows * kHeadDim];
    uint8_t k[kPfKeys * kHeadDim];
    uint16_t v[kPfKeys * kHeadDim];
    uint16_t p[kPfRows * kPfKeys];
    float k_scale[kPfKeys];
    float xch[2][kPfRows];            // exchange between the two threads of a row
    float rot[32 * 16];
    float cb[2][16];
    uint64_t bar_s, bar_o;
    uint32_t tmem_base;
};

// 32 index bytes (half a row) of one (token, head) from global memory; `align` is 16, 8 or 4.
__device__ __forceinline__ void load_idx32(const uint8_t* src, int align, uint32_t (&w)[8]) {
    if (align == 16) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 x = __ldg(reinterpret_cast<const uint4*>(src) + i);
            w[4 * i] = x.x; w[4 * i + 1] = x.y; w[4 * i + 2] = x.z; w[4 * i + 3] = x.w;
        }
    } else if (align == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint2 x = __ldg(reinterpret_cast<const uint2*>(src) + i);
            w[2 * i] = x.x; w[2 * i + 1] = x.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = __ldg(reinterpret_cast<const uint32_t*>(src) + i);
    }
}

// Four table bytes selected by the four nibbles of sel[15:0]; the table has 8 (BITS 3) or 16
// (BITS 4) byte entries in 2 or 4 registers.
template <int BITS>
__device__ __forceinline__ uint32_t byte_lookup(const uint32_t* tbl, uint32_t sel) {
    if constexpr (BITS == 3) {
        return prmt(tbl[0], tbl[1], sel);
    } else {
        const uint32_t s7 = sel & 0x7777u;
        const uint32_t y = prmt(sel, sel << 4, 0x5410);
        const uint32_t m = prmt(y, y, 0x9B8A);       // byte i = 0xFF when nibble i has its top bit set
        const uint32_t a = prmt(tbl[0], tbl[1], s7), b = prmt(tbl[2], tbl[3], s7);
        return (a & ~m) | (b & m);
    }
}

// int32 -> float for |x| < 2^22 without the conversion unit (which the exponentials need): adding x
// to the bit pattern of 1.5 * 2^23 gives the float 1.5 * 2^23 + x exactly.  |Q K^T| <= 128 * 127^2 < 2^21.
__device__ __forceinline__ float small_int_to_float(uint32_t x) {
    return __uint_as_float(x + 0x4B400000u) - 12582912.0f;
}

// Barrier of the two warps that share 32 rows (warp w and w ^ 4): ids 1..4.
__device__ __forceinline__ void pair_sync(int quarter) {
    asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
}

// 256 threads: thread (row = tid % 128, half = tid / 128).  Row r is TMEM lane r; the two threads
// of a row sit in warps w and w + 4, which may both address the lane quarter w % 4.  In the
// dequantisation phase `row` is the key of the tile and `half` the half of its 128 head-dims; in
// the softmax phase `row` is the query row and `half` the half of the 128 keys of the tile.
template <typename T, int KB, int VB>
__global__ void __launch_bounds__(kPfThreads, 2)
prefill_int8_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(smem_raw);
    constexpr int NK = 1 << KB, NV = 1 << VB;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int row = tid & (kPfRows - 1), half = tid >> 7, quarter = warp & 3;
    const int kvh = blockIdx.y, seq = blockIdx.z;
    const int q_begin = p.cu_seqlens_q ? __ldg(p.cu_seqlens_q + seq) : 0;
    const int q_end = p.cu_seqlens_q ? __ldg(p.cu_seqlens_q + seq + 1) : p.num_tokens;
    const int q_len = max(q_end - q_begin, 0);
    const int kv_len = max(__ldg(p.seq_lens + seq), 0);
    const int tiles_m = (q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
    // heavy (late) query tiles first
    const int m_tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
    if (m_tile >= tiles_m || kv_len == 0) {
        // rows of an empty sequence still get a defined (zero) output
        if (m_tile < tiles_m && half == 0) {
            const int tl = row / p.G, h = row % p.G;
            const int tok = m_tile * p.tokens_per_tile + tl;
            if (tl < p.tokens_per_tile && tok < q_len) {
                T* dst = static_cast<T*>(p.out) + (q_begin + tok) * p.o_stride_tok +
                         static_cast<int64_t>(kvh * p.G + h) * p.o_stride_head;
                for (int d = 0; d < kHeadDim; d += 8) *reinterpret_cast<uint4*>(dst + d) = make_uint4(0, 0, 0, 0);
            }
        }
        return;
    }

    // this thread's query row: token and head; absolute position of the token in its sequence
    const int tok_local = row / p.G, head_local = row % p.G;
    const int tok = m_tile * p.tokens_per_tile + tok_local;
    const bool row_valid = tok_local < p.tokens_per_tile && tok < q_len;
    const int pos = row_valid ? kv_len - q_len + tok : -1;
    const int last_tok = min(q_len, (m_tile + 1) * p.tokens_per_tile) - 1;
    const int max_pos = kv_len - q_len + last_tok;                  // >= 0 for the CTA
    const int n_tiles = min(max_pos, kv_len - 1) / kPfKeys + 1;

    // ---- set-up: barriers, TMEM, parameters ----
    if (tid == 0) {
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&sm.tmem_base, kTmemCols);
    for (int i = tid; i < 32 * 16; i += kPfThreads) {
        const int g = i >> 4, j = (i >> 2) & 3, k = i & 3;
        sm.rot[i] = __ldg(p.rotation + (4 * g + j) * kHeadDim + 4 * g + k);      // R[4g+j][4g+k]
    }
    if (tid < 32) {
        const int kv = tid >> 4, i = tid & 15;
        const int n = kv ? NV : NK;
        sm.cb[kv][i] = i < n ? __ldg((kv ? p.cent_v : p.cent_k) + i) : 0.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);   // this warp's TMEM lanes
    const uint32_t core_row_off = (row >> 3) * 1024 + (row & 7) * 16;                // q/k tiles: 8 chunks per row group

    // ---- Q: rotate, round, quantise the row to int8; each of the row's two threads handles half
    //      of the head-dims (16 rotation blocks, 4 chunks) and they exchange their maxima ----
    float q_scale = 0.0f;
    {
        uint32_t packed[32];                    // this half of the rotated, rounded row as T pairs (d, d+1)
        float mx = 0.0f;
        if (row_valid) {
            const T* src = static_cast<const T*>(p.q) + (q_begin + tok) * p.q_stride_tok +
                           static_cast<int64_t>(kvh * p.G + head_local) * p.q_stride_head + 64 * half;
#pragma unroll
            for (int b = 0; b < 16; ++b) {
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src + 4 * b));
                const float2 x01 = pf_unpack<T>(raw.x), x23 = pf_unpack<T>(raw.y);
                float r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 rr = *reinterpret_cast<const float4*>(&sm.rot[(16 * half + b) * 16 + j * 4]);
                    float acc = __fmul_rn(x01.x, rr.x);
                    acc = __fmaf_rn(x01.y, rr.y, acc);
                    acc = __fmaf_rn(x23.x, rr.z, acc);
                    acc = __fmaf_rn(x23.y, rr.w, acc);
                    r[j] = acc;
                }
                packed[2 * b] = pf_pack<T>(r[0], r[1]);
                packed[2 * b + 1] = pf_pack<T>(r[2], r[3]);
                const float2 a = pf_unpack<T>(packed[2 * b]), c = pf_unpack<T>(packed[2 * b + 1]);
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y))));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) packed[i] = 0u;
        }
        sm.xch[half][row] = mx;
        pair_sync(quarter);
        mx = fmaxf(mx, sm.xch[half ^ 1][row]);
        pair_sync(quarter);                     // xch is reused by the softmax
        const bool ok = mx > 0.0f && mx <= 3.0e38f;
        const float inv = ok ? __fdiv_rn(127.0f, mx) : 0.0f;
        q_scale = ok ? __fdiv_rn(mx, 127.0f) : 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {           // 16 head-dims = 16 bytes per chunk; chunks 4*half .. 4*half + 3
            uint32_t wds[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 a = pf_unpack<T>(packed[8 * c + 2 * w]), b = pf_unpack<T>(packed[8 * c + 2 * w + 1]);
                const int i0 = __float2int_rn(a.x * inv), i1 = __float2int_rn(a.y * inv);
                const int i2 = __float2int_rn(b.x * inv), i3 = __float2int_rn(b.y * inv);
                // position x holds head-dim x ^ 1
                wds[w] = (i1 & 0xFF) | ((i0 & 0xFF) << 8) | ((i3 & 0xFF) << 16) | ((i2 & 0xFF) << 24);
            }
            *reinterpret_cast<uint4*>(&sm.q[core_row_off + (4 * half + c) * 128]) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        }
    }
    const float row_factor = q_scale * p.qk_scale;

    // descriptors and instruction words
    const uint32_t idesc_s = (2u << 4) | (1u << 7) | (1u << 10) | ((kPfKeys >> 3) << 17) | ((kPfRows >> 4) << 24);
    const uint32_t idesc_o = (1u << 4) | (PfType<T>::kFmt << 7) | (PfType<T>::kFmt << 10) | (1u << 16) |
                             ((kHeadDim >> 3) << 17) | ((kPfRows >> 4) << 24);
    const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);

    const SlotLayout lay = slot_layout(p.H);
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);
    const int32_t* bt_row = p.block_table + seq * p.bt_stride;

    // index words and norms of this thread's half key, fetched one tile ahead
    uint32_t kw[8], vw[8];
    float norm_k = 0.0f, norm_v = 0.0f;
    auto load_key = [&](int tile) {
        const int kt = tile * kPfKeys + row;
        norm_k = 0.0f;
        norm_v = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { kw[i] = 0u; vw[i] = 0u; }
        if (tile < n_tiles && kt < kv_len) {
            int64_t blk = __ldg(bt_row + kt / p.block_size);
            blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
            const uint8_t* slot = p.cache + (blk * p.block_size + kt % p.block_size) * p.total_bytes;
            load_idx32(slot + lay.k_idx + kvh * kHalfDim + 32 * half, 16, kw);
            load_idx32(slot + lay.v_idx + kvh * kHalfDim + 32 * half, v_align, vw);
            norm_k = __ldg(reinterpret_cast<const float*>(slot + lay.k_norm) + kvh);
            norm_v = __ldg(reinterpret_cast<const float*>(slot + lay.v_norm) + kvh);
        }
    };
    load_key(0);

    float m_run = -INFINITY, l_run = 0.0f;      // l_run: sum over this thread's half of the keys
    uint32_t ph_s = 0, ph_o = 0;
    bool pv_pending = false, failed = false;

#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
        // ---- 1. dequantise half of key j*128 + row: K codes + scale, then V values ----
        {
            // K: int8 code table of this key (both threads of the key build it)
            float tv[NK];
            float mx = 0.0f;
#pragma unroll
            for (int i = 0; i < NK; ++i) {
                tv[i] = pf_round<T>(__fmul_rn(sm.cb[0][i], norm_k));
                mx = fmaxf(mx, fabsf(tv[i]));
            }
            const bool ok = mx > 0.0f && mx <= 3.0e38f;
            const float inv = ok ? __fdiv_rn(127.0f, mx) : 0.0f;
            if (half == 0) sm.k_scale[row] = ok ? __fdiv_rn(mx, 127.0f) : 0.0f;
            uint32_t ktbl[NK / 4];
#pragma unroll
            for (int i = 0; i < NK / 4; ++i) {
                const int c0 = __float2int_rn(tv[4 * i] * inv), c1 = __float2int_rn(tv[4 * i + 1] * inv);
                const int c2 = __float2int_rn(tv[4 * i + 2] * inv), c3 = __float2int_rn(tv[4 * i + 3] * inv);
                ktbl[i] = (c0 & 0xFF) | ((c1 & 0xFF) << 8) | ((c2 & 0xFF) << 16) | ((c3 & 0xFF) << 24);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {           // chunks 4*half .. 4*half + 3 of the key's 8
                const uint32_t a = kw[2 * c], b = kw[2 * c + 1];
                *reinterpret_cast<uint4*>(&sm.k[core_row_off + (4 * half + c) * 128]) =
                    make_uint4(byte_lookup<KB>(ktbl, a), byte_lookup<KB>(ktbl, a >> 16),
                               byte_lookup<KB>(ktbl, b), byte_lookup<KB>(ktbl, b >> 16));
            }
            // V: the previous tile's P V reads v and p until its barrier completes
            if (pv_pending) {
                failed |= !mbar_wait(&sm.bar_o, ph_o);
                ph_o ^= 1u;
                tc_fence_after();
                pv_pending = false;
            }
            // exact decompressed values, low- and high-byte planes of the T bit patterns
            uint32_t vlo[NV / 4], vhi[NV / 4];
#pragma unroll
            for (int i = 0; i < NV / 4; ++i) {
                const uint32_t p01 = pf_pack<T>(__fmul_rn(sm.cb[1][4 * i], norm_v), __fmul_rn(sm.cb[1][4 * i + 1], norm_v));
                const uint32_t p23 = pf_pack<T>(__fmul_rn(sm.cb[1][4 * i + 2], norm_v), __fmul_rn(sm.cb[1][4 * i + 3], norm_v));
                vlo[i] = prmt(p01, p23, 0x6420);
                vhi[i] = prmt(p01, p23, 0x7531);
            }
            uint8_t* vdst = reinterpret_cast<uint8_t*>(sm.v) + (row >> 3) * (16 * 128) + (row & 7) * 16;
#pragma unroll
            for (int c = 0; c < 8; ++c) {        // 8 head-dims = one 32-bit index word per chunk
                const uint32_t lo0 = byte_lookup<VB>(vlo, vw[c]), hi0 = byte_lookup<VB>(vhi, vw[c]);
                const uint32_t lo1 = byte_lookup<VB>(vlo, vw[c] >> 16), hi1 = byte_lookup<VB>(vhi, vw[c] >> 16);
                *reinterpret_cast<uint4*>(vdst + (8 * half + c) * 128) =
                    make_uint4(prmt(lo0, hi0, 0x5140), prmt(lo0, hi0, 0x7362),
                               prmt(lo1, hi1, 0x5140), prmt(lo1, hi1, 0x7362));
            }
        }
        load_key(j + 1);                             // lands while this tile's softmax runs
        fence_async_proxy();
        tc_fence_before();
        __syncthreads();

        // ---- 2. S = Q K^T ----
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int s = 0; s < 4; ++s)
                tc_mma_i8(tmem, smem_desc(q_addr + 256 * s, 128, 1024), smem_desc(k_addr + 256 * s, 128, 1024),
                          idesc_s, s > 0 ? 1u : 0u);
            tc_commit(&sm.bar_s);
        }
        failed |= !mbar_wait(&sm.bar_s, ph_s);
        ph_s ^= 1u;
        tc_fence_after();

        const float* const k_scale = sm.k_scale;

        // ---- 3. online softmax: this thread's row, keys 64*half .. 64*half + 63 of the tile ----
        // keys of this half that the row may see: columns 0 .. limit (>= 63: all of them)
        const int limit = pos - (j * kPfKeys + 64 * half);
        const bool unmasked = __all_sync(0xffffffffu, limit >= 63);
        uint8_t* prow = reinterpret_cast<uint8_t*>(sm.p) + (row >> 3) * (16 * 128) + (row & 7) * 16;
        auto softmax_half = [&](auto masked_tag) {
            constexpr bool kMasked = decltype(masked_tag)::value;
            // pass A: scale the integer sums by the key scales, row maximum.  The first 32 scaled sums
            // stay in registers, the other 32 go back to TMEM as floats until pass B.
            float m_half = -INFINITY;
            uint32_t r0[32];
            auto scale_chunk = [&](uint32_t (&r)[32], int ch) {
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 ks = *reinterpret_cast<const float4*>(&k_scale[64 * half + 32 * ch + 4 * c4]);
                    const float kk[4] = {ks.x, ks.y, ks.z, ks.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = 4 * c4 + e;
                        const float sv = small_int_to_float(r[c]) * kk[e];
                        r[c] = __float_as_uint(sv);
                        if (!kMasked || 32 * ch + c <= limit) m_half = fmaxf(m_half, sv);
                    }
                }
            };
            {
                uint32_t r1[32];
                tmem_ld32(lane_base + 64 * half + 32, r1);
                scale_chunk(r1, 1);
                tmem_st32(lane_base + 64 * half + 32, r1);
            }
            tmem_ld32(lane_base + 64 * half, r0);
            scale_chunk(r0, 0);
            sm.xch[half][row] = m_half;
            pair_sync(quarter);
            const float m_tile = fmaxf(m_half, sm.xch[half ^ 1][row]) * row_factor;     // row_factor >= 0
            // lazy reference: it moves only when the tile maximum exceeds it by more than 2^8
            const bool grew = m_tile > m_run + 8.0f;
            const float m_new = grew ? m_tile : m_run;
            const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
            const float alpha = grew ? ((m_run == -INFINITY) ? 0.0f : pf_ex2(m_run - m_use)) : 1.0f;
            if (j > 0 && __any_sync(0xffffffffu, grew)) {                // this thread's half of the O columns
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t r[32];
                    tmem_ld32(lane_base + kPfKeys + 64 * half + 32 * ch, r);
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                    tmem_st32(lane_base + kPfKeys + 64 * half + 32 * ch, r);
                }
            }
            l_run *= alpha;
            m_run = m_new;
            // pass B: probabilities -> shared P tile (K-major: 16 chunks of 8 keys per row)
            auto emit_chunk = [&](const uint32_t (&r)[32], int ch) {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    float p0 = pf_ex2(fmaf(__uint_as_float(r[c]), row_factor, -m_use));
                    float p1 = pf_ex2(fmaf(__uint_as_float(r[c + 1]), row_factor, -m_use));
                    if (kMasked) {
                        if (32 * ch + c > limit) p0 = 0.0f;
                        if (32 * ch + c + 1 > limit) p1 = 0.0f;
                    }
                    l_run += p0 + p1;
                    pk[c >> 1] = pf_pack<T>(p0, p1);
                }
#pragma unroll
                for (int kc = 0; kc < 4; ++kc)
                    *reinterpret_cast<uint4*>(prow + (8 * half + 4 * ch + kc) * 128) =
                        make_uint4(pk[4 * kc], pk[4 * kc + 1], pk[4 * kc + 2], pk[4 * kc + 3]);
            };
            emit_chunk(r0, 0);
            {
                uint32_t r1[32];
                tmem_ld32(lane_base + 64 * half + 32, r1);
                emit_chunk(r1, 1);
            }
        };
        // After the first tile the reference maximum rarely has to move, so the tile is first done in ONE
        // pass against the current reference (scaled sums and probabilities together, nothing parked in TMEM,
        // the raw sums left untouched); only when some row of the warp has outgrown its reference is the
        // tile redone by the two-pass code above, which also finds the new maximum.
        auto softmax_one_pass = [&](auto masked_tag) -> bool {
            constexpr bool kMasked = decltype(masked_tag)::value;
            const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
            float l_try = l_run;
#pragma unroll 1
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t r[32], pk[16];
                tmem_ld32(lane_base + 64 * half + 32 * ch, r);
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 ks = *reinterpret_cast<const float4*>(&k_scale[64 * half + 32 * ch + 4 * c4]);
                    const float kk[4] = {ks.x, ks.y, ks.z, ks.w};
                    float pr[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = 4 * c4 + e;
                        const float sv = small_int_to_float(r[c]) * kk[e];
                        pr[e] = pf_ex2(fmaf(sv, row_factor, -m_use));
                        if (kMasked && 32 * ch + c > limit) pr[e] = 0.0f;
                    }
                    l_try += pr[0] + pr[1];
                    l_try += pr[2] + pr[3];
                    pk[2 * c4] = pf_pack<T>(pr[0], pr[1]);
                    pk[2 * c4 + 1] = pf_pack<T>(pr[2], pr[3]);
                }
#pragma unroll
                for (int kc = 0; kc < 4; ++kc)
                    *reinterpret_cast<uint4*>(prow + (8 * half + 4 * ch + kc) * 128) =
                        make_uint4(pk[4 * kc], pk[4 * kc + 1], pk[4 * kc + 2], pk[4 * kc + 3]);
            }
            // The maximum is not tracked here: a row whose probabilities of this tile add up to more than 2^15
            // has outgrown its reference (every probability is below 2^15 otherwise, harmless for P in T
            // precision and for the fp32 sums), and so has a row that met its first visible key (its
            // reference is still -inf and some probability is exp2(score), unbounded): redo those tiles.
            sm.xch[half][row] = l_try - l_run;
            pair_sync(quarter);
            const float tile_sum = (l_try - l_run) + sm.xch[half ^ 1][row];
            // both warps that share these rows see the same sums, hence take the same decision
            const bool outgrown = !(tile_sum <= 32768.0f) || (m_run == -INFINITY && tile_sum > 0.0f);
            if (__any_sync(0xffffffffu, outgrown)) return false;
            l_run = l_try;
            return true;
        };
        bool done = false;
        if (j > 0) done = unmasked ? softmax_one_pass(std::false_type{}) : softmax_one_pass(std::true_type{});
        if (!done) {
            if (unmasked) softmax_half(std::false_type{});
            else softmax_half(std::true_type{});
        }
        fence_async_proxy();
        tc_fence_before();
        if (__syncthreads_or(failed)) { failed = true; break; }      // uniform exit

        // ---- 4. O += P V (completes while the next tile's K codes are built) ----
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int s = 0; s < 8; ++s)
                tc_mma_f16(tmem + kPfKeys, smem_desc(p_addr + 256 * s, 128, 2048),
                           smem_desc(v_addr + 4096 * s, 2048, 128), idesc_o, (j > 0 || s > 0) ? 1u : 0u);
            tc_commit(&sm.bar_o);
        }
        pv_pending = true;
    }
    if (pv_pending) {
        failed |= !mbar_wait(&sm.bar_o, ph_o);
        tc_fence_after();
    }
    failed = __syncthreads_or(failed);

    // ---- epilogue: O / l, round, rotate by R, round, store; this thread's half of the head-dims ----
    if (!failed) {
        sm.xch[half][row] = l_run;
        pair_sync(quarter);
        const float l_all = l_run + sm.xch[half ^ 1][row];
        const float inv_l = l_all > 0.0f ? 1.0f / l_all : 0.0f;
        T* dst = row_valid ? static_cast<T*>(p.out) + (q_begin + tok) * p.o_stride_tok +
                                 static_cast<int64_t>(kvh * p.G + head_local) * p.o_stride_head
                           : nullptr;
#pragma unroll 1
        for (int c2 = 0; c2 < 2; ++c2) {
            const int ch = 2 * half + c2;
            uint32_t r[32];
            tmem_ld32(lane_base + kPfKeys + 32 * ch, r);
            uint32_t outw[16];
#pragma unroll
            for (int b = 0; b < 8; ++b) {       // rotation block = head-dims 32ch + 4b .. + 3
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)    // column x of O holds head-dim x ^ 1
                    o[e] = pf_round<T>(__uint_as_float(r[(4 * b + e) ^ 1]) * inv_l);
                const float* rb = &sm.rot[(8 * ch + b) * 16];      // rb[k*4 + jj] = R[4g+k][4g+jj]
                float y[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    float acc = __fmul_rn(o[0], rb[jj]);
                    acc = __fmaf_rn(o[1], rb[4 + jj], acc);
                    acc = __fmaf_rn(o[2], rb[8 + jj], acc);
                    acc = __fmaf_rn(o[3], rb[12 + jj], acc);
                    y[jj] = acc;
                }
                outw[2 * b] = pf_pack<T>(y[0], y[1]);
                outw[2 * b + 1] = pf_pack<T>(y[2], y[3]);
            }
            if (dst != nullptr) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<uint4*>(dst + 32 * ch + 8 * i) =
                        make_uint4(outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]);
            }
        }
    } else if (tid == 0 && p.error_flag != nullptr) {
        atomicExch(p.error_flag, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---- staged path: scratch records ----------------------------------------------------------
//
// prefill_stage_kernel decompresses every (sequence, KV head, 128-key tile) once into a record of
// kStageRecord bytes: the K codes and the V values in exactly the shared-memory operand order of
// the attention kernel, then the 128 key scales.  Record index: (seq * tiles_per_seq + tile) * H + head.
constexpr int kStageRecord = 3 * kPfKeys * kHeadDim + kPfKeys * 4;      // 16 KB + 32 KB + 512 B

struct __align__(128) AttnSmem {
    uint8_t q[kPfRows * kHeadDim];
    uint8_t k[kPfKeys * kHeadDim];
    uint16_t v[kPfKeys * kHeadDim];
    uint16_t p[kPfRows * kPfKeys];
    float k_scale[2][kPfKeys];
    float xch[2][kPfRows];
    float rot[32 * 16];
    uint64_t bar_s, bar_o, bar_k, bar_v;
    uint32_t tmem_base;
};

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
}
// Contiguous global -> shared copy of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completing on the mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar_addr) : "memory");
}

// One CTA of 128 threads per (tile, KV head, sequence): thread = key.  Writes the record of the tile.
template <typename T, int KB, int VB>
__global__ void __launch_bounds__(128)
prefill_stage_kernel(const PrefillParams p) {
    constexpr int NK = 1 << KB, NV = 1 << VB;
    const int tid = threadIdx.x;
    const int tile = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int kv_len = max(__ldg(p.seq_lens + seq), 0);
    if (tile * kPfKeys >= kv_len) return;
    uint8_t* rec = p.stage + ((static_cast<int64_t>(seq) * p.stage_tiles_per_seq + tile) * p.H + kvh) * kStageRecord;
    const SlotLayout lay = slot_layout(p.H);
    const int v_align = (lay.v_idx % 16 == 0) ? 16 : ((lay.v_idx % 8 == 0) ? 8 : 4);
    const int kt = tile * kPfKeys + tid;
    uint32_t kw[16], vw[16];
    float norm_k = 0.0f, norm_v = 0.0f;
    if (kt < kv_len) {
        int64_t blk = __ldg(p.block_table + seq * p.bt_stride + kt / p.block_size);
        blk = blk < 0 ? 0 : (blk >= p.num_blocks ? p.num_blocks - 1 : blk);
        const uint8_t* slot = p.cache + (blk * p.block_size + kt % p.block_size) * p.total_bytes;
        load_idx64(slot + lay.k_idx + kvh * kHalfDim, 16, kw);
        load_idx64(slot + lay.v_idx + kvh * kHalfDim, v_align, vw);
        norm_k = __ldg(reinterpret_cast<const float*>(slot + lay.k_norm) + kvh);
        norm_v = __ldg(reinterpret_cast<const float*>(slot + lay.v_norm) + kvh);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) { kw[i] = 0u; vw[i] = 0u; }
    }
    // K: int8 code table of this key
    float tv[NK];
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < NK; ++i) {
        tv[i] = pf_round<T>(__fmul_rn(__ldg(p.cent_k + i), norm_k));
        mx = fmaxf(mx, fabsf(tv[i]));
    }
    const bool ok = mx > 0.0f && mx <= 3.0e38f;
    const float inv = ok ? __fdiv_rn(127.0f, mx) : 0.0f;
    reinterpret_cast<float*>(rec + 3 * kPfKeys * kHeadDim)[tid] = ok ? __fdiv_rn(mx, 127.0f) : 0.0f;
    uint32_t ktbl[NK / 4];
#pragma unroll
    for (int i = 0; i < NK / 4; ++i) {
        const int c0 = __float2int_rn(tv[4 * i] * inv), c1 = __float2int_rn(tv[4 * i + 1] * inv);
        const int c2 = __float2int_rn(tv[4 * i + 2] * inv), c3 = __float2int_rn(tv[4 * i + 3] * inv);
        ktbl[i] = (c0 & 0xFF) | ((c1 & 0xFF) << 8) | ((c2 & 0xFF) << 16) | ((c3 & 0xFF) << 24);
    }
    uint8_t* kdst = rec + (tid >> 3) * 1024 + (tid & 7) * 16;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint32_t a = kw[2 * c], b = kw[2 * c + 1];
        *reinterpret_cast<uint4*>(kdst + c * 128) =
            make_uint4(byte_lookup<KB>(ktbl, a), byte_lookup<KB>(ktbl, a >> 16),
                       byte_lookup<KB>(ktbl, b), byte_lookup<KB>(ktbl, b >> 16));
    }
    // V: exact decompressed values, low- and high-byte planes of the T bit patterns
    uint32_t vlo[NV / 4], vhi[NV / 4];
#pragma unroll
    for (int i = 0; i < NV / 4; ++i) {
        const uint32_t p01 = pf_pack<T>(__fmul_rn(__ldg(p.cent_v + 4 * i), norm_v), __fmul_rn(__ldg(p.cent_v + 4 * i + 1), norm_v));
        const uint32_t p23 = pf_pack<T>(__fmul_rn(__ldg(p.cent_v + 4 * i + 2), norm_v), __fmul_rn(__ldg(p.cent_v + 4 * i + 3), norm_v));
        vlo[i] = prmt(p01, p23, 0x6420);
        vhi[i] = prmt(p01, p23, 0x7531);
    }
    uint8_t* vdst = rec + kPfKeys * kHeadDim + (tid >> 3) * (16 * 128) + (tid & 7) * 16;
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        const uint32_t lo0 = byte_lookup<VB>(vlo, vw[c]), hi0 = byte_lookup<VB>(vhi, vw[c]);
        const uint32_t lo1 = byte_lookup<VB>(vlo, vw[c] >> 16), hi1 = byte_lookup<VB>(vhi, vw[c] >> 16);
        *reinterpret_cast<uint4*>(vdst + c * 128) =
            make_uint4(prmt(lo0, hi0, 0x5140), prmt(lo0, hi0, 0x7362),
                       prmt(lo1, hi1, 0x5140), prmt(lo1, hi1, 0x7362));
    }
}

// The attention kernel of the staged path: the same CTA shape, query set-up, softmax and epilogue
// as prefill_int8_kernel, but the K codes, key scales and V values of a tile arrive ready-made from
// the scratch written by prefill_stage_kernel: one thread starts three bulk copies per tile
// (cp.async.bulk, 16 KB + 512 B + 32 KB, already in operand order) that complete on mbarriers.  K of
// tile j+1 and V of tile j are requested as soon as S_j is finished, so both land under the softmax.
template <typename T>
__global__ void __launch_bounds__(kPfThreads, 2)
prefill_attn_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int row = tid & (kPfRows - 1), half = tid >> 7, quarter = warp & 3;
    const int kvh = blockIdx.y, seq = blockIdx.z;
    const int q_begin = p.cu_seqlens_q ? __ldg(p.cu_seqlens_q + seq) : 0;
    const int q_end = p.cu_seqlens_q ? __ldg(p.cu_seqlens_q + seq + 1) : p.num_tokens;
    const int q_len = max(q_end - q_begin, 0);
    const int kv_len = max(__ldg(p.seq_lens + seq), 0);
    const int tiles_m = (q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
    // heavy (late) query tiles first
    const int m_tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
    if (m_tile >= tiles_m || kv_len == 0) {
        // rows of an empty sequence still get a defined (zero) output
        if (m_tile < tiles_m && half == 0) {
            const int tl = row / p.G, h = row % p.G;
            const int tok = m_tile * p.tokens_per_tile + tl;
            if (tl < p.tokens_per_tile && tok < q_len) {
                T* dst = static_cast<T*>(p.out) + (q_begin + tok) * p.o_stride_tok +
                         static_cast<int64_t>(kvh * p.G + h) * p.o_stride_head;
                for (int d = 0; d < kHeadDim; d += 8) *reinterpret_cast<uint4*>(dst + d) = make_uint4(0, 0, 0, 0);
            }
        }
        return;
    }

    // this thread's query row: token and head; absolute position of the token in its sequence
    const int tok_local = row / p.G, head_local = row % p.G;
    const int tok = m_tile * p.tokens_per_tile + tok_local;
    const bool row_valid = tok_local < p.tokens_per_tile && tok < q_len;
    const int pos = row_valid ? kv_len - q_len + tok : -1;
    const int last_tok = min(q_len, (m_tile + 1) * p.tokens_per_tile) - 1;
    const int max_pos = kv_len - q_len + last_tok;                  // >= 0 for the CTA
    // never past the staged records (max_seq_len of the call bounds every sequence)
    const int n_tiles = min(min(max_pos, kv_len - 1) / kPfKeys + 1, p.stage_tiles_per_seq);

    // ---- set-up: barriers, TMEM, parameters ----
    if (tid == 0) {
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_init(&sm.bar_k, 1);
        mbar_init(&sm.bar_v, 1);
        fence_async_proxy();
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&sm.tmem_base, kTmemCols);
    for (int i = tid; i < 32 * 16; i += kPfThreads) {
        const int g = i >> 4, j = (i >> 2) & 3, k = i & 3;
        sm.rot[i] = __ldg(p.rotation + (4 * g + j) * kHeadDim + 4 * g + k);      // R[4g+j][4g+k]
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);   // this warp's TMEM lanes
    const uint32_t core_row_off = (row >> 3) * 1024 + (row & 7) * 16;                // q/k tiles: 8 chunks per row group

    // ---- Q: rotate, round, quantise the row to int8; each of the row's two threads handles half
    //      of the head-dims (16 rotation blocks, 4 chunks) and they exchange their maxima ----
    float q_scale = 0.0f;
    {
        uint32_t packed[32];                    // this half of the rotated, rounded row as T pairs (d, d+1)
        float mx = 0.0f;
        if (row_valid) {
            const T* src = static_cast<const T*>(p.q) + (q_begin + tok) * p.q_stride_tok +
                           static_cast<int64_t>(kvh * p.G + head_local) * p.q_stride_head + 64 * half;
#pragma unroll
            for (int b = 0; b < 16; ++b) {
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src + 4 * b));
                const float2 x01 = pf_unpack<T>(raw.x), x23 = pf_unpack<T>(raw.y);
                float r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 rr = *reinterpret_cast<const float4*>(&sm.rot[(16 * half + b) * 16 + j * 4]);
                    float acc = __fmul_rn(x01.x, rr.x);
                    acc = __fmaf_rn(x01.y, rr.y, acc);
                    acc = __fmaf_rn(x23.x, rr.z, acc);
                    acc = __fmaf_rn(x23.y, rr.w, acc);
                    r[j] = acc;
                }
                packed[2 * b] = pf_pack<T>(r[0], r[1]);
                packed[2 * b + 1] = pf_pack<T>(r[2], r[3]);
                const float2 a = pf_unpack<T>(packed[2 * b]), c = pf_unpack<T>(packed[2 * b + 1]);
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y))));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) packed[i] = 0u;
        }
        sm.xch[half][row] = mx;
        pair_sync(quarter);
        mx = fmaxf(mx, sm.xch[half ^ 1][row]);
        pair_sync(quarter);                     // xch is reused by the softmax
        const bool ok = mx > 0.0f && mx <= 3.0e38f;
        const float inv = ok ? __fdiv_rn(127.0f, mx) : 0.0f;
        q_scale = ok ? __fdiv_rn(mx, 127.0f) : 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {           // 16 head-dims = 16 bytes per chunk; chunks 4*half .. 4*half + 3
            uint32_t wds[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 a = pf_unpack<T>(packed[8 * c + 2 * w]), b = pf_unpack<T>(packed[8 * c + 2 * w + 1]);
                const int i0 = __float2int_rn(a.x * inv), i1 = __float2int_rn(a.y * inv);
                const int i2 = __float2int_rn(b.x * inv), i3 = __float2int_rn(b.y * inv);
                // position x holds head-dim x ^ 1
                wds[w] = (i1 & 0xFF) | ((i0 & 0xFF) << 8) | ((i3 & 0xFF) << 16) | ((i2 & 0xFF) << 24);
            }
            *reinterpret_cast<uint4*>(&sm.q[core_row_off + (4 * half + c) * 128]) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        }
    }
    const float row_factor = q_scale * p.qk_scale;
    fence_async_proxy();                 // the Q tile is read by the tensor core
    __syncthreads();

    // descriptors and instruction words
    const uint32_t idesc_s = (2u << 4) | (1u << 7) | (1u << 10) | ((kPfKeys >> 3) << 17) | ((kPfRows >> 4) << 24);
    const uint32_t idesc_o = (1u << 4) | (PfType<T>::kFmt << 7) | (PfType<T>::kFmt << 10) | (1u << 16) |
                             ((kHeadDim >> 3) << 17) | ((kPfRows >> 4) << 24);
    const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);

    // scratch records of this (sequence, KV head): [K codes 16 KB | V values 32 KB | key scales 512 B] per tile
    const uint8_t* const records = p.stage + (static_cast<int64_t>(seq) * p.stage_tiles_per_seq * p.H + kvh) * kStageRecord;
    const int64_t record_stride = static_cast<int64_t>(p.H) * kStageRecord;
    auto issue_k = [&](int tile) {                  // thread 0 only
        const uint8_t* rec = records + tile * record_stride;
        const uint32_t bar = smem_u32(&sm.bar_k);
        mbar_expect_tx(bar, kPfKeys * kHeadDim + kPfKeys * 4);
        bulk_load(smem_u32(sm.k), rec, kPfKeys * kHeadDim, bar);
        bulk_load(smem_u32(sm.k_scale[tile & 1]), rec + 3 * kPfKeys * kHeadDim, kPfKeys * 4, bar);
    };
    auto issue_v = [&](int tile) {                  // thread 0 only
        const uint8_t* rec = records + tile * record_stride;
        const uint32_t bar = smem_u32(&sm.bar_v);
        mbar_expect_tx(bar, 2 * kPfKeys * kHeadDim);
        bulk_load(smem_u32(sm.v), rec + kPfKeys * kHeadDim, 2 * kPfKeys * kHeadDim, bar);
    };
    if (tid == 0) {
        issue_k(0);
        issue_v(0);
    }

    float m_run = -INFINITY, l_run = 0.0f;      // l_run: sum over this thread's half of the keys
    uint32_t ph_s = 0, ph_o = 0, ph_k = 0, ph_v = 0;
    bool pv_pending = false, failed = false;

#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
        // ---- 1, 2. K codes and key scales of this tile have landed: S = Q K^T ----
        failed |= !mbar_wait(&sm.bar_k, ph_k);
        ph_k ^= 1u;
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int s = 0; s < 4; ++s)
                tc_mma_i8(tmem, smem_desc(q_addr + 256 * s, 128, 1024), smem_desc(k_addr + 256 * s, 128, 1024),
                          idesc_s, s > 0 ? 1u : 0u);
            tc_commit(&sm.bar_s);
        }
        failed |= !mbar_wait(&sm.bar_s, ph_s);
        ph_s ^= 1u;
        tc_fence_after();
        // the previous tile's P V has normally finished by now: its V tile and the P tile are free
        if (pv_pending) {
            failed |= !mbar_wait(&sm.bar_o, ph_o);
            ph_o ^= 1u;
            tc_fence_after();
            pv_pending = false;
        }
        if (tid == 0) {
            if (j + 1 < n_tiles) issue_k(j + 1);
            if (j > 0) issue_v(j);
        }
        const float* const k_scale = sm.k_scale[j & 1];

        // ---- 3. online softmax: this thread's row, keys 64*half .. 64*half + 63 of the tile ----
        // keys of this half that the row may see: columns 0 .. limit (>= 63: all of them)
        const int limit = pos - (j * kPfKeys + 64 * half);
        const bool unmasked = __all_sync(0xffffffffu, limit >= 63);
        uint8_t* prow = reinterpret_cast<uint8_t*>(sm.p) + (row >> 3) * (16 * 128) + (row & 7) * 16;
        auto softmax_half = [&](auto masked_tag) {
            constexpr bool kMasked = decltype(masked_tag)::value;
            // pass A: scale the integer sums by the key scales, row maximum.  The first 32 scaled sums
            // stay in registers, the other 32 go back to TMEM as floats until pass B.
            float m_half = -INFINITY;
            uint32_t r0[32];
            auto scale_chunk = [&](uint32_t (&r)[32], int ch) {
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 ks = *reinterpret_cast<const float4*>(&k_scale[64 * half + 32 * ch + 4 * c4]);
                    const float kk[4] = {ks.x, ks.y, ks.z, ks.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = 4 * c4 + e;
                        const float sv = small_int_to_float(r[c]) * kk[e];
                        r[c] = __float_as_uint(sv);
                        if (!kMasked || 32 * ch + c <= limit) m_half = fmaxf(m_half, sv);
                    }
                }
            };
            {
                uint32_t r1[32];
                tmem_ld32(lane_base + 64 * half + 32, r1);
                scale_chunk(r1, 1);
                tmem_st32(lane_base + 64 * half + 32, r1);
            }
            tmem_ld32(lane_base + 64 * half, r0);
            scale_chunk(r0, 0);
            sm.xch[half][row] = m_half;
            pair_sync(quarter);
            const float m_tile = fmaxf(m_half, sm.xch[half ^ 1][row]) * row_factor;     // row_factor >= 0
            // lazy reference: it moves only when the tile maximum exceeds it by more than 2^8
            const bool grew = m_tile > m_run + 8.0f;
            const float m_new = grew ? m_tile : m_run;
            const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
            const float alpha = grew ? ((m_run == -INFINITY) ? 0.0f : pf_ex2(m_run - m_use)) : 1.0f;
            if (j > 0 && __any_sync(0xffffffffu, grew)) {                // this thread's half of the O columns
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t r[32];
                    tmem_ld32(lane_base + kPfKeys + 64 * half + 32 * ch, r);
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                    tmem_st32(lane_base + kPfKeys + 64 * half + 32 * ch, r);
                }
            }
            l_run *= alpha;
            m_run = m_new;
            // pass B: probabilities -> shared P tile (K-major: 16 chunks of 8 keys per row)
            auto emit_chunk = [&](const uint32_t (&r)[32], int ch) {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    float p0 = pf_ex2(fmaf(__uint_as_float(r[c]), row_factor, -m_use));
                    float p1 = pf_ex2(fmaf(__uint_as_float(r[c + 1]), row_factor, -m_use));
                    if (kMasked) {
                        if (32 * ch + c > limit) p0 = 0.0f;
                        if (32 * ch + c + 1 > limit) p1 = 0.0f;
                    }
                    l_run += p0 + p1;
                    pk[c >> 1] = pf_pack<T>(p0, p1);
                }
#pragma unroll
                for (int kc = 0; kc < 4; ++kc)
                    *reinterpret_cast<uint4*>(prow + (8 * half + 4 * ch + kc) * 128) =
                        make_uint4(pk[4 * kc], pk[4 * kc + 1], pk[4 * kc + 2], pk[4 * kc + 3]);
            };
            emit_chunk(r0, 0);
            {
                uint32_t r1[32];
                tmem_ld32(lane_base + 64 * half + 32, r1);
                emit_chunk(r1, 1);
            }
        };
        // After the first tile the reference maximum rarely has to move, so the tile is first done in ONE
        // pass against the current reference (scaled sums and probabilities together, nothing parked in TMEM,
        // the raw sums left untouched); only when some row of the warp has outgrown its reference is the
        // tile redone by the two-pass code above, which also finds the new maximum.
        auto softmax_one_pass = [&](auto masked_tag) -> bool {
            constexpr bool kMasked = decltype(masked_tag)::value;
            const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
            float l_try = l_run;
#pragma unroll 1
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t r[32], pk[16];
                tmem_ld32(lane_base + 64 * half + 32 * ch, r);
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const float4 ks = *reinterpret_cast<const float4*>(&k_scale[64 * half + 32 * ch + 4 * c4]);
                    const float kk[4] = {ks.x, ks.y, ks.z, ks.w};
                    float pr[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = 4 * c4 + e;
                        const float sv = small_int_to_float(r[c]) * kk[e];
                        pr[e] = pf_ex2(fmaf(sv, row_factor, -m_use));
                        if (kMasked && 32 * ch + c > limit) pr[e] = 0.0f;
                    }
                    l_try += pr[0] + pr[1];
                    l_try += pr[2] + pr[3];
                    pk[2 * c4] = pf_pack<T>(pr[0], pr[1]);
                    pk[2 * c4 + 1] = pf_pack<T>(pr[2], pr[3]);
                }
#pragma unroll
                for (int kc = 0; kc < 4; ++kc)
                    *reinterpret_cast<uint4*>(prow + (8 * half + 4 * ch + kc) * 128) =
                        make_uint4(pk[4 * kc], pk[4 * kc + 1], pk[4 * kc + 2], pk[4 * kc + 3]);
            }
            // The maximum is not tracked here: a row whose probabilities of this tile add up to more than 2^15
            // has outgrown its reference (every probability is below 2^15 otherwise, harmless for P in T
            // precision and for the fp32 sums), and so has a row that met its first visible key (its
            // reference is still -inf and some probability is exp2(score), unbounded): redo those tiles.
            sm.xch[half][row] = l_try - l_run;
            pair_sync(quarter);
            const float tile_sum = (l_try - l_run) + sm.xch[half ^ 1][row];
            // both warps that share these rows see the same sums, hence take the same decision
            const bool outgrown = !(tile_sum <= 32768.0f) || (m_run == -INFINITY && tile_sum > 0.0f);
            if (__any_sync(0xffffffffu, outgrown)) return false;
            l_run = l_try;
            return true;
        };
        bool done = false;
        if (j > 0) done = unmasked ? softmax_one_pass(std::false_type{}) : softmax_one_pass(std::true_type{});
        if (!done) {
            if (unmasked) softmax_half(std::false_type{});
            else softmax_half(std::true_type{});
        }
        failed |= !mbar_wait(&sm.bar_v, ph_v);                   // the V tile has landed
        ph_v ^= 1u;
        fence_async_proxy();
        tc_fence_before();
        if (__syncthreads_or(failed)) { failed = true; break; }      // uniform exit

        // ---- 4. O += P V (completes under the next tile's S and row maxima) ----
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int s = 0; s < 8; ++s)
                tc_mma_f16(tmem + kPfKeys, smem_desc(p_addr + 256 * s, 128, 2048),
                           smem_desc(v_addr + 4096 * s, 2048, 128), idesc_o, (j > 0 || s > 0) ? 1u : 0u);
            tc_commit(&sm.bar_o);
        }
        pv_pending = true;
    }
    if (pv_pending) {
        failed |= !mbar_wait(&sm.bar_o, ph_o);
        tc_fence_after();
    }
    failed = __syncthreads_or(failed);

    // ---- epilogue: O / l, round, rotate by R, round, store; this thread's half of the head-dims ----
    if (!failed) {
        sm.xch[half][row] = l_run;
        pair_sync(quarter);
        const float l_all = l_run + sm.xch[half ^ 1][row];
        const float inv_l = l_all > 0.0f ? 1.0f / l_all : 0.0f;
        T* dst = row_valid ? static_cast<T*>(p.out) + (q_begin + tok) * p.o_stride_tok +
                                 static_cast<int64_t>(kvh * p.G + head_local) * p.o_stride_head
                           : nullptr;
#pragma unroll 1
        for (int c2 = 0; c2 < 2; ++c2) {
            const int ch = 2 * half + c2;
            uint32_t r[32];
            tmem_ld32(lane_base + kPfKeys + 32 * ch, r);
            uint32_t outw[16];
#pragma unroll
            for (int b = 0; b < 8; ++b) {       // rotation block = head-dims 32ch + 4b .. + 3
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)    // column x of O holds head-dim x ^ 1
                    o[e] = pf_round<T>(__uint_as_float(r[(4 * b + e) ^ 1]) * inv_l);
                const float* rb = &sm.rot[(8 * ch + b) * 16];      // rb[k*4 + jj] = R[4g+k][4g+jj]
                float y[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    float acc = __fmul_rn(o[0], rb[jj]);
                    acc = __fmaf_rn(o[1], rb[4 + jj], acc);
                    acc = __fmaf_rn(o[2], rb[8 + jj], acc);
                    acc = __fmaf_rn(o[3], rb[12 + jj], acc);
                    y[jj] = acc;
                }
                outw[2 * b] = pf_pack<T>(y[0], y[1]);
                outw[2 * b + 1] = pf_pack<T>(y[2], y[3]);
            }
            if (dst != nullptr) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<uint4*>(dst + 32 * ch + 8 * i) =
                        make_uint4(outw[4 * i], outw[4 * i + 1], outw[4 * i + 2], outw[4 * i + 3]);
            }
        }
    } else if (tid == 0 && p.error_flag != nullptr) {
        atomicExch(p.error_flag, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---- host side --------------------------------------------------------------------------------

template <typename T, int KB, int VB>
static int launch_prefill(const PrefillParams& p, int m_tiles, int num_seqs, cudaStream_t st) {
    dim3 grid(m_tiles, p.H, num_seqs);
    if (p.stage != nullptr) {
        dim3 sgrid(p.stage_tiles_per_seq, p.H, num_seqs);
        prefill_stage_kernel<T, KB, VB><<<sgrid, 128, 0, st>>>(p);
        if (int e = check_cuda(cudaGetLastError(), "rq_prefill_int8 stage launch")) return e;
        const size_t smem = sizeof(AttnSmem);
        if (int e = ensure_smem(prefill_attn_kernel<T>, smem)) return e;
        prefill_attn_kernel<T><<<grid, kPfThreads, smem, st>>>(p);
        return check_cuda(cudaGetLastError(), "rq_prefill_int8 attention launch");
    }
    const size_t smem = sizeof(PrefillSmem);
    if (int e = ensure_smem(prefill_int8_kernel<T, KB, VB>, smem)) return e;
    prefill_int8_kernel<T, KB, VB><<<grid, kPfThreads, smem, st>>>(p);
    return check_cuda(cudaGetLastError(), "rq_prefill_int8 launch");
}

template <typename T>
static int dispatch_prefill(const PrefillParams& p, int m_tiles, int num_seqs, int kb, int vb, cudaStream_t st) {
    if (kb == 3 && vb == 3) return launch_prefill<T, 3, 3>(p, m_tiles, num_seqs, st);
    if (kb == 4 && vb == 3) return launch_prefill<T, 4, 3>(p, m_tiles, num_seqs, st);
    if (kb == 3 && vb == 4) return launch_prefill<T, 3, 4>(p, m_tiles, num_seqs, st);
    return launch_prefill<T, 4, 4>(p, m_tiles, num_seqs, st);
}

static size_t stage_bytes(int num_seqs, int num_kv_heads, int max_seq_len) {
    if (num_seqs <= 0 || num_kv_heads <= 0 || max_seq_len <= 0) return 0;
    const size_t tiles = (static_cast<size_t>(max_seq_len) + kPfKeys - 1) / kPfKeys;
    return static_cast<size_t>(num_seqs) * tiles * num_kv_heads * kStageRecord;
}

}  // namespace rq

using namespace rq;

extern "C" size_t rq_prefill_workspace_bytes(int num_seqs, int num_kv_heads, int max_seq_len) {
    return stage_bytes(num_seqs, num_kv_heads, max_seq_len);
}

static int prefill_impl(const void* q, void* out, int dtype, int64_t q_stride_tok,
                        int64_t q_stride_head, int64_t o_stride_tok, int64_t o_stride_head,
                        const int32_t* cu_seqlens_q, int num_tokens, int num_seqs,
                        int max_q_len, int num_q_heads, int num_kv_heads, int head_dim,
                        const uint8_t* kv_cache, int64_t num_blocks, int block_size,
                        int total_bytes, const int32_t* block_table,
                        int64_t block_table_stride, const int32_t* seq_lens,
                        const float* centroids_k, int n_centroids_k,
                        const float* centroids_v, int n_centroids_v, const float* rotation,
                        float sm_scale, int* error_flag, int max_seq_len, void* workspace,
                        size_t workspace_bytes, void* stream) {
    if (num_tokens < 0 || num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_blocks < 0 ||
        block_size <= 0 || max_q_len < 0)
        return fail(RQ_ERR_INVALID_ARG, "rq_prefill_int8: negative or zero size");
    if (head_dim != kHeadDim)
        return fail(RQ_ERR_UNSUPPORTED, "rq_prefill_int8: head_dim %d (only 128)", head_dim);
    if (dtype != RQ_DTYPE_F16 && dtype != RQ_DTYPE_BF16)
        return fail(RQ_ERR_UNSUPPORTED, "rq_prefill_int8: query dtype must be f16 or bf16");
    if (num_q_heads % num_kv_heads != 0)
        return fail(RQ_ERR_INVALID_ARG, "rq_prefill_int8: %d query heads not a multiple of %d KV heads",
                    num_q_heads, num_kv_heads);
    const int G = num_q_heads / num_kv_heads;
    if (G > kPfRows)
        return fail(RQ_ERR_UNSUPPORTED, "rq_prefill_int8: %d query heads per KV head (at most 128)", G);
    if (total_bytes != num_kv_heads * kSlotPerHead)
        return fail(RQ_ERR_INVALID_ARG, "rq_prefill_int8: total_bytes %d != %d heads * 256", total_bytes,
                    num_kv_heads);
    if ((n_centroids_k != 8 && n_centroids_k != 16) || (n_centroids_v != 8 && n_centroids_v != 16))
        return fail(RQ_ERR_UNSUPPORTED, "rq_prefill_int8: codebooks must have 8 or 16 centroids");
    if (cu_seqlens_q == nullptr && num_seqs != 1)
        return fail(RQ_ERR_INVALID_ARG, "rq_prefill_int8: %d sequences need cu_seqlens_q", num_seqs);
    if (num_tokens == 0 || num_seqs == 0) return RQ_OK;
    if (num_seqs > 65535 || num_kv_heads > 65535)
        return fail(RQ_ERR_UNSUPPORTED, "rq_prefill_int8: too many sequences or heads for one launch");
    if (!q || !out || !kv_cache || !block_table || !seq_lens || !centroids_k || !centroids_v || !rotation)
        return fail(RQ_ERR_INVALID_ARG, "rq_prefill_int8: null pointer");
    if (!aligned(q, 8) || (q_stride_tok * 2) % 8 != 0 || (q_stride_head * 2) % 8 != 0)
        return fail(RQ_ERR_ALIGNMENT, "rq_prefill_int8: query rows must be 8-byte aligned");
    if (!aligned(out, 16) || (o_stride_tok * 2) % 16 != 0 || (o_stride_head * 2) % 16 != 0)
        return fail(RQ_ERR_ALIGNMENT, "rq_prefill_int8: output rows must be 16-byte aligned");
    if (!aligned(kv_cache, 16) || !aligned(rotation, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_prefill_int8: kv_cache and rotation must be 16-byte aligned");

    PrefillParams p{};
    p.q = q; p.out = out;
    p.q_stride_tok = q_stride_tok; p.q_stride_head = q_stride_head;
    p.o_stride_tok = o_stride_tok; p.o_stride_head = o_stride_head;
    p.cu_seqlens_q = cu_seqlens_q; p.num_tokens = num_tokens;
    p.H = num_kv_heads; p.Hq = num_q_heads; p.G = G;
    p.tokens_per_tile = kPfRows / G;
    p.cache = kv_cache; p.num_blocks = num_blocks; p.block_size = block_size;
    p.total_bytes = total_bytes; p.block_table = block_table; p.bt_stride = block_table_stride;
    p.seq_lens = seq_lens; p.cent_k = centroids_k; p.cent_v = centroids_v; p.rotation = rotation;
    p.qk_scale = sm_scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    if (workspace != nullptr) {
        if (max_seq_len <= 0)
            return fail(RQ_ERR_INVALID_ARG, "rq_prefill_int8_staged: max_seq_len must be positive");
        const size_t need = stage_bytes(num_seqs, num_kv_heads, max_seq_len);
        if (workspace_bytes < need)
            return fail(RQ_ERR_WORKSPACE, "rq_prefill_int8_staged: workspace of %zu bytes needed, %zu given", need,
                        workspace_bytes);
        if (!aligned(workspace, 128))
            return fail(RQ_ERR_ALIGNMENT, "rq_prefill_int8_staged: workspace must be 128-byte aligned");
        p.stage = static_cast<uint8_t*>(workspace);
        p.stage_tiles_per_seq = (max_seq_len + kPfKeys - 1) / kPfKeys;
    }
    const int longest = (max_q_len > 0 && max_q_len < num_tokens) ? max_q_len : num_tokens;
    const int m_tiles = (longest + p.tokens_per_tile - 1) / p.tokens_per_tile;
    const int kb = n_centroids_k == 8 ? 3 : 4, vb = n_centroids_v == 8 ? 3 : 4;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RQ_DTYPE_BF16) return dispatch_prefill<__nv_bfloat16>(p, m_tiles, num_seqs, kb, vb, st);
    return dispatch_prefill<__half>(p, m_tiles, num_seqs, kb, vb, st);
}

extern "C" int rq_prefill_int8(const void* q, void* out, int dtype, int64_t q_stride_tok,
                               int64_t q_stride_head, int64_t o_stride_tok, int64_t o_stride_head,
                               const int32_t* cu_seqlens_q, int num_tokens, int num_seqs,
                               int max_q_len, int num_q_heads, int num_kv_heads, int head_dim,
                               const uint8_t* kv_cache, int64_t num_blocks, int block_size,
                               int total_bytes, const int32_t* block_table,
                               int64_t block_table_stride, const int32_t* seq_lens,
                               const float* centroids_k, int n_centroids_k,
                               const float* centroids_v, int n_centroids_v, const float* rotation,
                               float sm_scale, int* error_flag, void* stream) {
    return prefill_impl(q, out, dtype, q_stride_tok, q_stride_head, o_stride_tok, o_stride_head, cu_seqlens_q,
                        num_tokens, num_seqs, max_q_len, num_q_heads, num_kv_heads, head_dim, kv_cache,
                        num_blocks, block_size, total_bytes, block_table, block_table_stride, seq_lens,
                        centroids_k, n_centroids_k, centroids_v, n_centroids_v, rotation, sm_scale, error_flag,
                        0, nullptr, 0, stream);
}

extern "C" int rq_prefill_int8_staged(const void* q, void* out, int dtype, int64_t q_stride_tok,
                                      int64_t q_stride_head, int64_t o_stride_tok, int64_t o_stride_head,
                                      const int32_t* cu_seqlens_q, int num_tokens, int num_seqs,
                                      int max_q_len, int num_q_heads, int num_kv_heads, int head_dim,
                                      const uint8_t* kv_cache, int64_t num_blocks, int block_size,
                                      int total_bytes, const int32_t* block_table,
                                      int64_t block_table_stride, const int32_t* seq_lens,
                                      const float* centroids_k, int n_centroids_k,
                                      const float* centroids_v, int n_centroids_v, const float* rotation,
                                      float sm_scale, int* error_flag, int max_seq_len, void* workspace,
                                      size_t workspace_bytes, void* stream) {
    if (workspace == nullptr)
        return fail(RQ_ERR_WORKSPACE, "rq_prefill_int8_staged: workspace missing");
    return prefill_impl(q, out, dtype, q_stride_tok, q_stride_head, o_stride_tok, o_stride_head, cu_seqlens_q,
                        num_tokens, num_seqs, max_q_len, num_q_heads, num_kv_heads, head_dim, kv_cache,
                        num_blocks, block_size, total_bytes, block_table, block_table_stride, seq_lens,
                        centroids_k, n_centroids_k, centroids_v, n_centroids_v, rotation, sm_scale, error_flag,
                        max_seq_len, workspace, workspace_bytes, stream);
}
