// Compress-on-cache-write for RotorQuant (IsoQuant / PlanarQuant), sm_100a.
//
// One pass over the new tokens: L2 norm, normalise, block-diagonal rotation, boundary bucketize,
// nibble pack, and the scatter into the paged cache.  Replaces the reference's per-row Triton
// kernel (triton/isoquant_compress.py:16-96) plus the row assembly and scatter in
// RQAttentionImpl._compress_and_store (vllm/rq_backend.py:585-657).
//
// Bit-exactness.  The bytes must equal the reference's PyTorch path
// (triton/isoquant_compress.py:161-190), so each value is produced by the IEEE-754 operations of
// that path in their order:
//   norm   : eight running sums s_l += x[8c+l]^2 (multiply and add rounded separately,
//            c ascending), combined left to right, correctly rounded sqrt
//   divide : x / (norm + 1e-10f), IEEE division
//   rotate : out_j = fma(x3,R[j][3], fma(x2,R[j][2], fma(x1,R[j][1], x0*R[j][0]))) per 4x4 block
//   bucket : number of boundaries strictly below the value
//
// Mapping.  The cache-write path (compress + store) gives a row of 128 values to four threads, 32
// elements, eight rotation blocks and one 16-byte store each; the plain rows-to-rows path gives it to
// sixteen threads of 8 elements.  Only the norm needs the whole row: the squares go through shared
// memory, a few threads of the row form the eight running sums in the prescribed order, and the
// left-to-right combination is done with shuffles.
#include "rq_common.cuh"

namespace rq {

constexpr int kCompressThreads = 256;                 // 16 rows per CTA
constexpr int kRowsPerCta = kCompressThreads / 16;
constexpr int kCompressGrid = 148 * 4;                // the grid walks the rows: at most 4 CTAs per SM
constexpr int kRowBatch = 2;                          // rows fetched ahead per 16-thread group and step
constexpr int64_t kWideFromRows = 16384;              // launches with this many rows per kind use four threads per row

struct CompressParams {
    const void* src[2];          // key, value (or x, unused)
    int64_t token_stride[2];     // elements
    int64_t head_stride[2];      // elements
    int64_t num_tokens;          // tokens (store variant) or rows (rows variant)
    int H;
    // cache destination (store variant)
    uint8_t* cache;
    int64_t num_slots;
    int total_bytes;
    const int64_t* slot_mapping;
    int write_padding;
    // plain-row destination (rows variant)
    uint8_t* packed_out;
    float* norms_out;
    // parameters
    const float* rotation;       // dense 128x128
    const float* bounds[2];
    int n_bounds[2];
    int h_shift;                 // log2(H) when H is a power of two, else -1
};

// Eight consecutive elements of a row, raw (converted only when they are used, so that a load
// issued ahead of time does not make its issuer wait).
template <typename T>
struct Raw8 {
    uint4 a, b;               // b only for 4-byte elements
};
template <typename T>
__device__ __forceinline__ Raw8<T> load_raw8(const T* src) {
    Raw8<T> r;
    r.a = __ldg(reinterpret_cast<const uint4*>(src));
    if constexpr (sizeof(T) == 4) r.b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    return r;
}
template <typename T>
__device__ __forceinline__ void unpack8(const Raw8<T>& r, float* x) {
    if constexpr (sizeof(T) == 4) {
        Chunk16<float>::unpack(r.a, x);
        Chunk16<float>::unpack(r.b, x + 4);
    } else {
        Chunk16<T>::unpack(r.a, x);
    }
}

// Eight consecutive elements of a row as fp32.
template <typename T>
__device__ __forceinline__ void load8(const T* src, float* x) {
    if constexpr (sizeof(T) == 4) {
        Chunk16<float>::unpack(__ldg(reinterpret_cast<const uint4*>(src)), x);
        Chunk16<float>::unpack(__ldg(reinterpret_cast<const uint4*>(src) + 1), x + 4);
    } else {
        Chunk16<T>::unpack(__ldg(reinterpret_cast<const uint4*>(src)), x);
    }
}

// What a thread needs of R for the whole launch: the two 4x4 blocks of its elements (thread j of a row owns
// blocks 2j and 2j + 1), as [half][out jj][in k].  The CTA keeps them in shared memory, 36 floats apart per
// thread slot so that the 16-byte chunks of eight consecutive threads fall into different banks (the two rows
// of a warp read the same addresses); keeping them in 32 registers per thread instead costs the fourth CTA per SM.
constexpr int kRotPitch = 36;
struct ThreadRotation {
    const float* s;
};
__device__ __forceinline__ ThreadRotation load_rotation(const float* __restrict__ rotation, int j) {
    __shared__ __align__(16) float rot_s[16 * kRotPitch];
    for (int i = threadIdx.x; i < 512; i += kCompressThreads) {
        const int t = i >> 5, e = i & 31;
        const int g = 2 * t + (e >> 4), jj = (e >> 2) & 3, k = e & 3;
        rot_s[t * kRotPitch + e] = __ldg(rotation + (4 * g + jj) * kHeadDim + 4 * g + k);
    }
    __syncthreads();
    return ThreadRotation{rot_s + j * kRotPitch};
}


// Number of boundaries strictly below v.  The boundaries ascend, so "bd[b] < v" is true for a
// prefix of them and a binary search over that prefix gives the count with log2(NB + 1) compares
// (a NaN compares false everywhere: 0, as the linear count gives).
template <int NB>
__device__ __forceinline__ uint32_t count_below(const float (&bd)[NB], float v) {
    if constexpr (NB == 7) {
        const bool c1 = bd[3] < v;
        const bool c2 = (c1 ? bd[5] : bd[1]) < v;
        const float lo = c2 ? bd[2] : bd[0], hi = c2 ? bd[6] : bd[4];
        const bool c3 = (c1 ? hi : lo) < v;
        return (c1 ? 4u : 0u) + (c2 ? 2u : 0u) + (c3 ? 1u : 0u);
    } else {
        static_assert(NB == 15, "7 or 15 boundaries");
        const bool c1 = bd[7] < v;
        const bool c2 = (c1 ? bd[11] : bd[3]) < v;
        const float m3a = c2 ? bd[5] : bd[1], m3b = c2 ? bd[13] : bd[9];
        const bool c3 = (c1 ? m3b : m3a) < v;
        // fourth level: boundary 8*c1 + 4*c2 + 2*c3
        const float q0 = c3 ? bd[2] : bd[0], q1 = c3 ? bd[6] : bd[4];
        const float q2 = c3 ? bd[10] : bd[8], q3 = c3 ? bd[14] : bd[12];
        const float h0 = c2 ? q1 : q0, h1 = c2 ? q3 : q2;
        const bool c4 = (c1 ? h1 : h0) < v;
        return (c1 ? 8u : 0u) + (c2 ? 4u : 0u) + (c3 ? 2u : 0u) + (c4 ? 1u : 0u);
    }
}

// The 16 threads of a row: returns this thread's packed word (8 indices) and the row norm.
// `x` are the thread's elements 8j..8j+7, `sq_row` the row's [16][8] exchange area in shared
// memory, `bd` the NB boundaries; all 32 lanes of the warp must call this.
template <int NB>
__device__ __forceinline__ uint32_t compress_chunk(const float (&x)[8], int j, float* sq_row,
                                                   const ThreadRotation& rot, const float (&bd)[NB],
                                                   float& norm_out) {
    // squares, published for the in-order lane sums
    float* mine = sq_row + 8 * j;
    *reinterpret_cast<float4*>(mine) = make_float4(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1]),
                                                   __fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3]));
    *reinterpret_cast<float4*>(mine + 4) = make_float4(__fmul_rn(x[4], x[4]), __fmul_rn(x[5], x[5]),
                                                       __fmul_rn(x[6], x[6]), __fmul_rn(x[7], x[7]));
    __syncwarp();
    float s = 0.0f;
    if (j < 8) {
        float v[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) v[c] = sq_row[8 * c + j];
        s = v[0];
#pragma unroll
        for (int c = 1; c < 16; ++c) s = __fadd_rn(s, v[c]);
    }
    float tot = __shfl_sync(0xffffffffu, s, 0, 16);
#pragma unroll
    for (int l = 1; l < 8; ++l) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, s, l, 16));
    __syncwarp();                                   // sq_row may be rewritten by the next row
    const float norm = __fsqrt_rn(tot);
    norm_out = norm;
    const float denom = __fadd_rn(norm, 1e-10f);

    uint32_t word = 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const float x0 = __fdiv_rn(x[4 * half], denom), x1 = __fdiv_rn(x[4 * half + 1], denom);
        const float x2 = __fdiv_rn(x[4 * half + 2], denom), x3 = __fdiv_rn(x[4 * half + 3], denom);
        uint32_t idx[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const float4 r4 = *reinterpret_cast<const float4*>(rot.s + 16 * half + 4 * jj);
            const float r[4] = {r4.x, r4.y, r4.z, r4.w};
            float acc = __fmul_rn(x0, r[0]);
            acc = __fmaf_rn(x1, r[1], acc);
            acc = __fmaf_rn(x2, r[2], acc);
            acc = __fmaf_rn(x3, r[3], acc);
            idx[jj] = count_below<NB>(bd, acc);
        }
        const uint32_t b0 = (idx[0] << 4) | idx[1];
        const uint32_t b1 = (idx[2] << 4) | idx[3];
        word |= (b0 | (b1 << 8)) << (16 * half);
    }
    return word;
}

// ---- store variant for small launches: sixteen threads per row -------------------------------------
//
// The decode step compresses one token per sequence: a few hundred rows.  With 8 elements per thread the
// dependency chain of a row is a quarter as long as with 32, and the rows spread over four times as many
// threads, which is what counts when the launch cannot fill the GPU anyway.  A fixed grid walks first all K
// rows (token-major, head-minor), then all V rows, two rows per warp at a time, the elements of a step's
// rows all requested before the first is processed.  Every row's 16 threads write its 64 index bytes and its
// norm straight into the token's cache slot; the K row of head 0 also zeroes the slot's padding.
template <typename T, int NB>
__device__ __forceinline__ void store_rows(const CompressParams& p, int kv, const ThreadRotation& rot,
                                           float* sq_row, int j) {
    float bd[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) bd[b] = __ldg(p.bounds[kv] + b);
    const int H = p.H;
    const SlotLayout lay = slot_layout(H);
    const uint32_t rows = static_cast<uint32_t>(p.num_tokens) * static_cast<uint32_t>(H);
    const uint32_t step = gridDim.x * kRowsPerCta;
    const uint32_t first = blockIdx.x * kRowsPerCta + (threadIdx.x >> 4);
    const T* src = static_cast<const T*>(p.src[kv]);
    auto locate = [&](uint32_t r, uint32_t& token, uint32_t& h) {
        if (p.h_shift >= 0) { token = r >> p.h_shift; h = r & (H - 1); }
        else { token = r / H; h = r - token * H; }
    };
    auto fetch = [&](uint32_t r, Raw8<T>& raw, int64_t& slot) {
        uint32_t token, h;
        locate(r < rows ? r : 0u, token, h);        // rows past the end compute on row 0 and store nothing
        raw = load_raw8<T>(src + token * p.token_stride[kv] + static_cast<int64_t>(h) * p.head_stride[kv] + 8 * j);
        slot = __ldg(p.slot_mapping + token);
    };
    // the two rows of a warp run in lock step (shuffles, __syncwarp): loop on the warp's first row.
    // A step fetches kRowBatch rows per thread group before it works on any of them, so that their
    // load latencies overlap.
    constexpr int B = kRowBatch;
    const uint32_t warp_first = first & ~1u;
    for (uint32_t wr = warp_first, r = first; wr < rows; wr += B * step, r += B * step) {
        Raw8<T> raw[B];
        int64_t slot[B];
#pragma unroll
        for (int b = 0; b < B; ++b)
            if (wr + b * step < rows) fetch(r + b * step, raw[b], slot[b]);
#pragma unroll
        for (int b = 0; b < B; ++b) {
            if (wr + b * step >= rows) break;               // warp-uniform
            const uint32_t rb = r + b * step;
            float x[8];
            unpack8<T>(raw[b], x);
            float norm;
            const uint32_t word = compress_chunk<NB>(x, j, sq_row, rot, bd, norm);
            if (rb < rows) {
                uint32_t token, h;
                locate(rb, token, h);
                if (slot[b] >= 0 && slot[b] < p.num_slots) {
                    uint8_t* dst = p.cache + slot[b] * p.total_bytes;
                    *reinterpret_cast<uint32_t*>(dst + (kv ? lay.v_idx : lay.k_idx) + h * kHalfDim + 4 * j) = word;
                    if (j == 0) *reinterpret_cast<float*>(dst + (kv ? lay.v_norm : lay.k_norm) + 4 * h) = norm;
                    if (p.write_padding && kv == 0 && h == 0) {
                        const int units = (lay.total - lay.payload_end) / 8;
                        for (int u = j; u < units; u += 16)
                            *reinterpret_cast<uint2*>(dst + lay.payload_end + 8 * u) = make_uint2(0u, 0u);
                    }
                }
            }
        }
    }
}
template <typename T>
__global__ void __launch_bounds__(kCompressThreads, 4)
compress_store_kernel(const CompressParams p) {
    __shared__ __align__(16) float sq[kRowsPerCta][16 * 8];
    const int j = threadIdx.x & 15;
    const ThreadRotation rot = load_rotation(p.rotation, j);
    float* sq_row = sq[threadIdx.x >> 4];
#pragma unroll 1
    for (int kv = 0; kv < 2; ++kv) {
        if (p.n_bounds[kv] <= 7) store_rows<T, 7>(p, kv, rot, sq_row, j);
        else store_rows<T, 15>(p, kv, rot, sq_row, j);
    }
}

// ---- store variant for large launches: four threads per row -----------------------------------------
//
// A fixed grid (two CTAs per SM) walks the rows: first all K rows (token-major, head-minor), then all V rows.
// Every row's threads write its 64 index bytes and its norm straight into the token's cache slot; the K row of
// head 0 also zeroes the slot's padding.  The arithmetic is that of compress_chunk with 32 elements per thread: thread t of a row owns elements 32t .. 32t + 31 (four
// 16-byte loads for 2-byte inputs, eight rotation blocks, one 16-byte store of packed indices), a warp works
// on eight rows at a time.  The per-row and per-thread overhead (addressing, slot lookup, the exchange for the
// in-order sums, the square root, stores) is spread over four times as many elements as with 16 threads per row.
// In-order sums: the squares go to shared memory as [c][l] (element 8c + l); thread t forms the running sums
// of lanes l = 2t and 2t + 1 over c = 0..15, and every thread then adds the eight lane sums left to right.
constexpr int kWideThreads = 256;
constexpr int kWideRowsPerWarp = 8;
constexpr int kWideRowsPerCta = (kWideThreads / 32) * kWideRowsPerWarp;   // 64
constexpr int kWideSqPitch = 136;            // floats per row of squares: 128 + 8, spreads rows over the banks
constexpr int kWideRotPitch = 132;           // floats per thread slot of rotation blocks: 8 x 16 + 4
constexpr int kWideGrid = 148 * 2;           // the grid walks the rows: two CTAs per SM

template <typename T, int NB>
__device__ __forceinline__ void store_rows_wide(const CompressParams& p, int kv, const float* rot_t, float* sq_row,
                                                int t) {
    float bd[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) bd[b] = __ldg(p.bounds[kv] + b);
    const int H = p.H;
    const SlotLayout lay = slot_layout(H);
    const uint32_t rows = static_cast<uint32_t>(p.num_tokens) * static_cast<uint32_t>(H);
    const uint32_t step = gridDim.x * kWideRowsPerCta;
    const int lane = threadIdx.x & 31;
    const uint32_t first = blockIdx.x * kWideRowsPerCta + (threadIdx.x >> 5) * kWideRowsPerWarp + (lane >> 2);
    const uint32_t warp_first = first - (lane >> 2);
    const T* src = static_cast<const T*>(p.src[kv]);

    // the eight rows of a warp run in lock step (__syncwarp around the exchange): loop on the warp's first row
    for (uint32_t wr = warp_first, r = first; wr < rows; wr += step, r += step) {
        const uint32_t rr = r < rows ? r : 0u;                      // rows past the end compute on row 0, store nothing
        uint32_t token, h;
        if (p.h_shift >= 0) { token = rr >> p.h_shift; h = rr & (H - 1); }
        else { token = rr / H; h = rr - token * H; }
        const T* row_src = src + token * p.token_stride[kv] + static_cast<int64_t>(h) * p.head_stride[kv] + 32 * t;
        const int64_t slot = __ldg(p.slot_mapping + token);
        float x[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) load8<T>(row_src + 8 * c, x + 8 * c);

        // squares, published for the in-order lane sums: sq_row[8 c + l], this thread's c = 4t .. 4t + 3
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float* dst = sq_row + 8 * (4 * t + c);
            *reinterpret_cast<float4*>(dst) = make_float4(__fmul_rn(x[8 * c], x[8 * c]), __fmul_rn(x[8 * c + 1], x[8 * c + 1]),
                                                         __fmul_rn(x[8 * c + 2], x[8 * c + 2]), __fmul_rn(x[8 * c + 3], x[8 * c + 3]));
            *reinterpret_cast<float4*>(dst + 4) = make_float4(__fmul_rn(x[8 * c + 4], x[8 * c + 4]), __fmul_rn(x[8 * c + 5], x[8 * c + 5]),
                                                             __fmul_rn(x[8 * c + 6], x[8 * c + 6]), __fmul_rn(x[8 * c + 7], x[8 * c + 7]));
        }
        __syncwarp();
        float s_even, s_odd;                                        // running sums of lanes 2t and 2t + 1
        {
            const float2 v0 = *reinterpret_cast<const float2*>(sq_row + 2 * t);
            s_even = v0.x; s_odd = v0.y;
#pragma unroll
            for (int c = 1; c < 16; ++c) {
                const float2 v = *reinterpret_cast<const float2*>(sq_row + 8 * c + 2 * t);
                s_even = __fadd_rn(s_even, v.x);
                s_odd = __fadd_rn(s_odd, v.y);
            }
        }
        const int row_lane0 = lane & ~3;
        float tot = __shfl_sync(0xffffffffu, s_even, row_lane0);
        tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, s_odd, row_lane0));
#pragma unroll
        for (int u = 1; u < 4; ++u) {
            tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, s_even, row_lane0 + u));
            tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, s_odd, row_lane0 + u));
        }
        __syncwarp();                                               // sq_row may be rewritten by the next row
        const float norm = __fsqrt_rn(tot);
        const float denom = __fadd_rn(norm, 1e-10f);

        // The 32 IEEE divisions x / denom, through double precision: (float)((double)x * (1.0 / (double)denom)) is
        // the correctly rounded fp32 quotient whenever that quotient is a normal number -- a quotient of two
        // 24-bit significands stays at least 2^-49 (relative) away from every midpoint between adjacent floats,
        // and the double-precision value is within 2^-52 of the exact quotient, so both round the same way;
        // zeros, infinities and NaNs come out as the division gives them.  Quotients in or next to the subnormal
        // range (coarser grid, exact ties possible) take the division instruction itself.  One reciprocal per
        // row and no branch per element: the quotients are independent instruction streams, not 32 basic blocks.
        {
            const double rcp = __ddiv_rn(1.0, static_cast<double>(denom));
            float q[32];
            bool tiny = false;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                q[i] = __double2float_rn(__dmul_rn(static_cast<double>(x[i]), rcp));
                tiny |= fabsf(q[i]) < 0x1p-124f && x[i] != 0.0f;        // (a zero quotient of a nonzero element too)
            }
            if (tiny) {
#pragma unroll
                for (int i = 0; i < 32; ++i) q[i] = __fdiv_rn(x[i], denom);
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = q[i];
        }
        uint32_t words[4];
#pragma unroll
        for (int b = 0; b < 8; ++b) {                               // rotation block 8t + b = elements 4b .. 4b + 3 of x
            const float x0 = x[4 * b], x1 = x[4 * b + 1], x2 = x[4 * b + 2], x3 = x[4 * b + 3];
            uint32_t idx[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const float4 r4 = *reinterpret_cast<const float4*>(rot_t + 16 * b + 4 * jj);
                float acc = __fmul_rn(x0, r4.x);
                acc = __fmaf_rn(x1, r4.y, acc);
                acc = __fmaf_rn(x2, r4.z, acc);
                acc = __fmaf_rn(x3, r4.w, acc);
                idx[jj] = count_below<NB>(bd, acc);
            }
            const uint32_t b0 = (idx[0] << 4) | idx[1];
            const uint32_t b1 = (idx[2] << 4) | idx[3];
            const uint32_t half16 = b0 | (b1 << 8);
            if (b & 1) words[b >> 1] |= half16 << 16;
            else words[b >> 1] = half16;
        }
        if (r < rows && slot >= 0 && slot < p.num_slots) {
            uint8_t* dst = p.cache + slot * p.total_bytes;
            uint8_t* idx_dst = dst + (kv ? lay.v_idx : lay.k_idx) + h * kHalfDim + 16 * t;
            if ((reinterpret_cast<uintptr_t>(idx_dst) & 15u) == 0) {
                *reinterpret_cast<uint4*>(idx_dst) = make_uint4(words[0], words[1], words[2], words[3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) reinterpret_cast<uint32_t*>(idx_dst)[i] = words[i];
            }
            if (t == 0) *reinterpret_cast<float*>(dst + (kv ? lay.v_norm : lay.k_norm) + 4 * h) = norm;
            if (p.write_padding && kv == 0 && h == 0) {
                const int units = (lay.total - lay.payload_end) / 8;
                for (int u = t; u < units; u += 4)
                    *reinterpret_cast<uint2*>(dst + lay.payload_end + 8 * u) = make_uint2(0u, 0u);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kWideThreads, 2)
compress_store_wide_kernel(const CompressParams p) {
    __shared__ __align__(16) float sq[kWideRowsPerCta * kWideSqPitch];
    __shared__ __align__(16) float rot_s[4 * kWideRotPitch];
    // rot_s[t][b][jj][k] = R[4g + jj][4g + k], g = 8t + b
    for (int i = threadIdx.x; i < 512; i += kWideThreads) {
        const int g = i >> 4, jj = (i >> 2) & 3, k = i & 3;
        rot_s[(g >> 3) * kWideRotPitch + (g & 7) * 16 + 4 * jj + k] = __ldg(p.rotation + (4 * g + jj) * kHeadDim + 4 * g + k);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, t = lane & 3;
    float* sq_row = sq + ((threadIdx.x >> 5) * kWideRowsPerWarp + (lane >> 2)) * kWideSqPitch;
    const float* rot_t = rot_s + t * kWideRotPitch;
#pragma unroll 1
    for (int kv = 0; kv < 2; ++kv) {
        if (p.n_bounds[kv] <= 7) store_rows_wide<T, 7>(p, kv, rot_t, sq_row, t);
        else store_rows_wide<T, 15>(p, kv, rot_t, sq_row, t);
    }
}

// Rows variant: x (rows, 128) -> packed (rows, 64) + norms, same walk.
template <typename T, int NB>
__device__ __forceinline__ void plain_rows(const CompressParams& p, const ThreadRotation& rot, float* sq_row, int j) {
    float bd[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) bd[b] = __ldg(p.bounds[0] + b);
    const int64_t rows = p.num_tokens;
    const int64_t step = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + (threadIdx.x >> 4);
    const T* src = static_cast<const T*>(p.src[0]);
    for (int64_t wr = first & ~1ll, r = first; wr < rows; wr += step, r += step) {
        float x[8];
        load8<T>(src + (r < rows ? r : 0) * p.token_stride[0] + 8 * j, x);
        float norm;
        const uint32_t word = compress_chunk<NB>(x, j, sq_row, rot, bd, norm);
        if (r < rows) {
            reinterpret_cast<uint32_t*>(p.packed_out + r * kHalfDim)[j] = word;
            if (j == 0) p.norms_out[r] = norm;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kCompressThreads)
compress_rows_kernel(const CompressParams p) {
    __shared__ __align__(16) float sq[kRowsPerCta][16 * 8];
    const int j = threadIdx.x & 15;
    const ThreadRotation rot = load_rotation(p.rotation, j);
    float* sq_row = sq[threadIdx.x >> 4];
    if (p.n_bounds[0] <= 7) plain_rows<T, 7>(p, rot, sq_row, j);
    else plain_rows<T, 15>(p, rot, sq_row, j);
}

// ---- decompress ------------------------------------------------------------

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Four threads per row; each expands 16 packed bytes into 32 output elements.
template <typename T>
__global__ void decompress_rows_kernel(const uint8_t* __restrict__ packed,
                                       const float* __restrict__ norms, int64_t num_rows,
                                       const float* __restrict__ centroids, int n_centroids,
                                       T* __restrict__ out) {
    __shared__ float cb[16];
    if (threadIdx.x < 16) cb[threadIdx.x] = threadIdx.x < n_centroids ? centroids[threadIdx.x] : 0.f;
    __syncthreads();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t row = i >> 2;
    const int q = static_cast<int>(i & 3);
    if (row >= num_rows) return;
    const uint4 pk = __ldg(reinterpret_cast<const uint4*>(packed + row * kHalfDim) + q);
    const float norm = __ldg(norms + row);
    const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
    T* dst = out + row * kHeadDim + 32 * q;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float f[8];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (w[k] >> (8 * b)) & 0xFFu;
            f[2 * b] = __fmul_rn(cb[byte >> 4], norm);
            f[2 * b + 1] = __fmul_rn(cb[byte & 15u], norm);
        }
        if constexpr (sizeof(T) == 4) {
            reinterpret_cast<float4*>(dst + 8 * k)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(dst + 8 * k)[1] = make_float4(f[4], f[5], f[6], f[7]);
        } else {
            *reinterpret_cast<uint4*>(dst + 8 * k) =
                make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]),
                           pack2<T>(f[6], f[7]));
        }
    }
}

// Paged decompress: the K and V rows of whole cache blocks, picked by a list of physical block
// numbers, straight out of the slot layout.  Four threads per (token, head, K|V) row; thread q expands
// index bytes 16q..16q+15.  Output row of (listed block j, position t, head h): (j * block_size + t) * H + h.
template <typename T>
__global__ void decompress_blocks_kernel(const uint8_t* __restrict__ cache, int total_bytes, int block_size, int H,
                                         const int32_t* __restrict__ blocks, int64_t num_listed, int64_t num_blocks,
                                         const float* __restrict__ cent_k, int n_k, const float* __restrict__ cent_v,
                                         int n_v, T* __restrict__ out_k, T* __restrict__ out_v) {
    __shared__ float cb[2][16];
    if (threadIdx.x < 32) {
        const int kv = threadIdx.x >> 4, i = threadIdx.x & 15;
        cb[kv][i] = i < (kv ? n_v : n_k) ? (kv ? cent_v : cent_k)[i] : 0.f;
    }
    __syncthreads();
    const int64_t rows_per_kind = num_listed * block_size * H;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t r2 = i >> 2;
    const int q = static_cast<int>(i & 3);
    if (r2 >= 2 * rows_per_kind) return;
    const int kind = r2 >= rows_per_kind ? 1 : 0;
    const int64_t r = r2 - kind * rows_per_kind;
    const int h = static_cast<int>(r % H);
    const int64_t tok = r / H;
    const int64_t j = tok / block_size;
    const int pos = static_cast<int>(tok % block_size);
    int64_t blk = blocks != nullptr ? static_cast<int64_t>(__ldg(blocks + j)) : j;
    blk = blk < 0 ? 0 : (blk >= num_blocks ? num_blocks - 1 : blk);
    const SlotLayout lay = slot_layout(H);
    const uint8_t* slot = cache + (blk * block_size + pos) * total_bytes;
    const uint8_t* src = slot + (kind ? lay.v_idx : lay.k_idx) + h * kHalfDim + 16 * q;   // 4-byte aligned at least
    const uint32_t w[4] = {__ldg(reinterpret_cast<const uint32_t*>(src)), __ldg(reinterpret_cast<const uint32_t*>(src) + 1),
                           __ldg(reinterpret_cast<const uint32_t*>(src) + 2), __ldg(reinterpret_cast<const uint32_t*>(src) + 3)};
    const float norm = __ldg(reinterpret_cast<const float*>(slot + (kind ? lay.v_norm : lay.k_norm)) + h);
    const float* c = cb[kind];
    T* dst = (kind ? out_v : out_k) + r * kHeadDim + 32 * q;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float f[8];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (w[k] >> (8 * b)) & 0xFFu;
            f[2 * b] = __fmul_rn(c[byte >> 4], norm);
            f[2 * b + 1] = __fmul_rn(c[byte & 15u], norm);
        }
        if constexpr (sizeof(T) == 4) {
            reinterpret_cast<float4*>(dst + 8 * k)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(dst + 8 * k)[1] = make_float4(f[4], f[5], f[6], f[7]);
        } else {
            *reinterpret_cast<uint4*>(dst + 8 * k) =
                make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]),
                           pack2<T>(f[6], f[7]));
        }
    }
}

// ---- host side -------------------------------------------------------------

static int check_bounds_count(int n, const char* what) {
    if (n != 7 && n != 15) return fail(RQ_ERR_UNSUPPORTED, "%s: %d boundaries (need 7 or 15)", what, n);
    return RQ_OK;
}

template <typename T>
static void launch_store(const CompressParams& p, cudaStream_t st) {
    const int64_t rows = p.num_tokens * p.H;                               // per kind
    if (rows >= kWideFromRows) {
        const int64_t want = (rows + kWideRowsPerCta - 1) / kWideRowsPerCta;
        const unsigned grid = static_cast<unsigned>(want < kWideGrid ? want : kWideGrid);
        compress_store_wide_kernel<T><<<grid, kWideThreads, 0, st>>>(p);
        return;
    }
    const int64_t want = (rows + kRowsPerCta - 1) / kRowsPerCta;
    const unsigned grid = static_cast<unsigned>(want < kCompressGrid ? want : kCompressGrid);
    compress_store_kernel<T><<<grid, kCompressThreads, 0, st>>>(p);
}
template <typename T>
static void launch_rows(const CompressParams& p, cudaStream_t st) {
    const int64_t want = (p.num_tokens + kRowsPerCta - 1) / kRowsPerCta;
    const unsigned grid = static_cast<unsigned>(want < kCompressGrid ? want : kCompressGrid);
    compress_rows_kernel<T><<<grid, kCompressThreads, 0, st>>>(p);
}

}  // namespace rq

using namespace rq;

extern "C" int rq_compress_store(const void* key, const void* value, int in_dtype,
                                 int64_t num_tokens, int num_kv_heads, int head_dim,
                                 int64_t k_token_stride, int64_t k_head_stride,
                                 int64_t v_token_stride, int64_t v_head_stride, uint8_t* kv_cache,
                                 int64_t num_slots, int total_bytes, const int64_t* slot_mapping,
                                 const float* rotation, const float* k_boundaries,
                                 int n_k_boundaries, const float* v_boundaries, int n_v_boundaries,
                                 int write_padding, void* stream) {
    if (num_tokens < 0 || num_kv_heads <= 0 || num_slots < 0)
        return fail(RQ_ERR_INVALID_ARG, "rq_compress_store: negative size");
    if (head_dim != kHeadDim)
        return fail(RQ_ERR_UNSUPPORTED, "rq_compress_store: head_dim %d (only 128)", head_dim);
    if (in_dtype < RQ_DTYPE_F32 || in_dtype > RQ_DTYPE_BF16)
        return fail(RQ_ERR_INVALID_ARG, "rq_compress_store: unknown dtype %d", in_dtype);
    if (total_bytes != num_kv_heads * kSlotPerHead)
        return fail(RQ_ERR_INVALID_ARG, "rq_compress_store: total_bytes %d != %d heads * 256",
                    total_bytes, num_kv_heads);
    if (int e = check_bounds_count(n_k_boundaries, "k_boundaries")) return e;
    if (int e = check_bounds_count(n_v_boundaries, "v_boundaries")) return e;
    if (num_tokens == 0) return RQ_OK;
    if (!key || !value || !kv_cache || !slot_mapping || !rotation || !k_boundaries || !v_boundaries)
        return fail(RQ_ERR_INVALID_ARG, "rq_compress_store: null pointer");
    const int eb = dtype_bytes(in_dtype);
    const int64_t strides[4] = {k_token_stride, k_head_stride, v_token_stride, v_head_stride};
    for (int64_t s : strides)
        if ((s * eb) % 16 != 0)
            return fail(RQ_ERR_ALIGNMENT, "rq_compress_store: stride %lld elements is not 16-byte aligned",
                        static_cast<long long>(s));
    if (!aligned(key, 16) || !aligned(value, 16) || !aligned(kv_cache, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_compress_store: key/value/kv_cache must be 16-byte aligned");
    if (num_tokens * num_kv_heads >= 0x3fffffffLL)
        return fail(RQ_ERR_UNSUPPORTED, "rq_compress_store: too many rows for one launch");

    CompressParams p{};
    p.src[0] = key; p.src[1] = value;
    p.token_stride[0] = k_token_stride; p.token_stride[1] = v_token_stride;
    p.head_stride[0] = k_head_stride; p.head_stride[1] = v_head_stride;
    p.num_tokens = num_tokens; p.H = num_kv_heads;
    p.h_shift = -1;
    for (int sft = 0; sft < 16; ++sft)
        if ((1 << sft) == num_kv_heads) p.h_shift = sft;
    p.cache = kv_cache; p.num_slots = num_slots; p.total_bytes = total_bytes;
    p.slot_mapping = slot_mapping; p.write_padding = write_padding;
    p.rotation = rotation;
    p.bounds[0] = k_boundaries; p.bounds[1] = v_boundaries;
    p.n_bounds[0] = n_k_boundaries; p.n_bounds[1] = n_v_boundaries;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case RQ_DTYPE_F32: launch_store<float>(p, st); break;
        case RQ_DTYPE_F16: launch_store<__half>(p, st); break;
        default: launch_store<__nv_bfloat16>(p, st); break;
    }
    return check_cuda(cudaGetLastError(), "rq_compress_store launch");
}

extern "C" int rq_compress(const void* x, int in_dtype, int64_t num_rows, int head_dim,
                           int64_t row_stride, const float* rotation, const float* boundaries,
                           int n_boundaries, uint8_t* packed_out, float* norms_out, void* stream) {
    if (num_rows < 0) return fail(RQ_ERR_INVALID_ARG, "rq_compress: negative size");
    if (head_dim != kHeadDim)
        return fail(RQ_ERR_UNSUPPORTED, "rq_compress: head_dim %d (only 128)", head_dim);
    if (in_dtype < RQ_DTYPE_F32 || in_dtype > RQ_DTYPE_BF16)
        return fail(RQ_ERR_INVALID_ARG, "rq_compress: unknown dtype %d", in_dtype);
    if (int e = check_bounds_count(n_boundaries, "boundaries")) return e;
    if (num_rows == 0) return RQ_OK;
    if (!x || !rotation || !boundaries || !packed_out || !norms_out)
        return fail(RQ_ERR_INVALID_ARG, "rq_compress: null pointer");
    if ((row_stride * dtype_bytes(in_dtype)) % 16 != 0 || !aligned(x, 16) || !aligned(packed_out, 4))
        return fail(RQ_ERR_ALIGNMENT, "rq_compress: rows must be 16-byte aligned");
    CompressParams p{};
    p.src[0] = x; p.token_stride[0] = row_stride; p.num_tokens = num_rows;
    p.packed_out = packed_out; p.norms_out = norms_out; p.rotation = rotation;
    p.bounds[0] = boundaries; p.n_bounds[0] = n_boundaries;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case RQ_DTYPE_F32: launch_rows<float>(p, st); break;
        case RQ_DTYPE_F16: launch_rows<__half>(p, st); break;
        default: launch_rows<__nv_bfloat16>(p, st); break;
    }
    return check_cuda(cudaGetLastError(), "rq_compress launch");
}

extern "C" int rq_decompress(const uint8_t* packed, const float* norms, int64_t num_rows,
                             int head_dim, const float* centroids, int n_centroids, void* out,
                             int out_dtype, void* stream) {
    if (num_rows < 0) return fail(RQ_ERR_INVALID_ARG, "rq_decompress: negative size");
    if (head_dim != kHeadDim)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decompress: head_dim %d (only 128)", head_dim);
    if (n_centroids != 8 && n_centroids != 16)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decompress: %d centroids (need 8 or 16)", n_centroids);
    if (out_dtype < RQ_DTYPE_F32 || out_dtype > RQ_DTYPE_BF16)
        return fail(RQ_ERR_INVALID_ARG, "rq_decompress: unknown dtype %d", out_dtype);
    if (num_rows == 0) return RQ_OK;
    if (!packed || !norms || !centroids || !out)
        return fail(RQ_ERR_INVALID_ARG, "rq_decompress: null pointer");
    if (!aligned(packed, 16) || !aligned(out, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_decompress: packed and out must be 16-byte aligned");
    const int threads = 256;
    const unsigned grid = static_cast<unsigned>((num_rows * 4 + threads - 1) / threads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
        case RQ_DTYPE_F32:
            decompress_rows_kernel<float><<<grid, threads, 0, st>>>(
                packed, norms, num_rows, centroids, n_centroids, static_cast<float*>(out));
            break;
        case RQ_DTYPE_F16:
            decompress_rows_kernel<__half><<<grid, threads, 0, st>>>(
                packed, norms, num_rows, centroids, n_centroids, static_cast<__half*>(out));
            break;
        default:
            decompress_rows_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(
                packed, norms, num_rows, centroids, n_centroids, static_cast<__nv_bfloat16*>(out));
            break;
    }
    return check_cuda(cudaGetLastError(), "rq_decompress launch");
}

extern "C" int rq_decompress_blocks(const uint8_t* kv_cache, int64_t num_blocks, int block_size, int total_bytes,
                                    int num_kv_heads, int head_dim, const int32_t* blocks, int64_t num_listed,
                                    const float* centroids_k, int n_centroids_k, const float* centroids_v,
                                    int n_centroids_v, void* out_k, void* out_v, int out_dtype, void* stream) {
    if (num_blocks < 0 || block_size <= 0 || num_kv_heads <= 0 || num_listed < 0)
        return fail(RQ_ERR_INVALID_ARG, "rq_decompress_blocks: negative or zero size");
    if (head_dim != kHeadDim)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decompress_blocks: head_dim %d (only 128)", head_dim);
    if (total_bytes != num_kv_heads * kSlotPerHead)
        return fail(RQ_ERR_INVALID_ARG, "rq_decompress_blocks: total_bytes %d != %d heads * 256", total_bytes,
                    num_kv_heads);
    if ((n_centroids_k != 8 && n_centroids_k != 16) || (n_centroids_v != 8 && n_centroids_v != 16))
        return fail(RQ_ERR_UNSUPPORTED, "rq_decompress_blocks: codebooks must have 8 or 16 centroids");
    if (out_dtype < RQ_DTYPE_F32 || out_dtype > RQ_DTYPE_BF16)
        return fail(RQ_ERR_INVALID_ARG, "rq_decompress_blocks: unknown dtype %d", out_dtype);
    if (num_listed == 0) return RQ_OK;
    if (num_blocks == 0) return fail(RQ_ERR_INVALID_ARG, "rq_decompress_blocks: blocks listed but the cache is empty");
    if (!kv_cache || !centroids_k || !centroids_v || !out_k || !out_v)
        return fail(RQ_ERR_INVALID_ARG, "rq_decompress_blocks: null pointer");
    if (!aligned(kv_cache, 16) || !aligned(out_k, 16) || !aligned(out_v, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_decompress_blocks: kv_cache and outputs must be 16-byte aligned");
    const int threads = 256;
    const int64_t work = 2 * num_listed * block_size * num_kv_heads * 4;
    if ((work + threads - 1) / threads > 0x7fffffffLL)
        return fail(RQ_ERR_UNSUPPORTED, "rq_decompress_blocks: too many rows for one launch");
    const unsigned grid = static_cast<unsigned>((work + threads - 1) / threads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (out_dtype) {
        case RQ_DTYPE_F32:
            decompress_blocks_kernel<float><<<grid, threads, 0, st>>>(
                kv_cache, total_bytes, block_size, num_kv_heads, blocks, num_listed, num_blocks, centroids_k,
                n_centroids_k, centroids_v, n_centroids_v, static_cast<float*>(out_k), static_cast<float*>(out_v));
            break;
        case RQ_DTYPE_F16:
            decompress_blocks_kernel<__half><<<grid, threads, 0, st>>>(
                kv_cache, total_bytes, block_size, num_kv_heads, blocks, num_listed, num_blocks, centroids_k,
                n_centroids_k, centroids_v, n_centroids_v, static_cast<__half*>(out_k), static_cast<__half*>(out_v));
            break;
        default:
            decompress_blocks_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(
                kv_cache, total_bytes, block_size, num_kv_heads, blocks, num_listed, num_blocks, centroids_k,
                n_centroids_k, centroids_v, n_centroids_v, static_cast<__nv_bfloat16*>(out_k),
                static_cast<__nv_bfloat16*>(out_v));
            break;
    }
    return check_cuda(cudaGetLastError(), "rq_decompress_blocks launch");
}
