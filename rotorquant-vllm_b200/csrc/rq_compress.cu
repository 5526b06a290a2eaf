// Compress-on-cache-write for RotorQuant (IsoQuant / PlanarQuant), sm_100a.
//
// One pass over the new tokens: L2 norm, normalise, block-diagonal rotation,
// boundary bucketize, nibble pack, and the scatter of whole cache slots.
// Replaces the reference's per-row Triton kernel (triton/isoquant_compress.py:16-96) plus the
// row assembly and scatter in RQAttentionImpl._compress_and_store (vllm/rq_backend.py:585-657).
//
// Bit-exactness.  The bytes must equal the reference's PyTorch path
// (triton/isoquant_compress.py:161-190), so every row is evaluated by ONE thread with the
// IEEE-754 operations of that path in their order:
//   norm   : eight running sums s_l += x[8c+l]^2 (multiply and add rounded separately,
//            c ascending), combined left to right, correctly rounded sqrt
//   divide : x / (norm + 1e-10f), IEEE division
//   rotate : out_j = fma(x3,R[j][3], fma(x2,R[j][2], fma(x1,R[j][1], x0*R[j][0]))) per 4x4 block
//   bucket : number of boundaries strictly below the value
// Rows are staged through shared memory so that global loads and the slot stores are
// coalesced 16-byte accesses although the arithmetic is thread-per-row.
#include "rq_common.cuh"

namespace rq {

constexpr int kCompressThreads = 128;       // rows per CTA pass
constexpr int kRowPitch = kHeadDim + 4;     // floats; +4 keeps float4 reads conflict-free

struct CompressParams {
    const void* src[2];          // key, value (or x, unused)
    int64_t token_stride[2];     // elements
    int64_t head_stride[2];      // elements
    int64_t num_tokens;
    int H;
    // cache destination (store variant)
    uint8_t* cache;
    int64_t num_slots;
    int total_bytes;
    const int64_t* slot_mapping;
    int write_padding;
    int tokens_per_cta;
    // plain-row destination (rows variant)
    uint8_t* packed_out;
    float* norms_out;
    // parameters
    const float* rotation;       // dense 128x128
    const float* bounds[2];
    int n_bounds[2];
};

// Compress one row held in shared memory as 128 floats.
__device__ __forceinline__ void compress_row(const float* __restrict__ x,
                                             const float* __restrict__ rot,   // [32][4][4]
                                             const float* __restrict__ bnd, int nb,
                                             uint32_t* packed, bool vec16, float& norm_out) {
    float s[8];
#pragma unroll
    for (int l = 0; l < 8; ++l) s[l] = 0.0f;
#pragma unroll 4
    for (int c = 0; c < kHeadDim / 8; ++c) {
        const float4 a = *reinterpret_cast<const float4*>(x + 8 * c);
        const float4 b = *reinterpret_cast<const float4*>(x + 8 * c + 4);
        s[0] = __fadd_rn(s[0], __fmul_rn(a.x, a.x));
        s[1] = __fadd_rn(s[1], __fmul_rn(a.y, a.y));
        s[2] = __fadd_rn(s[2], __fmul_rn(a.z, a.z));
        s[3] = __fadd_rn(s[3], __fmul_rn(a.w, a.w));
        s[4] = __fadd_rn(s[4], __fmul_rn(b.x, b.x));
        s[5] = __fadd_rn(s[5], __fmul_rn(b.y, b.y));
        s[6] = __fadd_rn(s[6], __fmul_rn(b.z, b.z));
        s[7] = __fadd_rn(s[7], __fmul_rn(b.w, b.w));
    }
    float tot = s[0];
#pragma unroll
    for (int l = 1; l < 8; ++l) tot = __fadd_rn(tot, s[l]);
    const float norm = __fsqrt_rn(tot);
    norm_out = norm;
    const float denom = __fadd_rn(norm, 1e-10f);

#pragma unroll 1
    for (int i = 0; i < 4; ++i) {               // 16 output bytes = 8 blocks of four values
        uint32_t words[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {           // one 32-bit word = two blocks = 8 indices
            uint32_t word = 0;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int g = 8 * i + 2 * w + half;
                const float4 xv = *reinterpret_cast<const float4*>(x + 4 * g);
                const float x0 = __fdiv_rn(xv.x, denom), x1 = __fdiv_rn(xv.y, denom);
                const float x2 = __fdiv_rn(xv.z, denom), x3 = __fdiv_rn(xv.w, denom);
                uint32_t idx[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 r = *reinterpret_cast<const float4*>(rot + g * 16 + j * 4);
                    float acc = __fmul_rn(x0, r.x);
                    acc = __fmaf_rn(x1, r.y, acc);
                    acc = __fmaf_rn(x2, r.z, acc);
                    acc = __fmaf_rn(x3, r.w, acc);
                    uint32_t n = 0;
                    for (int b = 0; b < nb; ++b) n += (bnd[b] < acc) ? 1u : 0u;
                    idx[j] = n > 15u ? 15u : n;
                }
                const uint32_t b0 = (idx[0] << 4) | idx[1];
                const uint32_t b1 = (idx[2] << 4) | idx[3];
                word |= (b0 | (b1 << 8)) << (16 * half);
            }
            words[w] = word;
        }
        // The V index region of a slot starts at H*68 bytes: 16-byte aligned only when H % 4 == 0.
        if (vec16) {
            reinterpret_cast<uint4*>(packed)[i] = make_uint4(words[0], words[1], words[2], words[3]);
        } else {
#pragma unroll
            for (int w = 0; w < 4; ++w) packed[4 * i + w] = words[w];
        }
    }
}

// Shared-memory carve-up (dynamic): rotation blocks, boundaries, row tile, slot images.
struct CompressSmem {
    float* rot;      // 32*16
    float* bnd;      // 2*16
    float* rows;     // kCompressThreads * kRowPitch
    uint8_t* stage;  // tokens_per_cta * total_bytes   (store variant only)
};
__device__ __forceinline__ CompressSmem carve(uint8_t* base) {
    CompressSmem s;
    s.rot = reinterpret_cast<float*>(base);
    s.bnd = s.rot + 32 * 16;
    s.rows = s.bnd + 32;
    s.stage = reinterpret_cast<uint8_t*>(s.rows + kCompressThreads * kRowPitch);
    return s;
}
static size_t compress_smem_bytes(int stage_bytes) {
    return sizeof(float) * (32 * 16 + 32 + kCompressThreads * kRowPitch) + stage_bytes;
}

__device__ __forceinline__ void load_params(const CompressParams& p, CompressSmem& sm) {
    for (int i = threadIdx.x; i < 32 * 16; i += blockDim.x) {
        const int g = i >> 4, j = (i >> 2) & 3, k = i & 3;
        sm.rot[i] = __ldg(p.rotation + (4 * g + j) * kHeadDim + 4 * g + k);
    }
    for (int i = threadIdx.x; i < 32; i += blockDim.x) {
        const int kv = i >> 4, b = i & 15;
        sm.bnd[i] = (p.bounds[kv] != nullptr && b < p.n_bounds[kv]) ? __ldg(p.bounds[kv] + b)
                                                                     : __int_as_float(0x7f800000);
    }
}

// Copy `rows_used` rows of 128 elements into the fp32 row tile with 16-byte global loads.
// row_src(r) returns the global address of row r or nullptr for a row that does not exist.
template <typename T, typename RowSrc>
__device__ __forceinline__ void stage_rows(float* rows, int rows_used, RowSrc row_src) {
    constexpr int E = Chunk16<T>::kElems;
    constexpr int CH = kHeadDim / E;
    for (int i = threadIdx.x; i < rows_used * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        const T* src = row_src(r);
        if (src == nullptr) continue;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + c * E));
        float f[E];
        Chunk16<T>::unpack(v, f);
        float* dst = rows + r * kRowPitch + c * E;
#pragma unroll
        for (int e = 0; e < E; e += 4)
            *reinterpret_cast<float4*>(dst + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kCompressThreads)
compress_store_kernel(const CompressParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    CompressSmem sm = carve(smem_raw);
    const int H = p.H;
    const int tpc = p.tokens_per_cta;
    const SlotLayout lay = slot_layout(H);
    const int64_t t0 = static_cast<int64_t>(blockIdx.x) * tpc;
    const int n_tok = static_cast<int>(min(static_cast<int64_t>(tpc), p.num_tokens - t0));

    load_params(p, sm);
    if (p.write_padding) {   // the tail of every slot image is zero
        const int pad = lay.total - lay.payload_end;
        for (int i = threadIdx.x; i < n_tok * (pad / 8); i += blockDim.x) {
            const int tl = i / (pad / 8), o = i % (pad / 8);
            *reinterpret_cast<uint2*>(sm.stage + tl * lay.total + lay.payload_end + 8 * o) =
                make_uint2(0u, 0u);
        }
    }

    // Rows of this CTA, K rows first: r = kv * (n_tok*H) + tl*H + h; passes of 128 rows.
    const int rows_total = 2 * n_tok * H;
    for (int r0 = 0; r0 < rows_total; r0 += kCompressThreads) {
        const int rows_used = min(kCompressThreads, rows_total - r0);
        __syncthreads();
        stage_rows<T>(sm.rows, rows_used, [&](int r) -> const T* {
            const int rr = r0 + r;
            const int kv = rr / (n_tok * H), rem = rr % (n_tok * H);
            const int tl = rem / H, h = rem % H;
            return static_cast<const T*>(p.src[kv]) + (t0 + tl) * p.token_stride[kv] +
                   static_cast<int64_t>(h) * p.head_stride[kv];
        });
        __syncthreads();
        if (threadIdx.x < rows_used) {
            const int rr = r0 + threadIdx.x;
            const int kv = rr / (n_tok * H), rem = rr % (n_tok * H);
            const int tl = rem / H, h = rem % H;
            float norm;
            uint8_t* slot = sm.stage + tl * lay.total;
            uint32_t* dst = reinterpret_cast<uint32_t*>(slot + (kv ? lay.v_idx : lay.k_idx) + h * kHalfDim);
            compress_row(sm.rows + threadIdx.x * kRowPitch, sm.rot, sm.bnd + 16 * kv,
                         p.n_bounds[kv], dst, (lay.v_idx % 16) == 0, norm);
            *reinterpret_cast<float*>(slot + (kv ? lay.v_norm : lay.k_norm) + 4 * h) = norm;
        }
    }
    __syncthreads();

    // Scatter whole slot images with coalesced 8-byte stores.
    const int nbytes = p.write_padding ? lay.total : lay.payload_end;
    const int units = nbytes / 8;
    for (int i = threadIdx.x; i < n_tok * units; i += blockDim.x) {
        const int tl = i / units, o = i % units;
        const int64_t slot = __ldg(p.slot_mapping + t0 + tl);
        if (slot < 0 || slot >= p.num_slots) continue;
        const uint2 v = *reinterpret_cast<const uint2*>(sm.stage + tl * lay.total + 8 * o);
        *reinterpret_cast<uint2*>(p.cache + slot * p.total_bytes + 8 * o) = v;
    }
}

template <typename T>
__global__ void __launch_bounds__(kCompressThreads)
compress_rows_kernel(const CompressParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    CompressSmem sm = carve(smem_raw);
    load_params(p, sm);
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * kCompressThreads;
    const int64_t left = p.num_tokens - r0;
    const int rows_used = left < kCompressThreads ? static_cast<int>(left) : kCompressThreads;
    stage_rows<T>(sm.rows, rows_used, [&](int r) -> const T* {
        return static_cast<const T*>(p.src[0]) + (r0 + r) * p.token_stride[0];
    });
    __syncthreads();
    if (threadIdx.x < rows_used) {
        float norm;
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.packed_out + (r0 + threadIdx.x) * kHalfDim);
        compress_row(sm.rows + threadIdx.x * kRowPitch, sm.rot, sm.bnd, p.n_bounds[0], dst, true, norm);
        p.norms_out[r0 + threadIdx.x] = norm;
    }
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

// ---- host side -------------------------------------------------------------

static int check_bounds_count(int n, const char* what) {
    if (n != 7 && n != 15) return fail(RQ_ERR_UNSUPPORTED, "%s: %d boundaries (need 7 or 15)", what, n);
    return RQ_OK;
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

    CompressParams p{};
    p.src[0] = key; p.src[1] = value;
    p.token_stride[0] = k_token_stride; p.token_stride[1] = v_token_stride;
    p.head_stride[0] = k_head_stride; p.head_stride[1] = v_head_stride;
    p.num_tokens = num_tokens; p.H = num_kv_heads;
    p.cache = kv_cache; p.num_slots = num_slots; p.total_bytes = total_bytes;
    p.slot_mapping = slot_mapping; p.write_padding = write_padding;
    p.rotation = rotation;
    p.bounds[0] = k_boundaries; p.bounds[1] = v_boundaries;
    p.n_bounds[0] = n_k_boundaries; p.n_bounds[1] = n_v_boundaries;
    int tpc = kCompressThreads / (2 * num_kv_heads);
    if (tpc < 1) tpc = 1;
    p.tokens_per_cta = tpc;
    const size_t smem = compress_smem_bytes(tpc * total_bytes);
    if (smem > 200 * 1024)
        return fail(RQ_ERR_UNSUPPORTED, "rq_compress_store: %d KV heads need too much shared memory",
                    num_kv_heads);
    const unsigned grid = static_cast<unsigned>((num_tokens + tpc - 1) / tpc);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case RQ_DTYPE_F32:
            if (int e = ensure_smem(compress_store_kernel<float>, smem)) return e;
            compress_store_kernel<float><<<grid, kCompressThreads, smem, st>>>(p);
            break;
        case RQ_DTYPE_F16:
            if (int e = ensure_smem(compress_store_kernel<__half>, smem)) return e;
            compress_store_kernel<__half><<<grid, kCompressThreads, smem, st>>>(p);
            break;
        default:
            if (int e = ensure_smem(compress_store_kernel<__nv_bfloat16>, smem)) return e;
            compress_store_kernel<__nv_bfloat16><<<grid, kCompressThreads, smem, st>>>(p);
            break;
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
    if ((row_stride * dtype_bytes(in_dtype)) % 16 != 0 || !aligned(x, 16) || !aligned(packed_out, 16))
        return fail(RQ_ERR_ALIGNMENT, "rq_compress: rows and packed_out must be 16-byte aligned");
    CompressParams p{};
    p.src[0] = x; p.token_stride[0] = row_stride; p.num_tokens = num_rows;
    p.packed_out = packed_out; p.norms_out = norms_out; p.rotation = rotation;
    p.bounds[0] = boundaries; p.n_bounds[0] = n_boundaries;
    const size_t smem = compress_smem_bytes(0);
    const unsigned grid = static_cast<unsigned>((num_rows + kCompressThreads - 1) / kCompressThreads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
        case RQ_DTYPE_F32:
            if (int e = ensure_smem(compress_rows_kernel<float>, smem)) return e;
            compress_rows_kernel<float><<<grid, kCompressThreads, smem, st>>>(p);
            break;
        case RQ_DTYPE_F16:
            if (int e = ensure_smem(compress_rows_kernel<__half>, smem)) return e;
            compress_rows_kernel<__half><<<grid, kCompressThreads, smem, st>>>(p);
            break;
        default:
            if (int e = ensure_smem(compress_rows_kernel<__nv_bfloat16>, smem)) return e;
            compress_rows_kernel<__nv_bfloat16><<<grid, kCompressThreads, smem, st>>>(p);
            break;
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
