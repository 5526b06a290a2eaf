/*
 * rq_b200.h -- C ABI of librq_b200.so: the RotorQuant KV-cache hot path for
 * NVIDIA B200 (sm_100a).
 *
 * Every entry point replaces one Python/Triton launcher of the reference
 * project (tpurtell/rotorquant-vllm, paths relative to its root).  All
 * pointers are raw device pointers owned by the caller unless stated
 * otherwise; the library allocates nothing, never synchronises the host and
 * only enqueues work on `stream` (a cudaStream_t passed as void*).  Functions
 * return RQ_OK (0) or a negative rq_status; rq_last_error() gives the message
 * of the last failure on the calling thread.
 *
 * Cache layout (src/rotorquant_vllm/vllm/rq_backend.py:155-188, :484-490):
 * uint8 (num_blocks, block_size, total_bytes), one slot per token:
 *
 *   [0, H*64)        K indices, 64 B per head: byte j = idx[2j] << 4 | idx[2j+1]
 *   [H*64, H*68)     K norms, fp32 little endian
 *   [H*68, H*132)    V indices
 *   [H*132, H*136)   V norms
 *   [H*136, H*256)   zero padding           total_bytes = H * 256  (head_dim 128)
 *
 * The rotation is passed the way the reference passes it: the dense row-major
 * (head_dim x head_dim) fp32 matrix R.  It must be block diagonal with 4x4
 * blocks (IsoQuant) or 2x2 blocks (PlanarQuant); only the 4x4 diagonal blocks
 * are read.
 */
#ifndef RQ_B200_H
#define RQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    RQ_OK = 0,
    RQ_ERR_INVALID_ARG = -1,  /* null pointer, negative size, inconsistent shapes      */
    RQ_ERR_UNSUPPORTED = -2,  /* head_dim != 128, bits not 3/4, group size > 16, ...    */
    RQ_ERR_ALIGNMENT = -3,    /* a pointer or stride breaks the stated alignment        */
    RQ_ERR_WORKSPACE = -4,    /* workspace missing or too small                         */
    RQ_ERR_CUDA = -5          /* a CUDA runtime call failed; message has the CUDA text  */
} rq_status;

typedef enum { RQ_DTYPE_F32 = 0, RQ_DTYPE_F16 = 1, RQ_DTYPE_BF16 = 2 } rq_dtype;

/* Library identification, e.g. "rq_b200 0.1 (sm_100a)". */
const char* rq_version(void);

/* Message of the most recent failure on this thread ("" if none). */
const char* rq_last_error(void);

/*
 * Compress new K and V tokens and write whole slots into the paged cache.
 * Replaces RQAttentionImpl._compress_and_store (vllm/rq_backend.py:585-657),
 * i.e. two iso_compress / planar_compress launches
 * (triton/isoquant_compress.py:104-158, triton/planarquant_compress.py:100-154)
 * plus the row assembly and scatter.  Bytes and norms equal the reference's
 * PyTorch path (triton/isoquant_compress.py:161-190) bit for bit.
 *
 *   key, value     (num_tokens, H, 128) in `in_dtype`, last dim contiguous; strides in elements;
 *                  rows must start on 16-byte boundaries
 *   slot_mapping   int64[num_tokens]: flat slot = block * block_size + offset; negative = skip
 *   boundaries     ascending fp32 Lloyd-Max boundaries, 7 (3-bit) or 15 (4-bit) entries
 *   write_padding  non-zero: zero bytes [H*136, H*256) of each written slot (reference behaviour)
 */
int rq_compress_store(const void* key, const void* value, int in_dtype, int64_t num_tokens,
                      int num_kv_heads, int head_dim, int64_t k_token_stride,
                      int64_t k_head_stride, int64_t v_token_stride, int64_t v_head_stride,
                      uint8_t* kv_cache, int64_t num_slots, int total_bytes,
                      const int64_t* slot_mapping, const float* rotation,
                      const float* k_boundaries, int n_k_boundaries, const float* v_boundaries,
                      int n_v_boundaries, int write_padding, void* stream);

/*
 * Compress rows without the cache: x (num_rows, 128) -> packed (num_rows, 64) uint8 and
 * norms (num_rows) fp32.  Replaces iso_compress / planar_compress
 * (triton/isoquant_compress.py:104-158, triton/planarquant_compress.py:100-154).
 */
int rq_compress(const void* x, int in_dtype, int64_t num_rows, int head_dim, int64_t row_stride,
                const float* rotation, const float* boundaries, int n_boundaries,
                uint8_t* packed_out, float* norms_out, void* stream);

/*
 * Decompress rows: packed (num_rows, 64) + norms (num_rows) -> out (num_rows, 128) in out_dtype,
 * centroid[idx] * norm rounded once; stays in rotated space.  Replaces iso_decompress /
 * planar_decompress (triton/isoquant_decompress.py:63-100, triton/planarquant_decompress.py:63-101).
 */
int rq_decompress(const uint8_t* packed, const float* norms, int64_t num_rows, int head_dim,
                  const float* centroids, int n_centroids, void* out, int out_dtype,
                  void* stream);

/*
 * Paged decompress: K and V of whole cache blocks, read straight from the slot layout.  Replaces the
 * gather + per-head slicing + two decompress launches of RQAttentionImpl._decompress_cache_paged
 * (vllm/rq_backend.py:737-852, the part after torch.unique) and of _decompress_cache (:663-735).
 *
 *   blocks        int32[num_listed] physical block numbers (device), or NULL for blocks 0..num_listed-1
 *   out_k, out_v  (num_listed, block_size, H, 128) in out_dtype: centroid[idx] * norm rounded once,
 *                 rotated space; 16-byte aligned
 */
int rq_decompress_blocks(const uint8_t* kv_cache, int64_t num_blocks, int block_size, int total_bytes,
                         int num_kv_heads, int head_dim, const int32_t* blocks, int64_t num_listed,
                         const float* centroids_k, int n_centroids_k, const float* centroids_v,
                         int n_centroids_v, void* out_k, void* out_v, int out_dtype, void* stream);

/*
 * Scratch bytes rq_decode needs for `num_splits` context splits (0 = let the library choose
 * from max_seq_len; the same choice rq_decode makes).
 */
size_t rq_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                 int max_seq_len, int num_splits);

/*
 * Fused paged decode attention, one query token per sequence.  Replaces
 * fused_paged_rq_decode (triton/fused_paged_rq_decode.py:214-312) including the two dense
 * rotations around the kernel (:271, :308): q is rotated by R^T, attention runs in rotated
 * space over centroid[idx] * norm, the result is rotated back by R.
 *
 *   q, out        (num_seqs, H_Q, 128) in `dtype` (f16 or bf16); strides in elements
 *   block_table   int32 (num_seqs, >= ceil(seq_len / block_size)), row stride in elements
 *   seq_lens      int32[num_seqs]; 0 gives a zero output row
 *   max_seq_len   upper bound of seq_lens (host value; sizes the grid, never read from device)
 *   workspace     >= rq_decode_workspace_bytes(...) bytes, 16-byte aligned
 *   num_splits    context splits per sequence, 0 = automatic
 *
 * Every device-side wait of the kernels (mbarriers of TMA copies and tcgen05 MMAs) is bounded to
 * about one second of SM clocks; if one expires the affected outputs are NaN and the kernels return.
 */
int rq_decode(const void* q, void* out, int dtype, int64_t q_stride_seq, int64_t q_stride_head,
              int64_t o_stride_seq, int64_t o_stride_head, int num_seqs, int num_q_heads,
              int num_kv_heads, int head_dim, const uint8_t* kv_cache, int64_t num_blocks,
              int block_size, int total_bytes, const int32_t* block_table,
              int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
              int n_centroids_k, const float* centroids_v, int n_centroids_v,
              const float* rotation, float sm_scale, int max_seq_len, void* workspace,
              size_t workspace_bytes, int num_splits, void* stream);

/*
 * Head-sharded decode for tensor parallelism: rq_decode on this GPU's KV heads whose merge kernel stores
 * every output row into `num_peers` buffers (host array of device pointers; one per GPU of the group, the
 * calling GPU's own among them; peer buffers are memory of other GPUs mapped into this process, e.g.
 * symmetric memory), at the offsets `o_stride_*` describe.  Each pointer addresses the place of THIS GPU's
 * heads inside that GPU's gathered buffer.  Plain stores over NVLink; nothing else differs from rq_decode
 * (same workspace, same bounded waits).  Follow it with rq_peer_barrier on every GPU of the group, and
 * alternate between two gathered buffers from step to step: a GPU may be one step ahead of a peer that
 * still reads the previous step's buffer.
 * No counterpart in the reference; replaces "decode + all-gather of the attention outputs" of a tensor-
 * parallel layer (vLLM runs that collective itself after the backend returns).
 */
int rq_decode_sharded(const void* q, int dtype, int64_t q_stride_seq, int64_t q_stride_head,
                      int64_t o_stride_seq, int64_t o_stride_head, int num_seqs, int num_q_heads,
                      int num_kv_heads, int head_dim, const uint8_t* kv_cache, int64_t num_blocks,
                      int block_size, int total_bytes, const int32_t* block_table,
                      int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
                      int n_centroids_k, const float* centroids_v, int n_centroids_v,
                      const float* rotation, float sm_scale, int max_seq_len, void* workspace,
                      size_t workspace_bytes, int num_splits, void* const* peer_out, int num_peers,
                      void* stream);

/*
 * Arrive-and-wait of the GPUs of a group, enqueued on `stream` after rq_decode_sharded: one warp writes this
 * GPU's step number into slot `rank` of every GPU's flag array and waits until all `world` slots of its own
 * array have reached it.  `peer_flags` is a host array of `world` device pointers (uint64[world] each, zeroed
 * once, this GPU's own array at index `rank`), `state` two uint64 on this GPU, zeroed once: state[0] counts
 * the steps, state[1] becomes 1 when a wait ran out.  The wait is bounded by `limit_cycles` SM clocks (0 =
 * about one second); on expiry the kernel records it and returns, it never traps.  Step numbers live on the
 * device, so the call can be captured in a CUDA graph.  No counterpart in the reference.
 */
int rq_peer_barrier(void* const* peer_flags, int world, int rank, void* state, long long limit_cycles,
                    void* stream);

/*
 * rq_decode for callers that cannot supply a workspace.  It has no counterpart in the reference.
 *
 * Who needs it: a caller that is unable to obtain device memory of its own when the decode call
 * is made -- for example a serving process that handed all free HBM to its KV-cache pool at
 * start-up and may not allocate afterwards, or a host runtime that bans allocator calls on its
 * request path.  The scratch lives in a fixed area of RQ_DECODE_STATIC_SCRATCH_BYTES bytes inside
 * the library image; every GPU that loads the library holds that area until the process exits.
 * The function calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * Arguments and results are those of rq_decode without `workspace` / `workspace_bytes`.
 *   - A call whose partial results need more than RQ_DECODE_STATIC_SCRATCH_BYTES (16 MiB; see
 *     rq_decode_workspace_bytes) is rejected with RQ_ERR_WORKSPACE; nothing is launched.
 *   - The first call on each device looks up the device address of the area
 *     (cudaGetSymbolAddress, with that device current).  Make that first call before any stream
 *     capture on the device.
 *   - All calls on a device share the one area, which keeps the previous call's contents.  The
 *     kernels write every scratch entry before they read it, so nothing needs clearing, but two
 *     calls that overlap on the GPU (different streams) race on it: keep them on one stream or
 *     order them yourself.
 */
#define RQ_DECODE_STATIC_SCRATCH_BYTES (16u << 20)
int rq_decode_static_scratch(const void* q, void* out, int dtype, int64_t q_stride_seq,
                             int64_t q_stride_head, int64_t o_stride_seq, int64_t o_stride_head,
                             int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                             const uint8_t* kv_cache, int64_t num_blocks, int block_size,
                             int total_bytes, const int32_t* block_table,
                             int64_t block_table_stride, const int32_t* seq_lens,
                             const float* centroids_k, int n_centroids_k,
                             const float* centroids_v, int n_centroids_v, const float* rotation,
                             float sm_scale, int max_seq_len, int num_splits, void* stream);

/*
 * Fused paged INT8 prefill attention: causal attention of new query tokens over the compressed
 * cache (which already holds those tokens).  Replaces fused_paged_rq_int8_prefill
 * (triton/fused_paged_rq_int8_prefill.py:247-363) including its two rotations (:322, :359).
 * QK^T runs on the tcgen05 INT8 tensor path with one scale per query row and per key, PV on the
 * tcgen05 16-bit path; both accumulate in tensor memory.
 *
 *   q, out         (num_tokens, H_Q, 128) in `dtype` (f16 or bf16); strides in elements
 *   cu_seqlens_q   int32[num_seqs + 1] device array: sequence s owns query rows
 *                  [cu[s], cu[s+1]); NULL = one sequence owning all rows (the reference contract)
 *   seq_lens       int32[num_seqs]: cached tokens per sequence, new tokens included; the query
 *                  rows of a sequence are its last rows (the reference requires q_len == seq_len)
 *   max_q_len      upper bound of the per-sequence query length (host value, 0 = num_tokens)
 *   error_flag     optional device int32, set to 1 if a bounded device-side wait expired
 */
int rq_prefill_int8(const void* q, void* out, int dtype, int64_t q_stride_tok,
                    int64_t q_stride_head, int64_t o_stride_tok, int64_t o_stride_head,
                    const int32_t* cu_seqlens_q, int num_tokens, int num_seqs, int max_q_len,
                    int num_q_heads, int num_kv_heads, int head_dim, const uint8_t* kv_cache,
                    int64_t num_blocks, int block_size, int total_bytes, const int32_t* block_table,
                    int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
                    int n_centroids_k, const float* centroids_v, int n_centroids_v,
                    const float* rotation, float sm_scale, int* error_flag, void* stream);

/*
 * rq_prefill_int8 in two steps, for callers that can lend scratch memory: every (sequence, KV head,
 * 128-key tile) is decompressed once into `workspace` (int8 K codes, key scales, V values, already
 * in tensor-core operand order) and the attention kernel streams those records with bulk copies
 * instead of rebuilding them for every block of query rows.  Same results as rq_prefill_int8.
 *
 *   max_seq_len      upper bound of seq_lens (host value); sequences longer than it are truncated
 *   workspace        >= rq_prefill_workspace_bytes(num_seqs, num_kv_heads, max_seq_len) bytes,
 *                    128-byte aligned; contents are scratch
 */
size_t rq_prefill_workspace_bytes(int num_seqs, int num_kv_heads, int max_seq_len);
int rq_prefill_int8_staged(const void* q, void* out, int dtype, int64_t q_stride_tok,
                           int64_t q_stride_head, int64_t o_stride_tok, int64_t o_stride_head,
                           const int32_t* cu_seqlens_q, int num_tokens, int num_seqs, int max_q_len,
                           int num_q_heads, int num_kv_heads, int head_dim, const uint8_t* kv_cache,
                           int64_t num_blocks, int block_size, int total_bytes,
                           const int32_t* block_table, int64_t block_table_stride,
                           const int32_t* seq_lens, const float* centroids_k, int n_centroids_k,
                           const float* centroids_v, int n_centroids_v, const float* rotation,
                           float sm_scale, int* error_flag, int max_seq_len, void* workspace,
                           size_t workspace_bytes, void* stream);

/*
 * Measurement helper (no counterpart in the reference): enqueue one launch that keeps the tcgen05
 * tensor pipe of every SM busy with back-to-back 128 x 256 MMAs from shared-memory operands --
 * kind 0: int8 (kind::i8), kind 1: bf16 (kind::f16) -- `iters` rounds of four K steps each.
 * *ops_out (host, optional) receives the operations (2 per multiply-add) of the launch; time the
 * launch with events on `stream` to get the achievable tensor rate the prefill roofline uses.
 * status_dev (device int, optional) is set to 1 if the kernel's bounded wait expired.
 */
int rq_probe_mma_peak(int kind, int iters, double* ops_out, int* status_dev, void* stream);

/*
 * Self test (no counterpart in the reference): one device thread waits, with the library's bounded
 * mbarrier wait and a limit of `limit_cycles` SM clocks, on a barrier that nobody arrives on.
 * status_dev[0] becomes 1 when the wait gave up as it must (0 if it reported completion),
 * status_dev[1] the clocks it took / 1024.  The context stays usable.
 */
int rq_selftest_bounded_wait(long long limit_cycles, int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RQ_B200_H */
