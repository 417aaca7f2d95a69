/*
 * kvq_b200 -- C ABI of the static per-channel INT8 KV-cache kernels for NVIDIA B200 (sm_100a).
 *
 * Drop-in boundary for the native module of ischencheng/int8-kvcache: each entry point below replaces one
 * function of the reference's pybind module (kvq/cuda/int8_kv.cu:674-679). The reference passes torch
 * tensors; here every tensor is a raw device pointer plus its sizes and element strides, and the CUDA
 * stream is explicit. Nothing in this library allocates device memory, synchronizes the device or
 * depends on PyTorch; all entry points only enqueue work on `stream` and can be captured in a CUDA graph.
 *
 * Conventions
 *   - bf16 tensors are `const void*` to 2-byte bfloat16 elements, int8 caches are `void*` to 1-byte elements.
 *   - Strides are in ELEMENTS of the tensor they describe. The innermost (head_dim) stride is always 1.
 *   - Caches are views [num_blocks, block_size, num_kv_heads, head_dim] with arbitrary block/slot/head
 *     strides (the vLLM layout interleaves K and V; separate contiguous caches work too).
 *   - Scales are fp32, contiguous: [num_kv_heads, head_dim] ("per channel") or [num_kv_heads] ("per head"),
 *     selected by the k_per_channel / v_per_channel flags. k_mu is always [num_kv_heads, head_dim].
 *   - head_dim is 64 or 128. Rows of bf16 tensors and cache rows must be 16-byte aligned.
 *   - Return value: KVQ_OK, or an error code with a message available from kvq_last_error() on the
 *     calling thread. Empty batches return KVQ_OK without launching anything.
 */
#ifndef KVQ_B200_H_
#define KVQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVQ_OK 0
#define KVQ_ERR_INVALID_ARGUMENT 1 /* shape / layout violation (the reference raises TORCH_CHECK -> RuntimeError) */
#define KVQ_ERR_CUDA 2             /* a CUDA runtime or driver call failed */
#define KVQ_ERR_WORKSPACE 3        /* workspace missing or too small */

/* cudaStream_t without pulling in the CUDA headers. */
typedef struct CUstream_st* kvq_stream_t;

/* Library version (major * 10000 + minor * 100 + patch). */
int kvq_version(void);

/* Message of the last error returned on this thread ("" if none). The pointer stays valid until the next
 * failing call on the same thread. */
const char* kvq_last_error(void);

/*
 * Fused static quantize + paged cache write.
 * Replaces quant_cache(key, value, kc, vc, slots, ks, vs, kmu), kvq/cuda/int8_kv.cu:554-575 (kernel :55-84).
 *   k_i8 = clamp(rne((f32(key) - k_mu) / k_scale), +-127), v_i8 = clamp(rne(f32(value) / v_scale), +-127),
 *   written to cache[slot / block_size][slot % block_size][head][:]. Rows with slot < 0 are skipped; rows of
 *   key/value beyond num_tokens are ignored. Bit-exact with the reference's torch quantizer.
 * key/value: bf16 [>= num_tokens, num_kv_heads, head_dim] with token/head strides; slots: int64 [num_tokens].
 */
int kvq_quant_cache(const void* key, const void* value, void* k_cache, void* v_cache, const int64_t* slots,
                    const float* k_scale, const float* v_scale, const float* k_mu, int64_t num_tokens,
                    int num_kv_heads, int head_dim, int block_size, int64_t key_stride_t, int64_t key_stride_h,
                    int64_t value_stride_t, int64_t value_stride_h, int64_t kc_stride_b, int64_t kc_stride_n,
                    int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h,
                    int k_per_channel, int v_per_channel, kvq_stream_t stream);

/*
 * Standalone q quantization: fold the per-channel K scale into q, one dynamic scale per `group` channels.
 * Replaces quant_q(q, ks, group), kvq/cuda/int8_kv.cu:577-598 (kernel :89-111). Unlike the reference this
 * entry point does not allocate: the caller passes q_i8 [T, Hq, head_dim] (contiguous int8) and
 * q_scale [T, Hq, head_dim / group] (contiguous fp32). head_dim must be 128 and group 128 or 32, as in the
 * reference. k_scale is [Hkv, 128] when k_per_channel, otherwise it is not read.
 */
int kvq_quant_q(const void* q, const float* k_scale, void* q_i8, float* q_scale, int64_t num_tokens,
                int num_q_heads, int num_kv_heads, int head_dim, int group, int64_t q_stride_t, int64_t q_stride_h,
                int k_per_channel, kvq_stream_t stream);

/*
 * Bytes of scratch kvq_int8_decode_attention needs on the current device for a batch of `num_seqs` requests
 * (split-KV partial results, the work plan, a status word). The size does not depend on context lengths.
 * Has no counterpart in the reference, which borrows vLLM's Triton split-KV buffers
 * (kvq/vllm_int8/backend.py:175-177).
 */
size_t kvq_decode_workspace_size(int num_seqs, int head_dim);

/*
 * INT8 paged attention for requests with 1 <= q_len <= qmax query tokens (decode, speculative-decoding
 * verification), causal inside the query. Requests with q_len == 0 or q_len > qmax are skipped and their
 * output rows are left untouched.
 * Replaces int8_decode_attention(...), kvq/cuda/int8_kv.cu:600-648 (kernels :168-463 and :472-503).
 *   q, out: bf16 [T, Hq, head_dim]; cu_q: int32 [num_seqs + 1]; seq_lens: int32 [>= num_seqs];
 *   block_table: int32 [>= num_seqs, bt_stride]; block_size: power of two >= 16; qmax <= 8.
 * Numerics ("implementation B"): q' = q * k_scale (per channel), quantized per (token, head); scores from
 * int8 x int8 -> int32 tensor-core products; fp32 online softmax; P quantized to int8 per (row, 32-key tile
 * at absolute positions); P.V in int8 -> int32; denominator from the quantized P; output * v_scale -> bf16.
 * Split-KV is chosen internally (work is divided over the SMs by the kernel itself, see kvq_debug_decode_split) and
 * merged by a second kernel; both
 * use `workspace` (>= kvq_decode_workspace_size bytes, 256-byte aligned). Calls that share a workspace must
 * not overlap on the GPU.
 */
int kvq_int8_decode_attention(const void* q, const void* k_cache, const void* v_cache, void* out,
                              const int32_t* cu_q, const int32_t* seq_lens, const int32_t* block_table,
                              const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
                              int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
                              int64_t q_stride_t, int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h,
                              int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h, int64_t vc_stride_b,
                              int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride, int k_per_channel,
                              int v_per_channel, int max_query_len, int qmax, void* workspace,
                              size_t workspace_bytes, kvq_stream_t stream);

/*
 * kvq_int8_decode_attention with a finer q quantization: one dynamic q scale per `q_group` channels instead of one
 * per (token, head) row. q_group = 32 computes the reference's q_gran="group32" numerics (kvq/int8_ref.py:120-130;
 * CONFIGS["B_channel_smooth_qgroup32"], :220): the integer dot product of every 32-channel slice is scaled by the
 * slice's own q scale and the slices are summed in fp32. q_group = 0 or head_dim is kvq_int8_decode_attention itself.
 * Everything else (arguments, workspace, skipped requests, P quantization, output) is unchanged. The reference's CUDA
 * kernel has no such mode (its group-32 scales exist only in the standalone quant_q and in the PyTorch
 * implementation); this entry point brings that accuracy option to the INT8 tensor-core path.
 */
int kvq_int8_decode_attention_qgroup(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int32_t* cu_q, const int32_t* seq_lens, const int32_t* block_table,
                                     const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
                                     int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                     int64_t num_blocks, int64_t q_stride_t, int64_t q_stride_h, int64_t o_stride_t,
                                     int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h,
                                     int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride,
                                     int k_per_channel, int v_per_channel, int max_query_len, int qmax, int q_group,
                                     void* workspace, size_t workspace_bytes, kvq_stream_t stream);

/*
 * Prefill / decode disaggregation: the raw int8 pages of a request as one contiguous buffer, and back. The reference
 * moves its int8_static pages between a prefill and a decode instance byte for byte through vLLM's KV connector and
 * never sends the static scales, which both sides load from the same file (docs/LOG.md:614-633: 26.5 KB per token
 * for 28 layers instead of 53 KB in bf16). kvq_pages_to_wire gathers cache pages page_ids[0 .. num_pages) of one
 * layer into wire[num_pages][2][block_size][num_kv_heads][head_dim] (K then V of each page, int8);
 * kvq_wire_to_pages scatters such a buffer into the pages page_ids[] of the receiving cache, which may use other page
 * ids and another cache layout (strides). 2 * num_kv_heads * head_dim bytes per token and layer cross the wire.
 */
int kvq_pages_to_wire(const void* k_cache, const void* v_cache, void* wire, const int32_t* page_ids, int64_t num_pages,
                      int num_kv_heads, int head_dim, int block_size, int64_t kc_stride_b, int64_t kc_stride_n,
                      int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h,
                      kvq_stream_t stream);
int kvq_wire_to_pages(const void* wire, void* k_cache, void* v_cache, const int32_t* page_ids, int64_t num_pages,
                      int num_kv_heads, int head_dim, int block_size, int64_t kc_stride_b, int64_t kc_stride_n,
                      int64_t kc_stride_h, int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h,
                      kvq_stream_t stream);

/*
 * Debug helper: copy the status word the attention kernels keep in `workspace` to the host (synchronizes
 * `stream`). 0 = clean; non-zero = a bounded wait inside a kernel expired. No reference counterpart.
 */
int kvq_decode_status(const void* workspace, int* status, kvq_stream_t stream);

/*
 * The same attention as kvq_int8_decode_attention for callers that cannot allocate device memory, so they
 * have no workspace to pass: an engine that gave all free HBM to its KV pool, code running inside another
 * framework's allocator or graph capture, a latency-critical loop that must never hit cudaMalloc's implicit
 * synchronization. This entry point has no counterpart in the reference. It allocates nothing (no cudaMalloc,
 * no cudaFree, no allocating library call): the scratch is a fixed array of kvq_static_workspace_bytes()
 * (10 MiB) inside the library's device image, resident on every GPU that loads the library until the process
 * exits. Inputs and outputs are still the caller's.
 *   - Limit: a batch whose minimal scratch exceeds the array is rejected with KVQ_ERR_WORKSPACE and a message;
 *     nothing is launched. 10 MiB covers GPUs of up to 148 SMs and about 150,000 requests per call. Multi-token
 *     queries run in the plain one-m-tile-per-item mode here (the grouped mode of kvq_int8_decode_attention needs
 *     four times the partial area), which gives the same results but re-reads K/V once per m tile.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and caches it; make that first call outside any stream capture.
 *   - All calls on a device share the one array, which keeps the previous call's contents. Nothing in it has
 *     to start at zero (each call rewrites the plan, the status word and every partial result it later reads),
 *     but two calls that overlap on the GPU (different streams without ordering) race on it.
 *   - kvq_decode_status does not apply (it needs a workspace pointer).
 */
size_t kvq_static_workspace_bytes(void);
int kvq_int8_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int32_t* cu_q, const int32_t* seq_lens, const int32_t* block_table,
                                      const float* k_scale, const float* v_scale, double softmax_scale, int num_seqs,
                                      int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                      int64_t num_blocks, int64_t q_stride_t, int64_t q_stride_h, int64_t o_stride_t,
                                      int64_t o_stride_h, int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h,
                                      int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride,
                                      int k_per_channel, int v_per_channel, int max_query_len, int qmax,
                                      kvq_stream_t stream);

/*
 * Profiling helper: when both arguments are non-null cudaEvent_t handles, every following
 * kvq_int8_decode_attention call records them on its stream immediately before and after the main attention
 * kernel (between the plan and merge kernels), so a benchmark can time that kernel alone. Pass nulls to stop.
 * Process-wide, not thread-safe, not for use under graph capture. No reference counterpart.
 */
int kvq_debug_kernel_events(void* start_event, void* stop_event);

/*
 * Inspection helper (host only, no GPU work): the split of a batch's work over num_ctas CTAs as
 * kvq_int8_decode_attention's kernel computes it for itself. A unit is one 32-key chunk of one (request, kv head,
 * group of m tiles) item, numbered request by request; CTA b processes units [ubeg[b], uend[b]). The ranges are equal
 * shares of a cost (one per unit plus item_cost per item start; pass item_cost < 0 for the library's figure), and a
 * share boundary that falls on an item start snaps to it. q_lens / seq_lens: host arrays [num_seqs]; grouped /
 * head_group: the kernel's modes (0 / 0 for single-token decode with fewer than 8 kv heads). No reference counterpart:
 * the reference gives every request 16 fixed segments (kvq/cuda/int8_kv.cu:196-198).
 */
int kvq_debug_decode_split(const int32_t* q_lens, const int32_t* seq_lens, int num_seqs, int group_size, int num_kv_heads,
                           int qmax, int grouped, int head_group, int item_cost, int num_ctas, int32_t* ubeg,
                           int32_t* uend);

/*
 * Dequantize pages of the INT8 cache into a temporary bf16 paged cache for the long-query (prefill) path.
 * Replaces dequant_pages(kc, vc, ko, vo, block_table, src_req, src_j, ks, vs), kvq/cuda/int8_kv.cu:650-672
 * (kernel :511-542). Output page p = bf16(rne(int8 page block_table[src_req[p]][src_j[p]] * scale)), laid out
 * contiguously as [num_pages, block_size, num_kv_heads, head_dim]; K stays (k - k_mu).
 */
int kvq_dequant_pages(const void* k_cache, const void* v_cache, void* k_out, void* v_out,
                      const int32_t* block_table, const int32_t* src_req, const int32_t* src_j,
                      const float* k_scale, const float* v_scale, int64_t num_pages, int num_kv_heads, int head_dim,
                      int block_size, int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h,
                      int64_t vc_stride_b, int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride,
                      int k_per_channel, int v_per_channel, kvq_stream_t stream);

/*
 * Causal attention for requests with MORE than min_query_len query tokens (prefill, chunked prefill), reading the
 * INT8 pages directly. Takes the place of the reference's long path as a whole - plan_long + dequant_pages into a
 * temporary bf16 cache + FlashAttention over it, kvq/cuda_kernels.py:80-131 - and computes the same quantity
 * ("implementation A", kvq/int8_ref.py:62-91): softmax(q . (k_i8 * k_scale)^T * softmax_scale) . (v_i8 * v_scale)
 * with the bottom-right causal mask (key n visible to query token t iff n < seq_len - q_len + 1 + t). Requests with
 * at most min_query_len query tokens are skipped and their output rows left untouched, so a mixed batch is served
 * by this call followed by kvq_int8_decode_attention with qmax = min_query_len. Arguments as for
 * kvq_int8_decode_attention; total_query_tokens = rows of q (sizes the grid). The workspace
 * (kvq_prefill_workspace_size(num_seqs) bytes, 256-byte aligned) holds the status word (int32 [0], non-zero after
 * an expired wait) and the work plan. Two launches on `stream`, no host synchronization, capturable.
 */
size_t kvq_prefill_workspace_size(int num_seqs);
int kvq_int8_prefill_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* cu_q,
                               const int32_t* seq_lens, const int32_t* block_table, const float* k_scale,
                               const float* v_scale, double softmax_scale, int num_seqs, int64_t total_query_tokens,
                               int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
                               int64_t q_stride_t, int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h,
                               int64_t kc_stride_b, int64_t kc_stride_n, int64_t kc_stride_h, int64_t vc_stride_b,
                               int64_t vc_stride_n, int64_t vc_stride_h, int64_t bt_stride, int k_per_channel,
                               int v_per_channel, int min_query_len, void* workspace, size_t workspace_bytes,
                               kvq_stream_t stream);

/*
 * Calibration statistics of one step's K/V rows, folded into running totals in place: per (kv head, channel) the
 * |x| maximum, signed maximum, signed minimum (fp32 [num_kv_heads, head_dim] each) and the sum (fp64), for K and
 * for V, plus the number of rows counted. One fused pass in place of the eight torch reductions of the
 * reference's capture hook `_record` (kvq/capture.py:25-44); rows with slots[t] < 0 are skipped like its
 * `slot_mapping >= 0` mask (slots may be null: every row counts). key / value are bf16 [num_tokens, num_kv_heads,
 * head_dim] with element strides; the caller initialises the totals (|x| max 0, max -inf, min +inf, sums 0,
 * tokens 0). Maxima are exact; sums are accumulated to ~48 bits per block and added in fp64 with atomics, so they
 * agree with the reference's double sum to ~1e-13 relative, not bit for bit.
 */
int kvq_calib_stats(const void* key, const void* value, const int64_t* slots, int64_t num_tokens, int num_kv_heads,
                    int head_dim, int64_t key_stride_t, int64_t key_stride_h, int64_t value_stride_t,
                    int64_t value_stride_h, float* k_absmax, float* k_max, float* k_min, double* k_sum,
                    float* v_absmax, float* v_max, float* v_min, double* v_sum, long long* tokens,
                    kvq_stream_t stream);

/*
 * Output all-gather of request-sharded decode over NVLink peer memory. The reference has no counterpart: it runs under
 * vLLM's tensor parallelism, whose collectives are vLLM's. Here requests are sharded over the GPUs of one node and the
 * one exchange on the path is every rank's output rows [T / world, Hq, D] reaching all ranks; at 114 KB per rank a
 * library all-gather is pure latency (~25 us next to a ~97 us attention call), so each rank stores its rows straight
 * into every peer's staging buffer and raises a flag there (plain peer stores, bounded waits, one launch).
 *   src             this rank's rows, bytes_per_rank bytes (a multiple of 16, 16-byte aligned), identical size on all ranks
 *   stage0/1[p]     rank p's two staging buffers (world * bytes_per_rank bytes each) as mapped into THIS process,
 *                   p < world <= 8; row block r of a staging buffer receives rank r's rows; steps alternate between the
 *                   two (a rank may be one step ahead of the slowest one). Host arrays, read during the call.
 *   flag_bufs[p]    rank p's flag array (64 uint32, zero before the first step) as mapped into this process
 *   out             this rank's result, world * bytes_per_rank bytes of ordinary device memory: rank r's rows at row
 *                   block r, complete when the call's kernel has finished
 *   counters        two uint32 in this rank's memory, zero before the first step: the kernel keeps the step count
 *                   there, so the launch has no per-step argument and may be replayed from a CUDA graph
 *   status          device int in this rank's memory: set to 1 when a wait for a peer ran out (about a second)
 * Every rank must make the same sequence of calls. One launch, no host synchronization, capturable.
 */
int kvq_peer_allgather(const void* src, size_t bytes_per_rank, void* const* stage0, void* const* stage1,
                       uint32_t* const* flag_bufs, void* out, int world, int rank, uint32_t* counters, int* status,
                       kvq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KVQ_B200_H_ */
