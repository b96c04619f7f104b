/*
 * ivab.h -- C ABI of libivab.so: paged-KV append, gather and single-query decode
 * attention for NVIDIA B200 (sm_100a).
 *
 * The reference project is pure Python; the operators this library replaces are Python
 * functions, cited per entry point below (paths inside the reference project).  A binding
 * needs only ctypes / cffi: every argument is a plain pointer, integer or float.
 *
 * Conventions
 *   - All data pointers are CUDA device pointers owned by the caller.  The library
 *     allocates no device memory at run time; scratch space is passed in as `workspace`.
 *     (One exception is static: the 8 MiB array behind ivab_paged_decode_attn_noalloc is part
 *     of the library image and occupies device memory on every GPU that loads the library.)
 *   - Strides are in ELEMENTS of `dtype`.  The innermost (head_dim) axis is contiguous.
 *   - `stream` is a cudaStream_t (NULL = legacy default stream).  Calls only enqueue work.
 *   - Return value: IVAB_OK (0) or a negative IVAB_ERR_* code; ivab_last_error() then
 *     returns a message for the calling thread.  Nothing throws or aborts.
 *   - Index data (slot ids, page ids, context lengths) lives on the device, so it cannot
 *     be validated before launch.  Kernels check every index, SKIP (or clamp) a bad access
 *     instead of faulting, and OR a bit into an int32 status word the caller supplies
 *     (`status`, may be NULL) or that lives in the decode workspace.
 *   - Page pool layout: element (head h, page p, offset o, dim d) is at
 *         pool + h*pool_stride_head + p*pool_stride_page + o*head_dim + d,
 *     i.e. each (head, page) block of page_size*head_dim elements is contiguous.
 *     The reference cache layout [1, H, num_pages*page_size, D]
 *     (src/kernels_t/kv_ops_triton.py:105) has pool_stride_page = page_size*D and
 *     pool_stride_head = num_pages*page_size*D.
 */
#ifndef IVAB_H_
#define IVAB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with -fvisibility=hidden */
#endif

#define IVAB_OK 0
#define IVAB_ERR_INVALID (-1)     /* bad argument (null pointer, misaligned, negative size ...) */
#define IVAB_ERR_UNSUPPORTED (-2) /* shape / dtype combination not compiled in */
#define IVAB_ERR_CUDA (-3)        /* a CUDA runtime call failed */
#define IVAB_ERR_WORKSPACE (-4)   /* workspace too small */
#define IVAB_ERR_DEVICE (-5)      /* device-side status word non-zero */

#define IVAB_F32 0
#define IVAB_F16 1
#define IVAB_BF16 2
#define IVAB_F8E4M3 3 /* 8-bit e4m3 KV storage: copy kernels and the *_fp8 entry points only */

/* bits of the device-side status word */
#define IVAB_STATUS_WAIT_TIMEOUT 1       /* a bounded in-kernel wait expired; the CTA unwound */
#define IVAB_STATUS_BAD_PAGE 2           /* block-table entry outside [0, num_pages) */
#define IVAB_STATUS_BAD_CTX_LEN 4        /* context length < 0 or beyond the block table */
#define IVAB_STATUS_BAD_SLOT 8           /* slot / index outside [0, num_slots) */
#define IVAB_STATUS_WORKSPACE_OVERFLOW 16

/* layouts of ivab_paged_gather's output */
#define IVAB_OUT_TOKEN_MAJOR 0 /* [total_tokens, H, D]                                  */
#define IVAB_OUT_HEAD_MAJOR 1  /* sequence s is [H, L_s, D] starting at out_offsets[s]*H*D */

const char* ivab_last_error(void);
int ivab_version(void);

/*
 * out[b,h,n,:] = cache[b,h,indices[n],:]
 * Replaces kv_gather_kernel + KVOpsTriton.forward(operation="gather")
 * (src/kernels_t/kv_ops_triton.py:18-40,111-123).  `indices` is int64[N], shared by all
 * batch rows and heads.  out_dtype == dtype, or IVAB_F32 to reproduce the reference's
 * always-fp32 output (kv_ops_triton.py:112).  head_dim*sizeof(dtype) must be a multiple
 * of 16 bytes and all base pointers / strides 16-byte aligned.
 */
int ivab_kv_gather(const void* cache, const int64_t* indices, void* out, int dtype, int out_dtype,
                   int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                   int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                   int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                   int32_t* status, void* stream);

/*
 * ivab_kv_gather with one index vector PER BATCH ROW: row b uses indices + b*indices_stride_b, and an
 * index of -1 is padding (the output row is left untouched, no status bit).  Together with
 * ivab_compact_indices this is the corrected form of kv_compact_kernel / kv_compact_triton
 * (src/kernels_t/kv_ops_triton.py:68-92,159-181), whose mask is [B,S] with independent rows.
 */
int ivab_kv_gather_rows(const void* cache, const int64_t* indices, int64_t indices_stride_b, void* out,
                        int dtype, int out_dtype,
                        int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                        int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                        int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                        int32_t* status, void* stream);

/*
 * Positions kept by a compaction mask: for every row b of `mask` (uint8 [batch, seq_len], non-zero = keep)
 *   indices[b, j] = position of the j-th kept entry for j < counts[b], and -1 behind them
 * (`indices` is int64 [batch, seq_len], `counts` int32 [batch]; one prefix scan per row, one launch).
 * This is the mask test of kv_compact_kernel (src/kernels_t/kv_ops_triton.py:82-84) turned into the
 * destination rows that kernel fails to compute (it writes survivor s to output row s, :86).
 */
int ivab_compact_indices(const uint8_t* mask, int64_t batch, int64_t seq_len, int64_t* indices,
                         int32_t* counts, void* stream);

/*
 * cache[b,h,indices[n],:] = values[b,h,n,:]   (IN PLACE)
 * Replaces kv_scatter_kernel (src/kernels_t/kv_ops_triton.py:43-65).  The reference clones
 * the whole cache first (kv_ops_triton.py:129); a caller that wants that behaviour clones
 * before calling.  Duplicate indices race, as they do in the reference.
 */
int ivab_kv_scatter(void* cache, const int64_t* indices, const void* values, int dtype,
                    int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                    int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                    int64_t values_stride_b, int64_t values_stride_h, int64_t values_stride_n,
                    int32_t* status, void* stream);

/*
 * Block-table append: K and V of T new tokens written to their slots in one launch.
 *   pool[h, slot_mapping[t]] = new[t, h, :]          slot = page*page_size + offset
 * The slot mapping is the `indices` vector of the reference scatter
 * (src/kernels_t/kv_ops_triton.py:58) read on the flattened slot axis; it also replaces the
 * concat-append of AttentionTorch.forward (src/core/attention.py:61-63).
 */
int ivab_paged_append(const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                      const int64_t* slot_mapping, void* k_pool, void* v_pool,
                      int64_t pool_stride_head, int64_t pool_stride_page, int dtype,
                      int64_t n_tokens, int64_t heads, int64_t head_dim, int64_t page_size,
                      int64_t num_pages, int32_t* status, void* stream);

/*
 * Block-table append into 8-bit (e4m3) pools: the new tokens arrive in `src_dtype` (IVAB_F16 or
 * IVAB_BF16) and are stored as  fp8( x / scale )  with saturation, K with k_scale and V with
 * v_scale (per-tensor scales chosen by the caller).  Strides of the pools are in 1-byte elements.
 * The reference only names fp8 KV storage in a config file (configs/quant_infer.yaml:22,52); there
 * is no reference implementation, so the contract is this library's own: decode attention on the
 * stored values is exact to the same tolerance as for 16-bit storage, the quantisation error is
 * the caller's trade-off.
 */
int ivab_paged_append_fp8(const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                          const int64_t* slot_mapping, void* k_pool, void* v_pool,
                          int64_t pool_stride_head, int64_t pool_stride_page, int src_dtype,
                          float k_scale, float v_scale,
                          int64_t n_tokens, int64_t heads, int64_t head_dim, int64_t page_size,
                          int64_t num_pages, int32_t* status, void* stream);

/*
 * Paged gather of every sequence to contiguous storage, through the block table:
 *   out[token out_offsets[s]+j, h, :] = pool[h, block_table[s][j/page_size], j%page_size, :]
 * for j < ctx_len[s].  Same semantics as the reference gather
 * (src/kernels_t/kv_ops_triton.py:33-40) called with each sequence's slot list.
 * out_offsets is int64[B+1] (cumulative lengths, in tokens).
 */
int ivab_paged_gather(const void* pool, int64_t pool_stride_head, int64_t pool_stride_page,
                      const int32_t* block_table, int64_t block_table_stride, const int32_t* ctx_len,
                      const int64_t* out_offsets, void* out, int out_layout, int dtype,
                      int64_t batch, int64_t heads, int64_t head_dim, int64_t page_size,
                      int64_t num_pages, int64_t max_pages_per_seq, int32_t* status, void* stream);

/*
 * Bytes of scratch ivab_paged_decode_attn needs on the current device for up to `batch`
 * sequences (plan, split-K partials, status word).
 */
int ivab_decode_workspace_bytes(int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                size_t* bytes_out);

/*
 * Single-query decode attention read through a block table:
 *   out[s,hq,:] = softmax_j( q[s,hq,:] . K[s,kvh(hq),j,:] * scale ) . V[s,kvh(hq),j,:]
 *                 over the keys j < ctx_len[s] with j < sink_tokens or j >= ctx_begin[s]
 *   lse[s,hq]   = log sum_j exp( q.K_j * scale )                       (natural log; may be NULL)
 * ctx_begin may be NULL (= 0 for every sequence).  With a sliding window it is ctx_len - window:
 * pages that lie wholly before it are never read, so their block-table entries may be stale and the
 * pages themselves may already be back in the pool (the keys a sliding-window mask would hide,
 * src/core/attention.py:83-87,115-129, are dropped instead of masked).  sink_tokens > 0 keeps the
 * first sink_tokens keys of every sequence visible in front of its window (attention sinks,
 * sink_cfg["sink_tokens"] of src/core/attention.py:131-148); their pages must stay allocated.
 * The math is AttentionTorch.forward lines 77, 99, 102 (src/core/attention.py) for one query
 * and no mask; it takes the place of the unusable attention_kernel
 * (src/kernels_t/attention_triton.py:18-71).  kvh(hq) = hq / (q_heads/kv_heads); the group
 * size may be 1 to 8 (3 runs in the kernels built for 4, 5-7 in those for 8) or a larger one that
 * splits into equal groups of at most 8 (16 = 2 x 8, 12 = 2 x 6, 64 = 8 x 8; each group is a work item
 * of its own, so the K/V of that head are read once per group); head_dim 32, 64, 128 (or 256 for
 * 16-bit types), page_size 16.
 * `dtype` is the type of q and of the pools.  `out_dtype` is the type of `out`: `dtype`, or
 * IVAB_F32 to receive the kernels' fp32 result without the final rounding to a 16-bit type (the
 * reference computes and returns fp32 for fp32 inputs, and its gather always returns fp32,
 * src/kernels_t/kv_ops_triton.py:112); out strides are in elements of `out_dtype`.
 * Enqueues up to three kernels: a planning kernel (batches above 32 sequences; smaller batches derive
 * their chunking inside the attention kernel), the persistent split-K attention kernel, and the logsumexp
 * merge kernel (not launched when no sequence can be split).  ctx_len[s] == 0
 * (or an empty window)
 * yields zeros and -inf.  `workspace` must be 256-byte aligned and hold
 * ivab_decode_workspace_bytes(); concurrent calls need distinct workspaces.
 */
int ivab_paged_decode_attn(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                           const void* k_pool, const void* v_pool,
                           int64_t pool_stride_head, int64_t pool_stride_page,
                           const int32_t* block_table, int64_t block_table_stride,
                           const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                           void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                           int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                           int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                           float scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * ivab_paged_decode_attn on 8-bit (e4m3) pools written by ivab_paged_append_fp8:
 *   K = k_scale * stored, V = v_scale * stored; q, out in `dtype` (IVAB_F16 or IVAB_BF16).
 * Pool strides are in 1-byte elements; head_dim 64 or 128.  The stored values are widened
 * exactly and all arithmetic is fp32, so results equal attention over the dequantised pools to
 * the tolerance of the 16-bit path.  With head_dim 128 (every head ratio) and head_dim 64 (grouped
 * queries) the tensor-core operands are built in registers straight from the stored bytes
 * (e4m3 -> fp16 is exact), about 1.35-1.7x the tokens/s of 16-bit storage at half the memory;
 * head_dim 64 multi-head attention widens on the fly on CUDA cores.  bf16 queries are converted to
 * fp16 (saturating) on the tensor-core path.
 * No counterpart in the reference (fp8 KV is only named in configs/quant_infer.yaml:52).
 */
int ivab_paged_decode_attn_fp8(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                               const void* k_pool, const void* v_pool,
                               int64_t pool_stride_head, int64_t pool_stride_page,
                               float k_scale, float v_scale,
                               const int32_t* block_table, int64_t block_table_stride,
                               const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                               void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                               int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                               int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                               float scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * One decode step in one call: append the newest token of every sequence, then attend over the cache
 * including it -- ivab_paged_append (one token per sequence) followed by ivab_paged_decode_attn[_fp8],
 * without the separate copy launch.  It replaces the pair cat-append + attention of
 * AttentionTorch.forward (src/core/attention.py:61-63 and :77,99,102) for a one-token step.
 *   k_new, v_new: [batch, kv_heads, head_dim] in `dtype` (strides new_stride_t per sequence, new_stride_h
 *   per head, in elements).  ctx_len[s] INCLUDES the new token: it is stored at position ctx_len[s] - 1,
 *   i.e. in page block_table[s][(ctx_len[s]-1) / page_size] -- the block table, not a slot mapping, says
 *   where (the page must already be in the table).  A sequence with ctx_len 0 appends nothing.
 *   kv_dtype: `dtype`, or IVAB_F8E4M3 with k_scale / v_scale (then the rows are quantised exactly as
 *   ivab_paged_append_fp8 does; pool strides in 1-byte elements).
 * The row is written by the CTA that reads that page (ordinary stores, ordered before its TMA reads), so the
 * pools end up bit-identical to the two-call sequence and so does the attention result.  q, k_new, v_new and
 * ctx_len may point into page-locked host memory that is addressable from the device: the kernels then read
 * the step's inputs in place, over the bus, with no upload in front of the step (the pools, the block table
 * and the workspace must be device memory).  Everything else as for ivab_paged_decode_attn.
 */
int ivab_paged_decode_step(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                           const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                           void* k_pool, void* v_pool, int64_t pool_stride_head, int64_t pool_stride_page,
                           int kv_dtype, float k_scale, float v_scale,
                           const int32_t* block_table, int64_t block_table_stride,
                           const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                           void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                           int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                           int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                           float scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Copies the status word of the last ivab_paged_decode_attn call on `workspace` to the host
 * (synchronises `stream`).  *status_out is a mask of IVAB_STATUS_* bits; returns
 * IVAB_ERR_DEVICE if it is non-zero.
 */
int ivab_decode_status(const void* workspace, int32_t* status_out, void* stream);

/*
 * ivab_paged_decode_attn without a workspace argument and without any allocation.
 * (No counterpart in the reference: it exists for callers of this library that cannot allocate.)
 *
 * Some callers have no way to obtain device scratch at the point where they decode: a serving
 * loop that handed out every byte of its memory budget at start-up, a plugin running inside a
 * host that owns the allocator and does not expose it, or a latency-critical path that may not
 * call cudaMalloc because it synchronises the whole device.  For them the split-K scratch is a
 * fixed 8 MiB array inside the library image; every GPU that loads the library holds those
 * 8 MiB until the process exits, whether or not this entry point is ever called.
 *
 * Arguments as ivab_paged_decode_attn; `status` (device int32, may be NULL) receives the
 * IVAB_STATUS_* bits of this call on `stream` (0 when batch is 0).  Limits and rules:
 *   - the problem must fit: ivab_decode_workspace_bytes(batch, ...) <= 8 MiB, else
 *     IVAB_ERR_WORKSPACE (e.g. 128 sequences x 32 query / 8 KV heads x head_dim 128 needs 6.9 MiB);
 *   - calls no cudaMalloc / cudaFree or other allocating routine;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture;
 *   - all calls on a device share the one array, which keeps the previous call's contents (the
 *     kernels re-initialise what they read): two calls that overlap on the GPU -- different
 *     streams, or different host threads -- race.  Serialise them.  (Looking up the array's
 *     address is itself safe from several host threads at once.)
 */
int ivab_paged_decode_attn_noalloc(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                   const void* k_pool, const void* v_pool,
                                   int64_t pool_stride_head, int64_t pool_stride_page,
                                   const int32_t* block_table, int64_t block_table_stride,
                                   const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                                   void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                                   int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                                   int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                                   float scale, int32_t* status, void* stream);

/*
 * All-gather of one small block per rank over peer-mapped memory, for the head-parallel decode of one long
 * sequence (every rank holds [batch, q_heads/world, head_dim + 1] fp32 rows after its attention call and needs
 * all ranks' rows).  It takes the place of the NCCL all-gather such a mode would otherwise call (the reference
 * has no parallel decode path; its collectives go through torch.distributed, src/utils/distributed.py:29-34).
 *   peer_bufs[r]  (host array of `world` device pointers) base of rank r's exchange buffer as mapped into THIS
 *                 process; peer_bufs[rank] is this rank's own buffer.  Every buffer has the layout
 *                 [slots][world][block_bytes] result rows, then at `staging_offset` a staging area of
 *                 [slots][world][2 * block_bytes] bytes that the peers write ({payload, step tag} 64-bit words),
 *                 and must be zero before its first use (all ranks, before any rank's first call).
 *   epoch         device uint32 of this rank, zero before the first call: steps exchanged so far.
 * After the call's kernel has run, result row r of slot (epoch_before % slots) of this rank's buffer holds rank
 * r's block.  Every rank must make the same sequence of calls.  Plain peer stores and local loads only, no
 * fence and no separate arrival flag (a word that carries the step's tag carries its payload); the wait for
 * the peers is bounded by wait_limit_ns and sets IVAB_STATUS_WAIT_TIMEOUT in *status (device int32, may be
 * NULL) when it expires.  world <= 16, slots >= 2, block_bytes a multiple of 16.
 */
int ivab_peer_allgather(const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world, int rank,
                        int slots, int64_t staging_offset, uint32_t* epoch, int32_t* status, int64_t wait_limit_ns,
                        void* stream);

/*
 * Head-parallel decode step with the all-gather folded into it: ivab_paged_decode_step (k_new / v_new may both
 * be NULL: attention only) whose fp32 output rows and logsumexp are written into `local_block` and exchanged
 * as ivab_peer_allgather would -- by the merge kernel's last CTA, so that no exchange kernel is launched
 * behind the step (a step whose block table is too narrow for any split has no merge kernel; the
 * stand-alone exchange kernel is launched then).  `out` (fp32, strides in elements) and `lse` must lie
 * inside [local_block, local_block + block_bytes); the exchange arguments are those of ivab_peer_allgather.
 * Every rank must make the same sequence of calls; batch must be positive.
 * No counterpart in the reference (it has no parallel decode path).
 */
int ivab_paged_decode_step_allgather(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                     const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                                     void* k_pool, void* v_pool, int64_t pool_stride_head, int64_t pool_stride_page,
                                     int kv_dtype, float k_scale, float v_scale,
                                     const int32_t* block_table, int64_t block_table_stride,
                                     const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                                     void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                                     int dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                                     int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                                     float scale, void* workspace, size_t workspace_bytes,
                                     const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world,
                                     int rank, int slots, int64_t staging_offset, uint32_t* epoch,
                                     int32_t* exchange_status, int64_t wait_limit_ns, void* stream);

/*
 * Number of kernels of this library launched by the calling process since load
 * (for benchmark bookkeeping).
 */
int64_t ivab_launch_count(void);

/*
 * Failure-detection self test: one CTA waits on a barrier that nothing will ever complete,
 * with the given limit; it must give up, set IVAB_STATUS_WAIT_TIMEOUT in *status (device
 * int32) and return normally.  Demonstrates that an in-kernel wait cannot hang the GPU.
 */
int ivab_selftest_bounded_wait(int32_t* status, int64_t limit_ns, void* stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* IVAB_H_ */
