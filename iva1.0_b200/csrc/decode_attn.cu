// Single-query decode attention through a block table (flash-decoding, split-K).
//
// Three kernels per call, all on the caller's stream:
//
//   1. plan_kernel   (1 CTA)      reads ctx_len (and the optional window start / sink count) on the
//                                 device, picks one chunk size (in pages) for the whole batch so
//                                 that the work list has a few items per resident CTA, orders the
//                                 sequences longest-first and writes the list of (sequence, page
//                                 range) chunks.  No host synchronisation: ragged batches never
//                                 stall the stream.
//   2. decode_kernel (persistent) one CTA per resident slot (2 per SM).  Work items are (kv head,
//                                 chunk) pairs taken from an atomic counter, kv-head-major so that
//                                 CTAs running at the same time read the same head's slab of the
//                                 pool.  Warp 4 is the producer: its item fetches (counter ->
//                                 descriptor -> block-table entries) are pipelined two items ahead,
//                                 and it issues a ring's worth of pages at a time with one lane per
//                                 page, each lane waiting for its own stage and issuing the TMA
//                                 copies of one K page and one V page (4 KB each for 16x128 bf16)
//                                 with an L2 evict-first policy.  The ring of shared-memory stages
//                                 is guarded by mbarriers and runs across item boundaries, so the
//                                 copy engine never drains between items.  Warps 0-3 consume: page
//                                 k of an item always goes to warp (seq + chunk + k) mod 4 (each
//                                 warp owns a quarter of the stages), so results do not depend on
//                                 scheduling.  Each warp keeps its own online-softmax state (running
//                                 max, sum and fp32 accumulators) for all query heads of the kv
//                                 head, so a page is read from HBM once per GQA group.  At the end
//                                 of an item every warp publishes its state to shared memory and
//                                 moves on; the warp that arrives last combines the four states (in
//                                 warp order) and writes the final output (one-chunk sequences) or
//                                 an fp32 partial (o, m, l).
//   3. merge_kernel               logsumexp-merge of the partials of split sequences: one warp per
//                                 (sequence, query head) for up to 32 chunks, one CTA per
//                                 (sequence, query head, 32-dim slice) beyond that.
//
// All waits are bounded (see mbar_wait_bounded); a wait that expires raises a CTA-wide abort
// flag, the status word gets IVAB_STATUS_WAIT_TIMEOUT and every warp unwinds.  Intra-CTA
// synchronisation uses mbarriers only (no bar.sync after start-up), so a warp that unwinds can
// never leave another one stuck at a barrier.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "decode_defs.cuh"      // constants, workspace layout, kernel parameters
#include "decode_dispatch.h"    // the per-dtype units that hold the attention and merge kernels

namespace ivab {

extern std::atomic<long long> g_launches;

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// The kernels handle up to 8 query heads per KV head.  A larger ratio is served by cutting the query
// heads of a KV head into `div` equal groups of at most 8, each a work item of its own that reads the
// same K/V slab ("virtual" KV heads: kv_heads * div of them, group = ratio / div query heads each).
// Returns div, or 0 when the ratio has no such split (a prime above 8, for example).
int split_ratio(int64_t ratio) {
    if (ratio < 1) return 0;
    if (ratio <= 8) return 1;
    for (int64_t div = (ratio + 7) / 8; div <= ratio / 2 + 1 && div <= 64; ++div)
        if (ratio % div == 0 && ratio / div <= 8) return (int)div;
    return 0;
}

int resident_slots() { return sm_count() * 2; }

// Work items per resident CTA the planner aims for.  More items = finer chunks = a shorter tail
// when the last CTAs finish, at the price of more split-K partials.  IVAB_ITEMS_PER_SLOT overrides
// the default for experiments (read once per process).
int items_per_slot() {
    static int v = [] {
        const char* e = std::getenv("IVAB_ITEMS_PER_SLOT");
        const int n = e ? std::atoi(e) : kItemsPerSlot;
        return n < 1 ? 1 : (n > 64 ? 64 : n);
    }();
    return v;
}

int target_chunks_for(int64_t kv_heads) {
    const int64_t items = (int64_t)resident_slots() * items_per_slot();
    int64_t t = (items + kv_heads - 1) / kv_heads;
    return (int)(t < 1 ? 1 : t);
}

// IVAB_DIRECT=0 sends small batches through the plan kernel as well (experiments, A/B runs).
bool use_direct_mode() {
    static bool v = [] {
        const char* e = std::getenv("IVAB_DIRECT");
        return !(e && std::atoi(e) == 0);
    }();
    return v;
}

// IVAB_PLAN_PDL=0 launches the plan kernel in plain stream order.
bool use_plan_pdl() {
    static bool v = [] {
        const char* e = std::getenv("IVAB_PLAN_PDL");
        const char* all = std::getenv("IVAB_PDL");
        return !(e && std::atoi(e) == 0) && !(all && std::atoi(all) == 0);
    }();
    return v;
}

// Order in which work items are handed out: 0 = kv-head-major, 1 = chunk-major, 2 = chunk-major when the plan
// kernel finds the batch ragged (IVAB_ITEM_ORDER, experiments).
int item_order() {
    static int v = [] {
        const char* e = std::getenv("IVAB_ITEM_ORDER");
        const int n = e ? std::atoi(e) : kDefaultItemOrder;
        return n < 0 || n > 2 ? kDefaultItemOrder : n;
    }();
    return v;
}

// Smallest chunk (pages) the plan-free mode cuts; IVAB_DIRECT_MIN_CHUNK overrides it for experiments.
int direct_min_chunk_pages() {
    static int v = [] {
        const char* e = std::getenv("IVAB_DIRECT_MIN_CHUNK");
        const int n = e ? std::atoi(e) : kDirectMinChunkPages;
        return n < 1 ? 1 : n;
    }();
    return v;
}

size_t carve_workspace(void* base, int64_t B, int64_t Hq, int64_t Hkv, int64_t D, Workspace* ws) {
    const int target = target_chunks_for(Hkv);
    const int64_t cap = B + target;
    size_t off = 0;
    char* p = static_cast<char*>(base);
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return p ? p + o : nullptr; };
    int* header = reinterpret_cast<int*>(take(kHdrWords * sizeof(int)));
    int* slots = reinterpret_cast<int*>(take(kStatusSlots * sizeof(int)));   // (ivab_decode_status reads header + slots in one copy)
#ifdef IVAB_PROFILE
    unsigned long long* prof_cta = reinterpret_cast<unsigned long long*>(take(kStatusSlots * 4 * sizeof(unsigned long long)));
    if (ws) ws->prof_cta = prof_cta;
#endif
    int* prefix = reinterpret_cast<int*>(take((B + 1) * sizeof(int)));
    int* order = reinterpret_cast<int*>(take(B * sizeof(int)));
    int* seq_first = reinterpret_cast<int*>(take(B * sizeof(int)));
    int* seq_count = reinterpret_cast<int*>(take(B * sizeof(int)));
    int* split_list = reinterpret_cast<int*>(take(B * sizeof(int)));
    ChunkDesc* chunks = reinterpret_cast<ChunkDesc*>(take(cap * sizeof(ChunkDesc)));
    float* ml = reinterpret_cast<float*>(take((size_t)cap * Hq * 2 * sizeof(float)));
    float* po = reinterpret_cast<float*>(take((size_t)cap * Hq * D * sizeof(float)));
    if (ws) { ws->header = header; ws->pos_prefix = prefix; ws->order = order; ws->seq_first = seq_first; ws->seq_count = seq_count;
              ws->split_list = split_list;
              ws->chunks = chunks; ws->part_ml = ml; ws->part_o = po; ws->status_slots = slots;
              ws->cap = (int)cap; ws->target_chunks = target; }
    return off;
}

// ------------------------------------------------------------------------------------------------
// 1. plan
// ------------------------------------------------------------------------------------------------

constexpr int kPlanThreads = 1024;
constexpr int kSortMax = 1024;   // largest batch whose sequences are ordered longest-first (rank sort, O(B) per thread)

__device__ int block_inclusive_scan(int v, int* warp_sums, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, v, off);
        if (lane >= off) v += t;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, w, off);
            if (lane >= off) w += t;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    if (warp > 0) v += warp_sums[warp - 1];
    *total = warp_sums[31];
    __syncthreads();
    return v;
}

__global__ void __launch_bounds__(kPlanThreads) plan_kernel(const int32_t* __restrict__ ctx_len,
                                                            const int32_t* __restrict__ ctx_begin, int sink_tokens, int B,
                                                            int page_size,
                                                            int max_pages, int target_chunks, int cap, int Hkv,
                                                            Workspace ws) {
    __shared__ int warp_sums[32];
    __shared__ long long s_total_pages;
    __shared__ int s_bad;
    __shared__ int s_pages[kSortMax];
    // Batches of up to kSortMax sequences keep the processing order and the chunk prefix in shared memory:
    // the chunk list is built by a binary search over the prefix per chunk, which through global memory
    // costs a dependent L2 round trip per step (seven for 128 sequences).
    __shared__ int s_order[kSortMax];
    __shared__ int s_prefix[kSortMax + 1];
    __shared__ int s_ragged, s_split, s_big;
    const int tid = threadIdx.x;
    // the attention kernel may be scheduled now: its set-up does not depend on the plan, and it
    // waits for this grid to complete before it reads the workspace
    grid_launch_dependents();
    // This kernel is itself launched as a programmatic dependent of the kernel before it in the stream, so
    // that its launch latency hides under that kernel (typically the append of the same step).  That kernel
    // may be the one that wrote ctx_len, and the attention kernel waits for THIS grid only: nothing is read,
    // and this grid cannot complete, before the predecessor has completed.
    grid_dependency_wait();
#ifdef IVAB_PROFILE
    if (tid == 0) {
        PROF_STAMP_SET(ws.header, 0)
        for (int i = 2; i < 8; ++i) PROF_STAMP_PTR(ws.header)[i] = (i == 5 || i == 7) ? 0ull : ~0ull;
        *reinterpret_cast<unsigned long long*>(ws.header + 14) = ~0ull;   // (words 8..12 belong to the plan-free counter and the merge count)
    }
#endif
    if (tid == 0) { s_total_pages = 0; s_bad = 0; s_ragged = 0; s_split = 0; s_big = 0; }
    __syncthreads();

    // (pages a sequence reads: seq_page_range in decode_defs.cuh; page_size is always kPage here)
    auto seq_range = [&](int s, int* L_out, int* begin_out, int* sink_pages_out) {
        return seq_page_range(ctx_len, ctx_begin, sink_tokens, max_pages, s, L_out, begin_out, sink_pages_out, nullptr);
    };

    // total pages of the batch
    long long local = 0;
    for (int s = tid; s < B; s += kPlanThreads) {
        const int L_raw = ctx_len[s];
        if (L_raw < 0 || (long long)L_raw > (long long)max_pages * page_size) s_bad = 1;
        if (ctx_begin != nullptr && (ctx_begin[s] < 0 || ctx_begin[s] > L_raw)) s_bad = 1;
        int L, b, sp;
        const int pg = seq_range(s, &L, &b, &sp);
        if (B <= kSortMax) s_pages[s] = pg;
        local += pg;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    if ((tid & 31) == 0 && local) atomicAdd(reinterpret_cast<unsigned long long*>(&s_total_pages), (unsigned long long)local);
    __syncthreads();
    const long long total_pages = s_total_pages;
    long long c64 = (total_pages + target_chunks - 1) / target_chunks;
    if (c64 < kMinChunkPages) c64 = kMinChunkPages;
    const int chunk_pages = (int)(c64 > 0x3fffffff ? 0x3fffffff : c64);

    // Processing order: longest sequence first (ties by index).  Work items are handed out in this
    // order, so the CTAs that finish last are working on the shortest items and the tail of the
    // kernel is short even for ragged batches.  Batches beyond kSortMax keep their natural order.
    auto clamped_pages = [&](int s) {
        int L, b, sp;
        return seq_range(s, &L, &b, &sp);
    };
    const bool sorted = B <= kSortMax;
    if (sorted) {
        for (int s = tid; s < B; s += kPlanThreads)
            if (s_pages[s] != s_pages[0]) s_ragged = 1;
        __syncthreads();
        const bool ragged = s_ragged != 0;   // a uniform batch needs no ordering
        for (int s = tid; s < B; s += kPlanThreads) {
            if (!ragged) { s_order[s] = s; continue; }
            const int mine = s_pages[s];
            int rank = 0;
            for (int t = 0; t < B; ++t) {
                const int other = s_pages[t];
                rank += (other > mine) || (other == mine && t < s);
            }
            s_order[rank] = s;
        }
    }
    __syncthreads();   // (larger batches keep their natural order: position = sequence)

    // chunks per position and their exclusive prefix
    int running = 0;
    for (int base = 0; base < B; base += kPlanThreads) {
        const int pos = base + tid;
        int n = 0, s = 0;
        if (pos < B) {
            s = sorted ? s_order[pos] : pos;
            const int pages = sorted ? s_pages[s] : clamped_pages(s);
            n = (pages + chunk_pages - 1) / chunk_pages;
            if (n < 1) n = 1;   // an empty sequence still gets one (empty) item, which writes zeros / -inf
        }
        int tile_total;
        const int incl = block_inclusive_scan(n, warp_sums, &tile_total);
        if (pos < B) {
            if (sorted) s_prefix[pos] = running + incl - n; else ws.pos_prefix[pos] = running + incl - n;
            ws.seq_first[s] = running + incl - n;
            ws.seq_count[s] = n;
            // order within either end of the list is irrelevant: every entry is merged on its own
            if (n > kMergeWarpMax) ws.split_list[B - 1 - atomicAdd(&s_big, 1)] = s;
            else if (n > 1) ws.split_list[atomicAdd(&s_split, 1)] = s;
        }
        running += tile_total;
    }
    int num_chunks = running;
    int overflow = 0;
    if (num_chunks > cap) { overflow = 1; num_chunks = 0; }   // cannot happen when cap = B + target_chunks
    if (tid == 0) {
        if (sorted) s_prefix[B] = running; else ws.pos_prefix[B] = running;
        ws.header[kHdrNumChunks] = num_chunks;
        ws.header[kHdrChunkPages] = chunk_pages;
        ws.header[kHdrCounter] = 0;
        ws.header[kHdrStatus] = (s_bad ? kStatusBadCtxLen : 0) | (overflow ? kStatusOverflow : 0);
        ws.header[kHdrTotalItems] = num_chunks * Hkv;
        ws.header[kHdrNumSplit] = overflow ? 0 : s_split;
        ws.header[kHdrNumBig] = overflow ? 0 : s_big;
        ws.header[kHdrChunkMajor] = sorted && s_ragged != 0;
#ifdef IVAB_PROFILE
        for (int i = 16; i < 48; ++i) ws.header[i] = 0;
#endif
    }
    __syncthreads();   // pos_prefix writes of this block are visible to this block

    for (int ci = tid; ci < num_chunks; ci += kPlanThreads) {
        int lo = 0, hi = B - 1;   // largest position with pos_prefix[pos] <= ci
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if ((sorted ? s_prefix[mid] : ws.pos_prefix[mid]) <= ci) lo = mid; else hi = mid - 1;
        }
        const int s = sorted ? s_order[lo] : lo;
        const int first = sorted ? s_prefix[lo] : ws.pos_prefix[lo];
        const int n = (sorted ? s_prefix[lo + 1] : ws.pos_prefix[lo + 1]) - first;
        const int j = ci - first;
        int L, begin, sink_pages;
        const int pages = seq_range(s, &L, &begin, &sink_pages);
        const int per = pages / n, rem = pages % n;   // even split: first `rem` chunks get one more page
        ChunkDesc d;
        d.seq = s;
        // position in the list of pages to read; page_of() turns it into a block-table index
        d.page_begin = j * per + (j < rem ? j : rem);
        d.n_pages = per + (j < rem ? 1 : 0);
        d.chunk_idx = j;
        d.n_chunks = n;
        d.pad0 = L;
        d.pad1 = begin;
        d.pad2 = sink_pages;
        ws.chunks[ci] = d;
    }
#ifdef IVAB_PROFILE
    __syncthreads();
    if (tid == 0) PROF_STAMP_SET(ws.header, 1)
#endif
}

// OR of the header's status word and of the per-CTA slots of the last call, into one device word.
__global__ void __launch_bounds__(kStatusSlots) status_fold_kernel(const int* ws, int n_slots, int* out) {
    const int mine = (int)threadIdx.x < n_slots ? ws[kHdrWords + threadIdx.x] : 0;
    int any = 0;
#pragma unroll
    for (int bit = 0; bit < 5; ++bit) any |= __syncthreads_or(mine & (1 << bit)) ? (1 << bit) : 0;
    if (threadIdx.x == 0) *out = any | ws[kHdrStatus];
}

__global__ void bounded_wait_selftest_kernel(int* status, uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    // Nothing ever arrives on `bar`: the wait must give up after limit_ns.
    const bool ok = mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag, limit_ns);
    if (!ok && threadIdx.x == 0) atomicOr(status, kStatusWaitTimeout);
}

}  // namespace
}  // namespace ivab

using namespace ivab;

extern "C" int ivab_decode_workspace_bytes(int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                                           size_t* bytes_out) {
    if (!bytes_out) return set_error(IVAB_ERR_INVALID, "ivab_decode_workspace_bytes: null bytes_out");
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || q_heads % kv_heads)
        return set_error(IVAB_ERR_INVALID, "ivab_decode_workspace_bytes: bad sizes");
    const int div = split_ratio(q_heads / kv_heads);
    *bytes_out = carve_workspace(nullptr, batch, q_heads, kv_heads * (div > 0 ? div : 1), head_dim, nullptr);
    return IVAB_OK;
}

namespace {

// Shared body of the decode entry points.  kv_dtype is the storage type of the pools (== dtype, or
// IVAB_F8E4M3 with per-tensor scales); pool strides are in elements of kv_dtype.
int decode_entry(const char* fn, const void* q, int64_t q_stride_b, int64_t q_stride_h,
                 const void* k_pool, const void* v_pool, int64_t pool_stride_head, int64_t pool_stride_page,
                 const int32_t* block_table, int64_t block_table_stride,
                 const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                 void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                 int dtype, int out_dtype, int kv_dtype, float k_scale, float v_scale,
                 int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                 int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq, float scale,
                 void* workspace, size_t workspace_bytes, void* stream,
                 const void* k_new = nullptr, const void* v_new = nullptr, int64_t new_stride_t = 0, int64_t new_stride_h = 0,
                 const PeerParams* xchg = nullptr) {
    const size_t esz = dtype_size(dtype);
    const size_t kv_esz = dtype_size(kv_dtype);
    if (esz == 0 || kv_esz == 0) return set_error(IVAB_ERR_INVALID, "%s: unknown dtype %d / %d", fn, dtype, kv_dtype);
    if (dtype == IVAB_F8E4M3) return set_error(IVAB_ERR_UNSUPPORTED, "%s: q and out must be fp32, fp16 or bf16", fn);
    if (kv_dtype == IVAB_F8E4M3 && dtype != IVAB_F16 && dtype != IVAB_BF16)
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: 8-bit pools need fp16 or bf16 queries", fn);
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || num_pages < 0 || max_pages_per_seq < 0)
        return set_error(IVAB_ERR_INVALID, "%s: bad sizes", fn);
    if (out_dtype != dtype && out_dtype != IVAB_F32)
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: out_dtype must be the dtype of q or IVAB_F32", fn);
    if (batch == 0) return IVAB_OK;
    if (num_pages == 0) return set_error(IVAB_ERR_INVALID, "%s: a pool of 0 pages cannot back a batch of %lld sequences", fn, (long long)batch);
    if (page_size != kPage) return set_error(IVAB_ERR_UNSUPPORTED, "%s: page_size %lld (supported: 16)", fn, (long long)page_size);
    if (!q || !k_pool || !v_pool || !block_table || !ctx_len || !out || !workspace)
        return set_error(IVAB_ERR_INVALID, "%s: null pointer", fn);
    auto mis = [](const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) != 0; };
    if (mis(q, 16) || mis(k_pool, 16) || mis(v_pool, 16) || mis(workspace, 256) || (q_stride_b * esz) % 16 ||
        (q_stride_h * esz) % 16 || (pool_stride_head * kv_esz) % 16 || (pool_stride_page * kv_esz) % 16)
        return set_error(IVAB_ERR_INVALID, "%s: q / pools must be 16-byte aligned (workspace 256) with 16-byte strides", fn);
    if (batch >= (1LL << 30) || max_pages_per_seq * page_size >= (1LL << 31))
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: batch or context too large", fn);
    if (sink_tokens < 0 || sink_tokens >= (1LL << 31)) return set_error(IVAB_ERR_INVALID, "%s: bad sink_tokens", fn);
    if ((k_new != nullptr) != (v_new != nullptr)) return set_error(IVAB_ERR_INVALID, "%s: k_new and v_new go together", fn);
    if (k_new != nullptr && (mis(k_new, 16) || mis(v_new, 16) || (new_stride_t * esz) % 16 || (new_stride_h * esz) % 16))
        return set_error(IVAB_ERR_INVALID, "%s: new tokens must be 16-byte aligned with 16-byte strides", fn);

    const int64_t ratio = q_heads / kv_heads;
    const int kv_div = split_ratio(ratio);
    if (kv_div == 0)
        return set_error(IVAB_ERR_UNSUPPORTED,
                         "%s: q_heads/kv_heads = %lld (supported: 1 to 8, and larger ratios that split into equal groups of at most 8)",
                         fn, (long long)ratio);
    const int64_t virt_heads = kv_heads * kv_div;   // work items are (virtual KV head, chunk) pairs
    Workspace ws;
    const size_t need = carve_workspace(workspace, batch, q_heads, virt_heads, head_dim, &ws);
    if (workspace_bytes < need)
        return set_error(IVAB_ERR_WORKSPACE, "%s: workspace of %zu bytes, need %zu", fn, workspace_bytes, need);
    if ((int64_t)ws.cap * virt_heads >= (1LL << 31)) return set_error(IVAB_ERR_UNSUPPORTED, "%s: too many work items", fn);
    // Pages of an 8-bit pool stream twice as fast, so the fixed work per item weighs more: cut a
    // quarter fewer, longer items (measured: C2 171.0 k -> 177.0 k, C3 587.2 k -> 594.6 k tokens/s).
    if (kv_dtype == IVAB_F8E4M3) ws.target_chunks = ws.target_chunks * 3 / 4 > 0 ? ws.target_chunks * 3 / 4 : 1;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Small batches skip the plan kernel: every CTA derives the chunking itself (decode_defs.cuh).  The
    // chunk list then holds at most target_items / heads + batch entries, which the capacity covers.
    const bool direct = batch <= kDirectMaxBatch && use_direct_mode();
    if (!direct) {
        // a programmatic dependent of whatever kernel precedes it in the stream (the append of the same
        // step): it is placed while that kernel runs and waits for it before it reads anything
        cudaLaunchAttribute pdl{};
        pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pdl.val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(1); cfg.blockDim = dim3(kPlanThreads); cfg.dynamicSmemBytes = 0; cfg.stream = st;
        cfg.attrs = &pdl; cfg.numAttrs = use_plan_pdl() ? 1 : 0;
        if (int rc = check_cuda(cudaLaunchKernelEx(&cfg, plan_kernel, ctx_len, ctx_begin, (int)sink_tokens, (int)batch,
                                                   (int)page_size, (int)max_pages_per_seq, ws.target_chunks, ws.cap,
                                                   (int)virt_heads, ws), "plan_kernel launch")) return rc;
        g_launches++;
    }

    DecodeParams p{};
    p.direct = direct ? 1 : 0;
    p.batch = (int)batch; p.max_pages = (int)max_pages_per_seq; p.n_virt_heads = (int)virt_heads;
    p.direct_min_chunk = direct_min_chunk_pages();
    p.chunk_major = item_order();
    p.ctx_len = ctx_len; p.ctx_begin = ctx_begin;
    p.q = q; p.q_sb = q_stride_b; p.q_sh = q_stride_h;
    p.k_pool = static_cast<const char*>(k_pool); p.v_pool = static_cast<const char*>(v_pool);
    p.pool_sh_bytes = pool_stride_head * (int64_t)kv_esz; p.pool_sp_bytes = pool_stride_page * (int64_t)kv_esz;
    p.block_table = block_table; p.bt_stride = block_table_stride;
    p.out = out; p.out_sb = out_stride_b; p.out_sh = out_stride_h; p.lse = lse;
    p.out_f32 = (out_dtype == IVAB_F32 && dtype != IVAB_F32) ? 1 : 0;
    p.Hq = (int)q_heads; p.num_pages = (int)num_pages; p.sink_tokens = (int)sink_tokens;
    p.group = (int)(ratio / kv_div);
    p.kv_div = kv_div;
    p.v_scale = v_scale;
    p.scale_log2 = scale * k_scale * 1.4426950408889634f;   // K = k_scale * stored value
    p.wait_limit_ns = kWaitLimitNs;
    p.ws = ws;
    p.k_new = static_cast<const char*>(k_new); p.v_new = static_cast<const char*>(v_new);
    p.new_st_bytes = new_stride_t * (int64_t)esz; p.new_sh_bytes = new_stride_h * (int64_t)esz;
    p.k_inv_scale = 1.f / k_scale; p.v_inv_scale = 1.f / v_scale;
    if (xchg != nullptr) { p.xchg_on = 1; p.xchg = *xchg; }
    const int G = p.group;
    if (kv_dtype == IVAB_F8E4M3) {
        if (dtype == IVAB_F16) return decode_dispatch_fp8_f16((int)head_dim, G, (int)kv_heads, p, (int)batch, st);
        return decode_dispatch_fp8_bf16((int)head_dim, G, (int)kv_heads, p, (int)batch, st);
    }
    switch (dtype) {
        case IVAB_F32: return decode_dispatch_f32((int)head_dim, G, (int)kv_heads, p, (int)batch, st);
        case IVAB_F16: return decode_dispatch_f16((int)head_dim, G, (int)kv_heads, p, (int)batch, st);
        default: return decode_dispatch_bf16((int)head_dim, G, (int)kv_heads, p, (int)batch, st);
    }
}

}  // namespace

extern "C" int ivab_paged_decode_attn(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                      const void* k_pool, const void* v_pool,
                                      int64_t pool_stride_head, int64_t pool_stride_page,
                                      const int32_t* block_table, int64_t block_table_stride,
                                      const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                                      void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                                      int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                                      int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                                      float scale, void* workspace, size_t workspace_bytes, void* stream) {
    if (dtype == IVAB_F8E4M3)
        return set_error(IVAB_ERR_UNSUPPORTED, "ivab_paged_decode_attn: 8-bit pools go through ivab_paged_decode_attn_fp8");
    return decode_entry("ivab_paged_decode_attn", q, q_stride_b, q_stride_h, k_pool, v_pool, pool_stride_head,
                        pool_stride_page, block_table, block_table_stride, ctx_len, ctx_begin, sink_tokens, out,
                        out_stride_b, out_stride_h, lse, dtype, out_dtype, dtype, 1.f, 1.f, batch, q_heads, kv_heads, head_dim,
                        page_size, num_pages, max_pages_per_seq, scale, workspace, workspace_bytes, stream);
}

extern "C" int ivab_paged_decode_attn_fp8(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                          const void* k_pool, const void* v_pool,
                                          int64_t pool_stride_head, int64_t pool_stride_page,
                                          float k_scale, float v_scale,
                                          const int32_t* block_table, int64_t block_table_stride,
                                          const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                                          void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                                          int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                                          int64_t head_dim, int64_t page_size, int64_t num_pages,
                                          int64_t max_pages_per_seq, float scale,
                                          void* workspace, size_t workspace_bytes, void* stream) {
    if (!(k_scale > 0.f) || !(v_scale > 0.f))
        return set_error(IVAB_ERR_INVALID, "ivab_paged_decode_attn_fp8: scales must be positive");
    return decode_entry("ivab_paged_decode_attn_fp8", q, q_stride_b, q_stride_h, k_pool, v_pool, pool_stride_head,
                        pool_stride_page, block_table, block_table_stride, ctx_len, ctx_begin, sink_tokens, out,
                        out_stride_b, out_stride_h, lse, dtype, out_dtype, IVAB_F8E4M3, k_scale, v_scale, batch, q_heads, kv_heads,
                        head_dim, page_size, num_pages, max_pages_per_seq, scale, workspace, workspace_bytes, stream);
}

extern "C" int ivab_paged_decode_step(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                      const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                                      void* k_pool, void* v_pool, int64_t pool_stride_head, int64_t pool_stride_page,
                                      int kv_dtype, float k_scale, float v_scale,
                                      const int32_t* block_table, int64_t block_table_stride,
                                      const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                                      void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                                      int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                                      int64_t head_dim, int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                                      float scale, void* workspace, size_t workspace_bytes, void* stream) {
    const char* fn = "ivab_paged_decode_step";
    if (batch > 0 && (!k_new || !v_new)) return set_error(IVAB_ERR_INVALID, "%s: null pointer", fn);
    if (kv_dtype != dtype && kv_dtype != IVAB_F8E4M3)
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: the pools hold the dtype of q, or IVAB_F8E4M3", fn);
    if (kv_dtype == IVAB_F8E4M3 && (!(k_scale > 0.f) || !(v_scale > 0.f)))
        return set_error(IVAB_ERR_INVALID, "%s: scales must be positive", fn);
    if (kv_dtype != IVAB_F8E4M3) k_scale = v_scale = 1.f;
    return decode_entry(fn, q, q_stride_b, q_stride_h, k_pool, v_pool, pool_stride_head, pool_stride_page, block_table,
                        block_table_stride, ctx_len, ctx_begin, sink_tokens, out, out_stride_b, out_stride_h, lse, dtype,
                        out_dtype, kv_dtype, k_scale, v_scale, batch, q_heads, kv_heads, head_dim, page_size, num_pages,
                        max_pages_per_seq, scale, workspace, workspace_bytes, stream, k_new, v_new, new_stride_t,
                        new_stride_h);
}

extern "C" int ivab_paged_decode_step_allgather(const void* q, int64_t q_stride_b, int64_t q_stride_h,
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
                                                int32_t* exchange_status, int64_t wait_limit_ns, void* stream) {
    const char* fn = "ivab_paged_decode_step_allgather";
    if ((k_new != nullptr) != (v_new != nullptr)) return set_error(IVAB_ERR_INVALID, "%s: k_new and v_new go together", fn);
    if (kv_dtype != dtype && kv_dtype != IVAB_F8E4M3)
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: the pools hold the dtype of q, or IVAB_F8E4M3", fn);
    if (kv_dtype == IVAB_F8E4M3 && (!(k_scale > 0.f) || !(v_scale > 0.f)))
        return set_error(IVAB_ERR_INVALID, "%s: scales must be positive", fn);
    if (kv_dtype != IVAB_F8E4M3) k_scale = v_scale = 1.f;
    if (batch <= 0) return set_error(IVAB_ERR_INVALID, "%s: every rank must take part in the exchange: batch must be positive", fn);
    PeerParams pp{};
    if (int rc = make_peer_params(fn, local_block, block_bytes, peer_bufs, world, rank, slots, staging_offset, epoch,
                                  exchange_status, wait_limit_ns, &pp)) return rc;
    // the rows this call writes are the block that is sent: fp32, inside [local_block, local_block + block_bytes)
    const char* lo = static_cast<const char*>(local_block);
    const char* o = static_cast<const char*>(out);
    if (!out || o < lo || o >= lo + block_bytes || (lse && (reinterpret_cast<const char*>(lse) < lo ||
                                                            reinterpret_cast<const char*>(lse) >= lo + block_bytes)))
        return set_error(IVAB_ERR_INVALID, "%s: out (and lse) must lie inside the block that is exchanged", fn);
    return decode_entry(fn, q, q_stride_b, q_stride_h, k_pool, v_pool, pool_stride_head, pool_stride_page, block_table,
                        block_table_stride, ctx_len, ctx_begin, sink_tokens, out, out_stride_b, out_stride_h, lse, dtype,
                        IVAB_F32, kv_dtype, k_scale, v_scale, batch, q_heads, kv_heads, head_dim, page_size, num_pages,
                        max_pages_per_seq, scale, workspace, workspace_bytes, stream, k_new, v_new, new_stride_t,
                        new_stride_h, &pp);
}

extern "C" int ivab_decode_status(const void* workspace, int32_t* status_out, void* stream) {
    if (!workspace || !status_out) return set_error(IVAB_ERR_INVALID, "ivab_decode_status: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the header, and behind it the per-CTA slots of which every call rewrites the first 2 x SMs
    static_assert(kHdrWords * sizeof(int) % 256 == 0, "the slots follow the header without a gap");
    int32_t words[kHdrWords + kStatusSlots];
    const int n_slots = 2 * sm_count() < kStatusSlots ? 2 * sm_count() : kStatusSlots;
    if (int rc = check_cuda(cudaMemcpyAsync(words, workspace, (kHdrWords + n_slots) * sizeof(int),
                                            cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(status)")) return rc;
    if (int rc = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return rc;
    int32_t v = words[kHdrStatus];
    for (int i = 0; i < n_slots; ++i) v |= words[kHdrWords + i];
    *status_out = v;
    if (v != 0) return set_error(IVAB_ERR_DEVICE, "device status 0x%x", v);
    return IVAB_OK;
}

extern "C" int ivab_selftest_bounded_wait(int32_t* status, int64_t limit_ns, void* stream) {
    if (!status || limit_ns <= 0 || limit_ns > 1000000000ll)
        return set_error(IVAB_ERR_INVALID, "ivab_selftest_bounded_wait: need status and 0 < limit_ns <= 1e9");
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, (uint64_t)limit_ns);
    g_launches++;
    return check_cuda(cudaGetLastError(), "bounded_wait_selftest_kernel launch");
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant: the scratch lives in the library image.
// ------------------------------------------------------------------------------------------------

// 8 MiB of device memory per GPU that loads this library, held until the process exits.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address
// a kernel can use has to be asked for, once per device, with that device current.
int static_scratch_ptr(unsigned char** out) {
    // Host threads may race to fill an entry; they all store the same address, and the atomic makes
    // the store and the later loads well defined.
    static std::atomic<unsigned char*> ptrs[kMaxDevices];
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= kMaxDevices) return set_error(IVAB_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
    unsigned char* addr = ptrs[dev].load(std::memory_order_acquire);
    if (addr == nullptr) {
        void* p = nullptr;
        if (int rc = check_cuda(cudaGetSymbolAddress(&p, g_static_scratch), "cudaGetSymbolAddress(static scratch)"))
            return rc;
        if (p == nullptr) return set_error(IVAB_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        addr = static_cast<unsigned char*>(p);
        ptrs[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return IVAB_OK;
}

}  // namespace

extern "C" int ivab_paged_decode_attn_noalloc(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                              const void* k_pool, const void* v_pool,
                                              int64_t pool_stride_head, int64_t pool_stride_page,
                                              const int32_t* block_table, int64_t block_table_stride,
                                              const int32_t* ctx_len, const int32_t* ctx_begin, int64_t sink_tokens,
                                              void* out, int64_t out_stride_b, int64_t out_stride_h, float* lse,
                                              int dtype, int out_dtype, int64_t batch, int64_t q_heads, int64_t kv_heads,
                                              int64_t head_dim, int64_t page_size, int64_t num_pages,
                                              int64_t max_pages_per_seq, float scale, int32_t* status, void* stream) {
    const char* fn = "ivab_paged_decode_attn_noalloc";
    if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || q_heads % kv_heads)
        return set_error(IVAB_ERR_INVALID, "%s: bad sizes", fn);
    const int div = split_ratio(q_heads / kv_heads);   // (an unsupported ratio is reported by the call below)
    const size_t need = carve_workspace(nullptr, batch, q_heads, kv_heads * (div > 0 ? div : 1), head_dim, nullptr);
    if (need > kStaticScratchBytes)
        return set_error(IVAB_ERR_WORKSPACE,
                         "%s: this problem needs %zu bytes of scratch, the built-in buffer holds %zu; use "
                         "ivab_paged_decode_attn with a caller-provided workspace", fn, need, kStaticScratchBytes);
    unsigned char* scratch = nullptr;
    if (int rc = static_scratch_ptr(&scratch)) return rc;
    // Nothing in the scratch has to start at zero: the plan kernel rewrites the header (work counter,
    // status word, chunk count) and every partial that is read was written by this call.
    if (int rc = ivab_paged_decode_attn(q, q_stride_b, q_stride_h, k_pool, v_pool, pool_stride_head, pool_stride_page,
                                        block_table, block_table_stride, ctx_len, ctx_begin, sink_tokens, out, out_stride_b,
                                        out_stride_h, lse,
                                        dtype, out_dtype, batch, q_heads, kv_heads, head_dim, page_size, num_pages,
                                        max_pages_per_seq, scale, scratch, kStaticScratchBytes, stream))
        return rc;
    if (status == nullptr) return IVAB_OK;
    if (batch == 0)   // nothing was launched, so nothing can have gone wrong: the caller still gets a defined word
        return check_cuda(cudaMemsetAsync(status, 0, sizeof(int), static_cast<cudaStream_t>(stream)), "cudaMemsetAsync(status)");
    const int n_slots = 2 * sm_count() < kStatusSlots ? 2 * sm_count() : kStatusSlots;
    status_fold_kernel<<<1, kStatusSlots, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const int*>(scratch), n_slots, status);
    g_launches++;
    return check_cuda(cudaGetLastError(), "status_fold_kernel launch");
}
