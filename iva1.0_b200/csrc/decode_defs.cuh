// Definitions shared by the plan, attention and merge kernels of decode_attn.cu and by the page
// engines in decode_engines.cuh: constants, the workspace layout, the kernel parameter block and the
// optional phase-timing macros.  The structs are shared by several translation units (the host side in
// decode_attn.cu and one unit of kernel instantiations per dtype); constants and helpers are internal.
#pragma once

#include <cstdint>

#include "common.cuh"
#include "peer_exchange.cuh"

namespace ivab {
namespace {

constexpr int kPage = 16;            // tokens per page (compile-time for the inner loops)
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kItemRing = 4;
constexpr int kMaxStages = 32;
static_assert(kMaxStages % kConsumerWarps == 0, "stage ring must divide among the consumer warps");
constexpr int kItemsPerSlot = 8;     // target work items per resident CTA
constexpr int kDirectSig0 = 0x49564142, kDirectSig1 = 0x5f637472, kDirectSig2 = 0x2e763031;
constexpr int kDirectBigKB = 768;     // plan-free mode: KB of K/V per CTA from which a batch counts as large (finer items, work counter)
constexpr int kMinChunkPages = 8;
constexpr int kDefaultItemOrder = 2;  // 0: kv-head-major, 1: chunk-major, 2: chunk-major for ragged batches only (see split_id)
// Plan-free ("direct") mode, for batches small enough that one warp holds a sequence per lane:
constexpr int kDirectMaxBatch = 32;
constexpr int kDirectItemsPerSlot = 2;       // work items per resident CTA the chunk size aims for
constexpr int kDirectMinChunkPages = 32;     // below this an item is cheaper to finish than to split and merge
constexpr int kStatusSlots = 512;            // per-CTA status words behind the header (at least 2 x SMs)
constexpr int kMergeWarpMax = 32;            // a sequence of at most this many chunks is merged by a single warp per query head
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s
constexpr int kMaxDevices = 64;      // device ordinals the per-device host caches cover

// Optional phase timing (debug builds only, -DIVAB_PROFILE): lane 0 of every warp accumulates
// clock64() deltas per phase and adds them to 64-bit counters in header words 16..47.
#ifdef IVAB_PROFILE
#define PROF_DECL long long prof_t0 = clock64(); long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define PROF_MARK(i) { const long long prof_t1 = clock64(); prof_acc[i] += prof_t1 - prof_t0; prof_t0 = prof_t1; }
#define PROF_FLUSH(base) if (lane == 0) { for (int i = 0; i < 8; ++i) atomicAdd(reinterpret_cast<unsigned long long*>(p.ws.header + 16) + (base) + i, (unsigned long long)prof_acc[i]); }
// Timeline stamps (%globaltimer, ns) in header words 48..63: [0] plan start, [1] plan end, [2] first
// attention CTA started, [3] first CTA past the dependency wait, [4] first page consumed, [5] last
// consumer warp done, [6] first merge CTA past its wait, [7] last merge CTA done.
#define PROF_STAMP_PTR(hdr) (reinterpret_cast<unsigned long long*>((hdr) + 48))
#define PROF_STAMP_SET(hdr, i) { PROF_STAMP_PTR(hdr)[i] = globaltimer_ns(); }
#define PROF_STAMP_MIN(hdr, i, t) atomicMin(PROF_STAMP_PTR(hdr) + (i), (unsigned long long)(t));
#define PROF_STAMP_MAX(hdr, i, t) atomicMax(PROF_STAMP_PTR(hdr) + (i), (unsigned long long)(t));
#else
#define PROF_DECL
#define PROF_MARK(i)
#define PROF_FLUSH(base)
#endif

// header words at the start of the workspace
enum { kHdrNumChunks = 0, kHdrChunkPages = 1, kHdrCounter = 2, kHdrStatus = 3, kHdrTotalItems = 4, kHdrNumSplit = 5, kHdrNumBig = 6,
       kHdrChunkMajor = 7,   // order in which the items are handed out, chosen by the plan kernel
       // Plan-free mode's work counter and three signature words (one 16-byte unit).  The merge kernel of every
       // plan-free call leaves {0, signature} behind once the attention kernel is done; an attention kernel that
       // finds the signature knows the counter is zero and hands the items of a large batch out through it; one
       // that does not (the first call on a workspace, whose memory is not initialised) assigns them statically,
       // as every call does for a batch that is not large.
       kHdrDirectCounter = 8, kHdrDirectSig = 9,
       kHdrMergeDone = 12,   // merge CTAs that have finished (zeroed by attention CTA 0 of the same call); the last one runs the peer exchange
       kHdrWords = 64 };
// Status protocol.  header[kHdrStatus] holds the bits of the planning step: written by the plan kernel,
// or (plan-free mode) by CTA 0 of the attention kernel.  Every CTA of the attention kernel additionally
// stores its own bits -- bad page ids, an expired wait -- into slot blockIdx.x of `status_slots` when its
// last warp leaves, unconditionally, so no word has to be cleared before a call: the status of a call is
// the OR of the header word and of the first 2 x SMs slots (a grid of one CTA per SM writes two each).

}  // namespace

struct ChunkDesc {
    int seq, page_begin, n_pages, chunk_idx, n_chunks, pad0, pad1, pad2;
};
static_assert(sizeof(ChunkDesc) == 32, "ChunkDesc is two 16-byte vectors");

struct Workspace {
    int* header;
    int* pos_prefix;      // [B+1] exclusive prefix of chunks over sequences in processing order
    int* order;           // [B]   sequence id at each position of the processing order
    int* seq_first;       // [B]   first chunk index of each sequence
    int* seq_count;       // [B]   number of chunks of each sequence
    int* split_list;      // [B]   ids of the sequences that were cut into more than one chunk: those with at most
                          //       kMergeWarpMax chunks from the front, those with more from the back
    ChunkDesc* chunks;    // [cap]
    float* part_ml;       // [cap*Hkv][G][2]   (running max in log2 units, sum)
    float* part_o;        // [cap*Hkv][G][D]
    int* status_slots;    // [kStatusSlots] per-CTA status words, directly behind the header
#ifdef IVAB_PROFILE
    unsigned long long* prof_cta;   // [kStatusSlots][4]: per CTA start, first page, last warp done (ns), items
#endif
    int cap;
    int target_chunks;
};


struct DecodeParams {
    const void* q; int64_t q_sb, q_sh;
    const char* k_pool; const char* v_pool; int64_t pool_sh_bytes, pool_sp_bytes;
    const int32_t* block_table; int64_t bt_stride;
    void* out; int64_t out_sb, out_sh; float* lse;
    int out_f32;             // out holds fp32 (strides in fp32 elements) instead of q's type
    int Hq, num_pages;
    int group;               // query heads per KV head; the kernels' template group size is this rounded up to 1, 2, 4 or 8
    int kv_div;              // work items number virtual KV heads; virtual head h reads the slab of KV head h / kv_div
    int sink_tokens;           // keys [0, sink_tokens) stay visible in front of a window (0 = none)
    float v_scale;             // 8-bit KV storage: V = v_scale * stored value (1 otherwise); K's scale is folded into scale_log2
    float scale_log2;          // scale * log2(e): scores are kept in base-2 units
    int stages;
    uint64_t wait_limit_ns;
    Workspace ws;
    // Plan-free mode (direct != 0): there is no plan kernel; every CTA derives the chunking from ctx_len
    // itself and takes the items blockIdx.x, blockIdx.x + gridDim.x, ... of the (kv head, chunk) list.
    int direct;
    int batch, max_pages, n_virt_heads;        // sequences, block-table width, KV heads the items number
    int direct_target_items, direct_min_chunk; // chunk size = max(min_chunk, ceil(total_pages * heads / target_items))
    int direct_grid;                           // CTAs of the attention launch
    int direct_dynamic;                        // 1: a merge kernel follows and re-arms the work counter, so the attention kernel may use it
    int direct_big_target_items;               // target_items of a large batch (0: same as direct_target_items)
    int direct_big_pages;                      // pages per CTA from which a batch counts as large
    int xchg_on;                               // head-parallel decode: the last merge CTA also runs the all-gather over peer memory
    PeerParams xchg;
    int status_slots_per_cta;                  // 2 when the grid is one CTA per SM, else 1
    int chunk_major;                           // order in which items are handed out: 0, 1, or 2 = as the plan kernel decided
    const int32_t* ctx_len; const int32_t* ctx_begin;
    // Fused decode step (k_new != nullptr): the newest token of every sequence -- position ctx_len - 1 -- is
    // written into its page by the CTA that is about to read that page (new tokens [batch, kv_heads, D] in q's
    // type, strides in bytes; 8-bit pools store fp8(x * inv_scale)).
    const char* k_new; const char* v_new; int64_t new_st_bytes, new_sh_bytes;
    float k_inv_scale, v_inv_scale;
};

namespace {

// v-th page a sequence reads -> index into its block table: `sink_pages` pages from the start, then
// the window's pages from begin / kPage on.
__device__ __forceinline__ int page_of(int v, int sink_pages, int begin) {
    return v < sink_pages ? v : v - sink_pages + begin / kPage;
}

// Sequence s attends the keys [0, sink) and [begin, L): L is ctx_len clamped to the block table, begin is
// ctx_begin (0 without one) clamped to [0, L], sink is sink_tokens clamped to begin.  Only the pages that
// hold such keys are read: `sink_pages` pages from the start of the block table, then the pages from
// begin / kPage on.  A sink page that is also the window's first page is read once, as a window page.
// Returns the number of pages to read; sets *bad when the raw values lie outside their ranges.
__device__ __forceinline__ int seq_page_range(const int32_t* ctx_len, const int32_t* ctx_begin, int sink_tokens, int max_pages,
                                              int s, int* L_out, int* begin_out, int* sink_pages_out, bool* bad) {
    const int L_raw = ctx_len[s];
    const long long cap_len = (long long)max_pages * kPage;
    int L = L_raw < 0 ? 0 : ((long long)L_raw > cap_len ? (int)cap_len : L_raw);
    const int b_raw = ctx_begin != nullptr ? ctx_begin[s] : 0;
    if (bad != nullptr) *bad = L_raw < 0 || (long long)L_raw > cap_len || b_raw < 0 || b_raw > L_raw;
    int b = b_raw < 0 ? 0 : (b_raw > L ? L : b_raw);
    if (sink_tokens >= b) b = 0;   // the sink keys reach the window: nothing is hidden
    const int sink = b > 0 ? sink_tokens : 0;
    const int first_window_page = b / kPage;
    int sp = (sink + kPage - 1) / kPage;
    if (sp > first_window_page) sp = first_window_page;
    // (when the window is empty its first page would hold no visible key: read sink pages only;
    //  a sink that ends on the window's page is then lost with it, so widen sp in that case)
    const int window_pages = b >= L ? 0 : (L + kPage - 1) / kPage - first_window_page;
    if (window_pages == 0) sp = (sink + kPage - 1) / kPage;
    *L_out = L; *begin_out = b; *sink_pages_out = sp;
    return sp + window_pages;
}

// The plan of the plan-free mode, held by one warp: lane s describes sequence s (lanes >= batch are empty).
struct DirectPlan {
    int pages, first, n;          // pages to read, index of the first chunk, number of chunks (>= 1 for lanes < batch)
    int L, begin, sink_pages;
    int num_chunks;               // warp-uniform: chunks of the whole batch
    bool bad;                     // warp-uniform: some ctx_len / ctx_begin was out of range
    bool big;                     // warp-uniform: a large batch (cut with big_target_items)
};

// Must be called by all 32 lanes.  Deterministic in its inputs, so every CTA of the attention kernel and of
// the merge kernel arrives at the same plan.  Sequences are split evenly into ceil(pages / c) chunks with
// c = max(min_chunk, ceil(total_pages * heads / target_items)) pages.  `big_target_items` (0 = none) replaces
// target_items from big_pages pages per CTA on: a batch of that size is served through the work counter
// (when it is armed), where finer items shorten the tail.
__device__ __forceinline__ DirectPlan direct_plan(const int32_t* ctx_len, const int32_t* ctx_begin, int sink_tokens, int max_pages,
                                                  int batch, int heads, int target_items, int min_chunk, int big_target_items,
                                                  int big_pages, int grid, int lane) {
    DirectPlan d{};
    bool bad = false;
    if (lane < batch) d.pages = seq_page_range(ctx_len, ctx_begin, sink_tokens, max_pages, lane, &d.L, &d.begin, &d.sink_pages, &bad);
    d.bad = __any_sync(0xffffffffu, bad);
    long long total = d.pages;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    // (one sequence alone is split evenly by construction: finer items would only add partial results to merge)
    d.big = big_target_items > 0 && batch > 1 && total * heads >= (long long)grid * big_pages;
    if (d.big) target_items = big_target_items;
    long long c64 = (total * heads + target_items - 1) / target_items;
    if (c64 < min_chunk) c64 = min_chunk;
    const int c = (int)(c64 > 0x3fffffff ? 0x3fffffff : c64);
    d.n = lane < batch ? (d.pages + c - 1) / c : 0;
    if (lane < batch && d.n < 1) d.n = 1;   // an empty sequence still gets one (empty) item, which writes zeros / -inf
    int incl = d.n;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    d.first = incl - d.n;
    d.num_chunks = __shfl_sync(0xffffffffu, incl, 31);
    return d;
}

// Chunk `ci` of the batch-wide chunk list as a descriptor (all lanes, warp-uniform result).
__device__ __forceinline__ ChunkDesc direct_desc(const DirectPlan& d, int ci, int batch, int lane) {
    const unsigned owners = __ballot_sync(0xffffffffu, lane < batch && d.first <= ci);
    const int s = owners ? 31 - __clz(owners) : 0;    // `first` increases strictly with the lane
    const int first = __shfl_sync(0xffffffffu, d.first, s), n = __shfl_sync(0xffffffffu, d.n, s);
    const int pages = __shfl_sync(0xffffffffu, d.pages, s);
    const int j = ci - first;
    const int per = n > 0 ? pages / n : 0, rem = n > 0 ? pages % n : 0;   // even split: the first `rem` chunks get one more page
    ChunkDesc c;
    c.seq = s;
    c.page_begin = j * per + (j < rem ? j : rem);
    c.n_pages = per + (j < rem ? 1 : 0);
    c.chunk_idx = j;
    c.n_chunks = n;
    c.pad0 = __shfl_sync(0xffffffffu, d.L, s);
    c.pad1 = __shfl_sync(0xffffffffu, d.begin, s);
    c.pad2 = __shfl_sync(0xffffffffu, d.sink_pages, s);
    return c;
}

// item ring entry (ints): what the producer tells the consumers about the next work item
enum { kItSeq = 0, kItHead = 1, kItPages = 2, kItPageBegin = 3, kItChunks = 4, kItIndex = 5, kItStart = 6, kItLen = 7,
       kItBegin = 8, kItSinkPages = 9, kItWords = 16 };

}  // namespace
}  // namespace ivab
