// Definitions shared by the plan, attention and merge kernels of decode_attn.cu and by the page
// engines in decode_engines.cuh: constants, the workspace layout, the kernel parameter block and the
// optional phase-timing macros.  The structs are shared by several translation units (the host side in
// decode_attn.cu and one unit of kernel instantiations per dtype); constants and helpers are internal.
#pragma once

#include <cstdint>

#include "common.cuh"

namespace ivab {
namespace {

constexpr int kPage = 16;            // tokens per page (compile-time for the inner loops)
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kItemRing = 4;
constexpr int kMaxStages = 32;
static_assert(kMaxStages % kConsumerWarps == 0, "stage ring must divide among the consumer warps");
constexpr int kItemsPerSlot = 8;     // target work items per resident CTA
constexpr int kMinChunkPages = 8;
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
       kHdrWords = 64 };

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
};

namespace {

// v-th page a sequence reads -> index into its block table: `sink_pages` pages from the start, then
// the window's pages from begin / kPage on.
__device__ __forceinline__ int page_of(int v, int sink_pages, int begin) {
    return v < sink_pages ? v : v - sink_pages + begin / kPage;
}

// item ring entry (ints): what the producer tells the consumers about the next work item
enum { kItSeq = 0, kItHead = 1, kItPages = 2, kItPageBegin = 3, kItChunks = 4, kItIndex = 5, kItStart = 6, kItLen = 7,
       kItBegin = 8, kItSinkPages = 9, kItWords = 16 };

}  // namespace
}  // namespace ivab
