// The persistent split-K attention kernel, the logsumexp merge kernel and their launch code.
// Included by the per-dtype instantiation units (decode_inst_*.cu); everything here has internal
// linkage, the units export one dispatch function each (decode_dispatch.h).
#pragma once

#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "decode_defs.cuh"      // constants, workspace layout, kernel parameters
#include "decode_engines.cuh"   // the page engines and the kernel's shared-memory layout

namespace ivab {

extern std::atomic<long long> g_launches;

namespace {

// ------------------------------------------------------------------------------------------------
// 2. persistent split-K attention
// ------------------------------------------------------------------------------------------------

// Fused decode step: one warp writes the newest token's K and V rows of one KV head into their slot of the
// pool (T: type of the new tokens = type of q; TKV: storage type of the pool).  The rows are copied verbatim,
// or -- 8-bit pools -- quantised exactly as the stand-alone append does (fp8(x * inv_scale), saturating).
// The loads (the block-table entry of the token's page and the two source rows, one 16-byte vector per lane
// and register) are issued one work item ahead; the stores follow when the item starts.
template <typename T, int D>
struct NewestRow {
    static constexpr int kVecs = D * (int)sizeof(T) / 16;      // 16-byte vectors per source row
    static constexpr int kRegs = (2 * kVecs + 31) / 32;
    uint4 v[kRegs];
    int pid;
    bool on;
};

template <typename T, int D>
__device__ __forceinline__ NewestRow<T, D> load_newest_row(const DecodeParams& p, const ChunkDesc& d, int slab, bool valid, int lane) {
    using R = NewestRow<T, D>;
    R r{};
    r.on = valid && p.k_new != nullptr && d.chunk_idx == d.n_chunks - 1 && d.pad0 > 0;
    if (!r.on) return r;
    r.pid = __ldg(p.block_table + (int64_t)d.seq * p.bt_stride + (d.pad0 - 1) / kPage);
    const int64_t row = (int64_t)d.seq * p.new_st_bytes + (int64_t)slab * p.new_sh_bytes;
#pragma unroll
    for (int k = 0; k < R::kRegs; ++k) {
        const int v = lane + 32 * k;
        if (v < 2 * R::kVecs)
            r.v[k] = __ldg(reinterpret_cast<const uint4*>((v >= R::kVecs ? p.v_new : p.k_new) + row) + (v >= R::kVecs ? v - R::kVecs : v));
    }
    return r;
}

template <typename T, typename TKV, int D>
__device__ __forceinline__ void store_newest_row(const DecodeParams& p, const NewestRow<T, D>& r, const ChunkDesc& d, int slab,
                                                 int* cta_status, int lane) {
    using R = NewestRow<T, D>;
    if (r.pid < 0 || r.pid >= p.num_pages) {
        if (lane == 0) atomicOr(cta_status, kStatusBadPage);    // skipped, never written out of range
        return;
    }
    const int pos = d.pad0 - 1;
    const int64_t off = (int64_t)slab * p.pool_sh_bytes + (int64_t)r.pid * p.pool_sp_bytes +
                        (int64_t)(pos % kPage) * (D * (int)sizeof(TKV));
#pragma unroll
    for (int k = 0; k < R::kRegs; ++k) {
        const int v = lane + 32 * k;
        if (v >= 2 * R::kVecs) continue;
        const bool is_v = v >= R::kVecs;
        const int i = is_v ? v - R::kVecs : v;
        char* dst = const_cast<char*>(is_v ? p.v_pool : p.k_pool) + off;
        if constexpr (std::is_same<T, TKV>::value) {
            *reinterpret_cast<uint4*>(dst + i * 16) = r.v[k];
        } else {
            static_assert(sizeof(T) == 2 && sizeof(TKV) == 1, "quantising append: 16-bit tokens into 8-bit pools");
            float f[8];
            Elt<T>::unpack(r.v[k], f);
            const float is = is_v ? p.v_inv_scale : p.k_inv_scale;
            uint2 q;
            q.x = (uint32_t)pack_fp8x2(f[0] * is, f[1] * is) | ((uint32_t)pack_fp8x2(f[2] * is, f[3] * is) << 16);
            q.y = (uint32_t)pack_fp8x2(f[4] * is, f[5] * is) | ((uint32_t)pack_fp8x2(f[6] * is, f[7] * is) << 16);
            *reinterpret_cast<uint2*>(dst + i * 8) = q;
        }
    }
}

template <typename T, int D, int G, int ENG, typename TKV = T>
__global__ void __launch_bounds__(kThreads, EngineSelect<ENG, T, TKV, D, G>::type::CTAS_PER_SM)
decode_kernel(const __grid_constant__ DecodeParams p, const __grid_constant__ TensorMaps tm) {
    using Eng = typename EngineSelect<ENG, T, TKV, D, G>::type;
    using C = SmemLayout<Eng::SCRATCH_PER_WARP, D, G>;
    extern __shared__ unsigned char smem_raw[];
    // the carve-up assumes a 1 KB-aligned base; the launch reserves 1 KB of slack for this
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = p.stages;
#ifdef IVAB_PROFILE
    const uint64_t prof_cta_start = globaltimer_ns();
#endif

    const uint32_t bars = smem_u32(smem + C::OFF_BARS);
    auto bar_full = [&](int s) { return bars + 8u * s; };
    auto bar_empty = [&](int s) { return bars + 8u * (kMaxStages + s); };
    auto bar_item_full = [&](int s) { return bars + 8u * (2 * kMaxStages + s); };
    auto bar_item_empty = [&](int s) { return bars + 8u * (2 * kMaxStages + kItemRing + s); };
    const uint32_t bar_combined = bars + 8u * (2 * kMaxStages + 2 * kItemRing);   // phase i completes when item i's states are combined
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_ABORT);
    int* merge_cnt = reinterpret_cast<int*>(smem + C::OFF_ABORT + 4);   // warps that have published the current item
    int* cta_status = reinterpret_cast<int*>(smem + C::OFF_ABORT + 8);  // IVAB_STATUS_* bits raised by this CTA
    int* exit_cnt = reinterpret_cast<int*>(smem + C::OFF_ABORT + 12);   // warps that have left the kernel
    volatile int* items = reinterpret_cast<volatile int*>(smem + C::OFF_ITEMS);
    unsigned char* stage_base = smem + C::OFF_STAGES;

    if constexpr (Eng::kTiled) {
        // (the descriptors are kernel parameters, so this needs nothing from the kernels before this one)
        if (threadIdx.x == kConsumerWarps * 32) { prefetch_tensormap(&tm.k); prefetch_tensormap(&tm.v); }
    }
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < stages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int s = 0; s < kItemRing; ++s) { mbar_init(bar_item_full(s), 1); mbar_init(bar_item_empty(s), kConsumerWarps); }
        mbar_init(bar_combined, 1);
        *merge_cnt = 0;
        *cta_status = 0;
        *exit_cnt = 0;
        fence_mbar_init();
    }
    __syncthreads();   // the only CTA-wide barrier: before any warp can have unwound

    // Everything above overlapped the plan kernel; the work list is read from here on.  The merge
    // kernel may be scheduled as soon as CTAs of this grid retire (it waits for the whole grid).
    grid_dependency_wait();
    grid_launch_dependents();
#ifdef IVAB_PROFILE
    if (threadIdx.x == 0) {
        PROF_STAMP_MIN(p.ws.header, 2, prof_cta_start)
        PROF_STAMP_MIN(p.ws.header, 3, globaltimer_ns())
    }
#endif

    const bool direct = p.direct != 0;
    int num_chunks = direct ? 0 : p.ws.header[kHdrNumChunks];
    int total_items = direct ? 0 : p.ws.header[kHdrTotalItems];
    int* counter = p.ws.header + kHdrCounter;
    const uint64_t limit = p.wait_limit_ns;
    // Every warp calls this exactly once, as the last thing it does.  The warp that arrives last stores the
    // bits this CTA raised into the CTA's status slot(s) -- unconditionally, so that the slots never need
    // clearing; in plan-free mode CTA 0 also defines the header's status word, which no plan kernel wrote.
    auto leave = [&]() {
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            if (atomicAdd(exit_cnt, 1) == kConsumerWarps) {
                __threadfence_block();
                const int st = *reinterpret_cast<volatile int*>(cta_status) | (*abort_flag ? kStatusWaitTimeout : 0);
                for (int k = 0; k < p.status_slots_per_cta; ++k) p.ws.status_slots[blockIdx.x + k * gridDim.x] = st;
                if (direct && blockIdx.x == 0) p.ws.header[kHdrStatus] = 0;
                if (p.xchg_on && blockIdx.x == 0) p.ws.header[kHdrMergeDone] = 0;   // counted up by the merge CTAs of this call
            }
        }
    };

    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp ------------------------------------------
        // The stage ring is split into one sub-ring per consumer warp (stage = slot*W + warp).
        // Page k of an item goes to warp (start + k) % W with start = (seq + chunk) % W, so which
        // warp sums which pages -- and therefore every fp32 rounding -- depends only on the
        // inputs, never on which CTA happened to pick the item up: results are bit-reproducible.
        int cnt[kConsumerWarps];   // pages issued to each warp so far
#pragma unroll
        for (int i = 0; i < kConsumerWarps; ++i) cnt[i] = 0;
        const int spw = stages / kConsumerWarps;   // stages per warp
        int published = 0;  // items published so far
        bool aborted = false;
        // The fetch of an item is three dependent global accesses (work counter -> chunk descriptor ->
        // block-table entries), about a microsecond each under load.  They are software-pipelined
        // across items: while the pages of item i are being issued, the block-table entries of item
        // i+1, the descriptor of item i+2 and the id of item i+3 are in flight, so the TMA issue
        // stream does not pause at item boundaries.
        // Plan-free mode: this warp derives the chunking from ctx_len itself (lane s holds sequence s) and
        // the CTA takes the items blockIdx.x, blockIdx.x + gridDim.x, ...: two dependent global accesses
        // (ctx_len, block-table entries) before the first page is requested.  Further items come from the
        // plan-free work counter when the batch is large and the previous call's merge kernel left the counter
        // armed (signature present), else statically: uninitialised workspace memory is never trusted.
        DirectPlan dplan{};
        int static_next = (int)blockIdx.x;
        bool dynamic = !direct;
        if (direct) {
            int4 sig = make_int4(0, 0, 0, 0);   // (in flight while the lengths are loaded and the plan is derived)
            if (p.direct_dynamic && lane == 0) sig = __ldcg(reinterpret_cast<const int4*>(p.ws.header + kHdrDirectCounter));
            // the block-table rows are needed right after the lengths: start them towards the L2 now
            if (lane < p.batch) prefetch_l2(p.block_table + (int64_t)lane * p.bt_stride);
            dplan = direct_plan(p.ctx_len, p.ctx_begin, p.sink_tokens, p.max_pages, p.batch, p.n_virt_heads,
                                p.direct_target_items, p.direct_min_chunk, p.direct_big_target_items, p.direct_big_pages, p.direct_grid, lane);
            num_chunks = dplan.num_chunks;
            total_items = num_chunks * p.n_virt_heads;
            if (dplan.big) {   // a large batch: through the work counter, if the previous call left it armed
                dynamic = __shfl_sync(0xffffffffu, sig.y == kDirectSig0 && sig.z == kDirectSig1 && sig.w == kDirectSig2, 0) != 0;
                if (dynamic) counter = p.ws.header + kHdrDirectCounter;
            }
            if (dplan.bad && lane == 0) atomicOr(cta_status, kStatusBadCtxLen);
            if (num_chunks > p.ws.cap) {   // cannot happen while target_items <= kItemsPerSlot x resident CTAs
                if (lane == 0) atomicOr(cta_status, kStatusOverflow);
                total_items = 0;
            }
        }
        auto fetch_id_async = [&]() {   // lane 0 holds the result; broadcast it only when it is needed
            int v = 0;
            if (!dynamic) { static_next += (int)gridDim.x; v = static_next; }
            else if (direct) {
                // Plan-free: a CTA's first two items are static; the counter hands out what lies beyond two
                // rounds over the grid.  Ids are claimed up to three items ahead, so claiming everything from
                // the counter would let the CTAs that ask first take most of a short list.
                if (static_next < (int)gridDim.x) { static_next += (int)gridDim.x; v = static_next; }
                else if (total_items <= 2 * (int)gridDim.x) v = total_items;
                else if (lane == 0) v = 2 * (int)gridDim.x + atomicAdd(counter, 1);
            }
            else if (lane == 0) v = (int)gridDim.x + atomicAdd(counter, 1);
            return v;
        };
        auto fetch_id = [&]() { return __shfl_sync(0xffffffffu, fetch_id_async(), 0); };
        // Item id -> (kv head, index in the chunk list).  Head-major order keeps the CTAs that run at the same
        // time on one or two heads' slabs of the pool; chunk-major order walks the chunk list (longest
        // sequences first) once for all heads, so the items handed out last are the shortest ones.
        // A batch of equal lengths is served head-major (measured 0.5-1 % faster: fewer slabs are open at a
        // time), a ragged one chunk-major (its long items must not be the ones that start last).
        const bool chunk_major = p.chunk_major == 2 ? (!direct && p.ws.header[kHdrChunkMajor] != 0) : p.chunk_major == 1;
        auto split_id = [&](int id, int* h_out, int* ci_out) {
            if (chunk_major) { const int ci = id / p.n_virt_heads; *ci_out = ci; *h_out = id - ci * p.n_virt_heads; }
            else { const int h = id / num_chunks; *h_out = h; *ci_out = id - h * num_chunks; }
        };
        auto load_desc = [&](int id, int* h_out) {
            ChunkDesc d{};
            *h_out = 0;
            int h = 0, ci = 0;
            if (id < total_items) split_id(id, &h, &ci);
            if (direct) {      // (every lane takes part in the shuffles, whatever the id)
                d = direct_desc(dplan, ci, p.batch, lane);
                if (id >= total_items) d = ChunkDesc{};
                *h_out = h;
            } else if (id < total_items) {
                const int4* src = reinterpret_cast<const int4*>(p.ws.chunks + ci);
                // written by the plan kernel of this call, which may still have been running when this
                // CTA started: not read-only data, so no ld.global.nc here
                const int4 a = __ldcg(src), b = __ldcg(src + 1);
                d.seq = a.x; d.page_begin = a.y; d.n_pages = a.z; d.chunk_idx = a.w; d.n_chunks = b.x; d.pad0 = b.y;
                d.pad1 = b.z; d.pad2 = b.w;
                *h_out = h;
            }
            return d;
        };
        auto load_pages = [&](const ChunkDesc& d, int p0) {   // this lane's entry of a 32-page batch
            // (the value is validated where it is used, so that this load stays a prefetch)
            int mine = 0;
            if (p0 + lane < d.n_pages)
                mine = __ldg(p.block_table + (int64_t)d.seq * p.bt_stride +
                             page_of(d.page_begin + p0 + lane, d.pad2, d.pad1));
            return mine;
        };
        PROF_DECL
        const uint64_t stream_policy = l2_policy_evict_first();   // K/V pages are read once
        // the first item of a CTA is its own index (no round trip to the work counter before the
        // first page can be requested); the counter hands out the items from gridDim.x on
        int id0 = (int)blockIdx.x, id1 = fetch_id_async(), id2 = fetch_id_async();   // (both round trips in flight at once)
        id1 = __shfl_sync(0xffffffffu, id1, 0); id2 = __shfl_sync(0xffffffffu, id2, 0);
        int h0, h1;
        ChunkDesc d0 = load_desc(id0, &h0);
        ChunkDesc d1 = load_desc(id1, &h1);
        int bt0 = id0 < total_items ? load_pages(d0, 0) : 0;
        NewestRow<T, D> nr0 = load_newest_row<T, D>(p, d0, h0 / p.kv_div, id0 < total_items, lane);
        for (;;) {
            const int item = id0, h = h0;
            const ChunkDesc d = d0;
            const bool done = item >= total_items;
            // prefetch for the following items (ids past the end of the list load nothing)
            int bt1 = 0, h2 = 0, id3_raw = 0;
            ChunkDesc d2{};
            NewestRow<T, D> nr1{};
            if (!done) {
                if (id1 < total_items) {
                    bt1 = load_pages(d1, 0);
                    nr1 = load_newest_row<T, D>(p, d1, h1 / p.kv_div, true, lane);
                }
                d2 = load_desc(id2, &h2);
                id3_raw = fetch_id_async();
            }
            PROF_MARK(0)   // fetch / prefetch issue
            const int slot = published % kItemRing;
            if (!mbar_wait_bounded(bar_item_empty(slot), ((published / kItemRing) & 1) ^ 1, abort_flag, limit)) {
                aborted = true; break;
            }
            PROF_MARK(1)   // wait for a free item slot
            if (lane == 0) {
                volatile int* it = items + slot * kItWords;
                it[kItSeq] = d.seq; it[kItHead] = h; it[kItPages] = done ? -1 : d.n_pages;
                int ci = 0, hh = 0;
                if (!done) split_id(item, &hh, &ci);
                // (where this item's partial result is stored: head-major, whatever the processing order)
                it[kItPageBegin] = d.page_begin; it[kItChunks] = d.n_chunks; it[kItIndex] = hh * num_chunks + ci;
                it[kItStart] = (d.seq + d.chunk_idx) % kConsumerWarps; it[kItLen] = d.pad0; it[kItBegin] = d.pad1; it[kItSinkPages] = d.pad2;
                mbar_arrive(bar_item_full(slot));
            }
            ++published;
            if (done) break;

            const int slab = h / p.kv_div;   // the KV head whose pages this item reads
            const char* kbase = p.k_pool + (int64_t)slab * p.pool_sh_bytes;
            const char* vbase = p.v_pool + (int64_t)slab * p.pool_sh_bytes;
            // Fused decode step: the item that ends a sequence reads the page of its newest token, so this
            // warp first writes that token's rows (position L - 1) of this KV head into the page -- from
            // registers, the loads went out one item ago -- and orders the stores before its own TMA reads
            // when it gets to the item's last request, which is the one that contains that page.  No other
            // CTA reads that page -- except, with more than 8 query heads per KV head, the items of the sibling
            // head groups, which write the same bytes themselves before they read.
            bool need_fence = false;
            if (nr0.on) {
                store_newest_row<T, TKV, D>(p, nr0, d, slab, cta_status, lane);
                need_fence = true;
            }
            const int start = (d.seq + d.chunk_idx) % kConsumerWarps;
            int bt_next = bt0;
            for (int p0 = 0; p0 < d.n_pages && !aborted; p0 += 32) {
                const int mine = bt_next;
                if (p0 + 32 < d.n_pages) bt_next = load_pages(d, p0 + 32);   // in flight while this batch is issued
                const int in_batch = min(32, d.n_pages - p0);
                PROF_MARK(2)   // block-table entries available
                // Pages are issued a ring's worth at a time, ONE LANE PER PAGE: every lane waits for
                // its own stage and issues its own copies, so the issue cost of up to `stages` pages
                // overlaps.  A sub-batch never exceeds the ring (spw pages per consumer warp): a lane
                // must not wait two phases ahead of a stage's barrier.
                int nb = 0;
                for (int q0 = 0; q0 < in_batch && !aborted; q0 += nb) {
                    nb = min(stages, in_batch - q0);
                    // the newest token's page goes out on its own, behind the fence: the pages before it need not wait
                    if (need_fence && p0 + q0 + nb >= d.n_pages && nb > 1) nb -= 1;
                    if (need_fence && p0 + q0 + nb >= d.n_pages) {   // the request that reads the newest token's page
                        fence_proxy_async_all();
                        __syncwarp();
                        need_fence = false;
                    }
                    int pid = __shfl_sync(0xffffffffu, mine, (q0 + lane) & 31);
                    if (lane < nb && (pid < 0 || pid >= p.num_pages)) {
                        atomicOr(cta_status, kStatusBadPage);   // flagged, and page 0 is read instead of faulting
                        pid = 0;
                    }
                    const int b0 = (start + p0 + q0) & (kConsumerWarps - 1);
                    const int w = (b0 + lane) & (kConsumerWarps - 1);          // consumer warp of this lane's page
                    const int nth = lane >> 2;                                  // its rank among that warp's pages here
                    int base_c = 0;
#pragma unroll
                    for (int i = 0; i < kConsumerWarps; ++i) if (i == w) base_c = cnt[i];
                    const int c = base_c + nth;
                    bool fail = false;
                    if (lane < nb) {
                        const int stage = (c % spw) * kConsumerWarps + w;
                        if (!mbar_wait_bounded(bar_empty(stage), ((c / spw) & 1) ^ 1, abort_flag, limit)) {
                            fail = true;
                        } else {
                            const uint32_t dst = smem_u32(stage_base + (size_t)stage * Eng::STAGE_BYTES);
                            mbar_arrive_expect_tx(bar_full(stage), Eng::STAGE_BYTES);
                            if constexpr (Eng::kTiled) {
#pragma unroll
                                for (int t = 0; t < Eng::TILES; ++t) {
                                    tma_tile4d_g2s_hint(dst + t * Eng::TILE_BYTES, &tm.k, t * Eng::TILE_COLS, 0, pid, slab, bar_full(stage),
                                                        stream_policy);
                                    tma_tile4d_g2s_hint(dst + Eng::PAGE_BYTES + t * Eng::TILE_BYTES, &tm.v, t * Eng::TILE_COLS, 0, pid, slab,
                                                        bar_full(stage), stream_policy);
                                }
                            } else {
                                tma_bulk_g2s_hint(dst, kbase + (int64_t)pid * p.pool_sp_bytes, Eng::PAGE_BYTES, bar_full(stage),
                                                  stream_policy);
                                tma_bulk_g2s_hint(dst + Eng::PAGE_BYTES, vbase + (int64_t)pid * p.pool_sp_bytes,
                                                  Eng::PAGE_BYTES, bar_full(stage), stream_policy);
                            }
                        }
                    }
                    if (__any_sync(0xffffffffu, fail)) aborted = true;
                    // pages handed to consumer warp i in this sub-batch: lanes r_i, r_i+4, ... below nb
#pragma unroll
                    for (int i = 0; i < kConsumerWarps; ++i) {
                        const int r_i = (i - b0) & (kConsumerWarps - 1);
                        cnt[i] += nb > r_i ? (nb - r_i + kConsumerWarps - 1) / kConsumerWarps : 0;
                    }
                    PROF_MARK(3)   // stage wait + TMA issue of a sub-batch
                }
            }
            PROF_MARK(4)   // TMA issue
            if (aborted) break;
            id0 = id1; h0 = h1; d0 = d1; bt0 = bt1; nr0 = nr1;
            id1 = id2; h1 = h2; d1 = d2;
            id2 = __shfl_sync(0xffffffffu, id3_raw, 0);
        }
        PROF_FLUSH(0)
        if (aborted) {
            // Copies already issued still target this CTA's shared memory: give each of the
            // most recent `stages` copies a bounded chance to land before the CTA retires.
            volatile int no_abort = 0;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                // the copy whose empty-wait just failed was counted but never issued
                for (int m = cnt[w] > spw ? cnt[w] - spw : 0; m < cnt[w]; ++m)
                    mbar_wait_bounded(bar_full((m % spw) * kConsumerWarps + w), (m / spw) & 1, &no_abort,
                                      limit < 100000000ull ? limit : 100000000ull);
            }
        }
        leave();
        return;
    }

    // ---------------------------------- consumer warps --------------------------------------------
    unsigned char* scratch = smem + C::OFF_SCRATCH + warp * Eng::SCRATCH_PER_WARP;   // this warp's private scratch
    float* mrg_ml = reinterpret_cast<float*>(smem + C::OFF_MRG_ML);
    float* mrg_o = reinterpret_cast<float*>(smem + C::OFF_MRG_O);
    T* outg = static_cast<T*>(p.out);
    Eng eng;
    eng.setup(lane);
    eng.attach(scratch, lane);

    const int spw = stages / kConsumerWarps;   // stages of this warp's sub-ring
    int taken = 0;      // pages this warp has consumed so far (position in its sub-ring)
    int consumed = 0;   // items consumed
    PROF_DECL
    for (;;) {
        const int slot = consumed % kItemRing;
        if (!mbar_wait_bounded(bar_item_full(slot), (consumed / kItemRing) & 1, abort_flag, limit)) break;
        PROF_MARK(0)   // wait for the next item
        // The slot stays with this warp until the end of the item: what only the epilogue needs (sequence,
        // head, chunk count, where the partial goes) is read again there instead of living in registers
        // through the page loop.
        volatile int* it = items + slot * kItWords;
        const int n_pages = it[kItPages], page_begin = it[kItPageBegin], start = it[kItStart], L = it[kItLen];
        const int begin = it[kItBegin], sink_pages = it[kItSinkPages];
        if (n_pages < 0) break;   // sentinel: the work list is exhausted

        eng.begin_item(p, it[kItSeq], it[kItHead], lane);   // query heads of this kv head into registers, state reset
        PROF_MARK(1)   // q load issue

        bool ok = true;
        const int k0 = (warp - start + kConsumerWarps) % kConsumerWarps;
        for (int k = k0; k < n_pages; k += kConsumerWarps, ++taken) {
            const int stage = (taken % spw) * kConsumerWarps + warp;
            if (!mbar_wait_bounded(bar_full(stage), (taken / spw) & 1, abort_flag, limit)) { ok = false; break; }
            PROF_MARK(2)   // wait for page data
#ifdef IVAB_PROFILE
            if (taken == 0 && lane == 0) {
                PROF_STAMP_MIN(p.ws.header, 4, globaltimer_ns())
                atomicCAS(p.ws.prof_cta + blockIdx.x * 4 + 1, 0ull, (unsigned long long)globaltimer_ns());   // this CTA's first page
            }
#endif
            // Token t of this page is key 16*pg + t.  It counts if it lies below L and outside the
            // hole [sink, begin) between the sink keys and the window; only the last page of the
            // sequence, the last sink page and the first window page are cut by these bounds.
            const int pg = page_of(page_begin + k, sink_pages, begin);
            const int n_valid = min(kPage, L - pg * kPage);
            const int hole_lo = min(kPage, max(0, min(p.sink_tokens, begin) - pg * kPage));
            const int hole_hi = min(kPage, max(0, begin - pg * kPage));
            eng.page(p, stage_base + (size_t)stage * Eng::STAGE_BYTES, n_valid, hole_lo, hole_hi, lane, scratch);
            if (lane == 0) mbar_arrive(bar_empty(stage));
            PROF_MARK(3)   // page math
        }
        if (!ok) break;

        // ---- end of item: no CTA-wide barrier.  Every warp publishes its state and moves on to the
        // next item at once; the warp that arrives LAST combines the four states (always in warp
        // order 0..3, so the sum does not depend on who arrived when) and writes the result.  A
        // stalled ring costs bandwidth directly, so three of four sub-rings keep draining while
        // one warp does the combine.  The scratch is reused by the next item: a warp may overwrite
        // its state only after the previous item's combine has finished.
        if (consumed > 0 && !mbar_wait_bounded(bar_combined, (consumed - 1) & 1, abort_flag, limit)) break;
        PROF_MARK(4)   // wait for the previous combine
        const int seq = it[kItSeq], h = it[kItHead], n_chunks = it[kItChunks], item = it[kItIndex];
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_item_empty(slot));
        eng.publish(p, mrg_ml + (warp * G) * 2, mrg_o + (size_t)(warp * G) * D, lane);
        __threadfence_block();
        __syncwarp();
        int arrival = 0;
        if (lane == 0) arrival = atomicAdd(merge_cnt, 1);
        arrival = __shfl_sync(0xffffffffu, arrival, 0);
        if (arrival == kConsumerWarps - 1) {
            __threadfence_block();
            const volatile float* all_ml = mrg_ml;
            const volatile float* all_o = mrg_o;
            const int Gr = p.group;   // real heads of this KV head: rows Gr..G-1 of the states are padding
            for (int idx = lane; idx < Gr * D; idx += 32) {
                const int g = idx / D, dd = idx % D;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, all_ml[(w * G + g) * 2]);
                float Lsum = 0.f, O = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    const float mw = all_ml[(w * G + g) * 2];
                    const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
                    Lsum = fmaf(all_ml[(w * G + g) * 2 + 1], f, Lsum);
                    O = fmaf(all_o[(size_t)(w * G + g) * D + dd], f, O);
                }
                O *= p.v_scale;
                const int hq = h * Gr + g;
                if (n_chunks == 1) {
                    const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
                    const int64_t oi = (int64_t)seq * p.out_sb + (int64_t)hq * p.out_sh + dd;
                    if (p.out_f32) static_cast<float*>(p.out)[oi] = O * inv;
                    else Elt<T>::store(outg + oi, O * inv);
                    if (dd == 0 && p.lse != nullptr)
                        p.lse[(int64_t)seq * p.Hq + hq] = Lsum > 0.f ? (M + log2f(Lsum)) * 0.6931471805599453f : -INFINITY;
                } else {
                    p.ws.part_o[((size_t)item * Gr + g) * D + dd] = O;
                    if (dd == 0) {
                        p.ws.part_ml[((size_t)item * Gr + g) * 2] = M;
                        p.ws.part_ml[((size_t)item * Gr + g) * 2 + 1] = Lsum;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) { *merge_cnt = 0; mbar_arrive(bar_combined); }
        }
        PROF_MARK(5)   // publish (+ combine if last)
        ++consumed;
    }
    PROF_FLUSH(8)
#ifdef IVAB_PROFILE
    if (lane == 0) {
        atomicMax(p.ws.prof_cta + blockIdx.x * 4 + 2, (unsigned long long)globaltimer_ns());
        if (warp == 0) { p.ws.prof_cta[blockIdx.x * 4 + 0] = prof_cta_start; p.ws.prof_cta[blockIdx.x * 4 + 3] = (unsigned long long)consumed; }
        PROF_STAMP_MAX(p.ws.header, 5, globaltimer_ns())
        atomicMin(reinterpret_cast<unsigned long long*>(p.ws.header + 14), (unsigned long long)globaltimer_ns());   // first warp done
    }
#endif
    leave();
}

// ------------------------------------------------------------------------------------------------
// 3. logsumexp merge of split-K partials
// ------------------------------------------------------------------------------------------------

constexpr int kMergeWarps = 8;

// VPL consecutive floats from a pointer aligned to VPL * 4 bytes (at most 16)
template <int VPL>
__device__ __forceinline__ void load_row(const float* src, float (&v)[VPL]) {
    if constexpr (VPL % 4 == 0) {
#pragma unroll
        for (int i = 0; i < VPL / 4; ++i) {
            const float4 t = reinterpret_cast<const float4*>(src)[i];
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    } else if constexpr (VPL == 2) {
        const float2 t = *reinterpret_cast<const float2*>(src);
        v[0] = t.x; v[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < VPL; ++i) v[i] = src[i];
    }
}

// Folds the partial results of the sequences that were split into chunks.  Two passes over the
// list the plan kernel left behind, both in a fixed summation order, so the result does not depend
// on scheduling:
//   A. a sequence of at most kMergeWarpMax chunks: one warp per (sequence, query head); lane j
//      holds the (max, sum) pair of chunk j, every lane owns D/32 consecutive dims.  No shared
//      memory, no barrier -- the common case (a few chunks per sequence) costs one round of loads.
//   B. a sequence of more chunks (one very long context on an otherwise idle GPU): one CTA per
//      (sequence, query head, 32-dim slice); the maximum over all chunks is taken first, then 32 groups of
//      eight lanes fold chunks g, g+32, ... with 16-byte loads, and the groups are summed in a fixed order.
template <typename T, int D>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_kernel(const __grid_constant__ DecodeParams p, int B) {
    const Workspace& ws = p.ws;
    const int Hq = p.Hq, G = p.group, out_f32 = p.out_f32;
    const int64_t out_sb = p.out_sb, out_sh = p.out_sh;
    float* lse = p.lse;
    T* out = static_cast<T*>(p.out);              // the output is of q's type T ...
    float* out32 = static_cast<float*>(p.out);    // ... or fp32 when out_f32 is set (strides in elements either way)
    constexpr int VPL = D / 32;   // dims per lane in pass A, 32-dim slices in pass B
    constexpr float kLn2 = 0.6931471805599453f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool direct = p.direct != 0;
    // Plan-free mode: every warp re-derives the chunking from ctx_len (inputs of the call, so this runs
    // before the wait below, under the attention kernel's tail) instead of reading the plan kernel's lists.
    DirectPlan dplan{};
    if (direct)
        dplan = direct_plan(p.ctx_len, p.ctx_begin, p.sink_tokens, p.max_pages, p.batch, p.n_virt_heads,
                            p.direct_target_items, p.direct_min_chunk, p.direct_big_target_items, p.direct_big_pages, p.direct_grid, lane);
    grid_dependency_wait();   // the attention kernel's partial results
    // Whatever follows as a programmatic dependent (the next step's plan or attention kernel, the peer exchange)
    // may be placed now: it waits for this grid to finish before it reads anything this kernel writes.
    grid_launch_dependents();
    // the attention kernel is done with the plan-free work counter: leave it zeroed and signed for the next call
    if (direct && p.direct_dynamic && blockIdx.x == 0 && threadIdx.x == 0)
        *reinterpret_cast<int4*>(ws.header + kHdrDirectCounter) = make_int4(0, kDirectSig0, kDirectSig1, kDirectSig2);
#ifdef IVAB_PROFILE
    if (threadIdx.x == 0) PROF_STAMP_MIN(ws.header, 6, globaltimer_ns())
#endif
    const int num_chunks = direct ? dplan.num_chunks : ws.header[kHdrNumChunks];
    const bool skip = direct && num_chunks > ws.cap;   // flagged by the attention kernel; nothing was computed
    // units of pass A / B: the plan kernel's lists of split sequences, or (plan-free) every sequence, of
    // which those with a fitting chunk count are taken
    const int n_small = skip ? 0 : (direct ? B : ws.header[kHdrNumSplit]);   // single-chunk sequences were written by the attention kernel
    const int n_big = skip ? 0 : (direct ? (__any_sync(0xffffffffu, dplan.n > kMergeWarpMax) ? B : 0) : ws.header[kHdrNumBig]);
    // a lane's VPL outputs go out as one store when every output row is aligned for it
    constexpr int kVecBytes = VPL * (int)sizeof(T);
    const bool vec_out = !out_f32 && VPL >= 2 && (sizeof(T) == 2 || VPL % 4 == 0) &&
                         ((reinterpret_cast<uintptr_t>(out) | (uintptr_t)(out_sb * (int64_t)sizeof(T)) |
                           (uintptr_t)(out_sh * (int64_t)sizeof(T))) % kVecBytes) == 0;

    // ---- pass A
    for (int unit = blockIdx.x * kMergeWarps + warp; unit < n_small * Hq; unit += gridDim.x * kMergeWarps) {
        const int s = direct ? unit / Hq : ws.split_list[unit / Hq], hq = unit % Hq;
        const int first = direct ? __shfl_sync(0xffffffffu, dplan.first, s) : ws.seq_first[s];
        const int n = direct ? __shfl_sync(0xffffffffu, dplan.n, s) : ws.seq_count[s];
        if (direct && (n < 2 || n > kMergeWarpMax)) continue;            // (warp-uniform)
        const int h = hq / G, g = hq % G;
        const size_t item0 = (size_t)h * num_chunks + first;
        const float* ml = ws.part_ml + (item0 * G + g) * 2;               // chunk j at ml + j*G*2
        const float* po = ws.part_o + (item0 * G + g) * D + lane * VPL;   // chunk j at po + j*G*D

        float mj = -INFINITY, lj = 0.f;
        if (lane < n) {
            const float2 v = *reinterpret_cast<const float2*>(ml + (size_t)lane * G * 2);
            mj = v.x; lj = v.y;
        }
        const float M = warp_max_f32(mj);
        const float f = (mj == -INFINITY) ? 0.f : fast_exp2(mj - M);
        float L = lj * f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);

        float acc[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
        int j = 0;
        for (; j + 4 <= n; j += 4) {   // four rows in flight
            float r[4][VPL];
#pragma unroll
            for (int u = 0; u < 4; ++u) load_row<VPL>(po + (size_t)(j + u) * G * D, r[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float fu = __shfl_sync(0xffffffffu, f, j + u);
#pragma unroll
                for (int i = 0; i < VPL; ++i) acc[i] = fmaf(r[u][i], fu, acc[i]);
            }
        }
        for (; j < n; ++j) {
            float r[VPL];
            load_row<VPL>(po + (size_t)j * G * D, r);
            const float fj = __shfl_sync(0xffffffffu, f, j);
#pragma unroll
            for (int i = 0; i < VPL; ++i) acc[i] = fmaf(r[i], fj, acc[i]);
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        const int64_t dst_i = (int64_t)s * out_sb + (int64_t)hq * out_sh + lane * VPL;
        T* dst = out + dst_i;
        if (out_f32) {
#pragma unroll
            for (int i = 0; i < VPL; ++i) out32[dst_i + i] = acc[i] * inv;
        } else if (vec_out) {
            // one store per lane (the output may be pinned host memory, where partial writes are expensive)
            if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int i = 0; i < VPL; i += 4)
                    *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i] * inv, acc[i + 1] * inv, acc[i + 2] * inv, acc[i + 3] * inv);
            } else if constexpr (VPL == 4) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack2<T>(acc[0] * inv, acc[1] * inv), pack2<T>(acc[2] * inv, acc[3] * inv));
            } else if constexpr (VPL == 8) {
                *reinterpret_cast<uint4*>(dst) = make_uint4(pack2<T>(acc[0] * inv, acc[1] * inv), pack2<T>(acc[2] * inv, acc[3] * inv),
                                                            pack2<T>(acc[4] * inv, acc[5] * inv), pack2<T>(acc[6] * inv, acc[7] * inv));
            } else {
                *reinterpret_cast<uint32_t*>(dst) = pack2<T>(acc[0] * inv, acc[1] * inv);
            }
        } else {
#pragma unroll
            for (int i = 0; i < VPL; ++i) Elt<T>::store(dst + i, acc[i] * inv);
        }
        if (lane == 0 && lse != nullptr) lse[(int64_t)s * Hq + hq] = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
    }

    // ---- pass B
    __shared__ float sh_m[kMergeWarps];
    __shared__ float sh_l[kMergeWarps];
    __shared__ __align__(16) float sh_o[kMergeWarps][32];
    for (int c = blockIdx.x; c < n_big * Hq * VPL; c += gridDim.x) {
        const int unit = c / VPL, slice = c % VPL;
        const int s = direct ? unit / Hq : ws.split_list[B - 1 - unit / Hq], hq = unit % Hq;
        const int first = direct ? __shfl_sync(0xffffffffu, dplan.first, s) : ws.seq_first[s];
        const int n = direct ? __shfl_sync(0xffffffffu, dplan.n, s) : ws.seq_count[s];
        if (direct && n <= kMergeWarpMax) continue;                      // (uniform over the CTA: no barrier is skipped by some)
        const int h = hq / G, g = hq % G;
        const size_t item0 = (size_t)h * num_chunks + first;
        const float* ml = ws.part_ml + (item0 * G + g) * 2;
        // 8 warps x 4 lane groups = 32 chunk groups; the 8 lanes of a group own four dims each of the slice
        const int grp = warp * 4 + (lane >> 3), dq = lane & 7;
        const float* po = ws.part_o + (item0 * G + g) * D + slice * 32 + dq * 4;

        // the maximum over all chunks first, so that every chunk is weighted once and no partial sum is rescaled
        float mx = -INFINITY;
        for (int j = threadIdx.x; j < n; j += kMergeWarps * 32) mx = fmaxf(mx, ml[(size_t)j * G * 2]);
        mx = warp_max_f32(mx);
        if (lane == 0) sh_m[warp] = mx;
        __syncthreads();
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMergeWarps; ++w) M = fmaxf(M, sh_m[w]);

        // chunk group `grp` folds chunks grp, grp + 32, ...: 16-byte loads, eight of them in flight per thread
        float lw = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int j = grp; j < n; j += kMergeWarps * 4) {
            const float2 v = *reinterpret_cast<const float2*>(ml + (size_t)j * G * 2);
            const float fj = (v.x == -INFINITY) ? 0.f : fast_exp2(v.x - M);
            const float4 o4 = *reinterpret_cast<const float4*>(po + (size_t)j * G * D);
            lw = fmaf(v.y, fj, lw);
            acc.x = fmaf(o4.x, fj, acc.x); acc.y = fmaf(o4.y, fj, acc.y);
            acc.z = fmaf(o4.z, fj, acc.z); acc.w = fmaf(o4.w, fj, acc.w);
        }
        // the four lane groups of a warp (fixed order: xor 8, then 16), then the eight warps through shared memory
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
            lw += __shfl_xor_sync(0xffffffffu, lw, off);
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
        }
        if (lane < 8) *reinterpret_cast<float4*>(&sh_o[warp][lane * 4]) = acc;
        if (lane == 0) sh_l[warp] = lw;
        __syncthreads();
        if (warp == 0) {
            float L = 0.f, O = 0.f;
#pragma unroll
            for (int w = 0; w < kMergeWarps; ++w) {
                L += sh_l[w];
                O += sh_o[w][lane];
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            const int64_t oi = (int64_t)s * out_sb + (int64_t)hq * out_sh + slice * 32 + lane;
            if (out_f32) out32[oi] = O * inv;
            else Elt<T>::store(out + oi, O * inv);
            if (slice == 0 && lane == 0 && lse != nullptr)
                lse[(int64_t)s * Hq + hq] = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
        }
        __syncthreads();   // the shared scratch is reused by the next unit
    }
#ifdef IVAB_PROFILE
    if (threadIdx.x == 0) PROF_STAMP_MAX(ws.header, 7, globaltimer_ns())
#endif
    // ---- head-parallel decode: the CTA that finishes last sends this rank's rows to the peers and collects theirs,
    // so the step needs no exchange launch behind this kernel.  (The rows also hold what the attention kernel
    // wrote for unsplit sequences: that grid finished before any CTA here passed its dependency wait.)
    if (p.xchg_on) {
        __shared__ int s_last;
        __syncthreads();   // this CTA's rows are written
        if (threadIdx.x == 0) {
            __threadfence();
            s_last = atomicAdd(ws.header + kHdrMergeDone, 1) == (int)gridDim.x - 1;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();   // the other CTAs' rows, published before their increments
            const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(p.xchg.epoch);
            peer_exchange_step(p.xchg, epoch, warp, kMergeWarps, lane);
            __syncthreads();
            if (threadIdx.x == 0) *p.xchg.epoch = epoch + 1u;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------

// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime so that the
// library does not link against libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// 4-D map of a page pool: (head_dim, token in page, page, kv head); box = one 128-byte column tile
// of one page (16 rows x 128 bytes: 64 16-bit or 128 8-bit elements), 128-byte swizzle -- or, for 8-bit
// pools with head_dim 64, the whole 16 x 64-byte page with 64-byte swizzle.  Returns false if the driver
// rejects the geometry (the caller then uses another engine).
bool encode_pool_map(CUtensorMap* tm, const void* pool, CUtensorMapDataType type, int64_t esz, int64_t D,
                     int64_t num_pages, int64_t Hkv, int64_t sp_bytes, int64_t sh_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t gdim[4] = {(cuuint64_t)D, (cuuint64_t)kPage, (cuuint64_t)num_pages, (cuuint64_t)Hkv};
    const cuuint64_t gstride[3] = {(cuuint64_t)(D * esz), (cuuint64_t)sp_bytes, (cuuint64_t)sh_bytes};
    const int64_t row_bytes = D * esz < 128 ? D * esz : 128;   // 64 only for 8-bit pools with head_dim 64
    if (row_bytes != 128 && row_bytes != 64) return false;
    const cuuint32_t box[4] = {(cuuint32_t)(row_bytes / esz), (cuuint32_t)kPage, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(tm, type, 4,
                          const_cast<void*>(pool), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Smallest q_heads/kv_heads ratio that takes a tensor-core engine.  By default multi-head attention
// (ratio 1) on 16-bit pools stays on CUDA cores, where it is HBM-bound, while 8-bit pools with
// head_dim 128 use the tensor cores at every ratio (the CUDA-core engine is issue-bound on
// them).  IVAB_TC_MIN_GROUP overrides both thresholds for experiments (1 = always, 99 = never).
int tc_min_group(int default_value) {
    static int v = [] {
        const char* e = std::getenv("IVAB_TC_MIN_GROUP");
        const int n = e ? std::atoi(e) : 0;
        return n < 1 ? 0 : n;
    }();
    return v ? v : default_value;
}

// Work items per resident CTA that the plan-free mode's chunk size aims for (IVAB_DIRECT_IPS overrides
// the default for experiments; read once per process).
int direct_items_per_slot() {
    static int v = [] {
        const char* e = std::getenv("IVAB_DIRECT_IPS");
        const int n = e ? std::atoi(e) : kDirectItemsPerSlot;
        return n < 1 ? 1 : (n > kItemsPerSlot ? kItemsPerSlot : n);   // the workspace is sized for kItemsPerSlot
    }();
    return v;
}

int env_int(const char* name, int dflt, int lo, int hi) {
    const char* e = std::getenv(name);
    if (!e) return dflt;
    const int n = std::atoi(e);
    return n < lo ? lo : (n > hi ? hi : n);
}

// Plan-free mode: IVAB_DIRECT_DYNAMIC=0 keeps the item ids static (CTA b takes b, b + grid, ...) even where the
// work counter could be used (experiments).
bool direct_dynamic_enabled() {
    static bool v = [] {
        const char* e = std::getenv("IVAB_DIRECT_DYNAMIC");
        return !(e && std::atoi(e) == 0);
    }();
    return v;
}

// Programmatic dependent launch of the attention and merge kernels; IVAB_PDL=0 turns it off.
bool use_dependent_launch() {
    static bool v = [] {
        const char* e = std::getenv("IVAB_PDL");
        return !(e && std::atoi(e) == 0);
    }();
    return v;
}

template <typename T, int D, int G, int ENG, typename TKV = T>
int launch_decode(const DecodeParams& p0, const TensorMaps& tm, int B, cudaStream_t st) {
    using Eng = typename EngineSelect<ENG, T, TKV, D, G>::type;
    using C = SmemLayout<Eng::SCRATCH_PER_WARP, D, G>;
    DecodeParams p = p0;
    constexpr int kCtas = Eng::CTAS_PER_SM;
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    int max_optin = 0;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev),
                            "cudaDeviceGetAttribute")) return rc;
    int per_sm = 0;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev),
                            "cudaDeviceGetAttribute")) return rc;
    // each resident CTA also pays 1 KB of system-reserved shared memory; 1 KB more is alignment slack
    int budget = per_sm / kCtas - 1024;
    if (budget > max_optin) budget = max_optin;
    int stages = (budget - C::OFF_STAGES - 1024) / Eng::STAGE_BYTES;
    if (stages > kMaxStages) stages = kMaxStages;
    // Pages go to consumer warps round-robin.  With a stage count that is a multiple of the warp
    // count, a stage is always consumed by the same warp, so a warp waiting for the next phase of a
    // stage has itself consumed the previous one -- the precondition of a parity wait.
    stages -= stages % kConsumerWarps;
    if (stages < kConsumerWarps) return set_error(IVAB_ERR_UNSUPPORTED, "decode attention: not enough shared memory for the stage ring");
    p.stages = stages;
    const size_t smem = (size_t)C::OFF_STAGES + 1024 + (size_t)stages * Eng::STAGE_BYTES;
    auto kern = decode_kernel<T, D, G, ENG, TKV>;
    // one flag per (kernel instantiation, device); concurrent host threads may both set the attribute, which is harmless
    static std::atomic<bool> configured[kMaxDevices];
    if (dev < 0 || dev >= kMaxDevices) return set_error(IVAB_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, max_optin),
                                "cudaFuncSetAttribute")) return rc;
        configured[dev].store(true, std::memory_order_release);
    }
    const int grid = sm_count() * kCtas;
    if (2 * sm_count() > kStatusSlots) return set_error(IVAB_ERR_UNSUPPORTED, "decode attention: %d SMs (status slots for %d)", sm_count(), kStatusSlots / 2);
    p.status_slots_per_cta = 2 / kCtas;   // the first 2 x SMs slots are written by every call, whatever the engine
    if (p.direct) {
        p.direct_target_items = grid * direct_items_per_slot();
        p.direct_grid = grid;
        // The work counter is usable when a merge kernel follows (it re-arms the counter for the next call);
        // a batch that turns out large (the lengths are known only on the device) is cut into finer items.
        p.direct_dynamic = direct_dynamic_enabled() && p.max_pages > p.direct_min_chunk ? 1 : 0;
        // (8-bit pools stream a page in half the time, so the fixed work per item weighs more: fewer, longer items
        //  and a threshold in bytes, not pages -- IVAB_DIRECT_BIG_IPS / IVAB_DIRECT_BIG_KB override both for experiments)
        static const int big_ips = env_int("IVAB_DIRECT_BIG_IPS", sizeof(TKV) == 1 ? kItemsPerSlot * 3 / 4 : kItemsPerSlot, 1, kItemsPerSlot);
        p.direct_big_target_items = p.direct_dynamic ? grid * big_ips : 0;
        const long long page_bytes = 2LL * kPage * D * (long long)sizeof(TKV);   // K and V
        static const int big_kb = env_int("IVAB_DIRECT_BIG_KB", kDirectBigKB, 1, 1 << 20);
        const long long big_pages = (long long)big_kb * 1024 / page_bytes;
        p.direct_big_pages = (int)(big_pages < 1 ? 1 : big_pages);
    }
    // Both launches below are programmatic dependents of the kernel before them (plan -> attention
    // -> merge): the launch latency and set-up of each overlap the tail of its predecessor.
    cudaLaunchAttribute pdl{};
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cfg.attrs = &pdl; cfg.numAttrs = use_dependent_launch() ? 1 : 0;
    if (int rc = check_cuda(cudaLaunchKernelEx(&cfg, kern, p, tm), "decode_kernel launch")) return rc;
    g_launches++;

    // pass A needs a warp, pass B D/32 CTAs per split (sequence, head); how many there are is known only on the device
    const long long units = (long long)B * p.Hq * (D / 32);
    const int merge_grid = (int)(units < (long long)sm_count() * 4 ? units : (long long)sm_count() * 4);
    cfg.gridDim = dim3(merge_grid); cfg.blockDim = dim3(kMergeWarps * 32); cfg.dynamicSmemBytes = 0;
    // plan-free mode with a block table no wider than the smallest chunk: no sequence can be split, nothing to merge
    if (p.direct && p.max_pages <= p.direct_min_chunk) return p.xchg_on ? launch_peer_allgather(p.xchg, st) : IVAB_OK;
    if (int rc = check_cuda(cudaLaunchKernelEx(&cfg, merge_kernel<T, D>, p, B), "merge_kernel launch")) {
        // (the counter stays as the attention kernel leaves it: drop the signature so that no later call trusts it)
        if (p.direct_dynamic) cudaMemsetAsync(p.ws.header + kHdrDirectCounter, 0, 4 * sizeof(int), st);
        return rc;
    }
    g_launches++;
    return IVAB_OK;
}

template <typename T> CUtensorMapDataType map_type() {
    return std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

template <typename T, int D, int G>
int choose_engine(const DecodeParams& p, int B, int Hkv, cudaStream_t st) {
    TensorMaps tm{};
    if constexpr (sizeof(T) == 2 && D % 64 == 0) {
        // head_dim 256 with two query heads per KV head is faster on the CUDA-core engine (6.1 against 5.8 TB/s)
        if (G >= tc_min_group(D >= 256 ? 3 : 2) && p.scale_log2 > 0.f &&
            encode_pool_map(&tm.k, p.k_pool, map_type<T>(), 2, D, p.num_pages, Hkv, p.pool_sp_bytes, p.pool_sh_bytes) &&
            encode_pool_map(&tm.v, p.v_pool, map_type<T>(), 2, D, p.num_pages, Hkv, p.pool_sp_bytes, p.pool_sh_bytes))
            return launch_decode<T, D, G, kEngMma>(p, tm, B, st);
    }
    return launch_decode<T, D, G, kEngSimt>(p, tm, B, st);
}

template <typename T, int D>
int dispatch_group(int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st) {
    // the kernels are instantiated for groups of 1, 2, 4 and 8 query heads; other ratios run in the
    // next larger one with the surplus rows empty (p.group holds the real ratio)
    switch (G) {
        case 1: return choose_engine<T, D, 1>(p, B, Hkv, st);
        case 2: return choose_engine<T, D, 2>(p, B, Hkv, st);
        case 3: case 4: return choose_engine<T, D, 4>(p, B, Hkv, st);
        case 5: case 6: case 7: case 8: return choose_engine<T, D, 8>(p, B, Hkv, st);
        default: return set_error(IVAB_ERR_UNSUPPORTED, "decode attention: q_heads/kv_heads = %d (supported: 1 to 8)", G);
    }
}

template <typename T>
int dispatch_dim(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st) {
    switch (D) {
        case 32: return dispatch_group<T, 32>(G, Hkv, p, B, st);
        case 64: return dispatch_group<T, 64>(G, Hkv, p, B, st);
        case 128: return dispatch_group<T, 128>(G, Hkv, p, B, st);
        case 256:
            if constexpr (sizeof(T) == 2) return dispatch_group<T, 256>(G, Hkv, p, B, st);
            [[fallthrough]];
        default:
            return set_error(IVAB_ERR_UNSUPPORTED,
                             "decode attention: head_dim %d (supported: 32, 64, 128; 256 for 16-bit types)", D);
    }
}

// IVAB_FP8_REG=0 keeps grouped-query 8-bit decode on the engine that widens pages in shared memory.
bool use_fp8_register_engine() {
    static bool v = [] {
        const char* e = std::getenv("IVAB_FP8_REG");
        return !(e && std::atoi(e) == 0);
    }();
    return v;
}

// 8-bit pools: multi-head attention (one query head per KV head) widens on the fly in the CUDA-core
// engine; grouped queries use the tensor cores -- with head_dim 128 on fragments built in registers
// from swizzled byte tiles, otherwise on pages widened to fp16 tiles in shared memory.
template <typename T>
int dispatch_fp8(int D, int G_real, int Hkv, const DecodeParams& p, int B, cudaStream_t st) {
    TensorMaps tm{};
    using F8 = __nv_fp8_e4m3;
    if (G_real < 1 || G_real > 8)
        return set_error(IVAB_ERR_UNSUPPORTED, "8-bit KV decode: q_heads/kv_heads = %d (supported: 1 to 8)", G_real);
    const int G = G_real <= 2 ? G_real : (G_real <= 4 ? 4 : 8);   // instantiated group sizes; p.group keeps the real one
    const bool simt = G < tc_min_group(2) || !(p.scale_log2 > 0.f);
    // head_dim 128: every ratio; head_dim 64: grouped queries (multi-head attention stays on CUDA cores there)
    if ((D == 128 || D == 64) && G >= tc_min_group(D == 128 ? 1 : 2) && p.scale_log2 > 0.f && use_fp8_register_engine() &&
        encode_pool_map(&tm.k, p.k_pool, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, p.num_pages, Hkv, p.pool_sp_bytes,
                        p.pool_sh_bytes) &&
        encode_pool_map(&tm.v, p.v_pool, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, p.num_pages, Hkv, p.pool_sp_bytes,
                        p.pool_sh_bytes)) {
        if (D == 128) {
            switch (G) {
                case 2: return launch_decode<T, 128, 2, kEngMmaFp8Reg, F8>(p, tm, B, st);
                case 4: return launch_decode<T, 128, 4, kEngMmaFp8Reg, F8>(p, tm, B, st);
                case 8: return launch_decode<T, 128, 8, kEngMmaFp8Reg, F8>(p, tm, B, st);
                case 1: return launch_decode<T, 128, 1, kEngMmaFp8Reg, F8>(p, tm, B, st);
                default: break;
            }
        } else {
            switch (G) {
                case 2: return launch_decode<T, 64, 2, kEngMmaFp8Reg, F8>(p, tm, B, st);
                case 4: return launch_decode<T, 64, 4, kEngMmaFp8Reg, F8>(p, tm, B, st);
                case 8: return launch_decode<T, 64, 8, kEngMmaFp8Reg, F8>(p, tm, B, st);
                case 1: return launch_decode<T, 64, 1, kEngMmaFp8Reg, F8>(p, tm, B, st);
                default: break;
            }
        }
    }
    // The CUDA-core engine on 8-bit pools is built for one and two query heads per KV head only (with four
    // or eight it needs several hundred bytes of spills per thread and was never the faster choice): larger
    // groups always take a tensor-core engine, which needs a positive softmax scale.
    if (simt && G > 2) {
        if (!(p.scale_log2 > 0.f))
            return set_error(IVAB_ERR_UNSUPPORTED, "8-bit KV decode with more than two query heads per KV head needs scale > 0");
    }
#define IVAB_FP8_CASE(DD, GG)                                                                   \
    if (D == DD && G == GG) {                                                                   \
        if constexpr (GG <= 2) {                                                                \
            if (simt) return launch_decode<T, DD, GG, kEngSimt, F8>(p, tm, B, st);              \
        }                                                                                       \
        return launch_decode<T, DD, GG, kEngMmaFp8, F8>(p, tm, B, st);                          \
    }
    IVAB_FP8_CASE(64, 1) IVAB_FP8_CASE(64, 2) IVAB_FP8_CASE(64, 4) IVAB_FP8_CASE(64, 8)
    IVAB_FP8_CASE(128, 1) IVAB_FP8_CASE(128, 2) IVAB_FP8_CASE(128, 4) IVAB_FP8_CASE(128, 8)
#undef IVAB_FP8_CASE
    return set_error(IVAB_ERR_UNSUPPORTED,
                     "8-bit KV decode: head_dim %d (supported: 64, 128)", D);
}

}  // namespace
}  // namespace ivab
