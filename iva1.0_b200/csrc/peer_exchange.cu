// All-gather of one small block per rank over peer-mapped memory (NVLink stores), for the head-parallel
// decode of one long sequence: every rank ends a step with a few KB of output rows, and every rank needs all
// of them.  One warp per peer: it stores this rank's block into that peer's staging area and collects that
// peer's block from its own.  No library collective, no host round trip: the exchange is one more kernel in
// the step's stream (or CUDA graph), launched as a programmatic dependent of the kernel before it.
//
// Flag-in-data protocol: every 32-bit payload word travels as one 64-bit store {payload, tag} with
// tag = step number + 1, and the receiver polls each 64-bit word until it carries the tag of the step.  A
// naturally aligned 64-bit access is single-copy atomic, so a word that shows the tag shows its payload:
// no fence, no separate arrival flag, and the latency of an exchange is one NVLink crossing instead of
// store -> fence -> flag (measured on two GPUs: 10-11 us per exchange with fence and flag).
//
// Buffer of every rank (same layout everywhere, mapped into every peer's address space by the caller):
//     [slots][world][block_bytes]       result rows: slot s, row r = rank r's block of a step with step % slots == s
//     [slots][world][2 * block_bytes]   staging: the same rows as {payload, tag} words, written by the peers
// The buffer is zero before the first step and tags start at 1 and only grow, so a stale word never matches.
// A rank cannot finish step k before every peer has sent step k, and a peer sends step k+1 only after its own
// step-k kernel has finished reading: two slots suffice as long as each rank consumes a step's rows in stream
// order before its next exchange but one.
//
// Only plain peer stores are used (loads are local) -- no multimem, no TMA, no cluster multicast.  The wait
// is bounded: when it expires the kernel sets IVAB_STATUS_WAIT_TIMEOUT and returns.
#include <atomic>

#include "common.cuh"

namespace ivab {

extern std::atomic<long long> g_launches;

namespace {

constexpr int kMaxPeers = 16;

struct PeerParams {
    const char* local;             // this rank's block
    char* peer[kMaxPeers];         // base of every rank's buffer, as mapped into this process (peer[rank] = own)
    int64_t block_bytes, flags_off;   // flags_off: offset of the staging area in every buffer
    int world, rank, slots;
    unsigned int* epoch;           // steps exchanged so far (this rank's device memory)
    int* status;
    uint64_t limit_ns;
};

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One CTA; warp r serves peer r: it sends this rank's block to rank r and collects rank r's block here.
__global__ void __launch_bounds__(kMaxPeers * 32) peer_allgather_kernel(const PeerParams pp) {
    grid_dependency_wait();   // the block is the output of the kernels before this one
    const int peer = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef IVAB_XCHG_STAMPS
    const uint64_t t_begin = globaltimer_ns();
#endif
    const unsigned int epoch = *pp.epoch;
    const unsigned long long tag = (unsigned long long)(epoch + 1u) << 32;
    const int slot = (int)(epoch % (unsigned)pp.slots);
    const int words = (int)(pp.block_bytes / 4);
    // send: word i of this rank's block -> staging row `rank` of the peer
    unsigned long long* to = reinterpret_cast<unsigned long long*>(pp.peer[peer] + pp.flags_off +
                                                                    ((int64_t)slot * pp.world + pp.rank) * 2 * pp.block_bytes);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pp.local);
    constexpr int kInFlight = 16;   // words of a lane whose loads (and, below, polls) overlap
    for (int base = lane; base < words; base += 32 * kInFlight) {
        unsigned int w[kInFlight];   // all loads first: the stores are asm volatile and would serialise them
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) w[u] = base + u * 32 < words ? mine[base + u * 32] : 0u;
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
            if (base + u * 32 < words) st_relaxed_sys_u64(to + base + u * 32, tag | w[u]);
    }
    // receive: staging row `peer` of this rank -> result row `peer`
    const unsigned long long* from = reinterpret_cast<const unsigned long long*>(pp.peer[pp.rank] + pp.flags_off +
                                                                                  ((int64_t)slot * pp.world + peer) * 2 * pp.block_bytes);
    unsigned int* row = reinterpret_cast<unsigned int*>(pp.peer[pp.rank] + ((int64_t)slot * pp.world + peer) * pp.block_bytes);
    const uint64_t t0 = globaltimer_ns();
    bool failed = false;
    // Up to kInFlight words of a lane are polled at once (their loads overlap: one L2 round trip per round, not
    // per word); words that do not carry the tag yet are loaded again in the next round.
    for (int base = lane; base < words && !failed; base += 32 * kInFlight) {
        unsigned long long v[kInFlight];
        unsigned int pending = 0;
#pragma unroll
        for (int u = 0; u < kInFlight; ++u)
            if (base + u * 32 < words) pending |= 1u << u;
        while (pending != 0) {
#pragma unroll
            for (int u = 0; u < kInFlight; ++u)
                if (pending >> u & 1u) v[u] = ld_relaxed_sys_u64(from + base + u * 32);
#pragma unroll
            for (int u = 0; u < kInFlight; ++u)
                if ((pending >> u & 1u) && (v[u] >> 32) == (tag >> 32)) {
                    row[base + u * 32] = (unsigned int)v[u];
                    pending &= ~(1u << u);
                }
            if (pending != 0 && globaltimer_ns() - t0 > pp.limit_ns) { failed = true; break; }
        }
    }
    if (failed && pp.status != nullptr) atomicOr(pp.status, kStatusWaitTimeout);
#ifdef IVAB_XCHG_STAMPS   // debug build: when this warp started, had sent, had received (status must hold 2 + 6 * world ints)
    if (lane == 0 && pp.status != nullptr) {
        unsigned long long* st = reinterpret_cast<unsigned long long*>(pp.status + 2) + 3 * peer;
        st[0] = t_begin; st[1] = t0; st[2] = globaltimer_ns();
    }
#endif
    __syncthreads();          // every warp has read the step counter and has collected its peer's block
    if (threadIdx.x == 0) *pp.epoch = epoch + 1u;
}

}  // namespace
}  // namespace ivab

using namespace ivab;

extern "C" int ivab_peer_allgather(const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world, int rank,
                                   int slots, int64_t staging_offset, uint32_t* epoch, int32_t* status, int64_t wait_limit_ns,
                                   void* stream) {
    const char* fn = "ivab_peer_allgather";
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || slots < 2)
        return set_error(IVAB_ERR_INVALID, "%s: world %d (1..%d), rank %d, slots %d (>= 2)", fn, world, kMaxPeers, rank, slots);
    if (!local_block || !peer_bufs || !epoch) return set_error(IVAB_ERR_INVALID, "%s: null pointer", fn);
    if (block_bytes <= 0 || block_bytes % 16 || (reinterpret_cast<uintptr_t>(local_block) & 15u))
        return set_error(IVAB_ERR_INVALID, "%s: the block must be 16-byte aligned and a multiple of 16 bytes", fn);
    if (staging_offset < (int64_t)slots * world * block_bytes || staging_offset % 16)
        return set_error(IVAB_ERR_INVALID, "%s: the staging area must lie behind the %d x %d result rows, 16-byte aligned", fn,
                         slots, world);
    if (wait_limit_ns <= 0) return set_error(IVAB_ERR_INVALID, "%s: wait_limit_ns must be positive", fn);
    PeerParams pp{};
    pp.local = static_cast<const char*>(local_block);
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || (reinterpret_cast<uintptr_t>(peer_bufs[r]) & 15u))
            return set_error(IVAB_ERR_INVALID, "%s: peer buffer %d is null or misaligned", fn, r);
        pp.peer[r] = static_cast<char*>(peer_bufs[r]);
    }
    pp.block_bytes = block_bytes; pp.flags_off = staging_offset;
    pp.world = world; pp.rank = rank; pp.slots = slots;
    pp.epoch = epoch; pp.status = status; pp.limit_ns = (uint64_t)wait_limit_ns;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute pdl{};
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(world * 32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cfg.attrs = &pdl; cfg.numAttrs = 1;
    if (int rc = check_cuda(cudaLaunchKernelEx(&cfg, peer_allgather_kernel, pp), "peer_allgather_kernel launch")) return rc;
    g_launches++;
    return IVAB_OK;
}
