// Device side of the all-gather over peer-mapped memory (the protocol is described in peer_exchange.cu).
// Shared by the stand-alone exchange kernel and by the merge kernel of the decode path, whose last CTA can
// run the exchange itself, so that a head-parallel decode step ends without one more launch.
#pragma once

#include "common.cuh"

namespace ivab {

constexpr int kMaxPeers = 16;

struct PeerParams {
    const char* local;             // this rank's block
    char* peer[kMaxPeers];         // base of every rank's buffer, as mapped into this process (peer[rank] = own)
    int64_t block_bytes, staging_off;
    int world, rank, slots;
    unsigned int* epoch;           // steps exchanged so far (this rank's device memory)
    int* status;
    uint64_t limit_ns;
};

int make_peer_params(const char* fn, const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world, int rank,
                     int slots, int64_t staging_offset, uint32_t* epoch, int32_t* status, int64_t wait_limit_ns, PeerParams* out);
int launch_peer_allgather(const PeerParams& pp, cudaStream_t st);

namespace {

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

constexpr int kPeerInFlight = 17;   // words of a lane whose loads (and polls) overlap: 32 x 17 covers the 4 x 129 fp32
                                    // words a rank sends when 32 query heads of head_dim 128 are split over 8 GPUs

// Called by `nwarps` whole warps (warp index `warp`).  The block is cut into units of at most 32 x kPeerInFlight
// words; the (peer, unit) pairs are dealt to the warps round-robin, so that few peers with large blocks keep
// as many warps busy as many peers with small ones.  A warp first sends its units, then collects the same units
// of its peers' blocks.  `epoch` is the value of *pp.epoch before the step (the caller reads it once and stores
// epoch + 1 when every warp is back).  The block is read with L1-bypassing loads: other CTAs of the calling grid
// may have written it.  Returns false when a wait expired (the status bit is set here).
__device__ __forceinline__ bool peer_exchange_step(const PeerParams& pp, unsigned int epoch, int warp, int nwarps, int lane) {
    const unsigned long long tag = (unsigned long long)(epoch + 1u) << 32;
    const int slot = (int)(epoch % (unsigned)pp.slots);
    const int words = (int)(pp.block_bytes / 4);
    const int units_per_peer = (words + 32 * kPeerInFlight - 1) / (32 * kPeerInFlight);
    const int unit_words = ((words + units_per_peer - 1) / units_per_peer + 31) / 32 * 32;   // balanced, <= 32 x kPeerInFlight
    const int total_units = pp.world * units_per_peer;
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pp.local);
    // send: word i of this rank's block -> staging row `rank` of the peer, as {payload, tag}
    for (int unit = warp; unit < total_units; unit += nwarps) {
        const int peer = unit / units_per_peer, first = (unit % units_per_peer) * unit_words;
        const int end = min(words, first + unit_words);
        unsigned long long* to = reinterpret_cast<unsigned long long*>(pp.peer[peer] + pp.staging_off +
                                                                        ((int64_t)slot * pp.world + pp.rank) * 2 * pp.block_bytes);
        unsigned int w[kPeerInFlight];   // all loads first: the stores are asm volatile and would serialise them
#pragma unroll
        for (int u = 0; u < kPeerInFlight; ++u) w[u] = first + lane + u * 32 < end ? __ldcg(mine + first + lane + u * 32) : 0u;
#pragma unroll
        for (int u = 0; u < kPeerInFlight; ++u)
            if (first + lane + u * 32 < end) st_relaxed_sys_u64(to + first + lane + u * 32, tag | w[u]);
    }
    // receive: staging row `peer` of this rank -> result row `peer`.  All words of a lane are polled at once (one
    // L2 round trip per round, not per word); words without the tag are loaded again.
    const uint64_t t0 = globaltimer_ns();
    bool failed = false;
    for (int unit = warp; unit < total_units && !failed; unit += nwarps) {
        const int peer = unit / units_per_peer, first = (unit % units_per_peer) * unit_words;
        const int end = min(words, first + unit_words);
        const unsigned long long* from = reinterpret_cast<const unsigned long long*>(
            pp.peer[pp.rank] + pp.staging_off + ((int64_t)slot * pp.world + peer) * 2 * pp.block_bytes);
        unsigned int* row = reinterpret_cast<unsigned int*>(pp.peer[pp.rank] + ((int64_t)slot * pp.world + peer) * pp.block_bytes);
        unsigned long long v[kPeerInFlight];
        unsigned int pending = 0;
#pragma unroll
        for (int u = 0; u < kPeerInFlight; ++u)
            if (first + lane + u * 32 < end) pending |= 1u << u;
        while (pending != 0) {
#pragma unroll
            for (int u = 0; u < kPeerInFlight; ++u)
                if (pending >> u & 1u) v[u] = ld_relaxed_sys_u64(from + first + lane + u * 32);
#pragma unroll
            for (int u = 0; u < kPeerInFlight; ++u)
                if ((pending >> u & 1u) && (v[u] >> 32) == (tag >> 32)) {
                    row[first + lane + u * 32] = (unsigned int)v[u];
                    pending &= ~(1u << u);
                }
            if (pending != 0 && globaltimer_ns() - t0 > pp.limit_ns) { failed = true; break; }
        }
    }
    failed = __any_sync(0xffffffffu, failed);
    if (failed && lane == 0 && pp.status != nullptr) atomicOr(pp.status, kStatusWaitTimeout);
    return !failed;
}

}  // namespace
}  // namespace ivab
