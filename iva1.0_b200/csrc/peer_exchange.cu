// All-gather of one small block per rank over peer-mapped memory (NVLink stores), for the head-parallel
// decode of one long sequence: every rank ends a step with a few KB of output rows, and every rank needs all
// of them.  The warps of one CTA share the (peer, unit of the block) pairs: each stores its units of this
// rank's block into the peers' staging areas and collects the same units of the peers' blocks from its own.  No library collective, no host round trip: the exchange is one more kernel in
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

#include "peer_exchange.cuh"

namespace ivab {

extern std::atomic<long long> g_launches;

namespace {

// One CTA of kExchangeWarps warps that share the (peer, unit of the block) pairs.
constexpr int kExchangeWarps = 16;
__global__ void __launch_bounds__(kExchangeWarps * 32) peer_allgather_kernel(const PeerParams pp) {
    grid_dependency_wait();   // the block is the output of the kernels before this one
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned int epoch = *pp.epoch;
    peer_exchange_step(pp, epoch, warp, (int)(blockDim.x >> 5), lane);
    __syncthreads();          // every warp has read the step counter and has collected its peers' blocks
    if (threadIdx.x == 0) *pp.epoch = epoch + 1u;
}

}  // namespace

// Checks the arguments of an exchange and fills the kernel's parameter block.
int make_peer_params(const char* fn, const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world, int rank,
                     int slots, int64_t staging_offset, uint32_t* epoch, int32_t* status, int64_t wait_limit_ns, PeerParams* out) {
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
    pp.block_bytes = block_bytes; pp.staging_off = staging_offset;
    pp.world = world; pp.rank = rank; pp.slots = slots;
    pp.epoch = epoch; pp.status = status; pp.limit_ns = (uint64_t)wait_limit_ns;
    *out = pp;
    return IVAB_OK;
}

// The exchange as a kernel of its own, a programmatic dependent of whatever precedes it in the stream.
int launch_peer_allgather(const PeerParams& pp, cudaStream_t st) {
    cudaLaunchAttribute pdl{};
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(kExchangeWarps * 32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cfg.attrs = &pdl; cfg.numAttrs = 1;
    if (int rc = check_cuda(cudaLaunchKernelEx(&cfg, peer_allgather_kernel, pp), "peer_allgather_kernel launch")) return rc;
    g_launches++;
    return IVAB_OK;
}

}  // namespace ivab

using namespace ivab;

extern "C" int ivab_peer_allgather(const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world, int rank,
                                   int slots, int64_t staging_offset, uint32_t* epoch, int32_t* status, int64_t wait_limit_ns,
                                   void* stream) {
    PeerParams pp{};
    if (int rc = make_peer_params("ivab_peer_allgather", local_block, block_bytes, peer_bufs, world, rank, slots, staging_offset,
                                  epoch, status, wait_limit_ns, &pp)) return rc;
    return launch_peer_allgather(pp, static_cast<cudaStream_t>(stream));
}
