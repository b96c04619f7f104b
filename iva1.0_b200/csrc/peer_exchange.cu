// All-gather of one small block per rank over peer-mapped memory (NVLink loads/stores), for the head-parallel
// decode of one long sequence: every rank ends a step with a few KB of output rows, and every rank needs all
// of them.  One warp per destination rank stores this rank's block straight into that rank's buffer, signals
// it, and waits for that rank's signal.  No library collective, no host round trip: the exchange is one
// more kernel in the step's stream (or CUDA graph), launched as a programmatic dependent of the kernel before it.
//
// Buffer of every rank (same layout everywhere, mapped into every peer's address space by the caller):
//     [slots][world][block_bytes]  data: slot s, row r = rank r's block of a step with epoch % slots == s
//     [world] uint32               arrival counters: entry r counts the blocks rank r has delivered here
// Counters only ever grow, so nothing is reset between steps; `epoch` (a device word of this rank) counts the
// steps this rank has exchanged.  A rank may run at most one step ahead of the slowest peer (it cannot finish
// step k before every peer has delivered step k), which is why two slots suffice as long as each rank consumes
// a step's data in stream order before its next exchange.
//
// Only plain peer stores / loads are used -- no multimem, no TMA, no cluster multicast.  The wait is bounded:
// when it expires the kernel sets IVAB_STATUS_WAIT_TIMEOUT and returns.
#include <atomic>

#include "common.cuh"

namespace ivab {

extern std::atomic<long long> g_launches;

namespace {

constexpr int kMaxPeers = 16;

struct PeerParams {
    const char* local;             // this rank's block
    char* peer[kMaxPeers];         // base of every rank's buffer, as mapped into this process (peer[rank] = own)
    int64_t block_bytes, flags_off;
    int world, rank, slots;
    unsigned int* epoch;           // steps exchanged so far (this rank's device memory)
    int* status;
    uint64_t limit_ns;
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One CTA; warp r serves destination rank r: it stores this rank's block into rank r's buffer, signals it,
// and waits for rank r's block to arrive here.
__global__ void __launch_bounds__(kMaxPeers * 32) peer_allgather_kernel(const PeerParams pp) {
    grid_dependency_wait();   // the block is the output of the kernels before this one
    const int dst = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned int epoch = *pp.epoch;
    const int slot = (int)(epoch % (unsigned)pp.slots);
    char* row = pp.peer[dst] + ((int64_t)slot * pp.world + pp.rank) * pp.block_bytes;
    for (int64_t off = (int64_t)lane * 16; off < pp.block_bytes; off += 32 * 16)
        *reinterpret_cast<uint4*>(row + off) = *reinterpret_cast<const uint4*>(pp.local + off);
    __threadfence_system();   // this lane's stores are performed at the destination ...
    __syncwarp();             // ... for every lane of the warp, before the one signal below
    if (lane == 0) {
        // one more block from `rank` has landed at `dst`
        red_release_sys_add(reinterpret_cast<unsigned int*>(pp.peer[dst] + pp.flags_off) + pp.rank, 1u);
        // and wait until rank `dst` has delivered ITS block of this step here
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(pp.peer[pp.rank] + pp.flags_off) + dst;
        const uint64_t t0 = globaltimer_ns();
        bool failed = false;
        // (counters wrap after 2^32 steps; the signed difference keeps the comparison right across the wrap)
        while ((int)(ld_acquire_sys(mine) - (epoch + 1u)) < 0) {
            if (globaltimer_ns() - t0 > pp.limit_ns) { failed = true; break; }
            __nanosleep(100);
        }
        if (failed && pp.status != nullptr) atomicOr(pp.status, kStatusWaitTimeout);
    }
    __syncthreads();          // every warp has read the step counter and has seen its peer's block
    if (threadIdx.x == 0) *pp.epoch = epoch + 1u;
}

}  // namespace
}  // namespace ivab

using namespace ivab;

extern "C" int ivab_peer_allgather(const void* local_block, int64_t block_bytes, void* const* peer_bufs, int world, int rank,
                                   int slots, int64_t flags_offset, uint32_t* epoch, int32_t* status, int64_t wait_limit_ns,
                                   void* stream) {
    const char* fn = "ivab_peer_allgather";
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || slots < 2)
        return set_error(IVAB_ERR_INVALID, "%s: world %d (1..%d), rank %d, slots %d (>= 2)", fn, world, kMaxPeers, rank, slots);
    if (!local_block || !peer_bufs || !epoch) return set_error(IVAB_ERR_INVALID, "%s: null pointer", fn);
    if (block_bytes <= 0 || block_bytes % 16 || (reinterpret_cast<uintptr_t>(local_block) & 15u))
        return set_error(IVAB_ERR_INVALID, "%s: the block must be 16-byte aligned and a multiple of 16 bytes", fn);
    if (flags_offset < (int64_t)slots * world * block_bytes || flags_offset % 16)
        return set_error(IVAB_ERR_INVALID, "%s: the arrival counters must lie behind the %d x %d data rows, 16-byte aligned", fn,
                         slots, world);
    if (wait_limit_ns <= 0) return set_error(IVAB_ERR_INVALID, "%s: wait_limit_ns must be positive", fn);
    PeerParams pp{};
    pp.local = static_cast<const char*>(local_block);
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || (reinterpret_cast<uintptr_t>(peer_bufs[r]) & 15u))
            return set_error(IVAB_ERR_INVALID, "%s: peer buffer %d is null or misaligned", fn, r);
        pp.peer[r] = static_cast<char*>(peer_bufs[r]);
    }
    pp.block_bytes = block_bytes; pp.flags_off = flags_offset;
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
