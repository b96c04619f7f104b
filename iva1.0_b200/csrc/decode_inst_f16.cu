// Decode-attention kernels for one type combination (see decode_dispatch.h); split from the other
// combinations so that the units compile in parallel.
#include "decode_dispatch.h"
#include "decode_kernel.cuh"

namespace ivab {

int decode_dispatch_f16(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st) {
    return dispatch_dim<__half>(D, G, Hkv, p, B, st);
}

}  // namespace ivab
