// Decode-attention kernels for one type combination (see decode_dispatch.h); split from the other
// combinations so that the units compile in parallel.
#include "decode_dispatch.h"
#include "decode_kernel.cuh"

namespace ivab {

int decode_dispatch_fp8_bf16(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st) {
    return dispatch_fp8<__nv_bfloat16>(D, G, Hkv, p, B, st);
}

}  // namespace ivab
