// Entry points of the per-dtype instantiation units of the decode-attention kernels.  Each unit
// (decode_inst_*.cu) compiles the kernels of one query / storage type combination and launches the
// attention and merge kernels for an already planned (or plan-free) call.
#pragma once

#include <cuda_runtime.h>

#include "decode_defs.cuh"

namespace ivab {

// q, out and the pools share one type (D: head_dim, G: query heads per KV head, 1..8)
int decode_dispatch_f32(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st);
int decode_dispatch_f16(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st);
int decode_dispatch_bf16(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st);
// 8-bit (e4m3) pools with fp16 / bf16 queries
int decode_dispatch_fp8_f16(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st);
int decode_dispatch_fp8_bf16(int D, int G, int Hkv, const DecodeParams& p, int B, cudaStream_t st);

}  // namespace ivab
