// KV append (scatter) and gather: pure vectorised copy kernels.
//
// The unit of work is one row of head_dim elements -- 128..512 bytes -- addressed on one side
// through an index (a slot id / a block-table entry) and on the other side densely.  Every
// thread moves 16-byte vectors; a CTA issues four independent loads per thread before the
// first store so that enough bytes are in flight to cover HBM latency.  Consecutive threads
// touch consecutive 16-byte vectors of the dense side, so dense traffic is fully coalesced and
// indexed traffic is coalesced per row (and per 4 KB page where slots are consecutive).
#include <atomic>

#include "common.cuh"

namespace ivab {

extern std::atomic<long long> g_launches;

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr uint32_t kTile = kThreads * kUnroll;

// Division of a number below 2^31 by a fixed divisor as one widening multiply and a shift:
// n / d == (n * mul) >> (31 + shift) with shift = ceil(log2 d), mul = ceil(2^(31 + shift) / d).
// (The rounding error of mul contributes less than n / 2^(31 + shift) * (e / d) < 1 / d, e < d <= 2^shift.)
struct FastDiv {
    uint32_t mul, shift, d;
};

FastDiv make_fastdiv(uint32_t d) {
    FastDiv f{};
    f.d = d;
    while ((1ull << f.shift) < d) ++f.shift;
    f.mul = (uint32_t)(((1ull << (31 + f.shift)) + d - 1) / d);
    return f;
}

__device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv& f) {
    return (uint32_t)(((uint64_t)n * f.mul) >> (31 + f.shift));
}

struct RowCopyParams {
    const char* src[2];
    char* dst[2];
    const int64_t* idx;
    int64_t idx_stride_b;   // batch row b reads idx + b * idx_stride_b (0: one index vector for all rows)
    int pad_ok;             // an index of -1 is padding: its row is skipped without raising a status bit
    // indexed side: offset(b,h,id) = b*ix_b + h*ix_h + (id / page_size)*ix_page + (id % page_size)*ix_slot
    int64_t ix_b, ix_h, ix_page, ix_slot;
    // dense side: offset(b,h,n) = b*dn_b + h*dn_h + n*dn_n
    int64_t dn_b, dn_h, dn_n;
    int64_t id_bound;       // valid ids are [0, id_bound)
    uint32_t N, H;
    uint32_t vec_per_row;   // 16-byte vectors per source row
    uint32_t total;         // N * H * vec_per_row (below 2^31)
    uint32_t page_size;
    FastDiv by_vpr, by_rows, by_page;   // divisors vec_per_row, (h_fastest ? H : N), page_size
    int h_fastest;          // row order on the dense side: 1 = (n, h), 0 = (h, n)
    int* status;
    float inv_scale[2];     // CVT 3/4 (quantising append): 1/scale per tensor
    int early_dependents;   // small grids: let a programmatically dependent kernel be scheduled at once
};

// Loads through the read-only path and default-policy stores: measured on the append/gather stress
// configuration against the streaming (.cs) variants of either, this pair was the fastest
// (append 5.97 -> 6.10 TB/s, gather 6.50 -> 6.60 TB/s on the same GPU).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
    *reinterpret_cast<uint4*>(p) = v;
}

// GATHER: indexed side is the source.  SCATTER: indexed side is the destination.
// CVT: 0 = raw copy, 1 = fp16 -> fp32, 2 = bf16 -> fp32 (gather only; the reference's gather
// always returns fp32, src/kernels_t/kv_ops_triton.py:112), 3 = fp16 -> e4m3, 4 = bf16 -> e4m3
// (scatter only: quantising append, 8 output bytes per 16-byte source vector).
template <bool GATHER, int CVT>
__global__ void __launch_bounds__(kThreads) row_copy_kernel(const RowCopyParams p) {
    const char* __restrict__ src = p.src[blockIdx.z];
    char* __restrict__ dst = p.dst[blockIdx.z];
    const int64_t b = blockIdx.y;
    const uint32_t n_tiles = (p.total + kTile - 1) / kTile;
    // A kernel launched behind this one as a programmatic dependent (the planning / attention kernels of
    // the same decode step) may be placed on the SMs this small grid leaves free; it waits for this grid
    // to complete before it reads the pool.  Large grids keep the SMs to themselves until they retire.
    if (p.early_dependents) grid_launch_dependents();

    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const uint32_t base = tile * kTile + threadIdx.x;
        uint4 v[kUnroll];
        int64_t doff[kUnroll];
        bool ok[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const uint32_t i = base + k * kThreads;
            ok[k] = i < p.total;
            doff[k] = 0;
            v[k] = make_uint4(0, 0, 0, 0);
            if (ok[k]) {
                // all quotients by multiply-and-shift: generic divisions here made the kernel issue-bound
                const uint32_t r = fdiv(i, p.by_vpr);
                const uint32_t vec = i - r * p.vec_per_row;
                const uint32_t outer = fdiv(r, p.by_rows), inner = r - outer * p.by_rows.d;
                const uint32_t h = p.h_fastest ? inner : outer, n = p.h_fastest ? outer : inner;
                const int64_t id = __ldg(p.idx + b * p.idx_stride_b + n);
                if (id < 0 || id >= p.id_bound) {
                    // Out-of-range index: record it and skip the row instead of faulting.
                    if (p.status != nullptr && vec == 0 && !(p.pad_ok && id == -1)) atomicOr(p.status, kStatusBadSlot);
                    ok[k] = false;
                } else {
                    const uint32_t uid = static_cast<uint32_t>(id);
                    const uint32_t page = fdiv(uid, p.by_page), in_page = uid - page * p.page_size;
                    const int64_t ix = b * p.ix_b + h * p.ix_h + (int64_t)page * p.ix_page + (int64_t)in_page * p.ix_slot;
                    const int64_t dn = b * p.dn_b + h * p.dn_h + (int64_t)n * p.dn_n;
                    const int64_t soff = (GATHER ? ix : dn) + (int64_t)vec * 16;
                    doff[k] = (GATHER ? dn : ix) + (int64_t)vec * (CVT == 0 ? 16 : (CVT <= 2 ? 32 : 8));
                    v[k] = ld_stream(src + soff);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            if (!ok[k]) continue;
            if (CVT == 0) {
                st_stream(dst + doff[k], v[k]);
            } else if (CVT >= 3) {
                float f[8];
                if (CVT == 3) Elt<__half>::unpack(v[k], f); else Elt<__nv_bfloat16>::unpack(v[k], f);
                const float is = p.inv_scale[blockIdx.z];
                uint2 q;
                q.x = (uint32_t)pack_fp8x2(f[0] * is, f[1] * is) | ((uint32_t)pack_fp8x2(f[2] * is, f[3] * is) << 16);
                q.y = (uint32_t)pack_fp8x2(f[4] * is, f[5] * is) | ((uint32_t)pack_fp8x2(f[6] * is, f[7] * is) << 16);
                __stcs(reinterpret_cast<uint2*>(dst + doff[k]), q);
            } else {
                float f[8];
                if (CVT == 1) Elt<__half>::unpack(v[k], f); else Elt<__nv_bfloat16>::unpack(v[k], f);
                st_stream(dst + doff[k], *reinterpret_cast<uint4*>(&f[0]));
                st_stream(dst + doff[k] + 16, *reinterpret_cast<uint4*>(&f[4]));
            }
        }
    }
}

struct PagedGatherParams {
    const char* pool;
    char* out;
    const int32_t* block_table;
    const int32_t* ctx_len;
    const int64_t* out_offsets;
    int64_t bt_stride;
    int64_t pool_sh, pool_sp;   // bytes
    uint32_t H, vec_per_row, page_size;
    int32_t num_pages, max_pages;
    int head_major;
    int* status;
};

// One CTA per (page index, sequence): copies that page of every head.  Within a head the page
// is one contiguous block of the pool, so reads are up to 4 KB sequential.
__global__ void __launch_bounds__(kThreads) paged_gather_kernel(const PagedGatherParams p) {
    const int s = blockIdx.y;
    int L = p.ctx_len[s];
    const int64_t cap = (int64_t)p.max_pages * p.page_size;
    if (L < 0 || L > cap) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && p.status) atomicOr(p.status, kStatusBadCtxLen);
        L = L < 0 ? 0 : (int)cap;
    }
    const uint32_t n_pages = (L + p.page_size - 1) / p.page_size;
    const int64_t row_bytes = (int64_t)p.vec_per_row * 16;
    const int64_t off = p.out_offsets[s];

    for (uint32_t pg = blockIdx.x; pg < n_pages; pg += gridDim.x) {
        int pid = p.block_table[(int64_t)s * p.bt_stride + pg];
        if (pid < 0 || pid >= p.num_pages) {
            if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusBadPage);
            continue;   // skip the page instead of reading outside the pool
        }
        const uint32_t first = pg * p.page_size;
        const uint32_t n_valid = min(p.page_size, (uint32_t)L - first);
        const uint32_t per_head = n_valid * p.vec_per_row;
        const uint32_t total = per_head * p.H;
        const char* __restrict__ src0 = p.pool + (int64_t)pid * p.pool_sp;
        for (uint32_t base = threadIdx.x; base < total; base += kTile) {
            uint4 v[kUnroll];
            int64_t doff[kUnroll];
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) {
                const uint32_t j = base + k * kThreads;
                if (j < total) {
                    const uint32_t h = j / per_head;
                    const uint32_t rem = j - h * per_head;
                    v[k] = ld_stream(src0 + (int64_t)h * p.pool_sh + (int64_t)rem * 16);
                    if (p.head_major) {
                        doff[k] = (off * p.H + (int64_t)h * L + first) * row_bytes + (int64_t)rem * 16;
                    } else {
                        const uint32_t tok = rem / p.vec_per_row;
                        const uint32_t vec = rem - tok * p.vec_per_row;
                        doff[k] = ((off + first + tok) * p.H + h) * row_bytes + (int64_t)vec * 16;
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) {
                const uint32_t j = base + k * kThreads;
                if (j < total) st_stream(p.out + doff[k], v[k]);
            }
        }
    }
}

// Positions of the non-zero entries of each mask row, in order: indices[b, j] = position of the j-th survivor of
// row b for j < counts[b], -1 behind them.  One CTA per batch row; the row is scanned in tiles of kScanThreads
// entries with a running offset.
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads) compact_index_kernel(const uint8_t* __restrict__ mask, int64_t S,
                                                                     int64_t* __restrict__ indices, int32_t* __restrict__ counts) {
    __shared__ int warp_sums[32];
    __shared__ int tile_total;
    const int64_t b = blockIdx.x;
    const uint8_t* row = mask + b * S;
    int64_t* out = indices + b * S;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int running = 0;
    for (int64_t base = 0; base < S; base += kScanThreads) {
        const int64_t pos = base + threadIdx.x;
        const int keep = pos < S && row[pos] != 0;
        int v = keep;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, v, off);
            if (lane >= off) v += t;
        }
        if (lane == 31) warp_sums[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, off);
                if (lane >= off) w += t;
            }
            warp_sums[lane] = w;
            if (lane == 31) tile_total = w;
        }
        __syncthreads();
        if (warp > 0) v += warp_sums[warp - 1];
        if (keep) out[running + v - 1] = pos;
        running += tile_total;
        __syncthreads();   // warp_sums / tile_total are rewritten by the next tile
    }
    for (int64_t j = running + threadIdx.x; j < S; j += kScanThreads) out[j] = -1;
    if (threadIdx.x == 0) counts[b] = running;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_row_copy(bool gather, int cvt, const RowCopyParams& p0, int64_t batch, int n_tensors, cudaStream_t st) {
    if (p0.total == 0 || batch == 0) return IVAB_OK;
    RowCopyParams p = p0;
    p.by_vpr = make_fastdiv(p.vec_per_row);
    p.by_rows = make_fastdiv(p.h_fastest ? p.H : p.N);
    p.by_page = make_fastdiv(p.page_size);
    const uint32_t n_tiles = (p.total + kTile - 1) / kTile;
    // One tile of kTile vectors per CTA.  A capped, grid-stride launch (148 x 16 CTAs) was measured 6 % slower
    // on the 131 072-token append (6.10 vs 6.48 TB/s): with plain CTAs the hardware scheduler keeps the SMs'
    // accesses spread over the whole range instead of marching through it in lockstep.
    const uint32_t max_x = 0x7fffffffu;
    dim3 grid(n_tiles < max_x ? n_tiles : max_x, (unsigned)batch, (unsigned)n_tensors);
    p.early_dependents = (uint64_t)grid.x * grid.y * grid.z <= (uint64_t)sm_count() ? 1 : 0;
    if (gather) {
        if (cvt == 0) row_copy_kernel<true, 0><<<grid, kThreads, 0, st>>>(p);
        else if (cvt == 1) row_copy_kernel<true, 1><<<grid, kThreads, 0, st>>>(p);
        else row_copy_kernel<true, 2><<<grid, kThreads, 0, st>>>(p);
    } else {
        if (cvt == 0) row_copy_kernel<false, 0><<<grid, kThreads, 0, st>>>(p);
        else if (cvt == 3) row_copy_kernel<false, 3><<<grid, kThreads, 0, st>>>(p);
        else row_copy_kernel<false, 4><<<grid, kThreads, 0, st>>>(p);
    }
    g_launches++;
    return check_cuda(cudaGetLastError(), "row_copy_kernel launch");
}

int common_checks(const char* fn, int dtype, int64_t head_dim, size_t* esz) {
    *esz = dtype_size(dtype);
    if (*esz == 0) return set_error(IVAB_ERR_INVALID, "%s: unknown dtype %d", fn, dtype);
    if (head_dim <= 0 || (head_dim * (int64_t)*esz) % 16 != 0)
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: head_dim*sizeof(dtype) = %lld bytes is not a multiple of 16",
                         fn, (long long)(head_dim * (int64_t)*esz));
    return IVAB_OK;
}

}  // namespace
}  // namespace ivab

using namespace ivab;

static int kv_gather_body(const char* fn, const void* cache, const int64_t* indices, int64_t indices_stride_b, int pad_ok,
                          void* out, int dtype, int out_dtype,
                          int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                          int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                          int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                          int32_t* status, void* stream);

extern "C" int ivab_kv_gather(const void* cache, const int64_t* indices, void* out, int dtype, int out_dtype,
                              int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                              int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                              int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                              int32_t* status, void* stream) {
    return kv_gather_body("ivab_kv_gather", cache, indices, 0, 0, out, dtype, out_dtype, batch, heads, seq_len, head_dim,
                          n_indices, cache_stride_b, cache_stride_h, cache_stride_s, out_stride_b, out_stride_h,
                          out_stride_n, status, stream);
}

extern "C" int ivab_kv_gather_rows(const void* cache, const int64_t* indices, int64_t indices_stride_b, void* out,
                                   int dtype, int out_dtype,
                                   int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                                   int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                                   int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                                   int32_t* status, void* stream) {
    if (indices_stride_b < 0) return set_error(IVAB_ERR_INVALID, "ivab_kv_gather_rows: negative indices_stride_b");
    return kv_gather_body("ivab_kv_gather_rows", cache, indices, indices_stride_b, 1, out, dtype, out_dtype, batch, heads,
                          seq_len, head_dim, n_indices, cache_stride_b, cache_stride_h, cache_stride_s, out_stride_b,
                          out_stride_h, out_stride_n, status, stream);
}

extern "C" int ivab_compact_indices(const uint8_t* mask, int64_t batch, int64_t seq_len, int64_t* indices,
                                    int32_t* counts, void* stream) {
    if (batch < 0 || seq_len < 0) return set_error(IVAB_ERR_INVALID, "ivab_compact_indices: negative size");
    if (batch == 0) return IVAB_OK;
    if (!mask || !indices || !counts) return set_error(IVAB_ERR_INVALID, "ivab_compact_indices: null pointer");
    if (batch >= (1LL << 31)) return set_error(IVAB_ERR_UNSUPPORTED, "ivab_compact_indices: batch too large");
    compact_index_kernel<<<(unsigned)batch, kScanThreads, 0, static_cast<cudaStream_t>(stream)>>>(mask, seq_len, indices, counts);
    g_launches++;
    return check_cuda(cudaGetLastError(), "compact_index_kernel launch");
}

static int kv_gather_body(const char* fn_name, const void* cache, const int64_t* indices, int64_t indices_stride_b, int pad_ok,
                          void* out, int dtype, int out_dtype,
                          int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                          int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                          int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                          int32_t* status, void* stream) {
    (void)fn_name;
    size_t esz;
    if (int rc = common_checks("ivab_kv_gather", dtype, head_dim, &esz)) return rc;
    if (batch < 0 || heads < 0 || seq_len < 0 || n_indices < 0)
        return set_error(IVAB_ERR_INVALID, "ivab_kv_gather: negative size");
    if (batch == 0 || heads == 0 || n_indices == 0) return IVAB_OK;
    if (!cache || !indices || !out) return set_error(IVAB_ERR_INVALID, "ivab_kv_gather: null pointer");
    int cvt = 0;
    size_t osz = esz;
    if (out_dtype != dtype) {
        if (out_dtype != IVAB_F32 || (dtype != IVAB_F16 && dtype != IVAB_BF16))
            return set_error(IVAB_ERR_UNSUPPORTED, "ivab_kv_gather: out_dtype must equal dtype, or be fp32 for a 16-bit cache");
        cvt = dtype == IVAB_F16 ? 1 : 2;
        osz = 4;
    }
    if (!aligned16(cache) || !aligned16(out) || (cache_stride_b * esz) % 16 || (cache_stride_h * esz) % 16 ||
        (cache_stride_s * esz) % 16 || (out_stride_b * osz) % 16 || (out_stride_h * osz) % 16 ||
        (out_stride_n * osz) % 16)
        return set_error(IVAB_ERR_INVALID, "ivab_kv_gather: pointers and strides must be 16-byte aligned");
    if (batch > 65535) return set_error(IVAB_ERR_UNSUPPORTED, "ivab_kv_gather: batch > 65535");
    const int64_t vpr = head_dim * (int64_t)esz / 16;
    const int64_t total = n_indices * heads * vpr;
    if (total >= (1LL << 31) - 4096 || seq_len >= (1LL << 31))
        return set_error(IVAB_ERR_UNSUPPORTED, "ivab_kv_gather: more than 2^31 16-byte vectors per batch row; split the call");
    RowCopyParams p{};
    p.src[0] = static_cast<const char*>(cache);
    p.dst[0] = static_cast<char*>(out);
    p.idx = indices; p.idx_stride_b = indices_stride_b; p.pad_ok = pad_ok;
    p.ix_b = cache_stride_b * esz; p.ix_h = cache_stride_h * esz; p.ix_page = cache_stride_s * esz; p.ix_slot = 0;
    p.dn_b = out_stride_b * osz; p.dn_h = out_stride_h * osz; p.dn_n = out_stride_n * osz;
    p.id_bound = seq_len; p.N = (uint32_t)n_indices; p.H = (uint32_t)heads; p.vec_per_row = (uint32_t)vpr;
    p.total = (uint32_t)total; p.page_size = 1; p.h_fastest = out_stride_h < out_stride_n; p.status = status;
    return launch_row_copy(true, cvt, p, batch, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int ivab_kv_scatter(void* cache, const int64_t* indices, const void* values, int dtype,
                               int64_t batch, int64_t heads, int64_t seq_len, int64_t head_dim, int64_t n_indices,
                               int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_s,
                               int64_t values_stride_b, int64_t values_stride_h, int64_t values_stride_n,
                               int32_t* status, void* stream) {
    size_t esz;
    if (int rc = common_checks("ivab_kv_scatter", dtype, head_dim, &esz)) return rc;
    if (batch < 0 || heads < 0 || seq_len < 0 || n_indices < 0)
        return set_error(IVAB_ERR_INVALID, "ivab_kv_scatter: negative size");
    if (batch == 0 || heads == 0 || n_indices == 0) return IVAB_OK;
    if (!cache || !indices || !values) return set_error(IVAB_ERR_INVALID, "ivab_kv_scatter: null pointer");
    if (!aligned16(cache) || !aligned16(values) || (cache_stride_b * esz) % 16 || (cache_stride_h * esz) % 16 ||
        (cache_stride_s * esz) % 16 || (values_stride_b * esz) % 16 || (values_stride_h * esz) % 16 ||
        (values_stride_n * esz) % 16)
        return set_error(IVAB_ERR_INVALID, "ivab_kv_scatter: pointers and strides must be 16-byte aligned");
    if (batch > 65535) return set_error(IVAB_ERR_UNSUPPORTED, "ivab_kv_scatter: batch > 65535");
    const int64_t vpr = head_dim * (int64_t)esz / 16;
    const int64_t total = n_indices * heads * vpr;
    if (total >= (1LL << 31) - 4096 || seq_len >= (1LL << 31))
        return set_error(IVAB_ERR_UNSUPPORTED, "ivab_kv_scatter: more than 2^31 16-byte vectors per batch row; split the call");
    RowCopyParams p{};
    p.src[0] = static_cast<const char*>(values);
    p.dst[0] = static_cast<char*>(cache);
    p.idx = indices;
    p.ix_b = cache_stride_b * esz; p.ix_h = cache_stride_h * esz; p.ix_page = cache_stride_s * esz; p.ix_slot = 0;
    p.dn_b = values_stride_b * esz; p.dn_h = values_stride_h * esz; p.dn_n = values_stride_n * esz;
    p.id_bound = seq_len; p.N = (uint32_t)n_indices; p.H = (uint32_t)heads; p.vec_per_row = (uint32_t)vpr;
    p.total = (uint32_t)total; p.page_size = 1; p.h_fastest = values_stride_h < values_stride_n; p.status = status;
    return launch_row_copy(false, 0, p, batch, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int ivab_paged_append(const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                                 const int64_t* slot_mapping, void* k_pool, void* v_pool,
                                 int64_t pool_stride_head, int64_t pool_stride_page, int dtype,
                                 int64_t n_tokens, int64_t heads, int64_t head_dim, int64_t page_size,
                                 int64_t num_pages, int32_t* status, void* stream) {
    size_t esz;
    if (int rc = common_checks("ivab_paged_append", dtype, head_dim, &esz)) return rc;
    if (n_tokens < 0 || heads < 0 || page_size <= 0 || num_pages < 0)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_append: bad size");
    if (n_tokens == 0 || heads == 0) return IVAB_OK;
    if (!k_new || !v_new || !slot_mapping || !k_pool || !v_pool)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_append: null pointer");
    if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(k_pool) || !aligned16(v_pool) ||
        (new_stride_t * esz) % 16 || (new_stride_h * esz) % 16 || (pool_stride_head * esz) % 16 ||
        (pool_stride_page * esz) % 16)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_append: pointers and strides must be 16-byte aligned");
    const int64_t vpr = head_dim * (int64_t)esz / 16;
    const int64_t total = n_tokens * heads * vpr;
    if (total >= (1LL << 31) - 4096 || num_pages * page_size >= (1LL << 31))
        return set_error(IVAB_ERR_UNSUPPORTED, "ivab_paged_append: more than 2^31 16-byte vectors; split the call");
    RowCopyParams p{};
    p.src[0] = static_cast<const char*>(k_new); p.src[1] = static_cast<const char*>(v_new);
    p.dst[0] = static_cast<char*>(k_pool); p.dst[1] = static_cast<char*>(v_pool);
    p.idx = slot_mapping;
    p.ix_b = 0; p.ix_h = pool_stride_head * esz; p.ix_page = pool_stride_page * esz; p.ix_slot = head_dim * esz;
    p.dn_b = 0; p.dn_h = new_stride_h * esz; p.dn_n = new_stride_t * esz;
    p.id_bound = num_pages * page_size; p.N = (uint32_t)n_tokens; p.H = (uint32_t)heads;
    p.vec_per_row = (uint32_t)vpr; p.total = (uint32_t)total; p.page_size = (uint32_t)page_size;
    p.h_fastest = new_stride_h < new_stride_t; p.status = status;
    return launch_row_copy(false, 0, p, 1, 2, static_cast<cudaStream_t>(stream));
}

extern "C" int ivab_paged_gather(const void* pool, int64_t pool_stride_head, int64_t pool_stride_page,
                                 const int32_t* block_table, int64_t block_table_stride, const int32_t* ctx_len,
                                 const int64_t* out_offsets, void* out, int out_layout, int dtype,
                                 int64_t batch, int64_t heads, int64_t head_dim, int64_t page_size,
                                 int64_t num_pages, int64_t max_pages_per_seq, int32_t* status, void* stream) {
    size_t esz;
    if (int rc = common_checks("ivab_paged_gather", dtype, head_dim, &esz)) return rc;
    if (batch < 0 || heads < 0 || page_size <= 0 || num_pages < 0 || max_pages_per_seq < 0)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_gather: bad size");
    if (batch == 0 || heads == 0 || max_pages_per_seq == 0) return IVAB_OK;
    if (!pool || !block_table || !ctx_len || !out_offsets || !out)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_gather: null pointer");
    if (out_layout != IVAB_OUT_TOKEN_MAJOR && out_layout != IVAB_OUT_HEAD_MAJOR)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_gather: unknown out_layout %d", out_layout);
    if (!aligned16(pool) || !aligned16(out) || (pool_stride_head * esz) % 16 || (pool_stride_page * esz) % 16)
        return set_error(IVAB_ERR_INVALID, "ivab_paged_gather: pointers and strides must be 16-byte aligned");
    if (batch > 65535) return set_error(IVAB_ERR_UNSUPPORTED, "ivab_paged_gather: batch > 65535; split the call");
    if (page_size * heads * head_dim * (int64_t)esz / 16 >= (1LL << 31) || max_pages_per_seq * page_size >= (1LL << 31))
        return set_error(IVAB_ERR_UNSUPPORTED, "ivab_paged_gather: page too large");
    PagedGatherParams p{};
    p.pool = static_cast<const char*>(pool); p.out = static_cast<char*>(out);
    p.block_table = block_table; p.ctx_len = ctx_len; p.out_offsets = out_offsets;
    p.bt_stride = block_table_stride; p.pool_sh = pool_stride_head * esz; p.pool_sp = pool_stride_page * esz;
    p.H = (uint32_t)heads; p.vec_per_row = (uint32_t)(head_dim * esz / 16); p.page_size = (uint32_t)page_size;
    p.num_pages = (int32_t)num_pages; p.max_pages = (int32_t)max_pages_per_seq;
    p.head_major = out_layout == IVAB_OUT_HEAD_MAJOR; p.status = status;
    const int64_t gx = max_pages_per_seq < 65535 * 32 ? max_pages_per_seq : 65535 * 32;
    dim3 grid((unsigned)gx, (unsigned)batch, 1);
    paged_gather_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    g_launches++;
    return check_cuda(cudaGetLastError(), "paged_gather_kernel launch");
}

extern "C" int ivab_paged_append_fp8(const void* k_new, const void* v_new, int64_t new_stride_t, int64_t new_stride_h,
                                     const int64_t* slot_mapping, void* k_pool, void* v_pool,
                                     int64_t pool_stride_head, int64_t pool_stride_page, int src_dtype,
                                     float k_scale, float v_scale,
                                     int64_t n_tokens, int64_t heads, int64_t head_dim, int64_t page_size,
                                     int64_t num_pages, int32_t* status, void* stream) {
    const char* fn = "ivab_paged_append_fp8";
    if (src_dtype != IVAB_F16 && src_dtype != IVAB_BF16)
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: new tokens must be fp16 or bf16", fn);
    if (!(k_scale > 0.f) || !(v_scale > 0.f)) return set_error(IVAB_ERR_INVALID, "%s: scales must be positive", fn);
    if (n_tokens < 0 || heads < 0 || page_size <= 0 || num_pages < 0 || head_dim <= 0 || head_dim % 16)
        return set_error(IVAB_ERR_INVALID, "%s: bad size (head_dim must be a multiple of 16)", fn);
    if (n_tokens == 0 || heads == 0) return IVAB_OK;
    if (!k_new || !v_new || !slot_mapping || !k_pool || !v_pool) return set_error(IVAB_ERR_INVALID, "%s: null pointer", fn);
    if (!aligned16(k_new) || !aligned16(v_new) || !aligned16(k_pool) || !aligned16(v_pool) ||
        (new_stride_t * 2) % 16 || (new_stride_h * 2) % 16 || pool_stride_head % 16 || pool_stride_page % 16)
        return set_error(IVAB_ERR_INVALID, "%s: pointers and strides must be 16-byte aligned", fn);
    const int64_t vpr = head_dim * 2 / 16;   // source vectors per row
    const int64_t total = n_tokens * heads * vpr;
    if (total >= (1LL << 31) - 4096 || num_pages * page_size >= (1LL << 31))
        return set_error(IVAB_ERR_UNSUPPORTED, "%s: more than 2^31 16-byte vectors; split the call", fn);
    RowCopyParams p{};
    p.src[0] = static_cast<const char*>(k_new); p.src[1] = static_cast<const char*>(v_new);
    p.dst[0] = static_cast<char*>(k_pool); p.dst[1] = static_cast<char*>(v_pool);
    p.idx = slot_mapping;
    p.ix_b = 0; p.ix_h = pool_stride_head; p.ix_page = pool_stride_page; p.ix_slot = head_dim;   // 1-byte elements
    p.dn_b = 0; p.dn_h = new_stride_h * 2; p.dn_n = new_stride_t * 2;
    p.id_bound = num_pages * page_size; p.N = (uint32_t)n_tokens; p.H = (uint32_t)heads;
    p.vec_per_row = (uint32_t)vpr; p.total = (uint32_t)total; p.page_size = (uint32_t)page_size;
    p.h_fastest = new_stride_h < new_stride_t; p.status = status;
    p.inv_scale[0] = 1.f / k_scale; p.inv_scale[1] = 1.f / v_scale;
    return launch_row_copy(false, src_dtype == IVAB_F16 ? 3 : 4, p, 1, 2, static_cast<cudaStream_t>(stream));
}
