// Page engines of the decode-attention kernel: what a consumer warp does with one staged page of K
// and V (16 tokens), plus the shared-memory layout of the kernel.  An engine provides
//   setup(lane), attach(scratch, lane), begin_item(params, seq, kv head, lane), page(params, stage, n_valid,
//   hole_lo, hole_hi, lane, scratch), publish(params, ml, o, lane)
// and the constants kTiled, STAGE_BYTES, PAGE_BYTES, SCRATCH_PER_WARP, CTAS_PER_SM (tiled engines also
// TILES, TILE_COLS, TILE_BYTES).  Included by decode_attn.cu only (internal linkage).
#pragma once

#include <cuda.h>

#include <type_traits>

#include "decode_defs.cuh"

namespace ivab {
namespace {

template <typename T, int D, int G>
struct Cfg {
    static constexpr int EPL = 16 / (int)sizeof(T);   // elements per lane per 16-byte vector
    static constexpr int LPR = D / EPL;               // lanes covering one row
    static constexpr int RPI = 32 / LPR;              // rows (tokens) per warp-wide load
    static constexpr int NV = kPage / RPI;            // warp-wide loads per page
    static constexpr int DUP = LPR / NV;              // lanes holding the same score after the reduce
    static constexpr int PAGE_BYTES = kPage * D * (int)sizeof(T);
    static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
    static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "row must map onto a power-of-two lane group");
    static_assert(NV >= 1 && NV <= LPR, "page too large for the transposing reduce");
};

// shared memory carve-up of the decode kernel (bytes) for an engine with SCRATCH bytes per consumer warp
template <int SCRATCH, int D, int G>
struct SmemLayout {
    static constexpr int OFF_BARS = 0;                                  // 2*kMaxStages + 2*kItemRing + 1 barriers
    static constexpr int OFF_ABORT = 1024 - 16;
    static constexpr int OFF_ITEMS = 1024;                              // kItemRing * kItWords ints
    static constexpr int OFF_MRG_ML = OFF_ITEMS + kItemRing * kItWords * 4;          // [W][G][2]
    static constexpr int OFF_MRG_O = OFF_MRG_ML + kConsumerWarps * G * 2 * 4;        // [W][G][D]
    static constexpr int OFF_SCRATCH = (OFF_MRG_O + kConsumerWarps * G * D * 4 + 127) / 128 * 128;   // [W][SCRATCH]
    static constexpr int OFF_STAGES = (OFF_SCRATCH + kConsumerWarps * SCRATCH + 1023) / 1024 * 1024;  // swizzled tiles need 1 KB alignment
};

enum { kEngSimt = 0, kEngMma = 1, kEngMmaFp8 = 2, kEngMmaFp8Reg = 3 };

// Sum NV per-lane values across the LPR lanes of a row group.  While more than one value is
// left, each step trades half of them with the partner lane (so the number of shuffles halves
// every step); the remaining steps are plain butterflies.  Returns the fully reduced value this
// lane ends up owning; which one that is is given by owned_index().
template <int NV, int OFF>
__device__ __forceinline__ float transpose_reduce(float (&v)[NV], int lane) {
    if constexpr (OFF == 0) {
        return v[0];
    } else if constexpr (NV > 1) {
        float h[NV / 2];
        const bool upper = (lane & OFF) != 0;
#pragma unroll
        for (int i = 0; i < NV / 2; ++i) {
            const float send = upper ? v[i] : v[i + NV / 2];
            const float keep = upper ? v[i + NV / 2] : v[i];
            h[i] = keep + __shfl_xor_sync(0xffffffffu, send, OFF);
        }
        return transpose_reduce<NV / 2, OFF / 2>(h, lane);
    } else {
        float h[1];
        h[0] = v[0] + __shfl_xor_sync(0xffffffffu, v[0], OFF);
        return transpose_reduce<1, OFF / 2>(h, lane);
    }
}

template <int NV, int LPR>
__device__ __forceinline__ int owned_index(int lane) {
    int idx = 0, nv = NV;
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) {
        if (nv > 1) { nv >>= 1; if (lane & off) idx += nv; }
    }
    return idx;
}

// ------------------------------------------------------------------------------------------------
// Page engines: what a consumer warp does with one staged K/V page.
//
//   SimtEngine  CUDA cores.  Lanes own 16-byte vectors of a row; scores come from a transposing
//               shuffle reduction.  Pages are staged by one untiled TMA bulk copy each (row-major).
//               Used for fp32 and for multi-head attention (one query head per KV head), where
//               the kernel is HBM-bound at ~1/3 issue utilisation.
//   MmaEngine   Tensor cores for grouped-query attention with 16-bit K/V.  With G >= 2 query heads
//               per KV head the CUDA-core path becomes issue-bound (4 flop/byte, ~52 % issue
//               utilisation at 46 % DRAM in ncu), so the G heads form the M side of
//               mma.sync.m16n8k16 tiles: S^T[head, token] = Q K^T, then O[head, dim] += P^T V.
//               Pages are staged by tiled TMA copies (64-element column tiles, 128-byte swizzle)
//               so that ldmatrix / ldmatrix.trans read them without bank conflicts.  Putting heads
//               on M makes the S^T accumulator fragment identical to the A fragment of the second
//               product: P never moves between lanes.
//
// Both engines leave the same per-warp state in shared memory (m in log2 units, l, o[G][D]) so
// the merge / epilogue code of the kernel is shared.
// ------------------------------------------------------------------------------------------------

// TKV: storage type of the pages; TQ: type of q (and of the output).  They differ only for 8-bit KV
// storage, where a lane's 16-byte vector holds 16 keys' worth of one row and q is still 16-bit.
template <typename TKV, typename TQ, int D, int G>
struct SimtEngine {
    using T = TKV;
    using C = Cfg<TKV, D, G>;
    static constexpr bool kTiled = false;
    static constexpr int PAGE_BYTES = C::PAGE_BYTES;
    static constexpr int STAGE_BYTES = C::STAGE_BYTES;
    static constexpr int SCRATCH_PER_WARP = G * kPage * 4;   // the page's softmax weights, [G][kPage] floats
    static constexpr int CTAS_PER_SM = (G >= 8) ? 1 : 2;      // G = 8 needs ~250 registers per thread

    float qf[G][C::EPL];
    float m_run[G], l_run[G], acc[G][C::EPL];
    int r, c, own_tok;
    bool owner;

    __device__ __forceinline__ void attach(unsigned char*, int) {}
    __device__ __forceinline__ void setup(int lane) {
        r = lane / C::LPR;             // which of the RPI rows of a warp-wide load this lane reads
        c = lane % C::LPR;             // which 16-byte vector of the row
        own_tok = owned_index<C::NV, C::LPR>(c) * C::RPI + r;   // token whose score this lane ends up owning
        owner = (c & (C::DUP - 1)) == 0;                        // one lane of each duplicate group
    }

    __device__ __forceinline__ void begin_item(const DecodeParams& p, int seq, int h, int lane) {
        const TQ* qg = static_cast<const TQ*>(p.q);
        constexpr int QV = C::EPL / Elt<TQ>::kPerVec;   // 16-byte loads covering this lane's EPL dims of q
        static_assert(QV >= 1 && QV * Elt<TQ>::kPerVec == C::EPL, "q type must not be narrower than the KV type");
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const TQ* qp = qg + (int64_t)seq * p.q_sb + (int64_t)(h * p.group + g) * p.q_sh + c * C::EPL;
#pragma unroll
            for (int v = 0; v < QV; ++v) {
                // heads past the real group size (template G is the group rounded up) are all-zero rows
                const uint4 u = g < p.group ? __ldg(reinterpret_cast<const uint4*>(qp) + v) : make_uint4(0, 0, 0, 0);
                Elt<TQ>::unpack(u, &qf[g][v * Elt<TQ>::kPerVec]);
            }
#pragma unroll
            for (int e = 0; e < C::EPL; ++e) qf[g][e] *= p.scale_log2;   // scores in base-2 units
            m_run[g] = -INFINITY; l_run[g] = 0.f;
#pragma unroll
            for (int e = 0; e < C::EPL; ++e) acc[g][e] = 0.f;
        }
    }

    // tokens t >= n_valid and hole_lo <= t < hole_hi of the page do not count
    __device__ __forceinline__ void page(const DecodeParams&, const unsigned char* stage, int n_valid, int hole_lo,
                                         int hole_hi, int lane, unsigned char* scratch) {
        float* p_smem = reinterpret_cast<float*>(scratch);
        const uint4* kp = reinterpret_cast<const uint4*>(stage) + lane;
        const uint4* vp = kp + C::PAGE_BYTES / 16;
        // ---- scores: q . k for the page's 16 tokens, all G heads
        float sc[G][C::NV];
#pragma unroll
        for (int i = 0; i < C::NV; ++i) {
            const uint4 u = kp[i * 32];
            float kf[C::EPL];
            Elt<T>::unpack(u, kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < C::EPL; ++e) a = fmaf(qf[g][e], kf[e], a);
                sc[g][i] = a;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s = transpose_reduce<C::NV, C::LPR / 2>(sc[g], c);
            if (own_tok >= n_valid || (own_tok >= hole_lo && own_tok < hole_hi))
                s = -INFINITY;                           // select, not arithmetic: stale slots may hold NaN
            const float m_page = warp_max_f32(s);
            if (m_page > m_run[g]) {                     // warp-uniform
                const float alpha = fast_exp2(m_run[g] - m_page);
                l_run[g] *= alpha;
#pragma unroll
                for (int e = 0; e < C::EPL; ++e) acc[g][e] *= alpha;
                m_run[g] = m_page;
            }
            const float pr = fast_exp2(s - m_run[g]);
            if (owner) { l_run[g] += pr; p_smem[g * kPage + own_tok] = pr; }
        }
        __syncwarp();
        // ---- weighted sum of V
        if (n_valid == kPage && hole_hi <= hole_lo) {
#pragma unroll
            for (int i = 0; i < C::NV; ++i) {
                const uint4 u = vp[i * 32];
                float vf[C::EPL];
                Elt<T>::unpack(u, vf);
                const int tok = i * C::RPI + r;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pg = p_smem[g * kPage + tok];
#pragma unroll
                    for (int e = 0; e < C::EPL; ++e) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
                }
            }
        } else {
            // a page cut by ctx_len, the sink or the window: rows that do not count are skipped, never multiplied
#pragma unroll
            for (int i = 0; i < C::NV; ++i) {
                const int tok = i * C::RPI + r;
                if (tok < n_valid && !(tok >= hole_lo && tok < hole_hi)) {
                    const uint4 u = vp[i * 32];
                    float vf[C::EPL];
                    Elt<T>::unpack(u, vf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float pg = p_smem[g * kPage + tok];
#pragma unroll
                        for (int e = 0; e < C::EPL; ++e) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
                    }
                }
            }
        }
        __syncwarp();
    }

    // fold the row groups of this warp and publish (m, l, o) of every head
    __device__ __forceinline__ void publish(const DecodeParams&, float* my_ml, float* my_o, int lane) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int off = C::LPR; off < 32; off <<= 1) {
#pragma unroll
                for (int e = 0; e < C::EPL; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], off);
            }
            l_run[g] = warp_sum_f32(l_run[g]);
        }
        if (r == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
#pragma unroll
                for (int e = 0; e < C::EPL; ++e) my_o[g * D + c * C::EPL + e] = acc[g][e];
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) { my_ml[g * 2] = m_run[g]; my_ml[g * 2 + 1] = l_run[g]; }
        }
    }
};

// TT: 16-bit type of the tiles fed to the tensor cores; TQ: type of q in global memory.
template <typename TT, typename TQ, int D, int G>
struct MmaCore {
    using T = TT;
    static_assert(sizeof(T) == 2 && D % 64 == 0 && G >= 1 && G <= 8, "tensor-core engine: 16-bit K/V, D % 64 == 0, G <= 8");
    static constexpr int TILES = D / 64;               // 64-element (128-byte) column tiles per row
    static constexpr int TILE_COLS = 64;               // elements per tile row (the TMA box's inner extent)
    static constexpr int TILE_BYTES = kPage * 128;     // 16 rows x 128 B, swizzled in 16-byte units
    static constexpr int PAGE_BYTES = TILES * TILE_BYTES;
    static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
    static constexpr int KSTEPS = D / 16;              // k-steps of Q K^T
    static constexpr int NBLK = D / 8;                 // 8-wide output blocks of P^T V

    // With head_dim 256 the accumulators alone take 128 registers.  The 32 registers of Q fragments then live in
    // this warp's scratch instead -- rows of D*2 + 16 bytes, so that the eight heads' rows start four banks
    // apart and a fragment load is conflict-free -- and are re-read for every k-step (measured faster than
    // keeping them in registers; with eight heads the merge area leaves no room for the scratch).
    static constexpr bool kQSmem = D >= 256 && G < 8;   // (eight heads x head_dim 256 run one CTA per SM with 255 registers)
    static constexpr int Q_ROW_WORDS = D / 2 + 4;
    static constexpr int Q_SCRATCH = kQSmem ? 8 * Q_ROW_WORDS * 4 : 0;
    uint32_t qa[kQSmem ? 1 : KSTEPS][2];    // A fragments of Q: head lane/4; rows 8..15 of the tile are zero
    uint32_t* qsm;             // kQSmem: this lane's first fragment word in the warp's scratch
    // Accumulators of P^T V for head lane/4, dims 8j + 2*(lane%4) + {0,1}: [0],[1] collect the 16-bit
    // weights (rows 0..7 of the A tile), [2],[3] the 16-bit corrections (rows 8..15); their sum is O.
    float o[NBLK][4];
    float m_run, l_run;        // running max (raw score units) and this lane's share of the sum

    __device__ __forceinline__ void setup(int) {}
    __device__ __forceinline__ void attach(unsigned char* scratch, int lane) {
        qsm = reinterpret_cast<uint32_t*>(scratch) + (lane >> 2) * Q_ROW_WORDS + (lane & 3);
    }

    // two consecutive q elements as one register of tile type (bf16 -> fp16 saturates at the fp16 range)
    __device__ __forceinline__ static uint32_t load_q_pair(const TQ* ptr) {
        const uint32_t raw = __ldg(reinterpret_cast<const uint32_t*>(ptr));
        if constexpr (std::is_same<TT, TQ>::value) {
            return raw;
        } else {
            const float2 f = unpack2<TQ>(raw);
            return pack2<TT>(fminf(fmaxf(f.x, -65504.f), 65504.f), fminf(fmaxf(f.y, -65504.f), 65504.f));
        }
    }

    __device__ __forceinline__ void begin_item(const DecodeParams& p, int seq, int h, int lane) {
        const int g = lane >> 2, c = lane & 3;
        if constexpr (kQSmem) {
            __syncwarp();   // every lane is done with the previous item's fragments
            const TQ* qrow = static_cast<const TQ*>(p.q) + (int64_t)seq * p.q_sb + (int64_t)(h * p.group + g) * p.q_sh;
#pragma unroll
            for (int s = 0; s < KSTEPS; ++s) {
                qsm[8 * s] = g < p.group ? load_q_pair(qrow + 16 * s + 2 * c) : 0u;
                qsm[8 * s + 4] = g < p.group ? load_q_pair(qrow + 16 * s + 2 * c + 8) : 0u;
            }
            __syncwarp();
        } else if (g < p.group) {
            const TQ* qrow = static_cast<const TQ*>(p.q) + (int64_t)seq * p.q_sb + (int64_t)(h * p.group + g) * p.q_sh;
#pragma unroll
            for (int s = 0; s < KSTEPS; ++s) {
                qa[s][0] = load_q_pair(qrow + 16 * s + 2 * c);
                qa[s][1] = load_q_pair(qrow + 16 * s + 2 * c + 8);
            }
        } else {
#pragma unroll
            for (int s = 0; s < KSTEPS; ++s) qa[s][0] = qa[s][1] = 0u;
        }
#pragma unroll
        for (int j = 0; j < NBLK; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        m_run = -INFINITY;
        l_run = 0.f;
    }

    // byte offset of 16-byte chunk `q` (0 .. D/8-1) of row `token` inside a swizzled page
    __device__ __forceinline__ static uint32_t chunk_off(int token, int q) {
        return (uint32_t)((q >> 3) * TILE_BYTES + token * 128 + (((q & 7) ^ (token & 7)) << 4));
    }

    // One page whose K and V tiles (swizzled, TILES x 2 KB each) sit at shared addresses kbase / vbase.
    // Rows of V that do not count must already be zero (see the engines).
    __device__ __forceinline__ void compute(const DecodeParams& p, uint32_t kbase, uint32_t vbase, int n_valid,
                                            int hole_lo, int hole_hi, int lane) {
        const int c = lane & 3;
        const int mi = lane >> 3, rr = lane & 7;   // ldmatrix: this lane addresses row rr of matrix mi
        const bool partial = n_valid < kPage || hole_hi > hole_lo;

        // ---- S^T[head, token] = Q K^T : two 8-token column blocks, KSTEPS k-steps each
        // (even and odd k-steps accumulate separately: four independent MMA chains instead of two)
        float s[2][2];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            float se[2] = {0.f, 0.f}, so[2] = {0.f, 0.f};
            const int token = nb * 8 + rr;
#pragma unroll
            for (int sp = 0; sp < KSTEPS / 2; ++sp) {
                uint32_t b[4];
                ldmatrix_x4(kbase + chunk_off(token, 4 * sp + mi), b);     // k-steps 2sp (b0,b1) and 2sp+1 (b2,b3)
                if constexpr (kQSmem) {
                    mma_m16n8k16_top<T>(se, qsm[16 * sp], qsm[16 * sp + 4], b[0], b[1]);
                    mma_m16n8k16_top<T>(so, qsm[16 * sp + 8], qsm[16 * sp + 12], b[2], b[3]);
                } else {
                    mma_m16n8k16_top<T>(se, qa[2 * sp][0], qa[2 * sp][1], b[0], b[1]);
                    mma_m16n8k16_top<T>(so, qa[2 * sp + 1][0], qa[2 * sp + 1][1], b[2], b[3]);
                }
            }
            s[nb][0] = se[0] + so[0];
            s[nb][1] = se[1] + so[1];
        }
        // this lane: head lane/4, tokens 2c, 2c+1 (block 0) and 8+2c, 9+2c (block 1)
        if (partial) {
            auto masked = [&](int tok) { return tok >= n_valid || (tok >= hole_lo && tok < hole_hi); };
            if (masked(2 * c)) s[0][0] = -INFINITY;
            if (masked(2 * c + 1)) s[0][1] = -INFINITY;
            if (masked(8 + 2 * c)) s[1][0] = -INFINITY;
            if (masked(9 + 2 * c)) s[1][1] = -INFINITY;
        }
        float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float sl2 = p.scale_log2;
        if (__any_sync(0xffffffffu, m_new > m_run)) {
            const float alpha = fast_exp2((m_run - m_new) * sl2);          // exp2(-inf) = 0 on the first page
            l_run *= alpha;
#pragma unroll
            for (int j = 0; j < NBLK; ++j) { o[j][0] *= alpha; o[j][1] *= alpha; o[j][2] *= alpha; o[j][3] *= alpha; }
            m_run = m_new;
        }
        const float msl = m_run * sl2;
        const float p0 = fast_exp2(fmaf(s[0][0], sl2, -msl)), p1 = fast_exp2(fmaf(s[0][1], sl2, -msl));
        const float p2 = fast_exp2(fmaf(s[1][0], sl2, -msl)), p3 = fast_exp2(fmaf(s[1][1], sl2, -msl));
        l_run += (p0 + p1) + (p2 + p3);
        // The S^T accumulator layout (row = head, cols = tokens 2c, 2c+1) is the A-fragment layout of
        // the next product: a0a1 = tokens 2c,2c+1, a4a5 = tokens 8+2c, 9+2c.
        // The weights are carried as a 16-bit value plus a 16-bit correction (p = hi + lo) so that P^T V
        // is accurate to ~2^-17 instead of the 2^-9 of a single bf16 rounding (which alone would exceed
        // the 2e-3 output tolerance on contexts of a few tokens).  The G <= 8 heads fill only rows 0..7
        // of the 16-row A tile, so the corrections ride in rows 8..15 of the same MMA at no extra cost.
        const uint32_t pa0 = pack2<T>(p0, p1), pa2 = pack2<T>(p2, p3);
        const float2 h01 = unpack2<T>(pa0), h23 = unpack2<T>(pa2);
        const uint32_t pb0 = pack2<T>(p0 - h01.x, p1 - h01.y), pb2 = pack2<T>(p2 - h23.x, p3 - h23.y);

        // ---- O[head, dim] += P^T V : NBLK 8-wide blocks, one k-step of 16 tokens
        const int vtok = (mi & 1) * 8 + rr;
#pragma unroll
        for (int jp = 0; jp < NBLK / 2; ++jp) {
            uint32_t b[4];
            ldmatrix_x4_trans(vbase + chunk_off(vtok, 2 * jp + (mi >> 1)), b);   // blocks 2jp (b0,b1), 2jp+1 (b2,b3)
            mma_m16n8k16<T>(o[2 * jp], pa0, pb0, pa2, pb2, b[0], b[1]);
            mma_m16n8k16<T>(o[2 * jp + 1], pa0, pb0, pa2, pb2, b[2], b[3]);
        }
    }

    __device__ __forceinline__ void publish(const DecodeParams& p, float* my_ml, float* my_o, int lane) {
        const int g = lane >> 2, c = lane & 3;
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (g < G) {
#pragma unroll
            for (int j = 0; j < NBLK; ++j)
                *reinterpret_cast<float2*>(my_o + g * D + 8 * j + 2 * c) =
                    make_float2(o[j][0] + o[j][2], o[j][1] + o[j][3]);
            if (c == 0) {
                my_ml[g * 2] = (m_run == -INFINITY) ? -INFINITY : m_run * p.scale_log2;
                my_ml[g * 2 + 1] = l_run;
            }
        }
    }
};


// 16-bit pools: pages arrive as swizzled tiles straight from the tiled TMA copies.
template <typename T, int D, int G>
struct MmaEngine : MmaCore<T, T, D, G> {
    using Core = MmaCore<T, T, D, G>;
    static constexpr bool kTiled = true;
    static constexpr int SCRATCH_PER_WARP = Core::Q_SCRATCH;   // the Q fragments, for head_dim 256 only
    // head_dim 256 runs one CTA per SM: a stage is 16 KB and the merge area up to 32 KB, which at two CTAs per
    // SM leaves four to six stages (one per consumer warp: no pipelining), and the accumulators alone take 128
    // of the 168 registers two CTAs allow.  Measured on 64 sequences x 4096 keys (same GPU): four query heads
    // per KV head 4.50 TB/s at two CTAs with Q in registers, 5.31 with Q in shared memory, 5.61 at one CTA;
    // eight heads 3.04 -> 3.35 TB/s.
    static constexpr int CTAS_PER_SM = D >= 256 ? 1 : 2;
    using Core::TILES; using Core::TILE_BYTES; using Core::PAGE_BYTES;

    __device__ __forceinline__ void page(const DecodeParams& p, unsigned char* stage, int n_valid, int hole_lo,
                                         int hole_hi, int lane, unsigned char*) {
        const bool partial = n_valid < kPage || hole_hi > hole_lo;
        if (partial) {
            // A page cut by ctx_len, the sink or the window: rows that do not count may hold stale bits (NaN
            // included).  Their weights are exactly zero, but 0 * NaN is NaN inside the MMA, so clear
            // those V rows.  (Rows are 128 bytes in every tile; the swizzle only permutes within a row.)
            for (int t = 0; t < TILES; ++t) {
                unsigned char* tile = stage + PAGE_BYTES + t * TILE_BYTES;
                for (int i = lane; i < (kPage - n_valid) * 8; i += 32)
                    *reinterpret_cast<uint4*>(tile + n_valid * 128 + i * 16) = make_uint4(0, 0, 0, 0);
                for (int i = lane; i < (hole_hi - hole_lo) * 8; i += 32)
                    *reinterpret_cast<uint4*>(tile + hole_lo * 128 + i * 16) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
        }
        const uint32_t kbase = smem_u32(stage);
        this->compute(p, kbase, kbase + PAGE_BYTES, n_valid, hole_lo, hole_hi, lane);
        if (partial) fence_proxy_async_smem();   // order the row clearing before the next TMA write
        __syncwarp();
    }
};

// 8-bit (e4m3) pools with grouped queries.  Pages arrive row-major (one untiled TMA copy each, 16 x D
// bytes); every consumer warp widens its page to fp16 -- e4m3 -> f16x2 is one exact instruction per
// pair -- into a private pair of swizzled tiles in shared memory and then runs the tensor-core code on
// them.  Rows that do not count are written as zeros during the widening.
template <typename TQ, int D, int G>
struct MmaFp8Engine : MmaCore<__half, TQ, D, G> {
    using Core = MmaCore<__half, TQ, D, G>;
    static constexpr bool kTiled = false;
    static constexpr int PAGE_BYTES = kPage * D;             // stored bytes of one K or V page
    static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
    static constexpr int SCRATCH_PER_WARP = 2 * Core::PAGE_BYTES;   // fp16 K and V tiles
    static constexpr int CTAS_PER_SM = 2;

    __device__ __forceinline__ static void widen(const unsigned char* src, unsigned char* dst, int n_valid, int hole_lo,
                                                 int hole_hi, int lane, bool mask_rows) {
        constexpr int VEC_PER_ROW = D / 16;                   // 16-byte vectors (16 values) per stored row
#pragma unroll
        for (int v = lane; v < kPage * VEC_PER_ROW; v += 32) {
            const int token = v / VEC_PER_ROW, part = v % VEC_PER_ROW;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
            if (!mask_rows || (token < n_valid && !(token >= hole_lo && token < hole_hi))) {
                const uint4 u = *reinterpret_cast<const uint4*>(src + v * 16);
                const __nv_fp8x2_storage_t* p2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&u);
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(p2[i], __NV_E4M3);
                    w[i] = (uint32_t)h.x | ((uint32_t)h.y << 16);
                }
                lo = make_uint4(w[0], w[1], w[2], w[3]);
                hi = make_uint4(w[4], w[5], w[6], w[7]);
            }
            *reinterpret_cast<uint4*>(dst + Core::chunk_off(token, 2 * part)) = lo;
            *reinterpret_cast<uint4*>(dst + Core::chunk_off(token, 2 * part + 1)) = hi;
        }
    }

    __device__ __forceinline__ void page(const DecodeParams& p, unsigned char* stage, int n_valid, int hole_lo,
                                         int hole_hi, int lane, unsigned char* scratch) {
        const bool partial = n_valid < kPage || hole_hi > hole_lo;
        widen(stage, scratch, n_valid, hole_lo, hole_hi, lane, false);                      // K: scores are masked later
        widen(stage + PAGE_BYTES, scratch + Core::PAGE_BYTES, n_valid, hole_lo, hole_hi, lane, partial);   // V: zero rows
        __syncwarp();
        const uint32_t kbase = smem_u32(scratch);
        this->compute(p, kbase, kbase + Core::PAGE_BYTES, n_valid, hole_lo, hole_hi, lane);
        __syncwarp();   // the tiles are rewritten for the next page
    }
};

// 8-bit (e4m3) pools, head_dim 64 or 128: the MMA operands are built in registers straight from the
// stored bytes -- no widened copy of the page in shared memory.  Pages arrive as one swizzled tile of
// 16 rows x D bytes each for K and V (tiled TMA; 128-byte swizzle for D = 128, 64-byte for D = 64).
// Both products may number their summation index and their output columns freely as long as both
// operands agree, and the numbering is chosen so that every lane reads whole chunks (D = 128 in
// brackets, D = 64 halves every figure):
//   * Q K^T: lane (g = lane/4, c = lane%4) holds bytes [32c, 32c+32) of key row g; byte pair
//     (4s, 4s+1) is B-fragment register 0 and pair (4s+2, 4s+3) register 1 of k-step s, and the
//     query fragments are loaded in the same numbering ([32] consecutive elements per lane).
//   * P^T V: the lane reads dims [16g, 16g+16) of the four value rows 2c, 2c+1, 2c+8, 2c+9; byte j
//     of those rows is the B fragment of output block j, so block j, column n is dim [16]n + j and
//     the lane ends up with the [32] consecutive dims from [32]c on of head g.
// e4m3 -> fp16 is exact (one cvt per pair); the weights are carried as fp16 value + correction in
// rows 0..7 / 8..15 of the A tile like in the 16-bit engine.
template <typename TQ, int D, int G>
struct MmaFp8RegEngine {
    static_assert(D == 128 || D == 64, "one swizzled tile of 128- or 64-byte rows per page");
    static_assert(G >= 1 && G <= 8, "query heads of one kv head fill rows 0..7 of the A tile");
    using TT = __half;
    static constexpr bool kTiled = true;
    static constexpr int TILES = 1;
    static constexpr int TILE_COLS = D;
    static constexpr int TILE_BYTES = kPage * D;
    static constexpr int PAGE_BYTES = TILE_BYTES;
    static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
    static constexpr int SCRATCH_PER_WARP = 0;
    static constexpr int CTAS_PER_SM = 2;
    static constexpr int KSTEPS = D / 16;
    static constexpr int NBLK = D / 8;
    static constexpr int LANE_DIMS = D / 4;    // consecutive dims of q and of the output one lane holds

    uint32_t qa[KSTEPS][2];
    float o[NBLK][4];          // block j: [0],[1] dims LANE_DIMS*c + j and + NBLK + j (weights), [2],[3] the corrections
    float m_run, l_run;

    __device__ __forceinline__ void setup(int) {}
    __device__ __forceinline__ void attach(unsigned char*, int) {}

    __device__ __forceinline__ static uint32_t to_half2(uint32_t raw) {
        if constexpr (std::is_same<TQ, __half>::value) {
            return raw;
        } else {
            const float2 f = unpack2<TQ>(raw);
            return pack2<TT>(fminf(fmaxf(f.x, -65504.f), 65504.f), fminf(fmaxf(f.y, -65504.f), 65504.f));
        }
    }

    // byte offset of 16-byte chunk `chunk` of row `row` inside a swizzled tile
    __device__ __forceinline__ static int chunk_off(int row, int chunk) {
        if constexpr (D == 128) return row * 128 + ((chunk ^ (row & 7)) << 4);
        else return row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4);
    }

    __device__ __forceinline__ void begin_item(const DecodeParams& p, int seq, int h, int lane) {
        const int g = lane >> 2, c = lane & 3;
        if (g < p.group) {
            const TQ* qrow = static_cast<const TQ*>(p.q) + (int64_t)seq * p.q_sb + (int64_t)(h * p.group + g) * p.q_sh + LANE_DIMS * c;
#pragma unroll
            for (int v = 0; v < LANE_DIMS / 8; ++v) {   // 16 bytes = elements 8v .. 8v + 7 of the lane's dims = k-steps 2v, 2v+1
                const uint4 u = __ldg(reinterpret_cast<const uint4*>(qrow) + v);
                qa[2 * v][0] = to_half2(u.x); qa[2 * v][1] = to_half2(u.y);
                qa[2 * v + 1][0] = to_half2(u.z); qa[2 * v + 1][1] = to_half2(u.w);
            }
        } else {
#pragma unroll
            for (int s = 0; s < KSTEPS; ++s) qa[s][0] = qa[s][1] = 0u;
        }
#pragma unroll
        for (int j = 0; j < NBLK; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        m_run = -INFINITY;
        l_run = 0.f;
    }

    __device__ __forceinline__ void page(const DecodeParams& p, unsigned char* stage, int n_valid, int hole_lo,
                                         int hole_hi, int lane, unsigned char*) {
        const int g = lane >> 2, c = lane & 3;
        const bool partial = n_valid < kPage || hole_hi > hole_lo;
        auto masked = [&](int tok) { return tok >= n_valid || (tok >= hole_lo && tok < hole_hi); };

        // value rows first: their loads overlap the score computation.  NBLK bytes per row: dims
        // [NBLK*g, NBLK*(g+1)) -- a whole 16-byte chunk for D = 128, half a chunk for D = 64.
        const unsigned char* vt = stage + PAGE_BYTES;
        uint32_t vw[4][NBLK / 4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = 2 * c + (i & 1) + (i >> 1) * 8;
            if constexpr (D == 128) {
                const uint4 u = *reinterpret_cast<const uint4*>(vt + chunk_off(row, g));
                vw[i][0] = u.x; vw[i][1] = u.y; vw[i][2] = u.z; vw[i][3] = u.w;
            } else {
                const uint2 u = *reinterpret_cast<const uint2*>(vt + chunk_off(row, g >> 1) + (g & 1) * 8);
                vw[i][0] = u.x; vw[i][1] = u.y;
            }
        }

        // ---- S^T[head, token] = Q K^T
        float s[2][2];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            const int row = nb * 8 + g;
            uint32_t w[KSTEPS];   // the lane's LANE_DIMS bytes of this key row: word t is k-step t
#pragma unroll
            for (int i = 0; i < KSTEPS / 4; ++i) {
                const uint4 u = *reinterpret_cast<const uint4*>(stage + chunk_off(row, (KSTEPS / 4) * c + i));
                w[4 * i] = u.x; w[4 * i + 1] = u.y; w[4 * i + 2] = u.z; w[4 * i + 3] = u.w;
            }
            float se[2] = {0.f, 0.f}, so[2] = {0.f, 0.f};
#pragma unroll
            for (int sp = 0; sp < KSTEPS / 2; ++sp) {
                mma_m16n8k16_top<TT>(se, qa[2 * sp][0], qa[2 * sp][1], cvt_e4m3x2_to_f16x2((uint16_t)(w[2 * sp] & 0xffffu)),
                                     cvt_e4m3x2_to_f16x2((uint16_t)(w[2 * sp] >> 16)));
                mma_m16n8k16_top<TT>(so, qa[2 * sp + 1][0], qa[2 * sp + 1][1],
                                     cvt_e4m3x2_to_f16x2((uint16_t)(w[2 * sp + 1] & 0xffffu)),
                                     cvt_e4m3x2_to_f16x2((uint16_t)(w[2 * sp + 1] >> 16)));
            }
            s[nb][0] = se[0] + so[0];
            s[nb][1] = se[1] + so[1];
        }
        if (partial) {
            if (masked(2 * c)) s[0][0] = -INFINITY;
            if (masked(2 * c + 1)) s[0][1] = -INFINITY;
            if (masked(8 + 2 * c)) s[1][0] = -INFINITY;
            if (masked(9 + 2 * c)) s[1][1] = -INFINITY;
            // rows that do not count may hold stale bytes (NaN included), and 0 * NaN is NaN in the MMA
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (masked(2 * c + (i & 1) + (i >> 1) * 8)) {
#pragma unroll
                    for (int k = 0; k < NBLK / 4; ++k) vw[i][k] = 0u;
                }
        }
        float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float sl2 = p.scale_log2;
        if (__any_sync(0xffffffffu, m_new > m_run)) {
            const float alpha = fast_exp2((m_run - m_new) * sl2);
            l_run *= alpha;
#pragma unroll
            for (int j = 0; j < NBLK; ++j) { o[j][0] *= alpha; o[j][1] *= alpha; o[j][2] *= alpha; o[j][3] *= alpha; }
            m_run = m_new;
        }
        const float msl = m_run * sl2;
        const float p0 = fast_exp2(fmaf(s[0][0], sl2, -msl)), p1 = fast_exp2(fmaf(s[0][1], sl2, -msl));
        const float p2 = fast_exp2(fmaf(s[1][0], sl2, -msl)), p3 = fast_exp2(fmaf(s[1][1], sl2, -msl));
        l_run += (p0 + p1) + (p2 + p3);
        const uint32_t pa0 = pack2<TT>(p0, p1), pa2 = pack2<TT>(p2, p3);
        const float2 h01 = unpack2<TT>(pa0), h23 = unpack2<TT>(pa2);
        const uint32_t pb0 = pack2<TT>(p0 - h01.x, p1 - h01.y), pb2 = pack2<TT>(p2 - h23.x, p3 - h23.y);

        // ---- O[head, dim] += P^T V
#pragma unroll
        for (int w = 0; w < NBLK / 4; ++w) {
            // bytes of rows (2c, 2c+1) and (2c+8, 2c+9) for dims 4w..4w+3 of the lane's chunk, interleaved into fragment order
            const uint32_t a01 = byte_perm(vw[0][w], vw[1][w], 0x5140u), a23 = byte_perm(vw[0][w], vw[1][w], 0x7362u);
            const uint32_t b01 = byte_perm(vw[2][w], vw[3][w], 0x5140u), b23 = byte_perm(vw[2][w], vw[3][w], 0x7362u);
            mma_m16n8k16<TT>(o[4 * w], pa0, pb0, pa2, pb2, cvt_e4m3x2_to_f16x2((uint16_t)(a01 & 0xffffu)),
                             cvt_e4m3x2_to_f16x2((uint16_t)(b01 & 0xffffu)));
            mma_m16n8k16<TT>(o[4 * w + 1], pa0, pb0, pa2, pb2, cvt_e4m3x2_to_f16x2((uint16_t)(a01 >> 16)),
                             cvt_e4m3x2_to_f16x2((uint16_t)(b01 >> 16)));
            mma_m16n8k16<TT>(o[4 * w + 2], pa0, pb0, pa2, pb2, cvt_e4m3x2_to_f16x2((uint16_t)(a23 & 0xffffu)),
                             cvt_e4m3x2_to_f16x2((uint16_t)(b23 & 0xffffu)));
            mma_m16n8k16<TT>(o[4 * w + 3], pa0, pb0, pa2, pb2, cvt_e4m3x2_to_f16x2((uint16_t)(a23 >> 16)),
                             cvt_e4m3x2_to_f16x2((uint16_t)(b23 >> 16)));
        }
        __syncwarp();   // every lane has read the stage before lane 0 hands it back
    }

    __device__ __forceinline__ void publish(const DecodeParams& p, float* my_ml, float* my_o, int lane) {
        const int g = lane >> 2, c = lane & 3;
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (g < G) {
            float* dst = my_o + g * D + LANE_DIMS * c;
#pragma unroll
            for (int j = 0; j < NBLK; j += 4) {
                *reinterpret_cast<float4*>(dst + j) = make_float4(o[j][0] + o[j][2], o[j + 1][0] + o[j + 1][2],
                                                                  o[j + 2][0] + o[j + 2][2], o[j + 3][0] + o[j + 3][2]);
                *reinterpret_cast<float4*>(dst + NBLK + j) = make_float4(o[j][1] + o[j][3], o[j + 1][1] + o[j + 1][3],
                                                                         o[j + 2][1] + o[j + 2][3], o[j + 3][1] + o[j + 3][3]);
            }
            if (c == 0) {
                my_ml[g * 2] = (m_run == -INFINITY) ? -INFINITY : m_run * p.scale_log2;
                my_ml[g * 2 + 1] = l_run;
            }
        }
    }
};

struct alignas(64) TensorMaps {
    CUtensorMap k, v;   // 4-D maps of the K and V pools: (dim, token in page, page, head)
};

// ENG picks the page engine; T is the type of q and of the output, TKV the storage type of the pools.
template <int ENG, typename T, typename TKV, int D, int G> struct EngineSelect;
template <typename T, typename TKV, int D, int G> struct EngineSelect<kEngSimt, T, TKV, D, G> { using type = SimtEngine<TKV, T, D, G>; };
template <typename T, typename TKV, int D, int G> struct EngineSelect<kEngMma, T, TKV, D, G> { using type = MmaEngine<T, D, G>; };
template <typename T, typename TKV, int D, int G> struct EngineSelect<kEngMmaFp8, T, TKV, D, G> { using type = MmaFp8Engine<T, D, G>; };
template <typename T, typename TKV, int D, int G> struct EngineSelect<kEngMmaFp8Reg, T, TKV, D, G> { using type = MmaFp8RegEngine<T, D, G>; };

}  // namespace
}  // namespace ivab
