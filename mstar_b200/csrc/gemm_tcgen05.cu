// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T (+bias, +residual, SwiGLU/GELU
// epilogues), fp32 accumulation in TMEM.
//
// One kernel serves both serving regimes:
//   * decode (M <= 128 tokens): "swapped" — the weight rows run along the UMMA M dimension (128 per tile)
//     and the few tokens along UMMA N, so no tensor-core rows are wasted and the kernel is a pure weight
//     stream. Split-K spreads a skinny weight over all 148 SMs; partials meet in a scratch workspace and the
//     last CTA of a tile reduces them in a fixed order (deterministic) and runs the epilogue.
//   * prefill / DiT (large M): tokens along UMMA M, weight rows along UMMA N (tile 128 x 256 or 128 x 128).
//
// Structure per CTA (192 threads): warp 0 = TMA producer, warp 1 = UMMA issuer and TMEM owner, warps 2-5 =
// epilogue (one TMEM lane quarter each). Operand tiles are K-major, 64 bf16 (128 bytes) wide, SWIZZLE_128B,
// moved by non-multicast TMA through a multi-stage mbarrier ring.
//
// Counterpart in the reference: every dense projection there is a cuBLAS call through F.linear
// (mstar/model/components/distributed/linear.py:8-419, mstar/model/components/mlp.py).
#include <cuda.h>
#include "common.cuh"
#include "host_common.h"
#include "comm_device.cuh"

namespace mstar {

// Optional tensor-parallel reduction fused into the epilogue (decode layout): every rank publishes its partial
// output tile in its symmetric-heap slot, raises the tile's flag at the peers, waits (bounded) for theirs and
// sums all ranks' tiles in rank order over NVLink, so the transfer of one tile overlaps the math of the others.
struct GemmAllReduce {
    PeerTable t;
    long long slot_bytes;       // two slots per rank, used in turn
    unsigned int* epoch;        // local: completed fused calls
    unsigned int* arrive;       // local: tiles finished in this launch
    int channel_base;
    int enabled;
};


struct GemmParams {
    int M, N, K;               // logical problem: C[M,N] = A[M,K] B[N,K]^T
    int swap;                  // 1: P operand (UMMA M) = B rows, Q operand (UMMA N) = A rows
    int splits;                // split-K factor (grid.z)
    int w_packed = 0;          // 1: the weight operand B is stored tile by tile: [ceil(N/128)][ceil(K/64)] tiles of
                               //    128 rows x 64 columns, each 16 KB contiguous (one TMA box = one DRAM burst run)
    unsigned long long* trace = nullptr;   // optional [CTAs][8] globaltimer stamps of the CTA's phases (bench only)
    int cluster_reduce = 0;    // 1: the splits of a tile form one thread-block cluster (1, 1, splits) and sum their
                               //    partial tiles through distributed shared memory (decode layout only)
    int kblocks_per_split;     // 64-wide K blocks handled by one split
    int kblocks_total;
    int epilogue;              // 0 none, 1 SwiGLU on interleaved (gate,up) output columns, 2 GELU(tanh)
    int out_f32;               // 1: C is fp32
    int ldc;                   // elements
    int ld_res;                // elements
    void* C;
    const __nv_bfloat16* bias;      // [N] or null
    const __nv_bfloat16* residual;  // [M, ld_res] or null
    float* workspace;               // split-K partials
    unsigned int* counters;         // one per output tile, zero on entry, zero again on exit
    KernelStatus* status;
    unsigned long long wait_limit_ns;
    float out_scale;                // multiplies the accumulator before bias (1.0 by default)
    GemmAllReduce ar;
    // grouped (mixture-of-experts) mode, decode layout only: the token rows (Q operand) are sorted by expert in
    // blocks of BN rows; block b multiplies with expert block_expert[b], whose weight rows start at
    // block_expert[b] * N in the stacked [E * N, K] weight. Blocks at or beyond *num_blocks do nothing.
    const int* block_expert;
    const int* num_blocks;
    const float* row_scale;         // optional per-token-row factor (routing weight), applied to the output row
    void* const* row_dst;           // optional per-token-row destination pointers (expert-parallel combine: the
                                    // row is stored straight into its owner's buffer, possibly on a peer GPU)
    // L2 management of the weight-streaming regime: while this kernel runs, its CTAs ask the L2 for the weights of
    // the kernel that follows; with l2_hints its own weight tiles (decode layout) are marked evict-first
    const void* pf_ptr = nullptr;
    unsigned long long pf_bytes = 0;
    int l2_hints = 0;
    // RMSNorm folded into its neighbours (decode layout): a projection whose output is the new residual stream also
    // accumulates, per token, the sum of squares of the bf16 values it stores (ss_out); the projection that consumes
    // the stream takes it un-normalised (its weight carries the norm's gain) and multiplies every output row by
    // rsqrt(ss_in[token] * ss_inv_h + ss_eps). ss_zero: ss_zero_n floats that this kernel clears after the previous
    // kernel has finished (the accumulator that the NEXT producer will add into).
    const float* ss_in = nullptr;
    float* ss_out = nullptr;
    float* ss_zero = nullptr;
    int ss_zero_n = 0;
    float ss_inv_h = 0.f, ss_eps = 0.f;
};

#define MSTAR_TRACE(i)                                                                                      \
    do {                                                                                                    \
        if (p.trace != nullptr)                                                                             \
            p.trace[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (i)] = \
                globaltimer_ns();                                                                           \
    } while (0)

constexpr int BM = 128;  // UMMA M (P-tile rows)
constexpr int BK = 64;   // bf16 elements per K block = 128 bytes = one swizzle atom
constexpr int UMMA_K = 16;

__host__ __device__ constexpr int gemm_stage_bytes(int BN) { return BM * BK * 2 + BN * BK * 2; }
__host__ __device__ constexpr int gemm_smem_bytes(int BN, int stages, int ksub = 1) {
    return stages * ksub * gemm_stage_bytes(BN) + 1024 /*alignment slack*/ + 256 /*barriers*/;
}

// Apply bias / activation / residual to a run of 32 accumulator values and store them.
// non-swapped: the thread owns output row m and 32 consecutive columns starting at n0.
template <bool OUT_F32>
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, int m, int n0, float* v, int ncols) {
    if (m >= p.M) return;
    if (p.out_scale != 1.0f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= p.out_scale;
    }
    if (p.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < ncols && n0 + i < p.N) v[i] += __bfloat162float(p.bias[n0 + i]);
    }
    if (p.epilogue == 1) {
        // (gate, up) interleaved along n: out column = n/2
        const int o0 = n0 >> 1;
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc + o0;
        const int half = ncols >> 1;
        const int No = p.N >> 1;
        if (half == 16 && o0 + 16 <= No && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float a = silu_f(v[4 * i]) * v[4 * i + 1];
                float b = silu_f(v[4 * i + 2]) * v[4 * i + 3];
                w[i] = pack_bf16x2(a, b);
            }
            reinterpret_cast<uint4*>(out)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(out)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            for (int i = 0; i < half; ++i)
                if (o0 + i < No) out[i] = __float2bfloat16(silu_f(v[2 * i]) * v[2 * i + 1]);
        }
        return;
    }
    if (p.epilogue == 2) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_f(v[i]);
    }
    if (p.residual != nullptr) {
        const __nv_bfloat16* r = p.residual + (size_t)m * p.ld_res + n0;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < ncols && n0 + i < p.N) v[i] += __bfloat162float(r[i]);
    }
    if constexpr (OUT_F32) {
        float* out = reinterpret_cast<float*>(p.C) + (size_t)m * p.ldc + n0;
        if (ncols == 32 && n0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(out)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
            for (int i = 0; i < ncols; ++i)
                if (n0 + i < p.N) out[i] = v[i];
        }
    } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc + n0;
        if (ncols == 32 && n0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(out)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        } else {
            for (int i = 0; i < ncols; ++i)
                if (n0 + i < p.N) out[i] = __float2bfloat16(v[i]);
        }
    }
}

// copy_out_staged for a projection with a folded RMSNorm on either side (see GemmParams::ss_in / ss_out). bf16 output
// only. Every lane of a warp runs the same number of trips (lanes beyond the last unit idle through them), because
// the sum of squares of a token row is first added up over the 16 lanes (8 for SwiGLU) that hold the row's units
// and only then sent to the accumulator: one atomic per token row and tile slice.
template <bool OUT_F32>
__device__ __noinline__ void copy_out_staged_norm(const GemmParams& pp, const float* stage, int rows, int m_base,
                                                  int n_in_base, int tid, bool dry) {
    struct {
        int M, N, ldc, ld_res, epilogue;
        float out_scale;
        void* C;
        const __nv_bfloat16* bias;
        const __nv_bfloat16* residual;
        const float* ss_in;
        float* ss_out;
        float inv_h, eps;
    } p = {pp.M, pp.N, pp.ldc, pp.ld_res, pp.epilogue, pp.out_scale, pp.C, pp.bias, pp.residual, pp.ss_in, pp.ss_out,
           pp.ss_inv_h, pp.ss_eps};
    constexpr int EPV = 8;
    const int ipo = p.epilogue == 1 ? 2 : 1;
    const int row_out = BM / ipo;
    const int units_per_row = row_out / EPV;             // 16, or 8 with SwiGLU: a power of two that divides 32
    const int total = rows * units_per_row;
    const int total_up = (total + 31) & ~31;
    const int n_out_base = n_in_base / ipo;
    const int n_limit = p.N / ipo;
    const bool vec_ok = (p.ldc % EPV == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        (p.residual == nullptr || (p.ld_res % 8 == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
    for (int u = tid; u < total_up; u += 128) {
        const int r = u / units_per_row, c = (u - r * units_per_row) * EPV;
        const int m = m_base + r, n = n_out_base + c;
        const bool live = u < total && m < p.M && n < n_limit;
        float ssq = 0.f;
        if (live) {
            const float* sp = stage + r * BM + c * ipo;
            const float sc = p.out_scale * (p.ss_in != nullptr ? rsqrtf(p.ss_in[m] * p.inv_h + p.eps) : 1.f);
            float x[EPV];
            if (ipo == 2) {
                float in[2 * EPV];
#pragma unroll
                for (int j = 0; j < 2 * EPV; j += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(sp + j);
                    in[j] = t.x; in[j + 1] = t.y; in[j + 2] = t.z; in[j + 3] = t.w;
                }
#pragma unroll
                for (int j = 0; j < 2 * EPV; ++j) {
                    const int nb = n_in_base + c * 2 + j;
                    in[j] = in[j] * sc + ((p.bias != nullptr && nb < p.N) ? __bfloat162float(p.bias[nb]) : 0.f);
                }
#pragma unroll
                for (int j = 0; j < EPV; ++j) x[j] = silu_f(in[2 * j]) * in[2 * j + 1];
            } else {
#pragma unroll
                for (int j = 0; j < EPV; j += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(sp + j);
                    x[j] = t.x; x[j + 1] = t.y; x[j + 2] = t.z; x[j + 3] = t.w;
                }
#pragma unroll
                for (int j = 0; j < EPV; ++j)
                    x[j] = x[j] * sc + ((p.bias != nullptr && n + j < n_limit) ? __bfloat162float(p.bias[n + j]) : 0.f);
                if (p.epilogue == 2) {
#pragma unroll
                    for (int j = 0; j < EPV; ++j) x[j] = gelu_tanh_f(x[j]);
                }
            }
            if (p.residual != nullptr) {
#pragma unroll
                for (int j = 0; j < EPV; ++j)
                    if (n + j < n_limit) x[j] += __bfloat162float(p.residual[(size_t)m * p.ld_res + n + j]);
            }
            // what is stored is what the next norm sees: square the bf16-rounded values
            __align__(16) __nv_bfloat16 o[EPV];
#pragma unroll
            for (int j = 0; j < EPV; ++j) {
                o[j] = __float2bfloat16(x[j]);
                const float f = __bfloat162float(o[j]);
                if (n + j < n_limit) ssq += f * f;
            }
            if (!dry) {
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc + n;
                if (vec_ok && n + EPV <= n_limit) {
                    *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(o);
                } else {
                    for (int j = 0; j < EPV; ++j)
                        if (n + j < n_limit) out[j] = o[j];
                }
            }
        }
        if (p.ss_out != nullptr) {
            for (int d = units_per_row >> 1; d > 0; d >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, d);
            if (live && !dry && (tid & (units_per_row - 1)) == 0) atomicAdd(p.ss_out + m, ssq);
        }
    }
}

// Swapped layout epilogue. Accumulators are first dumped raw into a shared-memory tile [token][weight row] (fp32;
// a few dozen instructions, so that the once-per-CTA epilogue does not pay instruction-cache misses for 32
// unrolled copies of the activation code), then one compact loop applies scale / bias / activation / residual
// and writes 16 bytes per lane, contiguous along the output columns.
// dry: run every instruction but keep the stores off. The epilogue warps call it once while the main loop streams,
// so that the real call after the last UMMA finds its code in the instruction cache (each CTA is the first on its SM
// for a one-wave decode GEMM: the cold epilogue measured 7 us of a 26 us kernel).
template <bool OUT_F32>
__device__ __noinline__ void copy_out_staged(const GemmParams& pp, const float* stage, int rows, int m_base,
                                             int n_in_base, int tid, bool dry = false) {
    // The kernel parameters are reached through a reference here, and the loop below stores to global memory: read
    // from the reference inside the loop, every field would be re-loaded after every store (measured: 4 us for eight
    // trips per thread). Local copies live in registers.
    struct {
        int M, N, ldc, ld_res, epilogue;
        float out_scale;
        void* C;
        const __nv_bfloat16* bias;
        const __nv_bfloat16* residual;
        const float* row_scale;
        void* const* row_dst;
    } p = {pp.M, pp.N, pp.ldc, pp.ld_res, pp.epilogue, pp.out_scale, pp.C, pp.bias, pp.residual, pp.row_scale, pp.row_dst};
    if (pp.ss_in != nullptr || pp.ss_out != nullptr) {
        copy_out_staged_norm<OUT_F32>(pp, stage, rows, m_base, n_in_base, tid, dry);
        return;
    }
    constexpr int EPV = OUT_F32 ? 4 : 8;                 // outputs per 16-byte store
    const int ipo = p.epilogue == 1 ? 2 : 1;             // accumulator columns per output (SwiGLU pairs)
    const int row_out = BM / ipo;
    const int units_per_row = row_out / EPV;
    const int total = rows * units_per_row;
    const int n_out_base = n_in_base / ipo;
    const int n_limit = p.N / ipo;
    const bool vec_ok = (p.ldc % EPV == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        (p.residual == nullptr || (p.ld_res % 8 == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
    for (int u = tid; u < total; u += 128) {
        const int r = u / units_per_row, c = (u - r * units_per_row) * EPV;
        const int m = m_base + r, n = n_out_base + c;
        if (m >= p.M || n >= n_limit) continue;
        const float* sp = stage + r * BM + c * ipo;
        float x[EPV];
        const bool full = n + EPV <= n_limit;
        if (ipo == 2) {
            float in[2 * EPV];
#pragma unroll
            for (int j = 0; j < 2 * EPV; j += 4) {
                const float4 t = *reinterpret_cast<const float4*>(sp + j);
                in[j] = t.x; in[j + 1] = t.y; in[j + 2] = t.z; in[j + 3] = t.w;
            }
            if (p.bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 2 * EPV; ++j) {
                    const int nb = n_in_base + c * 2 + j;
                    in[j] = in[j] * p.out_scale + (nb < p.N ? __bfloat162float(p.bias[nb]) : 0.f);
                }
            } else if (p.out_scale != 1.0f) {
#pragma unroll
                for (int j = 0; j < 2 * EPV; ++j) in[j] *= p.out_scale;
            }
#pragma unroll
            for (int j = 0; j < EPV; ++j) x[j] = silu_f(in[2 * j]) * in[2 * j + 1];
        } else {
#pragma unroll
            for (int j = 0; j < EPV; j += 4) {
                const float4 t = *reinterpret_cast<const float4*>(sp + j);
                x[j] = t.x; x[j + 1] = t.y; x[j + 2] = t.z; x[j + 3] = t.w;
            }
            if (p.bias != nullptr) {
#pragma unroll
                for (int j = 0; j < EPV; ++j)
                    x[j] = x[j] * p.out_scale + (n + j < n_limit ? __bfloat162float(p.bias[n + j]) : 0.f);
            } else if (p.out_scale != 1.0f) {
#pragma unroll
                for (int j = 0; j < EPV; ++j) x[j] *= p.out_scale;
            }
            if (p.epilogue == 2) {
#pragma unroll
                for (int j = 0; j < EPV; ++j) x[j] = gelu_tanh_f(x[j]);
            }
        }
        if (p.row_scale != nullptr) {
            const float rs = p.row_scale[m];
#pragma unroll
            for (int j = 0; j < EPV; ++j) x[j] *= rs;
        }
        if (p.row_dst != nullptr) {
            // expert-parallel combine: the destination row may live on a peer GPU; 16-byte peer stores
            if constexpr (!OUT_F32) {
                __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.row_dst[m]);
                if (drow != nullptr && !dry) {
                    if (full) {
                        *reinterpret_cast<uint4*>(drow + n) = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]),
                                                                           pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
                    } else {
                        for (int j = 0; j < EPV; ++j)
                            if (n + j < n_limit) drow[n + j] = __float2bfloat16(x[j]);
                    }
                }
            }
            continue;
        }
        if (p.residual != nullptr) {
            if (vec_ok && full) {
                const __nv_bfloat16* rp = p.residual + (size_t)m * p.ld_res + n;
                if constexpr (OUT_F32) {
                    const uint2 rv = *reinterpret_cast<const uint2*>(rp);
                    const float2 f0 = unpack_bf16x2(rv.x), f1 = unpack_bf16x2(rv.y);
                    x[0] += f0.x; x[1] += f0.y; x[2] += f1.x; x[3] += f1.y;
                } else {
                    const uint4 rv = *reinterpret_cast<const uint4*>(rp);
                    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = unpack_bf16x2(rw[j]);
                        x[2 * j] += f.x; x[2 * j + 1] += f.y;
                    }
                }
            } else {
                for (int j = 0; j < EPV; ++j)
                    if (n + j < n_limit) x[j] += __bfloat162float(p.residual[(size_t)m * p.ld_res + n + j]);
            }
        }
        if (dry) continue;
        if (vec_ok && full) {
            if constexpr (OUT_F32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + (size_t)m * p.ldc + n) =
                    make_float4(x[0], x[1], x[2], x[3]);
            } else {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc + n) =
                    make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                               pack_bf16x2(x[6], x[7]));
            }
        } else {
            for (int j = 0; j < EPV; ++j) {
                if (n + j >= n_limit) break;
                if constexpr (OUT_F32) reinterpret_cast<float*>(p.C)[(size_t)m * p.ldc + n + j] = x[j];
                else reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)m * p.ldc + n + j] = __float2bfloat16(x[j]);
            }
        }
    }
}

// Swapped-layout epilogue with the cross-rank sum. stage: [rows][BM] fp32 partial of this rank (rows of one exchange
// unit: a whole tile, or the slice of a tile that one CTA of a split-K cluster owns). PUSH protocol: the partial is
// rounded to bf16 and stored into EVERY PEER's slot (region [this rank] of the slot) with plain 16-byte stores over
// NVLink, which pipeline freely; one flag per unit tells the peers the stores are out; after the (bounded) wait for
// the peers' flags every read is local. An earlier pull version (each rank reading the peers' slots) paid one NVLink
// round trip per loop iteration: 57 us per fused GEMM against 18 us for the GEMM alone. Every rank adds the same
// bf16-rounded contributions in rank order, so all ranks hold bit-identical results.
__device__ __noinline__ void copy_out_allreduce(const GemmParams& pp, float* stage, int rows, int m_base, int n_base,
                                                int unit, int nunits, int tid, volatile int* flags) {
    const GemmAllReduce ar = pp.ar;          // local copies: see copy_out_staged
    struct {
        int M, N, ldc, ld_res;
        float out_scale;
        void* C;
        const __nv_bfloat16* bias;
        const __nv_bfloat16* residual;
        KernelStatus* status;
        unsigned long long wait_limit_ns;
    } p = {pp.M, pp.N, pp.ldc, pp.ld_res, pp.out_scale, pp.C, pp.bias, pp.residual, pp.status, pp.wait_limit_ns};
    if (tid == 0) flags[2] = (int)(*ar.epoch + 1u);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const unsigned int epoch = (unsigned int)flags[2];
    const long long slot_off = (long long)(epoch & 1u) * ar.slot_bytes;
    const long long region = (long long)p.M * p.N * 2;           // bytes of one rank's [M][N] bf16 contribution
    constexpr int EPV = 8;
    const int units_per_row = BM / EPV;
    const int total = rows * units_per_row;
    const int W = ar.t.world, R = ar.t.rank;
    // 1) round my partial, keep the rounded values in the staging tile, push them to the peers
    for (int u = tid; u < total; u += 128) {
        const int r = u / units_per_row, c = (u - r * units_per_row) * EPV;
        const int m = m_base + r, n = n_base + c;
        if (m >= p.M || n >= p.N) continue;
        float* sp = stage + r * BM + c;
        float x[EPV];
#pragma unroll
        for (int j = 0; j < EPV; j += 4) {
            const float4 t4 = *reinterpret_cast<const float4*>(sp + j);
            x[j] = t4.x; x[j + 1] = t4.y; x[j + 2] = t4.z; x[j + 3] = t4.w;
        }
#pragma unroll
        for (int j = 0; j < EPV; ++j) {
            x[j] *= p.out_scale;
            if (p.bias != nullptr && n + j < p.N) x[j] += __bfloat162float(p.bias[n + j]);
        }
        const uint4 packed = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]),
                                        pack_bf16x2(x[6], x[7]));
        const uint32_t pw[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = unpack_bf16x2(pw[j]);
            sp[2 * j] = f.x; sp[2 * j + 1] = f.y;
        }
        for (int q = 0; q < W; ++q) {
            if (q == R) continue;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(ar.t.buf[q]) + slot_off +
                                                                  (long long)R * region);
            *reinterpret_cast<uint4*>(dst + (size_t)m * p.N + n) = packed;
        }
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // 2) flags: tell the peers this unit is out, wait for theirs
    if (tid == 0) {
        const bool ok = signal_and_wait_all(ar.t, ar.channel_base + unit, epoch, p.status, p.wait_limit_ns, 0x40);
        flags[3] = ok ? 1 : 0;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // 3) sum in rank order (mine from the staging tile, the peers' from my own slot), add the residual, store
    if (flags[3]) {
        const char* mine = reinterpret_cast<const char*>(ar.t.buf[R]) + slot_off;
        for (int u = tid; u < total; u += 128) {
            const int r = u / units_per_row, c = (u - r * units_per_row) * EPV;
            const int m = m_base + r, n = n_base + c;
            if (m >= p.M || n >= p.N) continue;
            float acc[EPV];
#pragma unroll
            for (int j = 0; j < EPV; ++j) acc[j] = 0.f;
            for (int q = 0; q < W; ++q) {
                if (q == R) {
                    const float* sp = stage + r * BM + c;
#pragma unroll
                    for (int j = 0; j < EPV; ++j) acc[j] += sp[j];
                } else {
                    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(
                        reinterpret_cast<const __nv_bfloat16*>(mine + (long long)q * region) + (size_t)m * p.N + n));
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = unpack_bf16x2(w[j]);
                        acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
                    }
                }
            }
            if (p.residual != nullptr) {
                const uint4 v = *reinterpret_cast<const uint4*>(p.residual + (size_t)m * p.ld_res + n);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(w[j]);
                    acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
                }
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)m * p.ldc + n) =
                make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                           pack_bf16x2(acc[6], acc[7]));
        }
    }
    // 4) the last unit of the launch publishes the epoch for the next fused call
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(ar.arrive, 1u);
        if (old == (unsigned int)(nunits - 1)) {
            *ar.arrive = 0u;
            *ar.epoch = epoch;
        }
    }
}

// KSUB: 64-wide K blocks per pipeline stage. With KSUB = 1 every TMA box takes 128 bytes from each of 128 weight
// rows that lie a whole row pitch apart, and the next 128 bytes of those rows are only asked for a stage later: a
// weight-streaming (decode) GEMM then opens a DRAM page per 128 bytes and measured 1.3-2.2 TB/s. With KSUB = 2 or 4
// one stage asks for 256 or 512 contiguous bytes of every row back to back.
// SWAP: the layout is a template parameter so that a decode launch carries no token-major epilogue code (and the
// other way round): the once-per-CTA code of a one-wave decode GEMM stalled on instruction fetch (ncu no_instruction
// 4.9 per issue with both layouts compiled into one kernel).
template <int BN, int STAGES, int MINB, int KSUB = 1, bool SWAP = true>
__global__ void __launch_bounds__(192, MINB)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                         const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int P_BYTES = BM * BK * 2;                 // one 64-wide P sub-tile
    constexpr int Q_BYTES = BN * BK * 2;                 // one 64-wide Q sub-tile
    constexpr int STAGE_BYTES = KSUB * (P_BYTES + Q_BYTES);
    constexpr int Q_OFF = KSUB * P_BYTES;                // Q sub-tiles follow the P sub-tiles of the stage
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_slot + 1);  // [0] abort, [1] is_last, [2] epoch, [3] peers ok

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Blocks are scheduled x-fastest. Taking (x, y) as the tile directly makes a wave of CTAs share ONE Q tile and
    // stream the whole P operand past it, once per Q tile (measured: 3.2 GB of DRAM reads for 157 MB of operands
    // on 16384 x 9216 x 3072). Instead a wave covers a compact block of the tile grid: groups of GROUP_P tile rows,
    // inside a group the P index runs fastest, so a wave touches ~16 P tiles x ~9 Q tiles and L2 serves the re-use.
    int tile_p = blockIdx.x, tile_q = blockIdx.y;
    {
        constexpr int GROUP_P = 16;
        const int tiles_p = gridDim.x, tiles_q = gridDim.y;
        if (tiles_p >= 2 * GROUP_P && tiles_q > 1) {
            const int lin = blockIdx.y * tiles_p + blockIdx.x;
            const int per_group = GROUP_P * tiles_q;
            const int group = lin / per_group, within = lin - group * per_group;
            const int p0 = group * GROUP_P;
            const int gp = min(GROUP_P, tiles_p - p0);
            tile_p = p0 + within % gp;
            tile_q = within / gp;
        }
    }
    const int split = blockIdx.z;
    const int kb_begin = split * p.kblocks_per_split;
    int kb_end = kb_begin + p.kblocks_per_split;
    if (kb_end > p.kblocks_total) kb_end = p.kblocks_total;
    const int nkb = kb_end - kb_begin;  // host guarantees >= 1
    pdl_launch_dependents();
    if (threadIdx.x == 0) MSTAR_TRACE(0);
    int p_row0 = tile_p * BM;       // first row of this tile in the P operand
    if (p.block_expert != nullptr) {
        pdl_wait();
        if (tile_q >= *p.num_blocks) return;
        p_row0 += p.block_expert[tile_q] * p.N;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        flags[0] = 0;
        flags[1] = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmP);
        tma_prefetch_desc(&tmQ);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) MSTAR_TRACE(1);
    if (p.pf_bytes != 0 && threadIdx.x == 64)       // an epilogue warp, idle until the accumulator is complete
        l2_prefetch_slice(p.pf_ptr, p.pf_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                          gridDim.x * gridDim.y * gridDim.z, p.l2_hints != 0);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const bool w_stream = SWAP && p.l2_hints != 0;      // weight tiles are read once: first out of the L2
            const uint64_t pol_w = w_stream ? l2_policy_evict_first() : 0ull;
            // packed weights: tile (row tile t, K block kb) starts at row (t * kblocks_total + kb) * 128 of a
            // [tiles * 128, 64] matrix; the weight is the P operand in the decode layout, the Q operand otherwise
            const bool p_packed = p.w_packed && SWAP, q_packed = p.w_packed && !SWAP;
            auto load_P = [&](uint8_t* dst, uint64_t* bar, int kb) {
                const int x = p_packed ? 0 : kb * BK;
                const int y = p_packed ? ((p_row0 / BM) * p.kblocks_total + kb) * BM : p_row0;
                if (w_stream) tma_load_2d_hint(dst, &tmP, bar, x, y, pol_w);
                else tma_load_2d(dst, &tmP, bar, x, y);
            };
            auto load_Q = [&](uint8_t* dst, uint64_t* bar, int kb) {
                if (q_packed) {
#pragma unroll
                    for (int h = 0; h < (BN >= 128 ? BN / 128 : 1); ++h)
                        tma_load_2d(dst + h * (128 * BK * 2), &tmQ, bar, 0,
                                    ((tile_q * (BN / 128) + h) * p.kblocks_total + kb) * 128);
                } else {
                    tma_load_2d(dst, &tmQ, bar, kb * BK, tile_q * BN);
                }
            };
            int issued = 0;
            const int ngroups = (nkb + KSUB - 1) / KSUB;           // pipeline steps of up to KSUB K blocks
            auto group_subs = [&](int g) { return (nkb - g * KSUB) < KSUB ? (nkb - g * KSUB) : KSUB; };
            // The weight operand does not depend on the previous kernel: when it is the P operand (decode), fill
            // the ring with weight tiles first, and only then wait for the predecessor before touching activations.
            const int npre = SWAP ? (ngroups < STAGES ? ngroups : STAGES) : 0;
            for (int g = 0; g < npre; ++g) {
                const int ns = group_subs(g);
                mbar_expect_tx(&full_bar[g], ns * (P_BYTES + Q_BYTES));
                for (int u = 0; u < ns; ++u)
                    load_P(smem + g * STAGE_BYTES + u * P_BYTES, &full_bar[g], kb_begin + g * KSUB + u);
            }
            pdl_wait();
            for (int g = 0; g < npre; ++g) {
                const int ns = group_subs(g);
                for (int u = 0; u < ns; ++u)
                    load_Q(smem + g * STAGE_BYTES + Q_OFF + u * Q_BYTES, &full_bar[g], kb_begin + g * KSUB + u);
            }
            issued = npre;
            for (int g = npre; g < ngroups; ++g) {
                const int s = g % STAGES;
                const uint32_t ph = (g / STAGES) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_GEMM, 1, g, s);
                    flags[0] = 1;
                    break;
                }
                if (flags[0]) break;
                uint8_t* sp = smem + s * STAGE_BYTES;
                const int ns = group_subs(g);
                mbar_expect_tx(&full_bar[s], ns * (P_BYTES + Q_BYTES));
                for (int u = 0; u < ns; ++u) {
                    load_P(sp + u * P_BYTES, &full_bar[s], kb_begin + g * KSUB + u);
                    load_Q(sp + Q_OFF + u * Q_BYTES, &full_bar[s], kb_begin + g * KSUB + u);
                }
                issued = g + 1;
            }
            if (flags[0]) {
                // error path: let copies already in flight land before the CTA leaves
                for (int g = (issued > STAGES ? issued - STAGES : 0); g < issued; ++g)
                    mbar_wait(&full_bar[g % STAGES], (g / STAGES) & 1, 1000000ull);
            }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1);
            bool ok = true;
            const int ngroups = (nkb + KSUB - 1) / KSUB;
            for (int g = 0; g < ngroups; ++g) {
                const int s = g % STAGES;
                const uint32_t ph = (g / STAGES) & 1;
                if (!mbar_wait(&full_bar[s], ph, p.wait_limit_ns)) {
                    report_status(p.status, KID_GEMM, 2, g, s);
                    flags[0] = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (g == 0) MSTAR_TRACE(3);
                const uint32_t sp = smem_u32(smem + s * STAGE_BYTES);
                const int ns = (nkb - g * KSUB) < KSUB ? (nkb - g * KSUB) : KSUB;
                for (int u = 0; u < ns; ++u) {
                    const uint64_t da = umma_smem_desc_sw128(sp + u * P_BYTES);
                    const uint64_t db = umma_smem_desc_sw128(sp + Q_OFF + u * Q_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // +32 bytes per K slice inside the 128-byte swizzle atom (encoded >> 4)
                        umma_f16_ss(tmem_base, da + 2 * k, db + 2 * k, idesc, (g | u | k) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(&empty_bar[s]);
            }
            if (ok) umma_commit(acc_bar);
            MSTAR_TRACE(4);
        }
    } else {
        // ---------------- epilogue warps (TMEM lane quarter = warp % 4) ----------------
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;  // accumulator row (TMEM lane) owned by this thread
        pdl_wait();
        if (p.ss_zero != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
            // the previous kernel is complete: nobody reads this accumulator any more, the next producer adds into it
            for (int i = threadIdx.x - 64; i < p.ss_zero_n; i += 128) p.ss_zero[i] = 0.f;
        }
        if (SWAP && !p.ar.enabled) {
            // instruction-cache warm-up (see copy_out_staged); reads an untouched corner of the staging area
            if (p.out_f32) copy_out_staged<true>(p, reinterpret_cast<const float*>(smem), 1, tile_q * BN, tile_p * BM, threadIdx.x - 64, true);
            else copy_out_staged<false>(p, reinterpret_cast<const float*>(smem), 1, tile_q * BN, tile_p * BM, threadIdx.x - 64, true);
        }
        bool ok = mbar_wait(acc_bar, 0, p.wait_limit_ns + 500000000ull);
        if (!ok) {
            report_status(p.status, KID_GEMM, 3, 0, 0);
            flags[0] = 1;
        }
        tc_fence_after();
        if (threadIdx.x == 64) MSTAR_TRACE(5);
        const int pidx = tile_p * BM + row;  // index along the P operand's rows
        constexpr int CH = BN < 32 ? BN : 32;
        const int tile_lin = tile_q * gridDim.x + tile_p;
        bool do_final = ok;

        if (p.cluster_reduce) {
            // the partial tile goes to this CTA's staging tile; the cluster sums the tiles after the role branches
            do_final = false;
            if (ok) {
                float* stage = reinterpret_cast<float*>(smem);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += CH) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0;
                    if constexpr (CH == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < CH; ++i) stage[(c0 + i) * BM + row] = __uint_as_float(r[i]);
                }
            }
        } else if (ok && p.splits > 1) {
            // 1) publish this split's partial tile: layout [col][row] so that a warp writes 128 B per column
            float* wsp = p.workspace + ((size_t)(split * gridDim.x * gridDim.y + tile_lin)) * (BM * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0;
                if constexpr (CH == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < CH; ++i) __stcg(&wsp[(size_t)(c0 + i) * BM + row], __uint_as_float(r[i]));
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
                unsigned int old = atomicAdd(&p.counters[tile_lin], 1u);
                flags[1] = (old == (unsigned int)(p.splits - 1)) ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            do_final = flags[1] != 0;
            if (do_final) __threadfence();
        }

        if (do_final) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                float v[32];
                if (p.splits > 1) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                    for (int z = 0; z < p.splits; ++z) {
                        const float* wsp =
                            p.workspace + ((size_t)(z * gridDim.x * gridDim.y + tile_lin)) * (BM * BN);
#pragma unroll
                        for (int i = 0; i < CH; ++i) v[i] += __ldcg(&wsp[(size_t)(c0 + i) * BM + row]);
                    }
                } else {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0;
                    if constexpr (CH == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < CH; ++i) v[i] = __uint_as_float(r[i]);
                }
                const int qidx = tile_q * BN + c0;
                if (SWAP) {
                    // the pipeline stages are idle by now (all TMA loads consumed): reuse them as staging tile
                    float* stage = reinterpret_cast<float*>(smem);
#pragma unroll
                    for (int i = 0; i < CH; ++i) stage[(c0 + i) * BM + row] = v[i];
                } else {
                    if (p.out_f32) store_row_chunk<true>(p, pidx, qidx, v, CH);
                    else store_row_chunk<false>(p, pidx, qidx, v, CH);
                }
            }
            if (SWAP) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) MSTAR_TRACE(2);
                if (p.ar.enabled) copy_out_allreduce(p, reinterpret_cast<float*>(smem), BN, tile_q * BN, tile_p * BM, tile_lin, gridDim.x * gridDim.y, threadIdx.x - 64, flags);
                else if (p.out_f32) copy_out_staged<true>(p, reinterpret_cast<const float*>(smem), BN, tile_q * BN, tile_p * BM, threadIdx.x - 64);
                else copy_out_staged<false>(p, reinterpret_cast<const float*>(smem), BN, tile_q * BN, tile_p * BM, threadIdx.x - 64);
            }
            if (p.splits > 1 && threadIdx.x == 64) p.counters[tile_lin] = 0u;  // ready for the next launch
        }
        if (threadIdx.x == 64) MSTAR_TRACE(6);
        tc_fence_before();
    }
    if (p.cluster_reduce) {
        // Split-K without a trip through global memory: every CTA of the cluster holds the partial tile of its K
        // range in shared memory [token][weight row]. After the cluster barrier CTA k sums token rows
        // [k * rows / splits, (k + 1) * rows / splits) over all peers (fixed order: deterministic) into its own copy
        // of those rows, which no peer reads, and finishes them (bias / activation / residual / store). The second
        // barrier keeps every CTA's shared memory alive until its peers have read it.
        __syncwarp();
        cluster_sync_all();
        if (warp >= 2) {
            const int tid = threadIdx.x - 64;
            const int nsp = p.splits;
            const int crank = (int)cluster_ctarank();
            const int m_base = tile_q * BN;
            int vr = p.M - m_base;
            vr = vr > BN ? BN : (vr < 0 ? 0 : vr);
            const int r0 = crank * vr / nsp, r1 = (crank + 1) * vr / nsp;
            float* stage = reinterpret_cast<float*>(smem);
            const bool live = r1 > r0 && !flags[0];
            if (live) {
                uint32_t peer[8];
                const uint32_t sbase = smem_u32(stage);
#pragma unroll
                for (int z = 0; z < 8; ++z) peer[z] = cluster_map_shared(sbase, (uint32_t)(z < nsp ? z : 0));
                for (int e = r0 * (BM / 4) + tid; e < r1 * (BM / 4); e += 128) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int z = 0; z < 8; ++z) {
                        if (z < nsp) {
                            const float4 v = ld_cluster_f4(peer[z] + (uint32_t)e * 16u);
                            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                        }
                    }
                    reinterpret_cast<float4*>(stage)[e] = acc;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!p.ar.enabled) {
                    if (p.out_f32) copy_out_staged<true>(p, stage + r0 * BM, r1 - r0, m_base + r0, tile_p * BM, tid);
                    else copy_out_staged<false>(p, stage + r0 * BM, r1 - r0, m_base + r0, tile_p * BM, tid);
                }
            }
            if (p.ar.enabled) {
                // tensor-parallel sum: every (tile, cluster rank) slice is its own exchange unit with its own flag
                // channel; an empty slice still signals and arrives so that the ranks stay in step
                const int tile_lin = tile_q * gridDim.x + tile_p;
                copy_out_allreduce(p, stage + r0 * BM, live ? r1 - r0 : 0, m_base + r0, tile_p * BM,
                                   tile_lin * nsp + crank, (int)(gridDim.x * gridDim.y) * nsp, tid, flags);
            }
        }
        if (threadIdx.x == 64) MSTAR_TRACE(7);
        __syncwarp();
        cluster_sync_all();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Row-parallel GEMM with the all-reduce INSIDE the kernel, overlapped tile group by tile group (large M).
//
// The persistent kernel below gets two kinds of CTAs in ONE launch: the first n_gemm CTAs walk the tile list and
// store their output tiles into this rank's copy of a symmetric region; the last n_comm CTAs reduce. Tiles are
// visited in groups of `group_p` row tiles (all column tiles of a group before the next group), so row groups are
// completed one after another while later groups are still being multiplied. For each group the communication CTAs
// wait (bounded) until all of its tiles are stored here (a local counter that the epilogues bump), tell the peers,
// wait for the peers' same message, and then sum THIS rank's share of the group's rows over all ranks' copies with
// plain peer loads and store the sum back into every rank's copy (an in-place all-reduce of the group, n (W - 1) / W
// bytes per direction per GPU). The last group's reduction is the only communication that is not hidden behind
// tensor-core work. GEMM CTAs never wait for communication CTAs, and all CTAs of the launch are co-resident (the grid
// is at most one CTA per SM), so no wait can be circular; every wait is bounded and reports through the status word.
// ---------------------------------------------------------------------------------------------
struct TileAR {
    PeerTable t;                 // region bases and flag bases of the group
    McastTable mc;               // only the flag multicast is used
    long long off;               // byte offset of C inside the region (C is [M, N] bf16, leading dimension N)
    long long stage_off;         // byte offset of the staging area: [W - 1 sources][the groups' shares, back to back] (16-byte vectors)
    int n_comm;                  // communication CTAs (the last CTAs of the grid)
    int group_p;                 // row tiles per group
    int channel_base;            // flag channels [base, base + 2 * groups)
    unsigned int* done;          // [groups] local: output tiles stored, per group
    unsigned int* push_done;     // [groups] local: communication CTAs that have pushed their slice of the group
    unsigned int* red_done;      // [groups] local: communication CTAs that have reduced their slice of the group
    unsigned int* epoch;         // local: completed calls
    unsigned int* arrive;        // local: communication CTAs finished
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};

// Geometry of one row group: vectors [v0, v1) of C, cut into W shares of `share` vectors (rank q owns share q).
struct TileARGroup { long long v0, v1, share; };
__device__ __forceinline__ TileARGroup tile_ar_group(const TileAR& ta, int g, int M, int N, int tiles_p) {
    const int tp0 = g * ta.group_p;
    const int gp = min(ta.group_p, tiles_p - tp0);
    const long long r0 = (long long)tp0 * BM;
    long long r1 = r0 + (long long)gp * BM;
    if (r1 > M) r1 = M;
    TileARGroup G;
    G.v0 = r0 * N / 8;
    G.v1 = r1 * N / 8;
    G.share = (G.v1 - G.v0 + ta.t.world - 1) / ta.t.world;
    return G;
}

// Untiled bulk copies (the TMA engine, no tensor map, never multicast): global -> shared with an mbarrier, and
// shared -> global (local or peer memory) in bulk groups. One thread keeps hundreds of KB in flight, which plain
// stores from the 192 threads of a CTA cannot (measured: about 6 GB/s of peer stores per communication CTA).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

constexpr int TAR_CHUNK = 8192;          // bytes per bulk copy
constexpr int TAR_MAX_STAGES = 16;

//   push(g):   for every peer q, copy this rank's partial of q's share of group g into q's staging slot for this rank
//              (local C -> shared memory -> peer memory, batches of up to 16 chunks in flight)
//   reduce(g): this rank's share of group g: the local partial and the W - 1 staged copies come into shared memory,
//              the threads add them in rank order (fp32), the sum leaves for every rank's C
// The communication CTAs do push(g), then reduce(g - 1): the wait for the peers' pushes of a group is covered by the
// push of the next. Remote traffic is stores only: a load over NVLink holds an SM's few outstanding-request slots for
// a round trip (measured: about 2 GB/s per SM when pulling).
__device__ __noinline__ void tile_ar_comm_role(const TileAR& ta, const int c, const int M, const int N,
                                               const int tiles_p, const int tiles_q, uint8_t* smem, const int smem_bytes) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch, s_batch;
    __shared__ __align__(8) uint64_t full[TAR_MAX_STAGES];
    if (threadIdx.x == 0) {
        s_epoch = *ta.epoch + 1;
        s_ok = 1;
        for (int i = 0; i < TAR_MAX_STAGES; ++i) mbar_init(&full[i], 1);
        mbar_fence_init();
    }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int W = ta.t.world, R = ta.t.rank;
    const int groups = (tiles_p + ta.group_p - 1) / ta.group_p;
    // every group but the last has the same share; a source's slot in the staging area holds the groups' shares
    // back to back
    const long long share_full = tile_ar_group(ta, 0, M, N, tiles_p).share;
    const long long slot_stride = (long long)(groups - 1) * share_full + tile_ar_group(ta, groups - 1, M, N, tiles_p).share;
    char* const local = static_cast<char*>(ta.t.buf[R]);
    constexpr int CV = TAR_CHUNK / 16;                                           // vectors per chunk
    const int push_stages = min(TAR_MAX_STAGES, smem_bytes / TAR_CHUNK);
    const int red_stages = min(TAR_MAX_STAGES, smem_bytes / ((W + 1) * TAR_CHUNK));
    unsigned int batch = 0;              // batches run so far: every stage barrier completes one phase per batch
    for (int g = 0; g <= groups && s_ok; ++g) {
        if (g < groups) {
            // ---- push(g) ----
            const int gp = min(ta.group_p, tiles_p - g * ta.group_p);
            if (threadIdx.x == 0 &&
                !wait_flag(ta.done + g, (unsigned int)(gp * tiles_q), ta.wait_limit_ns)) {
                report_status(ta.status, KID_GEMM_AR, 0x41, g, c);
                s_ok = 0;
            }
            __syncthreads();
            if (!s_ok) break;
            if (threadIdx.x == 0) {
                fence_proxy_async_all();         // the epilogues' stores, seen through the counter, before bulk reads
                const TileARGroup G = tile_ar_group(ta, g, M, N, tiles_p);
                for (int q = 0; q < W && s_ok; ++q) {
                    if (q == R) continue;
                    const long long a = min(G.v1, G.v0 + (long long)q * G.share), b = min(G.v1, a + G.share);
                    const long long per = (b > a ? (b - a + ta.n_comm - 1) / ta.n_comm : 0);
                    const long long ca = a + (long long)c * per, cb = min(b, ca + per);
                    const int slot = R < q ? R : R - 1;
                    const uint4* src = reinterpret_cast<const uint4*>(local + ta.off);
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(ta.t.buf[q]) + ta.stage_off) +
                                 (long long)slot * slot_stride + (long long)g * share_full - a;
                    for (long long v = ca; v < cb && s_ok; v += (long long)push_stages * CV, ++batch) {
                        for (int st = 0; st < push_stages; ++st) {
                            const long long vs = v + (long long)st * CV;
                            const long long n = vs < cb ? min((long long)CV, cb - vs) : 0;
                            mbar_expect_tx(&full[st], (uint32_t)(n * 16));
                            if (n > 0) bulk_load(smem + st * TAR_CHUNK, src + vs, (uint32_t)(n * 16), &full[st]);
                        }
                        for (int st = 0; st < push_stages; ++st) {
                            const long long vs = v + (long long)st * CV;
                            const long long n = vs < cb ? min((long long)CV, cb - vs) : 0;
                            if (!mbar_wait(&full[st], batch & 1u, ta.wait_limit_ns)) {
                                report_status(ta.status, KID_GEMM_AR, 0x44, g, st);
                                s_ok = 0;
                                break;
                            }
                            if (n > 0) bulk_store(dst + vs, smem + st * TAR_CHUNK, (uint32_t)(n * 16));
                        }
                        tma_store_commit();
                        bulk_wait_read_all();        // the stages may be refilled
                        for (int st = push_stages; st < TAR_MAX_STAGES; ++st) mbar_expect_tx(&full[st], 0);
                    }
                }
                tma_store_wait_all();                // this CTA's pushes of the group have been written
                fence_proxy_async_all();
                __threadfence_system();
                const unsigned int old = atomicAdd(ta.push_done + g, 1u);
                if (old == (unsigned int)ta.n_comm - 1u) {      // every slice of this rank's pushes of group g is out
                    __threadfence_system();
                    signal_all(ta.t, ta.mc, ta.channel_base + g, epoch);
                }
                s_batch = batch;
            }
            __syncthreads();
            batch = s_batch;                     // only thread 0 ran the push batches
        }
        if (g >= 1 && s_ok) {
            // ---- reduce(g - 1) ----
            const int h = g - 1;
            if (threadIdx.x == 0) {
                if (!wait_all(ta.t, ta.channel_base + h, epoch, ta.status, ta.wait_limit_ns, 0x42)) s_ok = 0;
                fence_proxy_async_all();         // the peers' pushes, seen through their flags, before bulk reads
            }
            __syncthreads();
            if (!s_ok) break;
            const TileARGroup G = tile_ar_group(ta, h, M, N, tiles_p);
            const long long a = min(G.v1, G.v0 + (long long)R * G.share), b = min(G.v1, a + G.share);
            const long long per = (b > a ? (b - a + ta.n_comm - 1) / ta.n_comm : 0);
            const long long ca = a + (long long)c * per, cb = min(b, ca + per);
            const uint4* mine = reinterpret_cast<const uint4*>(local + ta.off);
            const uint4* staged = reinterpret_cast<const uint4*>(local + ta.stage_off) + (long long)h * share_full - a;
            const int stage_bytes = (W + 1) * TAR_CHUNK;        // W inputs in rank order, then the sum
            for (long long v = ca; v < cb && s_ok; v += (long long)red_stages * CV, ++batch) {
                if (threadIdx.x == 0) {
                    for (int st = 0; st < TAR_MAX_STAGES; ++st) {
                        const long long vs = v + (long long)st * CV;
                        const long long n = (st < red_stages && vs < cb) ? min((long long)CV, cb - vs) : 0;
                        mbar_expect_tx(&full[st], (uint32_t)(n * 16 * W));
                        if (n == 0) continue;
                        for (int q = 0; q < W; ++q) {
                            const uint4* srcq = q == R ? mine + vs : staged + (long long)(q < R ? q : q - 1) * slot_stride + vs;
                            bulk_load(smem + st * stage_bytes + q * TAR_CHUNK, srcq, (uint32_t)(n * 16), &full[st]);
                        }
                    }
                }
                for (int st = 0; st < red_stages; ++st) {
                    const long long vs = v + (long long)st * CV;
                    const long long n = vs < cb ? min((long long)CV, cb - vs) : 0;
                    if (n == 0) break;                   // uniform: every thread sees the same bounds
                    const bool landed = mbar_wait(&full[st], batch & 1u, ta.wait_limit_ns);
                    uint4* in = reinterpret_cast<uint4*>(smem + st * stage_bytes);
                    uint4* out = in + W * CV;
                    if (landed) {
                        for (int i = threadIdx.x; i < (int)n; i += blockDim.x) {
                            float acc[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                            for (int q = 0; q < W; ++q) add_bf16x8(acc, in[q * CV + i]);
                            out[i] = pack8(acc);
                        }
                    } else {
                        if (threadIdx.x == 0) report_status(ta.status, KID_GEMM_AR, 0x45, h, st);
                        s_ok = 0;
                    }
                    fence_proxy_async_smem();        // the sums, written by threads, before the bulk stores read them
                    __syncthreads();
                    if (threadIdx.x == 0 && s_ok) {
                        for (int q = 0; q < W; ++q)
                            bulk_store(reinterpret_cast<uint4*>(static_cast<char*>(ta.t.buf[q]) + ta.off) + vs, out,
                                       (uint32_t)(n * 16));
                        tma_store_commit();
                    }
                }
                if (threadIdx.x == 0) bulk_wait_read_all();
                __syncthreads();                     // stages free, and s_ok agreed on
            }
            if (threadIdx.x == 0) {
                tma_store_wait_all();
                fence_proxy_async_all();
                __threadfence_system();
                const unsigned int old = atomicAdd(ta.red_done + h, 1u);
                if (old == (unsigned int)ta.n_comm - 1u) {      // this rank's share of the group is summed everywhere
                    __threadfence_system();
                    signal_all(ta.t, ta.mc, ta.channel_base + groups + h, epoch);
                }
            }
            __syncthreads();
        }
    }
    // the peers' shares of every group have landed here before the kernel (and with it the stream) moves on
    if (threadIdx.x == 0 && s_ok) {
        for (int g = c; g < groups; g += ta.n_comm)
            if (!wait_all(ta.t, ta.channel_base + groups + g, epoch, ta.status, ta.wait_limit_ns, 0x43)) break;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        tma_store_wait_all();
        __threadfence();
        const unsigned int old = atomicAdd(ta.arrive, 1u);
        if (old == (unsigned int)ta.n_comm - 1u) {
            for (int g = 0; g < groups; ++g) { ta.done[g] = 0u; ta.push_done[g] = 0u; ta.red_done[g] = 0u; }
            *ta.arrive = 0u;
            __threadfence();
            *ta.epoch = epoch;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Persistent variant for large token-major GEMMs (M > 128, one K split): one CTA per SM walks the tile list.
// Two TMEM accumulators of BN columns: while the four epilogue warps drain tile i (TMEM -> registers -> bias /
// activation / residual -> global), the UMMA warp is already accumulating tile i + 1 into the other buffer and the
// TMA warp is prefetching its operands; barrier set-up, TMEM allocation and pipeline fill are paid once per CTA
// instead of once per tile. Tiles are visited in the grouped order of the non-persistent kernel.
// ---------------------------------------------------------------------------------------------
template <int BN, int STAGES, bool FUSED = false>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_persistent_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                            const __grid_constant__ GemmParams p, const int tiles_p, const int tiles_q,
                            const __grid_constant__ TileAR ta) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int P_BYTES = BM * BK * 2;
    constexpr int STAGE_BYTES = gemm_stage_bytes(BN);
    constexpr int TMEM_COLS = 2 * BN;
    static_assert(TMEM_COLS <= 512, "two accumulators must fit in TMEM");
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;      // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_slot + 1);  // [0] abort

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = tiles_p * tiles_q;
    const int nkb = p.kblocks_total;
    pdl_launch_dependents();
    // tile walkers: all CTAs, or all but the communication CTAs at the end of the grid
    const int n_walk = FUSED ? (int)gridDim.x - ta.n_comm : (int)gridDim.x;
    if constexpr (FUSED) {
        if ((int)blockIdx.x >= n_walk) {
            pdl_wait();
            tile_ar_comm_role(ta, (int)blockIdx.x - n_walk, p.M, p.N, tiles_p, tiles_q, smem, STAGES * STAGE_BYTES);
            return;
        }
    }
    auto tile_coords = [&](int lin, int& tp, int& tq) {
        const int GROUP_P = FUSED ? ta.group_p : 16;
        if (FUSED || (tiles_p >= 2 * GROUP_P && tiles_q > 1)) {
            const int per_group = GROUP_P * tiles_q;
            const int group = lin / per_group, within = lin - group * per_group;
            const int p0 = group * GROUP_P;
            const int gp = min(GROUP_P, tiles_p - p0);
            tp = p0 + within % gp;
            tq = within / gp;
        } else {
            tp = lin % tiles_p;
            tq = lin / tiles_p;
        }
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
        flags[0] = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmP); tma_prefetch_desc(&tmQ); }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            long long g = 0;          // running k-block count over all tiles of this CTA: stage and phase
            int issued = 0;
            for (int t = blockIdx.x; t < ntiles && !flags[0]; t += n_walk) {
                int tp, tq;
                tile_coords(t, tp, tq);
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = (int)(g % STAGES);
                    const uint32_t ph = (uint32_t)((g / STAGES) & 1);
                    if (g >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1, p.wait_limit_ns)) {
                        report_status(p.status, KID_GEMM, 11, t, kb);
                        flags[0] = 1;
                        break;
                    }
                    uint8_t* sp = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    tma_load_2d(sp, &tmP, &full_bar[s], kb * BK, tp * BM);
                    if (p.w_packed) {
#pragma unroll
                        for (int h = 0; h < BN / 128; ++h)
                            tma_load_2d(sp + P_BYTES + h * (128 * BK * 2), &tmQ, &full_bar[s], 0,
                                        ((tq * (BN / 128) + h) * nkb + kb) * 128);
                    } else {
                        tma_load_2d(sp + P_BYTES, &tmQ, &full_bar[s], kb * BK, tq * BN);
                    }
                    ++issued;
                }
            }
            if (flags[0]) {      // let copies in flight land before the CTA leaves
                const long long lo = g > STAGES ? g - STAGES : 0;
                for (long long i = lo; i < g; ++i) mbar_wait(&full_bar[i % STAGES], (uint32_t)((i / STAGES) & 1), 1000000ull);
            }
            (void)issued;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1);
            long long g = 0;
            int it = 0;
            for (int t = blockIdx.x; t < ntiles && !flags[0]; t += n_walk, ++it) {
                const int a = it & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                if (it >= 2 && !mbar_wait(&acc_empty[a], (uint32_t)(((it >> 1) - 1) & 1), p.wait_limit_ns)) {
                    report_status(p.status, KID_GEMM, 12, t, it);
                    flags[0] = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(a * BN);
                bool ok = true;
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = (int)(g % STAGES);
                    const uint32_t ph = (uint32_t)((g / STAGES) & 1);
                    if (!mbar_wait(&full_bar[s], ph, p.wait_limit_ns)) {
                        report_status(p.status, KID_GEMM, 13, t, kb);
                        flags[0] = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sp = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = umma_smem_desc_sw128(sp);
                    const uint64_t db = umma_smem_desc_sw128(sp + P_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_f16_ss(d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                if (!ok) break;
                umma_commit(&acc_full[a]);
            }
        }
    } else {
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;
        int it = 0;
        for (int t = blockIdx.x; t < ntiles; t += n_walk, ++it) {
            const int a = it & 1;
            if (!mbar_wait(&acc_full[a], (uint32_t)((it >> 1) & 1), p.wait_limit_ns + 500000000ull)) {
                report_status(p.status, KID_GEMM, 14, t, it);
                flags[0] = 1;
                break;
            }
            tc_fence_after();
            int tp, tq;
            tile_coords(t, tp, tq);
            const int pidx = tp * BM + row;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                float v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * BN + c0), r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                const int qidx = tq * BN + c0;
                if (p.out_f32) store_row_chunk<true>(p, pidx, qidx, v, 32);
                else store_row_chunk<false>(p, pidx, qidx, v, 32);
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[a]);
            if constexpr (FUSED) {
                // the tile is in this rank's copy of the region: count it for its row group (release: every epilogue
                // thread fences its own stores, the four warps meet, one thread publishes)
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) atomicAdd(ta.done + tp / ta.group_p, 1u);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Block-scaled fp8 GEMM (e4m3 operands): C[m,n] = sum over 128-wide K blocks kb of
//     a_scale[m, kb] * w_scale[n / 128, kb] * sum_{k in kb} A8[m,k] * W8[n,k]
// (1 x 128 activation scales, 128 x 128 weight scales). One K block is 128 bytes = one swizzle atom = four
// kind::f8f6f4 UMMAs (K = 32). The tensor core cannot apply a different scale per K block inside one accumulation,
// so each K block is accumulated on its own into one of TWO TMEM buffers; the four epilogue warps drain buffer
// kb & 1 (tcgen05.ld), multiply by the block's scales and add into fp32 registers while the UMMA warp is already
// filling the other buffer with block kb + 1. Both layouts of the bf16 kernel: decode (weights on UMMA M, one weight
// scale per tile and K block, one activation scale per accumulator column) and token-major (tokens on UMMA M).
// The grouped mixture-of-experts form uses the decode layout with the bf16 kernel's block -> expert table.
// ---------------------------------------------------------------------------------------------
struct Fp8Scales {
    const float* a_scale_t;   // [kblocks, ld_as]: scale of token t and K block kb at kb * ld_as + t
    const float* w_scale;     // [ceil(rows / 128), kblocks] over the (stacked) weight rows
    int ld_as;
};

constexpr int F8_BK = 128;    // fp8 elements (= bytes) per K block

__host__ __device__ constexpr int gemm_fp8_smem_bytes(int BN, int stages) {
    return stages * (BM * F8_BK + BN * F8_BK) + 1024 /*alignment*/ + 1024 /*scales*/ + 256 /*barriers*/;
}

// EW: epilogue warps, 4 or 8. With 8 (token-major layout) two warps share a TMEM lane quarter and take half of the
// accumulator columns each: at large M the per-K-block drain (tcgen05.ld + one FMA per element) by four warps took
// longer than the block's four UMMAs.
template <int BN, int STAGES, bool SWAP, int EW = 4>
__global__ void __launch_bounds__(64 + EW * 32, 1)
gemm_fp8_blockscaled_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                            const __grid_constant__ GemmParams p, const __grid_constant__ Fp8Scales sc) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int P_BYTES = BM * F8_BK;
    constexpr int Q_BYTES = BN * F8_BK;
    constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    constexpr int ACC_COLS = BN < 32 ? 32 : BN;          // columns of one accumulator buffer
    // Four accumulator buffers (all 512 TMEM columns at BN = 128): the hand-over of one buffer (commit -> mbarrier ->
    // tcgen05.ld -> FMAs -> arrive -> UMMA warp wakes) takes several times the block's four UMMAs, and with two
    // buffers the tensor pipe was busy 25 % of the time.
    constexpr int NACC = 4;
    constexpr int TMEM_COLS = NACC * ACC_COLS;
    static_assert(TMEM_COLS <= 512 && BN <= 128, "four accumulators of at most 128 columns");
    static_assert(EW == 4 || (EW == 8 && !SWAP && BN >= 64), "eight epilogue warps: token-major layout only");
    constexpr int NCOL = BN / (EW / 4);                  // accumulator columns per epilogue thread
    float* scale_s = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES);           // [2][128]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + 1024);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;      // [NACC]
    uint64_t* acc_empty = acc_full + NACC;        // [NACC]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + NACC);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_slot + 1);  // [0] abort

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_p = blockIdx.x, tile_q = blockIdx.y;
    const int nkb = p.kblocks_total;
    pdl_launch_dependents();
    int p_row0 = tile_p * BM;
    if (p.block_expert != nullptr) {
        pdl_wait();
        if (tile_q >= *p.num_blocks) return;
        p_row0 += p.block_expert[tile_q] * p.N;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < NACC; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], EW * 32); }
        flags[0] = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmP); tma_prefetch_desc(&tmQ); }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            int issued = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (uint32_t)((kb / STAGES) & 1);
                if (kb >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_GEMM, 21, kb, s);
                    flags[0] = 1;
                    break;
                }
                if (flags[0]) break;
                uint8_t* sp = smem + s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(sp, &tmP, &full_bar[s], kb * F8_BK, p_row0);
                tma_load_2d(sp + P_BYTES, &tmQ, &full_bar[s], kb * F8_BK, tile_q * BN);
                issued = kb + 1;
            }
            if (flags[0]) {      // let copies in flight land before the CTA leaves
                for (int g = (issued > STAGES ? issued - STAGES : 0); g < issued; ++g)
                    mbar_wait(&full_bar[g % STAGES], (uint32_t)((g / STAGES) & 1), 1000000ull);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN, 0, 0);      // e4m3 x e4m3 -> f32
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES;
                const int a = kb % NACC;
                if (!mbar_wait(&full_bar[s], (uint32_t)((kb / STAGES) & 1), p.wait_limit_ns)) {
                    report_status(p.status, KID_GEMM, 22, kb, s);
                    flags[0] = 1;
                    break;
                }
                // the epilogue must have drained this accumulator buffer (K block kb - NACC)
                if (kb >= NACC && !mbar_wait(&acc_empty[a], (uint32_t)(((kb / NACC) - 1) & 1), p.wait_limit_ns)) {
                    report_status(p.status, KID_GEMM, 23, kb, a);
                    flags[0] = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t sp = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t da = umma_smem_desc_sw128(sp);
                const uint64_t db = umma_smem_desc_sw128(sp + P_BYTES);
                const uint32_t d = tmem_base + (uint32_t)(a * ACC_COLS);
#pragma unroll
                for (int k = 0; k < F8_BK / 32; ++k)      // 32 bytes per K slice inside the swizzle atom (encoded >> 4)
                    umma_f8_ss(d, da + 2 * k, db + 2 * k, idesc, k != 0 ? 1u : 0u);
                umma_commit(&empty_bar[s]);
                umma_commit(&acc_full[a]);
            }
        }
    } else {
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;          // accumulator row (TMEM lane) of this thread
        const int tid = threadIdx.x - 64;
        const int pidx = tile_p * BM + row;
        const int cb = ((warp - 2) >> 2) * NCOL; // first accumulator column of this thread
        pdl_wait();
        float acc[NCOL];
#pragma unroll
        for (int j = 0; j < NCOL; ++j) acc[j] = 0.f;
        const float* wsc = sc.w_scale + (size_t)((SWAP ? p_row0 : tile_q * BN) / 128) * nkb;
        bool ok = true;
        // The scales of K block kb + 1 are fetched while block kb is drained: a scale load at the top of every trip
        // put a global-memory round trip (long scoreboard) in front of each block's FMAs, longer than the block's UMMAs.
        auto load_w = [&](int kb) { return kb < nkb ? __ldg(wsc + kb) : 0.f; };
        auto load_a = [&](int kb) {
            if (kb >= nkb) return 0.f;
            if constexpr (SWAP) {
                const int t = tile_q * BN + tid;
                return (tid < BN && t < p.M) ? __ldg(sc.a_scale_t + (size_t)kb * sc.ld_as + t) : 0.f;
            } else {
                return pidx < p.M ? __ldg(sc.a_scale_t + (size_t)kb * sc.ld_as + pidx) : 0.f;
            }
        };
        float w_next = load_w(0), a_next = load_a(0);
        for (int kb = 0; kb < nkb; ++kb) {
            const int a = kb % NACC;          // accumulator buffer
            const int sb = kb & 1;            // scale staging buffer
            const float w_cur = w_next, a_cur = a_next;
            w_next = load_w(kb + 1);
            a_next = load_a(kb + 1);
            float rowfac;
            if constexpr (SWAP) {
                // one weight scale for the tile, one activation scale per column: staged through shared memory
                rowfac = w_cur;
                if (tid < BN) scale_s[sb * 128 + tid] = a_cur;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            } else {
                rowfac = a_cur * w_cur;
            }
            if (!mbar_wait(&acc_full[a], (uint32_t)((kb / NACC) & 1), p.wait_limit_ns + 500000000ull)) {
                report_status(p.status, KID_GEMM, 24, kb, a);
                flags[0] = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            constexpr int CH = NCOL < 32 ? NCOL : 32;
            if constexpr (NCOL >= 64) {
                // two 32-column loads in flight per wait
#pragma unroll
                for (int c0 = 0; c0 < NCOL; c0 += 64) {
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * ACC_COLS + cb + c0);
                    tmem_ld32(taddr, r0);
                    tmem_ld32(taddr + 32, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if constexpr (SWAP) {
                            acc[c0 + i] = fmaf(__uint_as_float(r0[i]), rowfac * scale_s[sb * 128 + c0 + i], acc[c0 + i]);
                            acc[c0 + 32 + i] = fmaf(__uint_as_float(r1[i]), rowfac * scale_s[sb * 128 + c0 + 32 + i], acc[c0 + 32 + i]);
                        } else {
                            acc[c0 + i] = fmaf(__uint_as_float(r0[i]), rowfac, acc[c0 + i]);
                            acc[c0 + 32 + i] = fmaf(__uint_as_float(r1[i]), rowfac, acc[c0 + 32 + i]);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int c0 = 0; c0 < NCOL; c0 += CH) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * ACC_COLS + cb + c0);
                    if constexpr (CH == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < CH; ++i) {
                        if constexpr (SWAP) acc[c0 + i] = fmaf(__uint_as_float(r[i]), rowfac * scale_s[sb * 128 + c0 + i], acc[c0 + i]);
                        else acc[c0 + i] = fmaf(__uint_as_float(r[i]), rowfac, acc[c0 + i]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[a]);
        }
        if (ok) {
            if constexpr (SWAP) {
                // every UMMA has completed (its accumulator was read above): the pipeline stages are free
                float* stage = reinterpret_cast<float*>(smem);
                asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
                for (int j = 0; j < BN; ++j) stage[j * BM + row] = acc[j];
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (p.out_f32) copy_out_staged<true>(p, stage, BN, tile_q * BN, tile_p * BM, tid);
                else copy_out_staged<false>(p, stage, BN, tile_q * BN, tile_p * BM, tid);
            } else {
#pragma unroll
                for (int c0 = 0; c0 < NCOL; c0 += 32) {
                    if (p.out_f32) store_row_chunk<true>(p, pidx, tile_q * BN + cb + c0, &acc[c0], 32);
                    else store_row_chunk<false>(p, pidx, tile_q * BN + cb + c0, &acc[c0], 32);
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// Split-K through a thread-block cluster (MSTAR_GEMM_CLUSTER=0 turns it off); cleared when a cluster launch fails.
static bool g_cluster_reduce_ok = true;
static bool cluster_reduce_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MSTAR_GEMM_CLUSTER");
        v = e ? atoi(e) : 1;
    }
    return v != 0 && g_cluster_reduce_ok;
}

template <int BN, int STAGES, int MINB, int KSUB = 1>
static int launch_gemm(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p, dim3 grid,
                       cudaStream_t stream) {
    constexpr int smem = gemm_smem_bytes(BN, STAGES, KSUB);
    using KernelFn = void (*)(CUtensorMap, CUtensorMap, GemmParams);
    const KernelFn kern = p.swap ? static_cast<KernelFn>(gemm_bf16_tcgen05_kernel<BN, STAGES, MINB, KSUB, true>)
                                 : static_cast<KernelFn>(gemm_bf16_tcgen05_kernel<BN, STAGES, MINB, KSUB, false>);
    static PerDeviceFlag configured[2];
    if (!configured[p.swap ? 1 : 0]()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error("gemm: cudaFuncSetAttribute failed", e);
        configured[p.swap ? 1 : 0]() = true;
    }
    if (p.cluster_reduce) {
        // Clusters are placed inside one GPC each, so a split factor that does not divide the GPCs' SM counts well
        // leaves SMs unusable and the grid runs in two waves (measured: 24 clusters of 6 CTAs did, 24 of 4 do not).
        // Ask the runtime how many clusters of each size are co-resident and take the largest factor, at most the
        // planned one, whose clusters all fit.
        static int max_active_dev[kMaxDevices][9] = {};
        int* max_active = max_active_dev[current_device()];
        const int tiles = (int)(grid.x * grid.y);
        int use = 0;
        for (int sp = (int)grid.z; sp >= 2 && use == 0; --sp) {
            if (max_active[sp] == 0) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(grid.x, grid.y, sp);
                cfg.blockDim = dim3(192);
                cfg.dynamicSmemBytes = smem;
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = sp;
                cfg.attrs = at; cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
                    (void)cudaGetLastError();
                    n = -1;
                }
                max_active[sp] = n > 0 ? n : -1;
            }
            if (max_active[sp] >= tiles) use = sp;
        }
        GemmParams pc = p;
        dim3 gc = grid;
        if (use >= 2 && use != (int)grid.z) {
            const int kpb = (p.kblocks_total + use - 1) / use;
            pc.splits = (p.kblocks_total + kpb - 1) / kpb;
            pc.kblocks_per_split = kpb;
            gc.z = pc.splits;
        }
        cudaError_t e = cudaErrorInvalidConfiguration;
        if (use >= 2 && gc.z >= 2)
            e = launch_pdl_cluster_z(kern, gc, dim3(192), smem, stream, gc.z,
                                     tmP, tmQ, pc);
        else if (use >= 2) {       // the K range collapsed to one split
            pc.cluster_reduce = 0;
            e = launch_pdl(kern, gc, dim3(192), smem, stream, tmP, tmQ, pc);
        }
        if (e == cudaSuccess) return 0;
        if (use == 0 && p.workspace != nullptr) {       // no cluster size fits this grid: scratch-buffer reduction
            GemmParams q = p;
            q.cluster_reduce = 0;
            e = launch_pdl(kern, grid, dim3(192), smem, stream, tmP, tmQ, q);
            if (e != cudaSuccess) return set_error("gemm: launch failed", e);
            return 0;
        }
        // this cluster shape cannot be launched here: remember it and take the scratch-buffer reduction
        (void)cudaGetLastError();
        g_cluster_reduce_ok = false;
        if (p.workspace == nullptr) return set_error("gemm: cluster launch failed and no split-K scratch was given", e);
        GemmParams q = p;
        q.cluster_reduce = 0;
        e = launch_pdl(kern, grid, dim3(192), smem, stream, tmP, tmQ, q);
        if (e != cudaSuccess) return set_error("gemm: launch failed", e);
        return 0;
    }
    cudaError_t e = launch_pdl(kern, grid, dim3(192), smem, stream, tmP, tmQ, p);
    if (e != cudaSuccess) return set_error("gemm: launch failed", e);
    return 0;
}

static bool persistent_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MSTAR_GEMM_PERSISTENT");
        v = e ? atoi(e) : 1;
    }
    return v != 0;
}

template <int BN, int STAGES>
static int launch_persistent(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p, dim3 grid,
                             cudaStream_t stream) {
    constexpr int smem = gemm_smem_bytes(BN, STAGES);
    static PerDeviceFlag configured;
    if (!configured()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_persistent_kernel<BN, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error("gemm: cudaFuncSetAttribute failed", e);
        configured() = true;
    }
    const int tiles = (int)(grid.x * grid.y);
    const int ctas = tiles < device_sm_count() ? tiles : device_sm_count();
    cudaError_t e = launch_pdl(gemm_bf16_persistent_kernel<BN, STAGES>, dim3(ctas), dim3(192), smem, stream, tmP, tmQ, p,
                               (int)grid.x, (int)grid.y, TileAR{});
    if (e != cudaSuccess) return set_error("gemm: launch failed", e);
    return 0;
}

// The fused form: `ta.n_comm` communication CTAs ride at the end of a grid of one CTA per SM.
template <int BN, int STAGES>
static int launch_persistent_fused(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p, int tiles_p,
                                   int tiles_q, const TileAR& ta, cudaStream_t stream) {
    constexpr int smem = gemm_smem_bytes(BN, STAGES);
    static PerDeviceFlag configured;
    if (!configured()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_persistent_kernel<BN, STAGES, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error("gemm+all-reduce: cudaFuncSetAttribute failed", e);
        configured() = true;
    }
    const int ctas = device_sm_count();         // every CTA resident: the communication CTAs wait for the walkers
    cudaError_t e = launch_pdl(gemm_bf16_persistent_kernel<BN, STAGES, true>, dim3(ctas), dim3(192), smem, stream, tmP, tmQ,
                               p, tiles_p, tiles_q, ta);
    if (e != cudaSuccess) return set_error("gemm+all-reduce: launch failed", e);
    return 0;
}

// Tile configuration by (Q tile width, layout). Decode (swapped) tiles stream weights: MSTAR_GEMM_KSUB picks how many
// 64-wide K blocks one pipeline stage fetches (1, 2, 4; 22 = two blocks per stage with two CTAs per SM).
static int dispatch_tile(int bn, int swap, const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p,
                         dim3 grid, cudaStream_t stream) {
    static int ksub = -1;
    if (ksub < 0) {
        const char* e = getenv("MSTAR_GEMM_KSUB");
        ksub = e ? atoi(e) : 2;      // measured on the 3B decode step: 5.99 ms (1), 5.80 (2), 5.83 (4), 6.05 (22)
    }
    if (swap && ksub == 2) {
        switch (bn) {
            case 16: return launch_gemm<16, 4, 1, 2>(tmP, tmQ, p, grid, stream);
            case 32: return launch_gemm<32, 4, 1, 2>(tmP, tmQ, p, grid, stream);
            case 64: return launch_gemm<64, 4, 1, 2>(tmP, tmQ, p, grid, stream);
            case 128: return launch_gemm<128, 3, 1, 2>(tmP, tmQ, p, grid, stream);
        }
    } else if (swap && ksub == 22) {
        switch (bn) {
            case 16: return launch_gemm<16, 3, 2, 2>(tmP, tmQ, p, grid, stream);
            case 32: return launch_gemm<32, 2, 2, 2>(tmP, tmQ, p, grid, stream);
            case 64: return launch_gemm<64, 2, 2, 2>(tmP, tmQ, p, grid, stream);
            case 128: return launch_gemm<128, 3, 1, 2>(tmP, tmQ, p, grid, stream);
        }
    } else if (swap && ksub == 4) {
        switch (bn) {
            case 16: return launch_gemm<16, 3, 1, 4>(tmP, tmQ, p, grid, stream);
            case 32: return launch_gemm<32, 2, 1, 4>(tmP, tmQ, p, grid, stream);
            case 64: return launch_gemm<64, 2, 1, 4>(tmP, tmQ, p, grid, stream);
            case 128: return launch_gemm<128, 3, 1, 2>(tmP, tmQ, p, grid, stream);
        }
    }
    switch (bn) {
        // decode tiles: 4 stages keep a CTA under 100 KB so that two CTAs share an SM and one CTA's prologue /
        // epilogue overlaps the other's weight stream
        case 16: return launch_gemm<16, 5, 2>(tmP, tmQ, p, grid, stream);
        case 32: return launch_gemm<32, 5, 2>(tmP, tmQ, p, grid, stream);
        case 64: return launch_gemm<64, 4, 2>(tmP, tmQ, p, grid, stream);
        case 128:
            if (swap) return launch_gemm<128, 3, 2>(tmP, tmQ, p, grid, stream);
            return launch_gemm<128, 6, 1>(tmP, tmQ, p, grid, stream);
        case 256:
            if (!swap && grid.z == 1 && p.block_expert == nullptr && !p.ar.enabled && persistent_enabled())
                return launch_persistent<256, 4>(tmP, tmQ, p, grid, stream);
            return launch_gemm<256, 4, 1>(tmP, tmQ, p, grid, stream);
    }
    return set_error("gemm: unsupported tile", cudaSuccess);
}

}  // namespace mstar

using namespace mstar;
static GemmAllReduce g_next_ar = {};

// Folded-norm arguments of the NEXT mstar_gemm_bf16 call on the current device (see GemmParams::ss_in): set by
// mstar_gemm_norm_hint, taken once. A call that cannot honour them (not the decode layout, fp32 output) fails.
struct NormHint { const float* ss_in; float* ss_out; float* ss_zero; int ss_zero_n; float inv_h, eps; int set; };
static NormHint g_norm_hint[kMaxDevices] = {};
static unsigned long long* g_trace = nullptr;

// Phase stamps for the benchmark: a device buffer of [CTAs][8] 64-bit words filled by later mstar_gemm_bf16 launches
// (entry, prologue done, accumulator staged, first tile landed, last UMMA issued, accumulator ready, epilogue done,
// cluster slice stored), or null to stop.
MSTAR_API void mstar_gemm_set_trace(void* buf) { g_trace = reinterpret_cast<unsigned long long*>(buf); }

// Arms the tensor-parallel reduction for the NEXT mstar_gemm_bf16 call of this thread of control: the output is
// summed over the ranks of the table inside the GEMM epilogue. state: two local device words [epoch, arrive].
MSTAR_API int mstar_gemm_arm_allreduce(void* const* bufs, void* const* flags, int world, int rank,
                                       long long slot_bytes, void* state, int channel_base) {
    if (world < 1 || world > MAX_RANKS) return set_error("gemm+allreduce: bad world size", cudaSuccess);
    for (int i = 0; i < MAX_RANKS; ++i) {
        g_next_ar.t.buf[i] = i < world ? bufs[i] : nullptr;
        g_next_ar.t.flags[i] = i < world ? reinterpret_cast<unsigned int*>(flags[i]) : nullptr;
    }
    g_next_ar.t.world = world;
    g_next_ar.t.rank = rank;
    g_next_ar.slot_bytes = slot_bytes;
    g_next_ar.epoch = reinterpret_cast<unsigned int*>(state);
    g_next_ar.arrive = g_next_ar.epoch + 1;
    g_next_ar.channel_base = channel_base;
    g_next_ar.enabled = 1;
    return 0;
}

// Workspace bytes needed for a given problem (0 when no split-K is used). Also returns the split factor.
MSTAR_API int mstar_gemm_plan(int M, int N, int K, int* swap_out, int* bn_out, int* splits_out,
                              long long* ws_bytes_out, int* tiles_out) {
    const int kblocks = (K + BK - 1) / BK;
    int swap = (M <= 128) ? 1 : 0;
    int bn;
    int tiles_p, tiles_q;
    if (swap) {
        bn = 16;
        while (bn < M) bn <<= 1;  // 16,32,64,128
        tiles_p = (N + BM - 1) / BM;
        tiles_q = 1;
    } else {
        bn = (N % 256 == 0 || N >= 2048) ? 256 : 128;
        if (N <= 128) bn = 128;
        tiles_p = (M + BM - 1) / BM;
        tiles_q = (N + bn - 1) / bn;
    }
    const int tiles = tiles_p * tiles_q;
    int splits = 1;
    const int sms = device_sm_count();
    const int target = sms;
    if (tiles < target) {
        splits = target / tiles;
        // keep at least 4 K blocks per split so the pipeline has something to stream
        int max_splits = kblocks / 4;
        if (max_splits < 1) max_splits = 1;
        if (splits > max_splits) splits = max_splits;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
    }
    int kpb = (kblocks + splits - 1) / splits;
    splits = (kblocks + kpb - 1) / kpb;  // no empty split
    if (swap_out) *swap_out = swap;
    if (bn_out) *bn_out = bn;
    if (splits_out) *splits_out = splits;
    if (tiles_out) *tiles_out = tiles;
    if (ws_bytes_out) *ws_bytes_out = splits > 1 ? (long long)splits * tiles * BM * bn * 4 : 0;
    return 0;
}

// Fold RMSNorms into the next mstar_gemm_bf16 call on this device. ss_in: per-token sums of squares of the activation
// rows (the call multiplies output row t by rsqrt(ss_in[t] * inv_h + eps)); ss_out: per-token accumulator that gets the
// sum of squares of the bf16 output rows (its N tiles add into it atomically: it must be zero on entry);
// ss_zero / ss_zero_n: floats cleared by the call once the previous kernel has finished. Any of the three may be null.
MSTAR_API void mstar_gemm_norm_hint(const void* ss_in, void* ss_out, void* ss_zero, int ss_zero_n, float inv_h, float eps) {
    NormHint& nh = g_norm_hint[current_device()];
    nh.ss_in = static_cast<const float*>(ss_in);
    nh.ss_out = static_cast<float*>(ss_out);
    nh.ss_zero = static_cast<float*>(ss_zero);
    nh.ss_zero_n = ss_zero != nullptr ? ss_zero_n : 0;
    nh.inv_h = inv_h;
    nh.eps = eps;
    nh.set = 1;
}

// C[M,N] = A[M,K] * B[N,K]^T with optional bias[N], residual[M,N] and epilogue.
// A, B bf16 row-major with leading dimensions lda, ldb (elements, multiples of 8); C bf16 or fp32.
// epilogue 1 (SwiGLU): B's rows interleave (gate_j, up_j); C has N/2 columns.
MSTAR_API int mstar_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                              const void* bias, const void* residual, int ld_res, int epilogue, int out_f32,
                              float out_scale, void* workspace, long long workspace_bytes, void* counters,
                              int n_counters, int force_splits, int b_packed, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((lda % 8) || (!b_packed && (ldb % 8)) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
        return set_error("gemm: operands must be 16-byte aligned with leading dimensions multiple of 8", cudaSuccess);
    int swap, bn, splits, tiles;
    long long ws_need;
    mstar_gemm_plan(M, N, K, &swap, &bn, &splits, &ws_need, &tiles);
    const int kblocks = (K + BK - 1) / BK;
    if (force_splits > 0) {
        splits = force_splits > kblocks ? kblocks : force_splits;
        int kpb = (kblocks + splits - 1) / splits;
        splits = (kblocks + kpb - 1) / kpb;
        ws_need = splits > 1 ? (long long)splits * tiles * BM * bn * 4 : 0;
    }
    if (splits > 1 && (workspace == nullptr || ws_need > workspace_bytes || tiles > n_counters)) {
        splits = 1;  // no scratch available: fall back to a single pass over K
    }
    GemmParams p;
    { const PrefetchHint h = take_prefetch_hint(); p.pf_ptr = h.ptr; p.pf_bytes = h.bytes; p.l2_hints = h.l2_hints; }
    p.M = M; p.N = N; p.K = K;
    p.swap = swap;
    p.splits = splits;
    p.kblocks_total = kblocks;
    p.kblocks_per_split = (kblocks + splits - 1) / splits;
    p.epilogue = epilogue;
    p.out_f32 = out_f32;
    p.ldc = ldc;
    p.ld_res = ld_res;
    p.C = C;
    p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
    p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
    p.workspace = reinterpret_cast<float*>(workspace);
    p.counters = reinterpret_cast<unsigned int*>(counters);
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    p.out_scale = out_scale;
    p.block_expert = nullptr;
    p.num_blocks = nullptr;
    p.row_scale = nullptr;
    p.row_dst = nullptr;
    p.ar = g_next_ar;
    g_next_ar.enabled = 0;
    {
        NormHint& nh = g_norm_hint[current_device()];
        if (nh.set) {
            nh.set = 0;
            if (!swap || out_f32 || p.ar.enabled)
                return set_error("gemm: a folded norm needs the decode layout (M <= 128), bf16 output and no fused all-reduce", cudaSuccess);
            p.ss_in = nh.ss_in; p.ss_out = nh.ss_out; p.ss_zero = nh.ss_zero; p.ss_zero_n = nh.ss_zero_n;
            p.ss_inv_h = nh.inv_h; p.ss_eps = nh.eps;
        }
    }
    if (p.ar.enabled) {
        if (!swap || epilogue != 0 || out_f32 || (N % 8) || ldc % 8 || (residual && ld_res % 8))
            return set_error("gemm+allreduce: needs the decode layout (M <= 128), bf16 output, no activation, N % 8 == 0", cudaSuccess);
        if ((long long)p.ar.t.world * M * N * 2 > p.ar.slot_bytes)
            return set_error("gemm+allreduce: the ranks' partial outputs do not fit the heap slot", cudaSuccess);
        if ((long long)tiles * splits > 480) return set_error("gemm+allreduce: more exchange units than flag channels", cudaSuccess);
        if ((long long)tiles * splits > 2LL * device_sm_count())
            return set_error("gemm+allreduce: grid must be co-resident", cudaSuccess);
    }

    p.cluster_reduce = (swap && splits > 1 && splits <= 8 && cluster_reduce_enabled()) ? 1 : 0;
    p.w_packed = b_packed ? 1 : 0;
    p.trace = g_trace;
    if (b_packed && !swap && bn < 128) return set_error("gemm: packed weights need a 128- or 256-wide tile", cudaSuccess);

    const void* Pp = swap ? B : A;
    const void* Qp = swap ? A : B;
    const int rowsP = swap ? N : M, rowsQ = swap ? M : N;
    const int ldP = swap ? ldb : lda, ldQ = swap ? lda : ldb;
    CUtensorMap tmP, tmQ;
    const int packed_rows = ((N + 127) / 128) * kblocks * 128;
    if (b_packed && swap) {
        if (make_tmap_2d_bf16(&tmP, Pp, packed_rows, BK, BK, BM, BK)) return -1;
    } else if (make_tmap_2d_bf16(&tmP, Pp, rowsP, K, ldP, BM, BK)) return -1;
    if (b_packed && !swap) {
        if (make_tmap_2d_bf16(&tmQ, Qp, packed_rows, BK, BK, 128, BK)) return -1;
    } else if (make_tmap_2d_bf16(&tmQ, Qp, rowsQ, K, ldQ, bn, BK)) return -1;
    dim3 grid((rowsP + BM - 1) / BM, (rowsQ + bn - 1) / bn, splits);
    return dispatch_tile(bn, swap, tmP, tmQ, p, grid, stream);
}

// Row-parallel projection of a tensor-parallel layer at large M with the all-reduce inside the kernel (see TileAR):
// C = sum over ranks of A_r[M, K] * B_r[N, K]^T (+ bias, + residual: pass them on ONE rank only), bf16, written in
// place at byte offset `off` of every rank's copy of a symmetric region (`bufs`), leading dimension N. `ctrs` is a
// local zero-initialised array of 3 * 64 + 4 unsigned ints that belongs to this call site (group counters, epoch,
// arrival counter); [stage_off, stage_off + stage_bytes) of the region is the staging area the peers push into
// ((W - 1) / W of C's size, rounded up per row group). N % 8 == 0, K % 8 == 0, at most 64 row groups. Every rank of the group must make the same call.
MSTAR_API int mstar_gemm_bf16_allreduce_tiles(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                                              const void* bias, const void* residual, int ld_res,
                                              void* const* bufs, void* const* flags, int world, int rank,
                                              void* mc_flags, long long off, long long stage_off, long long stage_bytes,
                                              void* ctrs, int channel_base, int n_comm, int group_p, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 || N % 8 || lda % 8 || ldb % 8 || off % 16)
        return set_error("gemm+all-reduce: K, N and the leading dimensions must be multiples of 8, the offset of 16", cudaSuccess);
    if (world < 2 || world > MAX_RANKS || rank < 0 || rank >= world)
        return set_error("gemm+all-reduce: bad group", cudaSuccess);
    const int sms = device_sm_count();
    if (n_comm <= 0) n_comm = 24;
    if (n_comm > sms / 2) n_comm = sms / 2;
    constexpr int bn = 256;
    const int tiles_p = (M + BM - 1) / BM, tiles_q = (N + bn - 1) / bn;
    if (group_p <= 0) {
        // about as many tiles per group as there are walkers, so that a group is roughly one wave
        group_p = (sms - n_comm + tiles_q - 1) / tiles_q;
        if (group_p < 1) group_p = 1;
    }
    const int groups = (tiles_p + group_p - 1) / group_p;
    if (groups > 64) return set_error("gemm+all-reduce: more than 64 row groups", cudaSuccess);
    {
        long long rows0 = (long long)group_p * BM;
        if (rows0 > M) rows0 = M;
        const long long share_full = (rows0 * N / 8 + world - 1) / world;
        const long long rows_last = M - (long long)(groups - 1) * group_p * BM;
        const long long share_last = (rows_last * N / 8 + world - 1) / world;
        if (stage_off % 16 || (long long)(world - 1) * ((groups - 1) * share_full + share_last) * 16 > stage_bytes)
            return set_error("gemm+all-reduce: the staging area is too small or misaligned", cudaSuccess);
    }
    GemmParams p;
    (void)take_prefetch_hint();
    p.M = M; p.N = N; p.K = K;
    p.swap = 0;
    p.splits = 1;
    p.kblocks_total = (K + BK - 1) / BK;
    p.kblocks_per_split = p.kblocks_total;
    p.epilogue = 0;
    p.out_f32 = 0;
    p.ldc = N;
    p.ld_res = ld_res;
    p.C = static_cast<char*>(bufs[rank]) + off;
    p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
    p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
    p.workspace = nullptr;
    p.counters = nullptr;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    p.out_scale = 1.0f;
    p.ar = GemmAllReduce{};
    p.block_expert = nullptr;
    p.num_blocks = nullptr;
    p.row_scale = nullptr;
    p.row_dst = nullptr;
    TileAR ta{};
    for (int i = 0; i < MAX_RANKS; ++i) {
        ta.t.buf[i] = i < world ? bufs[i] : nullptr;
        ta.t.flags[i] = i < world ? static_cast<unsigned int*>(flags[i]) : nullptr;
    }
    ta.t.world = world; ta.t.rank = rank;
    ta.mc.data = nullptr;
    ta.mc.flags = static_cast<unsigned int*>(mc_flags);
    ta.off = off;
    ta.stage_off = stage_off;
    ta.n_comm = n_comm;
    ta.group_p = group_p;
    ta.channel_base = channel_base;
    ta.done = static_cast<unsigned int*>(ctrs);
    ta.push_done = ta.done + 64;
    ta.red_done = ta.done + 128;
    ta.epoch = ta.done + 192;
    ta.arrive = ta.done + 193;
    ta.status = p.status;
    ta.wait_limit_ns = p.wait_limit_ns;
    CUtensorMap tmP, tmQ;
    if (make_tmap_2d_bf16(&tmP, A, M, K, lda, BM, BK)) return -1;
    if (make_tmap_2d_bf16(&tmQ, B, N, K, ldb, bn, BK)) return -1;
    const int rc = launch_persistent_fused<256, 4>(tmP, tmQ, p, tiles_p, tiles_q, ta, stream);
    return rc < 0 ? rc : groups;
}

// Grouped GEMM for mixture-of-experts layers (decode layout): rows of A are token copies sorted by expert in
// blocks of `block_rows` (16, 32, 64 or 128); block b uses expert block_expert[b]. W is the stacked expert
// weight [E * N, K]. C row i is the result of A row i (same sorted order), or is scattered through row_dst.
//   epilogue 1: SwiGLU over interleaved (gate, up) rows of each expert (C has N/2 columns)
//   row_scale:  optional per-row factor (routing weight); row_dst: optional per-row destination pointers
MSTAR_API int mstar_moe_grouped_gemm(const void* A, const void* W, void* C, int capacity_rows, int N, int K, int E,
                                     int block_rows, const int* block_expert, const int* num_blocks,
                                     const float* row_scale, void* const* row_dst, int epilogue, int ldc,
                                     void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (capacity_rows <= 0) return 0;
    if (block_rows != 16 && block_rows != 32 && block_rows != 64 && block_rows != 128)
        return set_error("moe gemm: block_rows must be 16, 32, 64 or 128", cudaSuccess);
    if (K % 8 || N % 8 || capacity_rows % block_rows)
        return set_error("moe gemm: K and N must be multiples of 8, capacity a multiple of block_rows", cudaSuccess);
    GemmParams p;
    { const PrefetchHint h = take_prefetch_hint(); p.pf_ptr = h.ptr; p.pf_bytes = h.bytes; p.l2_hints = h.l2_hints; }
    p.M = capacity_rows; p.N = N; p.K = K;
    p.swap = 1;
    p.splits = 1;
    p.kblocks_total = (K + BK - 1) / BK;
    p.kblocks_per_split = p.kblocks_total;
    p.epilogue = epilogue;
    p.out_f32 = 0;
    p.ldc = ldc;
    p.ld_res = 0;
    p.C = C;
    p.bias = nullptr;
    p.residual = nullptr;
    p.workspace = nullptr;
    p.counters = nullptr;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    p.out_scale = 1.0f;
    p.ar = GemmAllReduce{};
    p.block_expert = block_expert;
    p.num_blocks = num_blocks;
    p.row_scale = row_scale;
    p.row_dst = row_dst;
    CUtensorMap tmP, tmQ;
    if (make_tmap_2d_bf16(&tmP, W, E * N, K, K, BM, BK)) return -1;
    if (make_tmap_2d_bf16(&tmQ, A, capacity_rows, K, K, block_rows, BK)) return -1;
    dim3 grid((N + BM - 1) / BM, capacity_rows / block_rows, 1);
    switch (block_rows) {
        case 16: return launch_gemm<16, 5, 2>(tmP, tmQ, p, grid, stream);
        case 32: return launch_gemm<32, 5, 2>(tmP, tmQ, p, grid, stream);
        case 64: return launch_gemm<64, 4, 2>(tmP, tmQ, p, grid, stream);
        default: return launch_gemm<128, 3, 2>(tmP, tmQ, p, grid, stream);
    }
}

// ---------------------------------------------------------------------------------------------
// fp8 (e4m3) block-scaled GEMM entry points
// ---------------------------------------------------------------------------------------------
namespace mstar {

static int make_tmap_2d_u8(CUtensorMap* out, const void* base, long long rows, int cols, long long ld, int box_rows) {
    unsigned long long dims[2] = {(unsigned long long)cols, (unsigned long long)rows};
    unsigned long long strides[2] = {1ull, (unsigned long long)ld};
    unsigned int box[2] = {(unsigned int)F8_BK, (unsigned int)box_rows};
    return make_tmap(out, base, 1, 2, dims, strides, box, 1);
}

template <int BN, int STAGES, bool SWAP, int EW = 4>
static int launch_fp8(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p, const Fp8Scales& sc,
                      dim3 grid, cudaStream_t stream) {
    constexpr int smem = gemm_fp8_smem_bytes(BN, STAGES);
    static PerDeviceFlag configured;
    if (!configured()) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_blockscaled_kernel<BN, STAGES, SWAP, EW>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error("gemm_fp8: cudaFuncSetAttribute failed", e);
        configured() = true;
    }
    cudaError_t e = launch_pdl(gemm_fp8_blockscaled_kernel<BN, STAGES, SWAP, EW>, grid, dim3(64 + EW * 32), smem, stream,
                               tmP, tmQ, p, sc);
    if (e != cudaSuccess) return set_error("gemm_fp8: launch failed", e);
    return 0;
}

static int dispatch_fp8(int bn, int swap, const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p,
                        const Fp8Scales& sc, dim3 grid, cudaStream_t stream) {
    if (swap) {
        switch (bn) {
            case 16: return launch_fp8<16, 8, true>(tmP, tmQ, p, sc, grid, stream);
            case 32: return launch_fp8<32, 8, true>(tmP, tmQ, p, sc, grid, stream);
            case 64: return launch_fp8<64, 8, true>(tmP, tmQ, p, sc, grid, stream);
            case 128: return launch_fp8<128, 6, true>(tmP, tmQ, p, sc, grid, stream);
        }
    } else if (bn == 128) {
        return launch_fp8<128, 6, false, 8>(tmP, tmQ, p, sc, grid, stream);
    }
    return set_error("gemm_fp8: unsupported tile", cudaSuccess);
}

static void fill_fp8_params(GemmParams& p, int M, int N, int K, int swap, int epilogue, int out_f32, int ldc, void* C) {
    p.M = M; p.N = N; p.K = K;
    p.swap = swap;
    p.splits = 1;
    p.kblocks_total = (K + F8_BK - 1) / F8_BK;
    p.kblocks_per_split = p.kblocks_total;
    p.epilogue = epilogue;
    p.out_f32 = out_f32;
    p.ldc = ldc;
    p.ld_res = 0;
    p.C = C;
    p.bias = nullptr;
    p.residual = nullptr;
    p.workspace = nullptr;
    p.counters = nullptr;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    p.out_scale = 1.0f;
    p.ar = GemmAllReduce{};
    p.block_expert = nullptr;
    p.num_blocks = nullptr;
    p.row_scale = nullptr;
    p.row_dst = nullptr;
}

}  // namespace mstar

// C[M,N] = (A8 * a_scale) (W8 * w_scale)^T (+bias, +residual, epilogue as in mstar_gemm_bf16).
// A8 [M,K] and W8 [N,K] are e4m3 bytes, row-major, leading dimensions multiples of 16; a_scale_t is fp32
// [ceil(K/128), ld_as] (one scale per token and 128-wide K block, token index contiguous, ld_as >= the token count
// rounded up to the tile); w_scale is fp32 [ceil(N/128), ceil(K/128)].
MSTAR_API int mstar_gemm_fp8(const void* A8, const void* a_scale_t, int ld_as, const void* W8, const void* w_scale,
                             void* C, int M, int N, int K, int lda, int ldb, int ldc, const void* bias,
                             const void* residual, int ld_res, int epilogue, int out_f32, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A8) & 15) || (reinterpret_cast<uintptr_t>(W8) & 15))
        return set_error("gemm_fp8: operands must be 16-byte aligned with leading dimensions multiple of 16", cudaSuccess);
    const int swap = M <= 128 ? 1 : 0;
    int bn = 128;
    if (swap) {
        bn = 16;
        while (bn < M) bn <<= 1;
        if (ld_as < bn) return set_error("gemm_fp8: activation scale rows must be padded to the token tile", cudaSuccess);
    }
    GemmParams p;
    { const PrefetchHint h = take_prefetch_hint(); p.pf_ptr = h.ptr; p.pf_bytes = h.bytes; p.l2_hints = h.l2_hints; }
    fill_fp8_params(p, M, N, K, swap, epilogue, out_f32, ldc, C);
    p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
    p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
    p.ld_res = ld_res;
    Fp8Scales sc;
    sc.a_scale_t = reinterpret_cast<const float*>(a_scale_t);
    sc.w_scale = reinterpret_cast<const float*>(w_scale);
    sc.ld_as = ld_as;
    const void* Pp = swap ? W8 : A8;
    const void* Qp = swap ? A8 : W8;
    const int rowsP = swap ? N : M, rowsQ = swap ? M : N;
    const int ldP = swap ? ldb : lda, ldQ = swap ? lda : ldb;
    CUtensorMap tmP, tmQ;
    if (make_tmap_2d_u8(&tmP, Pp, rowsP, K, ldP, BM)) return -1;
    if (make_tmap_2d_u8(&tmQ, Qp, rowsQ, K, ldQ, bn)) return -1;
    dim3 grid((rowsP + BM - 1) / BM, (rowsQ + bn - 1) / bn, 1);
    return dispatch_fp8(bn, swap, tmP, tmQ, p, sc, grid, stream);
}

// Grouped form for mixture-of-experts layers: as mstar_moe_grouped_gemm with e4m3 token rows (scales
// [ceil(K/128), ld_as] over the sorted rows) and stacked e4m3 expert weights [E * N, K] (N a multiple of 128; scales
// [E * N / 128, ceil(K/128)]).
MSTAR_API int mstar_moe_grouped_gemm_fp8(const void* A8, const void* a_scale_t, int ld_as, const void* W8,
                                         const void* w_scale, void* C, int capacity_rows, int N, int K, int E,
                                         int block_rows, const int* block_expert, const int* num_blocks,
                                         const float* row_scale, void* const* row_dst, int epilogue, int ldc,
                                         void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (capacity_rows <= 0) return 0;
    if (block_rows != 16 && block_rows != 32 && block_rows != 64 && block_rows != 128)
        return set_error("moe gemm fp8: block_rows must be 16, 32, 64 or 128", cudaSuccess);
    if (K % 16 || N % 128 || capacity_rows % block_rows || ld_as < capacity_rows)
        return set_error("moe gemm fp8: K % 16, N % 128, capacity % block_rows and ld_as >= capacity are required", cudaSuccess);
    GemmParams p;
    { const PrefetchHint h = take_prefetch_hint(); p.pf_ptr = h.ptr; p.pf_bytes = h.bytes; p.l2_hints = h.l2_hints; }
    fill_fp8_params(p, capacity_rows, N, K, 1, epilogue, 0, ldc, C);
    p.block_expert = block_expert;
    p.num_blocks = num_blocks;
    p.row_scale = row_scale;
    p.row_dst = row_dst;
    Fp8Scales sc;
    sc.a_scale_t = reinterpret_cast<const float*>(a_scale_t);
    sc.w_scale = reinterpret_cast<const float*>(w_scale);
    sc.ld_as = ld_as;
    CUtensorMap tmP, tmQ;
    if (make_tmap_2d_u8(&tmP, W8, (long long)E * N, K, K, BM)) return -1;
    if (make_tmap_2d_u8(&tmQ, A8, capacity_rows, K, K, block_rows)) return -1;
    dim3 grid((N + BM - 1) / BM, capacity_rows / block_rows, 1);
    return dispatch_fp8(block_rows, 1, tmP, tmQ, p, sc, grid, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (declared in mstar_noalloc.h): the split-K scratch is a device array inside this
// library image instead of caller-provided memory.
// ---------------------------------------------------------------------------------------------
#include <stdio.h>
#include <stdlib.h>
#include "mstar_noalloc.h"

namespace {

struct NoAllocScratch {
    float partials[MSTAR_NOALLOC_WORKSPACE_BYTES / sizeof(float)];
    unsigned int counters[MSTAR_NOALLOC_MAX_TILES];
};
// In host code this name is only a handle for the runtime's symbol table, not a device address; the address that a
// kernel may use comes from cudaGetSymbolAddress (below), once per device.
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;

static NoAllocScratch* g_noalloc_ptr[kMaxDevices] = {};

}  // namespace

MSTAR_API int mstar_gemm_bf16_noalloc(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                      int ldc, void* stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
        return set_error("gemm_noalloc: operands must be 16-byte aligned with leading dimensions multiple of 8", cudaSuccess);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error("gemm_noalloc: cudaGetDevice failed", e);
    if (dev < 0 || dev >= kMaxDevices) return set_error("gemm_noalloc: device index out of range", cudaSuccess);
    if (g_noalloc_ptr[dev] == nullptr) {
        // set-up, once per device, with that device current
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) return set_error("gemm_noalloc: cudaGetSymbolAddress failed", e);
        g_noalloc_ptr[dev] = static_cast<NoAllocScratch*>(p);
    }
    NoAllocScratch* scratch = g_noalloc_ptr[dev];

    int swap, bn, splits, tiles;
    long long ws_need;
    mstar_gemm_plan(M, N, K, &swap, &bn, &splits, &ws_need, &tiles);
    if (ws_need > (long long)MSTAR_NOALLOC_WORKSPACE_BYTES) {
        char msg[200];
        snprintf(msg, sizeof(msg), "gemm_noalloc: this problem's split-K plan needs %lld scratch bytes, the built-in "
                 "maximum is %u", ws_need, (unsigned)MSTAR_NOALLOC_WORKSPACE_BYTES);
        return set_error(msg, cudaSuccess);
    }
    if (splits > 1 && tiles > MSTAR_NOALLOC_MAX_TILES)
        return set_error("gemm_noalloc: more output tiles than built-in arrival counters", cudaSuccess);
    if (splits > 1) {
        // counters must start at zero even if an earlier call was cut short
        e = cudaMemsetAsync(scratch->counters, 0, sizeof(unsigned int) * (size_t)tiles, stream);
        if (e != cudaSuccess) return set_error("gemm_noalloc: clearing the counters failed", e);
    }
    const int kblocks = (K + BK - 1) / BK;
    GemmParams p;
    { const PrefetchHint h = take_prefetch_hint(); p.pf_ptr = h.ptr; p.pf_bytes = h.bytes; p.l2_hints = h.l2_hints; }
    p.M = M; p.N = N; p.K = K;
    p.swap = swap;
    p.splits = splits;
    p.kblocks_total = kblocks;
    p.kblocks_per_split = (kblocks + splits - 1) / splits;
    p.epilogue = 0;
    p.out_f32 = 0;
    p.ldc = ldc;
    p.ld_res = 0;
    p.C = C;
    p.bias = nullptr;
    p.residual = nullptr;
    p.workspace = scratch->partials;
    p.counters = scratch->counters;
    p.status = nullptr;              // the status word is allocated memory, which this path must not create: its
                                     // waits stay bounded but a timeout is not reported (stated in the header)
    p.wait_limit_ns = wait_limit_ns();
    p.out_scale = 1.0f;
    p.ar = GemmAllReduce{};
    p.block_expert = nullptr;
    p.num_blocks = nullptr;
    p.row_scale = nullptr;
    p.row_dst = nullptr;
    const void* Pp = swap ? B : A;
    const void* Qp = swap ? A : B;
    const int rowsP = swap ? N : M, rowsQ = swap ? M : N;
    const int ldP = swap ? ldb : lda, ldQ = swap ? lda : ldb;
    CUtensorMap tmP, tmQ;
    if (make_tmap_2d_bf16(&tmP, Pp, rowsP, K, ldP, BM, BK)) return -1;
    if (make_tmap_2d_bf16(&tmQ, Qp, rowsQ, K, ldQ, bn, BK)) return -1;
    dim3 grid((rowsP + BM - 1) / BM, (rowsQ + bn - 1) / bn, splits);
    switch (bn) {
        case 16: return launch_gemm<16, 5, 2>(tmP, tmQ, p, grid, stream);
        case 32: return launch_gemm<32, 5, 2>(tmP, tmQ, p, grid, stream);
        case 64: return launch_gemm<64, 4, 2>(tmP, tmQ, p, grid, stream);
        case 128:
            if (swap) return launch_gemm<128, 3, 2>(tmP, tmQ, p, grid, stream);
            return launch_gemm<128, 6, 1>(tmP, tmQ, p, grid, stream);
        case 256: return launch_gemm<256, 4, 1>(tmP, tmQ, p, grid, stream);
    }
    return set_error("gemm_noalloc: unsupported tile", cudaSuccess);
}
