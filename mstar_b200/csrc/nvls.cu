// Collectives and fused consumers that use NVLS: loads, stores and reductions through the MULTICAST mapping of the
// symmetric heap, executed inside the NVSwitch. Every kernel also has a plain peer load / store path for groups
// without a multicast object (the host passes null multicast pointers), so results are the same on any box.
//
//   * allreduce_nvls          sum over the group. One-shot (small messages): every rank stages its input in its own
//                             heap, one flag round, then every rank load-reduces the whole message (the switch adds
//                             the ranks' values in fp32). Two-shot (large messages): rank r load-reduces share r and
//                             multicast-stores the sum to every rank's gather region: per GPU N/W bytes in and N/W
//                             out instead of the (W-1)/W * 2N of a ring.
//   * reduce_residual_norm    consumer half of a row-parallel projection under tensor parallelism. The GEMM writes its
//                             PARTIAL output into this rank's heap slot and returns without any communication; this
//                             kernel (the next one in the stream anyway: residual add + RMSNorm) raises the rank's
//                             flag, waits (bounded) for the peers' flags, and reads every row as one load-reduce over
//                             all ranks' slots while it normalises. The all-reduce is never materialised: its sum
//                             exists only in the registers of the norm kernel.
//   * allgather_cols          column-sharded outputs (vocabulary-parallel logits): every rank multicast-stores its
//                             [M, Ns] shard into every rank's [M, W * Ns] buffer, one flag round, and the sampler
//                             reads local memory.
//   * embed_gather_p2p        vocabulary-parallel embedding: the table shards live in the heap; a token's row is
//                             loaded straight from the owner's shard over NVLink (no mask, no all-reduce).
//
// Every wait is bounded and reports through the status word. No TMA and no cluster multicast is used here.
//
// Reference counterparts: RowParallelLinear all-reduce (mstar/model/components/distributed/linear.py:415), lm_head
// gather (mstar/model/orpheus/components/language_model.py:95, linear.py:105), VocabParallelEmbedding all-reduce
// (mstar/model/components/distributed/embedding.py:27-116) — separate NCCL kernels there.
#include <cstdlib>
#include "common.cuh"
#include "host_common.h"
#include "comm_device.cuh"

namespace mstar {

// Sum of 8 bf16 values at byte offset `off` of every rank's heap: one switch-side load-reduce, or W plain loads
// (own heap local, peers over NVLink) added in rank order.
__device__ __forceinline__ void load_sum8(const PeerTable& t, const McastTable& mc, long long off, float (&acc)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (mc.data != nullptr) {
        add_bf16x8(acc, multimem_ld_reduce_bf16x8(mc.data + off));
    } else {
        for (int q = 0; q < t.world; ++q)
            add_bf16x8(acc, __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(t.buf[q]) + off)));
    }
}

// ---------------------------------------------------------------------------------------------
// all-reduce
// ---------------------------------------------------------------------------------------------
struct NvlsARParams {
    PeerTable t;
    McastTable mc;
    const __nv_bfloat16* in;
    __nv_bfloat16* out;
    const __nv_bfloat16* residual;
    long long n;                 // elements, multiple of 8
    long long stage_off;         // byte offset of the staging area inside the data region (two slots by epoch parity)
    long long slot_bytes;        // bytes of one slot: [input n*2 | gathered result n*2] (two-shot uses both halves)
    int two_shot;
    unsigned int* epoch;
    unsigned int* arrive;
    int channel_base;            // flag channels [base, base + 2 * grid)
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};

__global__ void __launch_bounds__(512) allreduce_nvls_kernel(const __grid_constant__ NvlsARParams p) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) { s_epoch = *p.epoch + 1; s_ok = 1; }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int W = p.t.world, R = p.t.rank;
    const long long base = p.stage_off + (long long)(epoch & 1u) * p.slot_bytes;
    const long long nvec = p.n >> 3;
    const long long per = (nvec + gridDim.x - 1) / gridDim.x;
    const long long v0 = (long long)blockIdx.x * per;
    long long v1 = v0 + per;
    if (v1 > nvec) v1 = nvec;
    // stage my input in my own heap (local stores)
    const uint4* src = reinterpret_cast<const uint4*>(p.in);
    uint4* mine = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[R]) + base);
    {
        long long v = v0 + threadIdx.x;
        for (; v + 3LL * blockDim.x < v1; v += 4LL * blockDim.x) {
            const uint4 a0 = src[v], a1 = src[v + blockDim.x], a2 = src[v + 2LL * blockDim.x], a3 = src[v + 3LL * blockDim.x];
            mine[v] = a0; mine[v + blockDim.x] = a1; mine[v + 2LL * blockDim.x] = a2; mine[v + 3LL * blockDim.x] = a3;
        }
        for (; v < v1; v += blockDim.x) mine[v] = src[v];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        signal_all(p.t, p.mc, p.channel_base + blockIdx.x, epoch);
        if (!wait_all(p.t, p.channel_base + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x11)) s_ok = 0;
    }
    __syncthreads();
    if (s_ok && !p.two_shot) {
        for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
            float acc[8];
            load_sum8(p.t, p.mc, base + v * 16, acc);
            if (p.residual != nullptr) add_bf16x8(acc, reinterpret_cast<const uint4*>(p.residual)[v]);
            reinterpret_cast<uint4*>(p.out)[v] = pack8(acc);
        }
    } else if (s_ok && p.mc.data != nullptr) {
        // two-shot through the switch, four load-reduces in flight per thread (one per trip left the loop bound by
        // the round trip to the switch). The sum goes straight to every rank's OUTPUT region of the slot.
        const long long share = (v1 > v0 ? (v1 - v0 + W - 1) / W : 0);
        const long long a = v0 + (long long)R * share;
        long long b = a + share;
        if (b > v1) b = v1;
        const long long goff = base + p.n * 2;
        long long v = a + threadIdx.x;
        for (; v + 3LL * blockDim.x < b; v += 4LL * blockDim.x) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) r[u] = multimem_ld_reduce_bf16x8(p.mc.data + base + (v + (long long)u * blockDim.x) * 16);
#pragma unroll
            for (int u = 0; u < 4; ++u) multimem_st_v4(p.mc.data + goff + (v + (long long)u * blockDim.x) * 16, r[u]);
        }
        for (; v < b; v += blockDim.x)
            multimem_st_v4(p.mc.data + goff + v * 16, multimem_ld_reduce_bf16x8(p.mc.data + base + v * 16));
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            signal_all(p.t, p.mc, p.channel_base + gridDim.x + blockIdx.x, epoch);
            if (!wait_all(p.t, p.channel_base + gridDim.x + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x12)) s_ok = 0;
        }
        __syncthreads();
        if (s_ok) {
            const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[R]) + goff);
            const uint4* rs = reinterpret_cast<const uint4*>(p.residual);
            uint4* o = reinterpret_cast<uint4*>(p.out);
            long long w = v0 + threadIdx.x;
            for (; w + 3LL * blockDim.x < v1; w += 4LL * blockDim.x) {
                uint4 x[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) x[u] = __ldcg(g + w + (long long)u * blockDim.x);
                if (rs != nullptr) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float acc[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                        add_bf16x8(acc, x[u]);
                        add_bf16x8(acc, rs[w + (long long)u * blockDim.x]);
                        x[u] = pack8(acc);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) o[w + (long long)u * blockDim.x] = x[u];
            }
            for (; w < v1; w += blockDim.x) {
                uint4 x = __ldcg(g + w);
                if (rs != nullptr) {
                    float acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                    add_bf16x8(acc, x);
                    add_bf16x8(acc, rs[w]);
                    x = pack8(acc);
                }
                o[w] = x;
            }
        }
    } else if (s_ok) {
        // my share of this CTA's range: reduce in the switch, hand the sum to every rank's gather half
        const long long share = (v1 > v0 ? (v1 - v0 + W - 1) / W : 0);
        const long long a = v0 + (long long)R * share;
        long long b = a + share;
        if (b > v1) b = v1;
        const long long goff = base + p.n * 2;
        for (long long v = a + threadIdx.x; v < b; v += blockDim.x) {
            float acc[8];
            load_sum8(p.t, p.mc, base + v * 16, acc);
            const uint4 o = pack8(acc);
            if (p.mc.data != nullptr) {
                multimem_st_v4(p.mc.data + goff + v * 16, o);
            } else {
                for (int q = 0; q < W; ++q)
                    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + goff + v * 16) = o;
            }
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            signal_all(p.t, p.mc, p.channel_base + gridDim.x + blockIdx.x, epoch);
            if (!wait_all(p.t, p.channel_base + gridDim.x + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x12)) s_ok = 0;
        }
        __syncthreads();
        if (s_ok) {
            const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[R]) + goff);
            for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
                uint4 x = __ldcg(g + v);
                if (p.residual != nullptr) {
                    float acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                    add_bf16x8(acc, x);
                    add_bf16x8(acc, reinterpret_cast<const uint4*>(p.residual)[v]);
                    x = pack8(acc);
                }
                reinterpret_cast<uint4*>(p.out)[v] = x;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(p.arrive, 1u);
        if (old == gridDim.x - 1) {
            *p.arrive = 0u;
            *p.epoch = epoch;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// all-reduce in place, on a tensor that already lives at the same offset of every rank's symmetric region
// ---------------------------------------------------------------------------------------------
// The producer (a GEMM) wrote its partial straight into the region, so nothing is staged and nothing is copied out:
// one flag round ("my partial is complete"), then rank r load-reduces share r of every CTA's range in the switch and
// multicast-stores the sum over the same addresses of every rank, one more flag round, and every rank holds the sum
// where its partial was. Per GPU n/W bytes cross NVLink in each direction for the loads and again for the stores;
// HBM sees one read and one write of the tensor. Eight 16-byte requests are in flight per thread.
struct ARInplaceParams {
    PeerTable t;
    McastTable mc;
    long long off;               // byte offset of the tensor inside the region, 16-byte aligned
    long long n;                 // bf16 elements, multiple of 8
    unsigned int* epoch;
    unsigned int* arrive;
    int channel_base;            // flag channels [base, base + 2 * grid)
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};

__global__ void __launch_bounds__(512) allreduce_inplace_kernel(const __grid_constant__ ARInplaceParams p) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) { s_epoch = *p.epoch + 1; s_ok = 1; }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int W = p.t.world, R = p.t.rank;
    if (threadIdx.x == 0) {
        __threadfence_system();
        signal_all(p.t, p.mc, p.channel_base + blockIdx.x, epoch);
        if (!wait_all(p.t, p.channel_base + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x31)) s_ok = 0;
    }
    __syncthreads();
    const long long nvec = p.n >> 3;
    const long long per = (nvec + gridDim.x - 1) / gridDim.x;
    const long long v0 = (long long)blockIdx.x * per;
    long long v1 = v0 + per;
    if (v1 > nvec) v1 = nvec;
    if (s_ok && v1 > v0) {
        const long long share = (v1 - v0 + W - 1) / W;
        const long long a = v0 + (long long)R * share;
        long long b = a + share;
        if (b > v1) b = v1;
        constexpr int U = 8;
        long long v = a + threadIdx.x;
        if (p.mc.data != nullptr) {
            char* base = p.mc.data + p.off;
            for (; v + (long long)(U - 1) * blockDim.x < b; v += (long long)U * blockDim.x) {
                uint4 r[U];
#pragma unroll
                for (int u = 0; u < U; ++u) r[u] = multimem_ld_reduce_bf16x8(base + (v + (long long)u * blockDim.x) * 16);
#pragma unroll
                for (int u = 0; u < U; ++u) multimem_st_v4(base + (v + (long long)u * blockDim.x) * 16, r[u]);
            }
            for (; v < b; v += blockDim.x) multimem_st_v4(base + v * 16, multimem_ld_reduce_bf16x8(base + v * 16));
        } else {
            // plain peer loads and stores: this rank's share of every peer's partial comes in over NVLink once and
            // the sum goes out once, (W - 1) / W * n bytes per direction and nothing crosses the switch twice
            if (W == 2) v = p2p_share<2, 8>(p.t, p.off, v, b);
            else if (W <= 4) v = p2p_share<4, 4>(p.t, p.off, v, b);
            else v = p2p_share<MAX_RANKS, 2>(p.t, p.off, v, b);
            for (; v < b; v += blockDim.x) {
                float acc[8];
                load_sum8(p.t, p.mc, p.off + v * 16, acc);
                const uint4 o = pack8(acc);
                for (int q = 0; q < W; ++q)
                    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + p.off + v * 16) = o;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_ok) {
            signal_all(p.t, p.mc, p.channel_base + gridDim.x + blockIdx.x, epoch);
            wait_all(p.t, p.channel_base + gridDim.x + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x32);
        }
        __threadfence();
        const unsigned int old = atomicAdd(p.arrive, 1u);
        if (old == gridDim.x - 1) {
            *p.arrive = 0u;
            *p.epoch = epoch;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// reduce + residual + RMSNorm (consumer of a row-parallel GEMM's partial sums)
// ---------------------------------------------------------------------------------------------
struct RRNParams {
    PeerTable t;
    McastTable mc;
    long long slot_off;          // byte offset of the [M, N] bf16 partial inside every rank's data region
    int M, N;                    // N multiple of 8, at most RRN_MAX_N
    const __nv_bfloat16* residual_in;    // [M, N] or null
    __nv_bfloat16* residual_out;         // [M, N] or null: sum + residual_in (the new residual stream)
    const __nv_bfloat16* gamma;          // [N] or null (null: no normalisation, `out` gets the plain sum)
    __nv_bfloat16* out;                  // [M, N] normalised rows
    const __nv_bfloat16* bias;           // [N] or null, added once
    // two-shot form (large M): this rank reduces and normalises only rows [row_begin, row_end) and multicast-stores
    // them into every rank's h buffer at h_off of the region; the residual stream stays cut by rows
    // (residual_in / residual_out then hold this rank's rows only, row 0 = row_begin). out is unused.
    int two_shot, row_begin, row_end;
    long long h_off;
    float eps;
    unsigned int* epoch;
    unsigned int* arrive;
    int channel;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};
constexpr int RRN_THREADS = 256;
constexpr int RRN_MAX_VEC = 6;           // vectors of 8 per thread held in registers: N <= 256 * 6 * 8 = 12288

__global__ void __launch_bounds__(RRN_THREADS) reduce_residual_norm_kernel(const __grid_constant__ RRNParams p) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch;
    __shared__ float s_part[RRN_THREADS / 32];
    pdl_launch_dependents();
    pdl_wait();                  // the GEMM that wrote this rank's partial is complete and visible
    if (threadIdx.x == 0) { s_epoch = *p.epoch + 1; s_ok = 1; }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            signal_all(p.t, p.mc, p.channel, epoch);       // "my partial is in my slot"
        }
        if (!wait_all(p.t, p.channel, epoch, p.status, p.wait_limit_ns, 0x21)) s_ok = 0;
    }
    __syncthreads();
    const int nvec = p.N >> 3;
    const int m_first = p.two_shot ? p.row_begin : 0;
    const int m_last = p.two_shot ? p.row_end : p.M;
    if (s_ok) {
        for (int m = m_first + blockIdx.x; m < m_last; m += gridDim.x) {
            const size_t lm = (size_t)(m - m_first);      // row index inside the (possibly row-cut) residual tensors
            float x[RRN_MAX_VEC][8];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < RRN_MAX_VEC; ++i) {
                const int c = threadIdx.x + i * RRN_THREADS;
                if (c < nvec) {
                    load_sum8(p.t, p.mc, p.slot_off + ((long long)m * p.N + c * 8) * 2, x[i]);
                    if (p.bias != nullptr) add_bf16x8(x[i], reinterpret_cast<const uint4*>(p.bias)[c]);
                    if (p.residual_in != nullptr)
                        add_bf16x8(x[i], reinterpret_cast<const uint4*>(p.residual_in + lm * p.N)[c]);
                    const uint4 r8 = pack8(x[i]);
                    if (p.residual_out != nullptr) reinterpret_cast<uint4*>(p.residual_out + lm * p.N)[c] = r8;
                    // the norm sees the bf16-rounded residual stream, exactly as the unfused add + norm kernels do
                    const uint32_t w[4] = {r8.x, r8.y, r8.z, r8.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = unpack_bf16x2(w[j]);
                        x[i][2 * j] = f.x;
                        x[i][2 * j + 1] = f.y;
                        ss += f.x * f.x + f.y * f.y;
                    }
                }
            }
            if (p.gamma == nullptr && !p.two_shot) {
#pragma unroll
                for (int i = 0; i < RRN_MAX_VEC; ++i) {
                    const int c = threadIdx.x + i * RRN_THREADS;
                    if (c < nvec) reinterpret_cast<uint4*>(p.out + (size_t)m * p.N)[c] = pack8(x[i]);
                }
                continue;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < RRN_THREADS / 32; ++i) tot += s_part[i];
            __syncthreads();
            const float inv = p.gamma != nullptr ? rsqrtf(tot / (float)p.N + p.eps) : 1.f;
#pragma unroll
            for (int i = 0; i < RRN_MAX_VEC; ++i) {
                const int c = threadIdx.x + i * RRN_THREADS;
                if (c < nvec) {
                    float y[8];
                    if (p.gamma != nullptr) {
                        const uint4 g8 = reinterpret_cast<const uint4*>(p.gamma)[c];
                        const uint32_t gw[4] = {g8.x, g8.y, g8.z, g8.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 g = unpack_bf16x2(gw[j]);
                            y[2 * j] = x[i][2 * j] * inv * g.x;
                            y[2 * j + 1] = x[i][2 * j + 1] * inv * g.y;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) y[j] = x[i][j];
                    }
                    const uint4 o8 = pack8(y);
                    if (!p.two_shot) {
                        reinterpret_cast<uint4*>(p.out + (size_t)m * p.N)[c] = o8;
                    } else {
                        const long long dst = p.h_off + ((long long)m * p.N + c * 8) * 2;
                        if (p.mc.data != nullptr) {
                            multimem_st_v4(p.mc.data + dst, o8);
                        } else {
                            for (int q = 0; q < p.t.world; ++q)
                                *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + dst) = o8;
                        }
                    }
                }
            }
        }
    }
    if (p.two_shot) {
        // second flag round: every rank's rows of h are in place on this rank before the kernel (and with it the
        // stream) moves on to the GEMM that reads them
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0 && s_ok) {
            // block b of every rank signals on channel + 1 + b and waits for block b of the peers; all ranks launch the
            // same grid, so when all blocks of this rank are through, all blocks of all peers have stored their rows
            signal_all(p.t, p.mc, p.channel + 1 + blockIdx.x, epoch);
            if (!wait_all(p.t, p.channel + 1 + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x23)) s_ok = 0;
        }
        __syncthreads();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(p.arrive, 1u);
        if (old == gridDim.x - 1) {
            *p.arrive = 0u;
            *p.epoch = epoch;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// all-gather of column shards
// ---------------------------------------------------------------------------------------------
struct AGParams {
    PeerTable t;
    McastTable mc;
    long long shard_off;         // byte offset of this rank's [M, Ns] bf16 shard in its own heap (written by the GEMM)
    long long full_off;          // byte offset of the [M, W * Ns] gathered matrix in every rank's heap
    int M, Ns;                   // Ns multiple of 8
    unsigned int* epoch;
    unsigned int* arrive;
    int channel;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};

__global__ void __launch_bounds__(512) allgather_cols_kernel(const __grid_constant__ AGParams p) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) { s_epoch = *p.epoch + 1; s_ok = 1; }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int W = p.t.world, R = p.t.rank;
    const long long vec_per_row = p.Ns >> 3;
    const long long total = (long long)p.M * vec_per_row;
    const long long full_ld = (long long)W * p.Ns;       // elements
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[R]) + p.shard_off);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / vec_per_row, c = i - m * vec_per_row;
        const uint4 v = src[i];
        const long long dst = p.full_off + (m * full_ld + (long long)R * p.Ns + c * 8) * 2;
        if (p.mc.data != nullptr) {
            multimem_st_v4(p.mc.data + dst, v);
        } else {
            for (int q = 0; q < W; ++q) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + dst) = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    // every CTA signals on its own channel slot and waits for the same CTA of the peers: when all CTAs are through,
    // all shards are in place on this rank (a consumer kernel in the stream starts after this kernel ends)
    if (threadIdx.x == 0) {
        signal_all(p.t, p.mc, p.channel + blockIdx.x, epoch);
        if (!wait_all(p.t, p.channel + blockIdx.x, epoch, p.status, p.wait_limit_ns, 0x31)) s_ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(p.arrive, 1u);
        if (old == gridDim.x - 1) {
            *p.arrive = 0u;
            *p.epoch = epoch;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// vocabulary-parallel embedding
// ---------------------------------------------------------------------------------------------
struct EmbedP2PParams {
    PeerTable t;
    long long table_off;         // byte offset of every rank's [rows_per_rank, H] bf16 table shard in its heap
    int rows_per_rank, H;        // H multiple of 8
    const long long* ids;        // [T]
    __nv_bfloat16* out;          // [T, H]
    int T, vocab;
};

__global__ void __launch_bounds__(256) embed_gather_p2p_kernel(const __grid_constant__ EmbedP2PParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int vec = p.H >> 3;
    for (int tkn = blockIdx.x; tkn < p.T; tkn += gridDim.x) {
        long long id = p.ids[tkn];
        if (id < 0) id = 0;
        if (id >= p.vocab) id = p.vocab - 1;
        const int owner = (int)(id / p.rows_per_rank);
        const long long row = id - (long long)owner * p.rows_per_rank;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[owner]) + p.table_off +
                                                          row * (long long)p.H * 2);
        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)tkn * p.H);
        for (int c = threadIdx.x; c < vec; c += blockDim.x) dst[c] = __ldg(src + c);
    }
}

}  // namespace mstar

using namespace mstar;

static int fill_tables(PeerTable* t, McastTable* mc, void* const* bufs, void* const* flags, int world, int rank,
                       void* mc_data, void* mc_flags) {
    if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world)
        return set_error("nvls: world must be in [1, 8] and rank inside it", cudaSuccess);
    for (int i = 0; i < MAX_RANKS; ++i) {
        t->buf[i] = i < world ? bufs[i] : nullptr;
        t->flags[i] = i < world ? reinterpret_cast<unsigned int*>(flags[i]) : nullptr;
    }
    t->world = world;
    t->rank = rank;
    mc->data = reinterpret_cast<char*>(mc_data);
    mc->flags = reinterpret_cast<unsigned int*>(mc_flags);
    return 0;
}

// mode 1 = one-shot, 2 = two-shot, 0 = pick by size. Returns the number of CTAs used, or -1.
MSTAR_API int mstar_allreduce_nvls(void* const* bufs, void* const* flags, int world, int rank, void* mc_data,
                                   void* mc_flags, const void* in, void* out, const void* residual, long long n,
                                   long long stage_off, long long slot_bytes, void* state, int channel_base,
                                   int max_ctas, int mode, void* stream_) {
    if (n <= 0) return 0;
    if (n % 8) return set_error("allreduce_nvls: element count must be a multiple of 8", cudaSuccess);
    NvlsARParams p;
    if (fill_tables(&p.t, &p.mc, bufs, flags, world, rank, mc_data, mc_flags)) return -1;
    const long long bytes = n * 2;
    if (mode == 0) mode = bytes <= (1 << 20) ? 1 : 2;
    if ((mode == 1 ? bytes : 2 * bytes) > slot_bytes)
        return set_error("allreduce_nvls: message does not fit the staging slot", cudaSuccess);
    p.in = (const __nv_bfloat16*)in;
    p.out = (__nv_bfloat16*)out;
    p.residual = (const __nv_bfloat16*)residual;
    p.n = n;
    p.stage_off = stage_off;
    p.slot_bytes = slot_bytes;
    p.two_shot = mode == 2;
    p.epoch = reinterpret_cast<unsigned int*>(state);
    p.arrive = p.epoch + 1;
    p.channel_base = channel_base;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    long long ctas = (n / 8 + 2047) / 2048;
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;
    cudaError_t e = launch_pdl(allreduce_nvls_kernel, dim3((unsigned)ctas), dim3(512), 0, (cudaStream_t)stream_, p);
    if (e != cudaSuccess) return set_error("allreduce_nvls launch", e);
    return (int)ctas;
}

// The bandwidth-bound forms (in-place all-reduce, two-shot consumer reduce) move their DATA through the switch only
// from this group size on: a load-reduce also pulls the requester's own copy through NVLink and a multicast store
// comes back to the sender, (W + 1) / W * n bytes per direction against (W - 1) / W * n for plain peer loads and
// stores, which in small groups costs more than the switch-side addition saves. Flags still use the multicast.
static int nvls_data_min_world() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MSTAR_NVLS_DATA_MIN_WORLD");
        v = e != nullptr ? atoi(e) : 4;
        if (v < 2) v = 2;
    }
    return v;
}

// In-place sum of the [n] bf16 tensor at byte offset `off` of every rank's region (`bufs` / `mc_data` describe that
// region). Every rank must launch the same grid: it is sized from n and max_ctas only. Returns the grid size.
MSTAR_API int mstar_allreduce_inplace(void* const* bufs, void* const* flags, int world, int rank, void* mc_data,
                                      void* mc_flags, long long off, long long n, void* state, int channel_base,
                                      int max_ctas, void* stream_) {
    if (n <= 0) return 0;
    if (n % 8 || off % 16) return set_error("allreduce_inplace: count must be a multiple of 8, offset of 16", cudaSuccess);
    ARInplaceParams p;
    if (fill_tables(&p.t, &p.mc, bufs, flags, world, rank, mc_data, mc_flags)) return -1;
    if (world < nvls_data_min_world()) p.mc.data = nullptr;
    p.off = off;
    p.n = n;
    p.epoch = reinterpret_cast<unsigned int*>(state);
    p.arrive = p.epoch + 1;
    p.channel_base = channel_base;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    long long ctas = (n / 8 + 4095) / 4096;
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;
    cudaError_t e = launch_pdl(allreduce_inplace_kernel, dim3((unsigned)ctas), dim3(512), 0, (cudaStream_t)stream_, p);
    if (e != cudaSuccess) return set_error("allreduce_inplace launch", e);
    return (int)ctas;
}

// two_shot != 0: rows [row_begin, row_end) are this rank's; normalised rows go to h_off of every rank's region copy.
MSTAR_API int mstar_reduce_residual_norm(void* const* bufs, void* const* flags, int world, int rank, void* mc_data,
                                         void* mc_flags, long long slot_off, int M, int N, const void* residual_in,
                                         void* residual_out, const void* gamma, const void* bias, void* out, float eps,
                                         int two_shot, int row_begin, int row_end, long long h_off,
                                         void* state, int channel, void* stream_) {
    if (M <= 0) return 0;
    if (N % 8 || N > RRN_THREADS * RRN_MAX_VEC * 8)
        return set_error("reduce_residual_norm: N must be a multiple of 8 and at most 12288", cudaSuccess);
    RRNParams p;
    if (fill_tables(&p.t, &p.mc, bufs, flags, world, rank, mc_data, mc_flags)) return -1;
    p.slot_off = slot_off;
    p.M = M; p.N = N;
    p.residual_in = (const __nv_bfloat16*)residual_in;
    p.residual_out = (__nv_bfloat16*)residual_out;
    p.gamma = (const __nv_bfloat16*)gamma;
    p.bias = (const __nv_bfloat16*)bias;
    p.out = (__nv_bfloat16*)out;
    p.eps = eps;
    p.two_shot = two_shot ? 1 : 0;
    if (two_shot && world < nvls_data_min_world()) p.mc.data = nullptr;
    p.row_begin = row_begin;
    p.row_end = row_end;
    p.h_off = h_off;
    p.epoch = reinterpret_cast<unsigned int*>(state);
    p.arrive = p.epoch + 1;
    p.channel = channel;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    // the two-shot form uses one flag channel per block and needs the same grid on every rank: it is sized from the
    // largest row share, ceil(M / world), not from this rank's own share
    const int rows = two_shot ? (M + world - 1) / world : M;
    const int cap = two_shot ? 1024 : 4 * device_sm_count();
    int grid = rows < cap ? rows : cap;
    if (grid < 1) grid = 1;
    cudaError_t e = launch_pdl(reduce_residual_norm_kernel, dim3(grid), dim3(RRN_THREADS), 0, (cudaStream_t)stream_, p);
    return e == cudaSuccess ? 0 : set_error("reduce_residual_norm launch", e);
}

MSTAR_API int mstar_allgather_cols(void* const* bufs, void* const* flags, int world, int rank, void* mc_data,
                                   void* mc_flags, long long shard_off, long long full_off, int M, int Ns, void* state,
                                   int channel, int max_ctas, void* stream_) {
    if (M <= 0) return 0;
    if (Ns % 8) return set_error("allgather_cols: shard width must be a multiple of 8", cudaSuccess);
    AGParams p;
    if (fill_tables(&p.t, &p.mc, bufs, flags, world, rank, mc_data, mc_flags)) return -1;
    p.shard_off = shard_off;
    p.full_off = full_off;
    p.M = M; p.Ns = Ns;
    p.epoch = reinterpret_cast<unsigned int*>(state);
    p.arrive = p.epoch + 1;
    p.channel = channel;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    long long ctas = ((long long)M * (Ns / 8) + 4095) / 4096;
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;
    cudaError_t e = launch_pdl(allgather_cols_kernel, dim3((unsigned)ctas), dim3(512), 0, (cudaStream_t)stream_, p);
    if (e != cudaSuccess) return set_error("allgather_cols launch", e);
    return (int)ctas;
}

MSTAR_API int mstar_embed_gather_p2p(void* const* bufs, int world, int rank, long long table_off, int rows_per_rank,
                                     int H, const void* ids, void* out, int T, int vocab, void* stream_) {
    if (T <= 0) return 0;
    if (H % 8) return set_error("embed_gather_p2p: hidden size must be a multiple of 8", cudaSuccess);
    if (world < 1 || world > MAX_RANKS) return set_error("embed_gather_p2p: bad world size", cudaSuccess);
    EmbedP2PParams p;
    for (int i = 0; i < MAX_RANKS; ++i) { p.t.buf[i] = i < world ? bufs[i] : nullptr; p.t.flags[i] = nullptr; }
    p.t.world = world; p.t.rank = rank;
    p.table_off = table_off;
    p.rows_per_rank = rows_per_rank;
    p.H = H;
    p.ids = (const long long*)ids;
    p.out = (__nv_bfloat16*)out;
    p.T = T;
    p.vocab = vocab;
    const int cap = 8 * device_sm_count();
    cudaError_t e = launch_pdl(embed_gather_p2p_kernel, dim3(T < cap ? T : cap), dim3(256), 0, (cudaStream_t)stream_, p);
    return e == cudaSuccess ? 0 : set_error("embed_gather_p2p launch", e);
}
