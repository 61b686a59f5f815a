// Collectives over the symmetric heap: every rank maps every peer's heap (plain peer pointers over NVLink, no
// TMA and no multicast loads from peer memory). Signals are 32-bit epoch words written with release stores at
// system scope and polled with acquire loads; every poll is bounded and reports through the status word
// instead of hanging, so a missing peer turns into an error code on the host.
//
//   * allreduce_oneshot   small messages (decode): every rank copies its partial into its own heap slot, raises
//                         its flag at every peer, then sums all ranks' partials in rank order (identical
//                         result on every rank, which tensor-parallel greedy decoding relies on).
//   * allreduce_twoshot   large messages: rank r reduces slice r of the rows from all peers and stores the sum
//                         into every rank's output (reduce-scatter + all-gather in one kernel).
//   * a2a_heads           Ulysses exchange: [S_local, H, D] -> every peer gets its head group of these rows
//                         written straight into its [S_total, H / P, D] buffer (and the reverse direction).
//   * cfg_combine_peer    classifier-free guidance with the branches on different GPUs: the combine rank reads
//                         the peers' velocities over NVLink and applies guidance + renorm + Euler step.
//   * peer_barrier        device-side barrier over the flags (replaces a host barrier per forward).
//
// Reference counterparts: CommGroup all_reduce / all_to_all through NCCL (mstar/distributed/communication.py:
// 67-162), row-parallel all-reduce call sites (mstar/model/components/distributed/linear.py:415), Ulysses
// (mstar/model/components/distributed/sequence_parallel.py:84-176), CFG branch exchange over the tensor
// transport (mstar/model/bagel/submodules.py:1411-1570), per-forward tp barrier
// (mstar/engine/kv_cache_engine.py:1016).
#include "common.cuh"
#include "host_common.h"
#include "comm_device.cuh"

namespace mstar {

struct ARParams {
    PeerTable t;
    const __nv_bfloat16* in;     // local partial [n]
    __nv_bfloat16* out;          // local result [n]
    const __nv_bfloat16* residual;   // optional, added after the sum
    long long n;                 // elements (multiple of 8)
    long long slot_bytes;        // data region is split into 2 slots used in turn (parity of the epoch)
    unsigned int* epoch;         // local device word: number of completed calls on this channel set
    unsigned int* arrive;        // local device word: CTA arrival counter (reset by the last CTA)
    int channel_base;            // flag channels [channel_base, channel_base + gridDim.x)
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};

// Both kernels PUSH: a rank stores its data into its peers' slots with plain 16-byte stores over NVLink (which
// pipeline without waiting for anything), raises one flag per CTA slice, waits (bounded) for the peers' flags and
// then reads only local memory. The first versions pulled (each rank loading the peers' slots): every loop trip paid
// an NVLink round trip, 0.37-0.40 of the link rate on 86 MB where NCCL reached 0.57.
//
// One-shot: CTA b owns vectors [b*per, (b+1)*per) and flag channel b. Slot layout: region q (n elements) holds rank
// q's input. Traffic out per rank: (W - 1) * n. Used for small messages and for two ranks.
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const __grid_constant__ ARParams p) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) { s_epoch = *p.epoch + 1; s_ok = 1; }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int parity = epoch & 1;
    const int W = p.t.world, R = p.t.rank;
    const long long nvec = p.n >> 3;
    const long long per = (nvec + gridDim.x - 1) / gridDim.x;
    const long long v0 = (long long)blockIdx.x * per;
    long long v1 = v0 + per;
    if (v1 > nvec) v1 = nvec;
    const uint4* src = reinterpret_cast<const uint4*>(p.in);
    for (int q = 0; q < W; ++q) {
        if (q == R) continue;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + parity * p.slot_bytes) + (long long)R * nvec;
        // four local loads in flight per thread before the four peer stores (one load per trip left the copy bound by
        // the local load latency: 0.48 of the link rate on 86 MB)
        long long v = v0 + threadIdx.x;
        for (; v + 3LL * blockDim.x < v1; v += 4LL * blockDim.x) {
            const uint4 a0 = src[v], a1 = src[v + blockDim.x], a2 = src[v + 2LL * blockDim.x], a3 = src[v + 3LL * blockDim.x];
            dst[v] = a0; dst[v + blockDim.x] = a1; dst[v + 2LL * blockDim.x] = a2; dst[v + 3LL * blockDim.x] = a3;
        }
        for (; v < v1; v += blockDim.x) dst[v] = src[v];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!signal_and_wait_all(p.t, p.channel_base + blockIdx.x, epoch, p.status, p.wait_limit_ns, 1)) s_ok = 0;
    }
    __syncthreads();
    if (s_ok) {
        const uint4* mine = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[R]) + parity * p.slot_bytes);
#pragma unroll 4
        for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int r = 0; r < W; ++r) {       // rank order on every rank: bit-identical results
                const uint4 x = r == R ? src[v] : __ldcg(mine + (long long)r * nvec + v);
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(w[j]);
                    acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
                }
            }
            if (p.residual != nullptr) {
                const uint4 x = reinterpret_cast<const uint4*>(p.residual)[v];
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(w[j]);
                    acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
                }
            }
            reinterpret_cast<uint4*>(p.out)[v] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                            pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
        }
    }
    // the last CTA of the launch publishes the new epoch for the next call
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

// Two-shot (more than two ranks, large messages): inside CTA b's slice rank r owns the share [a_r, b_r). Phase 1
// (reduce-scatter by push): every rank stores its part of share r into rank r's slot, region [source rank], at the
// vector's own index. Phase 2: the owner sums its share in rank order, writes its own output and pushes the sum into
// every peer's gather region (second half of the slot). Phase 3: everyone copies the other shares from its gather
// region to the output. Traffic out per rank: 2 * (W - 1) / W * n.
__global__ void __launch_bounds__(512) allreduce_twoshot_kernel(const __grid_constant__ ARParams p) {
    __shared__ int s_ok;
    __shared__ unsigned int s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) { s_epoch = *p.epoch + 1; s_ok = 1; }
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int parity = epoch & 1;
    const long long nvec = p.n >> 3;
    const int W = p.t.world, R = p.t.rank;
    const long long half_bytes = p.slot_bytes >> 1;      // [shares received | gathered result]
    const long long per = (nvec + gridDim.x - 1) / gridDim.x;
    const long long v0 = (long long)blockIdx.x * per;
    long long v1 = v0 + per;
    if (v1 > nvec) v1 = nvec;
    const long long share = (v1 > v0 ? (v1 - v0 + W - 1) / W : 0);
    // the receive area of a slot is W regions of `cap` vectors; a vector of CTA b's share sits at b * share + offset
    const long long cap = (long long)gridDim.x * ((per + W - 1) / W);
    const long long share_cap = (per + W - 1) / W;
    const uint4* src = reinterpret_cast<const uint4*>(p.in);
    // phase 1
    for (int q = 0; q < W; ++q) {
        if (q == R) continue;
        const long long a = v0 + q * share;
        long long b = a + share;
        if (b > v1) b = v1;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + parity * p.slot_bytes) +
                     (long long)R * cap + (long long)blockIdx.x * share_cap;
        for (long long v = a + threadIdx.x; v < b; v += blockDim.x) dst[v - a] = src[v];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!signal_and_wait_all(p.t, p.channel_base + blockIdx.x, epoch, p.status, p.wait_limit_ns, 2)) s_ok = 0;
    }
    __syncthreads();
    const long long a = v0 + R * share;
    long long b = a + share;
    if (b > v1) b = v1;
    // phase 2
    if (s_ok) {
        const uint4* recv = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[R]) + parity * p.slot_bytes) +
                            (long long)blockIdx.x * share_cap;
        for (long long v = a + threadIdx.x; v < b; v += blockDim.x) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int r = 0; r < W; ++r) {
                const uint4 x = r == R ? src[v] : __ldcg(recv + (long long)r * cap + (v - a));
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(w[j]);
                    acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
                }
            }
            const uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                       pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
            for (int r = 0; r < W; ++r)
                if (r != R)
                    reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[r]) + parity * p.slot_bytes + half_bytes)[v] = o;
            uint4 x = o;
            if (p.residual != nullptr) {
                const uint4 rsd = reinterpret_cast<const uint4*>(p.residual)[v];
                const uint32_t a4[4] = {x.x, x.y, x.z, x.w}, b4[4] = {rsd.x, rsd.y, rsd.z, rsd.w};
                uint32_t o4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fa = unpack_bf16x2(a4[j]), fb = unpack_bf16x2(b4[j]);
                    o4[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
                }
                x = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
            reinterpret_cast<uint4*>(p.out)[v] = x;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && s_ok) {
        // second signal round uses its own channel range [base + grid, base + 2 * grid)
        if (!signal_and_wait_all(p.t, p.channel_base + gridDim.x + blockIdx.x, epoch, p.status, p.wait_limit_ns, 3)) s_ok = 0;
    }
    __syncthreads();
    // phase 3: the other ranks' shares
    if (s_ok) {
        const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.t.buf[R]) + parity * p.slot_bytes + half_bytes);
        for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
            if (v >= a && v < b) continue;
            uint4 x = __ldcg(g + v);
            if (p.residual != nullptr) {
                const uint4 rsd = reinterpret_cast<const uint4*>(p.residual)[v];
                const uint32_t a4[4] = {x.x, x.y, x.z, x.w}, b4[4] = {rsd.x, rsd.y, rsd.z, rsd.w};
                uint32_t o4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fa = unpack_bf16x2(a4[j]), fb = unpack_bf16x2(b4[j]);
                    o4[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
                }
                x = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
            reinterpret_cast<uint4*>(p.out)[v] = x;
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

// Device-side barrier over one flag channel (one CTA, one thread does the signalling).
struct BarrierParams {
    PeerTable t;
    unsigned int* epoch;
    int channel;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};
__global__ void peer_barrier_kernel(const __grid_constant__ BarrierParams p) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        const unsigned int e = *p.epoch + 1;
        __threadfence_system();
        signal_and_wait_all(p.t, p.channel, e, p.status, p.wait_limit_ns, 4);
        *p.epoch = e;
    }
}

// Ulysses head <-> sequence exchange by peer stores.
//   forward  (scatter heads, gather sequence): src [S_local, H, D] on each rank; rank q receives, for its head
//            group, rows [seq_off[r], seq_off[r] + S_local_r) of dst [S_total, H/P, D] from rank r.
//   backward (scatter sequence, gather heads): src [S_total, H/P, D]; rank q receives its rows with rank r's
//            head group into dst [S_local_q, H, D].
struct A2AParams {
    PeerTable t;
    const __nv_bfloat16* src;
    long long dst_offset_bytes;   // destination buffer offset inside every rank's data region
    int forward;
    int H, D;                      // full head count, head dim
    int seq_off[MAX_RANKS + 1];    // row offsets of the ranks' sequence shards
    unsigned int* epoch;
    unsigned int* arrive;
    int channel_base;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};
__global__ void __launch_bounds__(256) a2a_heads_kernel(const __grid_constant__ A2AParams p) {
    __shared__ unsigned int s_epoch;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) s_epoch = *p.epoch + 1;
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int W = p.t.world, R = p.t.rank;
    const int Hp = p.H / W;
    const int vec_per_head = p.D >> 3;
    const int S_total = p.seq_off[W];
    if (p.forward) {
        const int S_local = p.seq_off[R + 1] - p.seq_off[R];
        const long long total = (long long)S_local * p.H * vec_per_head;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
            const int v = (int)(i % vec_per_head);
            const long long hs = i / vec_per_head;
            const int h = (int)(hs % p.H);
            const long long s = hs / p.H;
            const int q = h / Hp, hl = h - q * Hp;
            const uint4 x = reinterpret_cast<const uint4*>(p.src)[i];
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + p.dst_offset_bytes);
            dst[((long long)(p.seq_off[R] + s) * Hp + hl) * vec_per_head + v] = x;
        }
    } else {
        const long long total = (long long)S_total * Hp * vec_per_head;
        for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
            const int v = (int)(i % vec_per_head);
            const long long hs = i / vec_per_head;
            const int hl = (int)(hs % Hp);
            const int s = (int)(hs / Hp);
            int q = 0;
            while (q + 1 < W && s >= p.seq_off[q + 1]) ++q;
            const uint4 x = reinterpret_cast<const uint4*>(p.src)[i];
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.t.buf[q]) + p.dst_offset_bytes);
            dst[((long long)(s - p.seq_off[q]) * p.H + R * Hp + hl) * vec_per_head + v] = x;
        }
    }
    __threadfence_system();
    __syncthreads();
    // grid-wide completion: the last CTA signals the peers and waits for theirs
    __shared__ int s_last;
    if (threadIdx.x == 0) {
        const unsigned int old = atomicAdd(p.arrive, 1u);
        s_last = (old == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence_system();
        signal_and_wait_all(p.t, p.channel_base, epoch, p.status, p.wait_limit_ns, 5);
        *p.arrive = 0u;
        *p.epoch = epoch;
    }
}

// QK-norm + RoPE with the Ulysses head scatter as its store: the rows of this sequence-parallel rank ([T_local,
// (Hq + 2 Hkv) * D], all heads of the tensor-parallel shard) are normalised and rotated, and every head's 256 bytes
// go straight into the buffer of the rank that attends with that head: q head h -> rank h / (Hq / P), row
// seq_off[R] + t of its [S_total, Hq / P, D] tensor; k and v likewise. No [T_local, H, D] intermediate and no
// stand-alone exchange kernel. One CTA per token; a head is handled by 16 lanes with 8 consecutive elements each
// (one 16-byte load and one 16-byte store per lane); the rotate-half partner sits 8 lanes away. Full rotary only
// (rot_dim == D). The end of the kernel is the exchange's flag round: the last CTA tells the peers that this rank's
// stores are out and waits (bounded) for theirs.
struct RopeScatterParams {
    PeerTable t;
    const __nv_bfloat16* qkv;
    long long ld_qkv;
    const int* positions;            // [n_axes, pos_stride]: positions of the LOCAL tokens
    long long pos_stride;
    const float* inv_freq;           // [D / 2]
    const signed char* axis_of_freq; // [D / 2] or null
    const __nv_bfloat16* q_norm_w;   // [D] or null
    const __nv_bfloat16* k_norm_w;
    long long q_off, k_off, v_off;   // byte offsets of the destination tensors inside every rank's data region
    int T, Hq, Hkv, D, interleaved;
    float norm_eps;
    int seq_off[MAX_RANKS + 1];
    unsigned int* epoch;
    unsigned int* arrive;
    int channel;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};

__global__ void __launch_bounds__(256) rope_scatter_kernel(const __grid_constant__ RopeScatterParams p) {
    __shared__ float s_cos[128], s_sin[128];
    __shared__ unsigned int s_epoch;
    __shared__ int s_last;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) s_epoch = *p.epoch + 1;
    const int W = p.t.world, R = p.t.rank;
    const int D = p.D, half = D >> 1;
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
        __syncthreads();                 // the previous token's table is no longer read
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int axis = p.axis_of_freq ? p.axis_of_freq[i] : 0;
            const float ang = (float)p.positions[(size_t)axis * p.pos_stride + t] * p.inv_freq[i];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            s_cos[i] = cs;
            s_sin[i] = sn;
        }
        __syncthreads();
        const int lanes = D >> 3;                        // lanes per head: 16 for D = 128, 8 for D = 64
        const int sub = threadIdx.x % lanes;             // which 8 elements of the head
        const int slot = threadIdx.x / lanes, nslots = blockDim.x / lanes;
        const int nheads = p.Hq + 2 * p.Hkv;
        const __nv_bfloat16* row = p.qkv + (size_t)t * p.ld_qkv;
        const long long drow = p.seq_off[R] + t;
        for (int h0 = 0; h0 < nheads; h0 += nslots) {
            const int h = h0 + slot;
            const bool on = h < nheads;
            const bool is_q = h < p.Hq, is_k = !is_q && h < p.Hq + p.Hkv;
            float x[8];
            if (on) {
                const uint4 raw = *reinterpret_cast<const uint4*>(row + (size_t)h * D + sub * 8);
                const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack_bf16x2(w4[j]);
                    x[2 * j] = f.x; x[2 * j + 1] = f.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = 0.f;
            }
            const bool rotate = on && (is_q || is_k);
            const __nv_bfloat16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
            if (p.q_norm_w != nullptr || p.k_norm_w != nullptr) {
                // per-head RMS norm (every lane of the warp takes part in the reduction, whatever its head is); the
                // norm's output is rounded to bf16 before the rotation, as a separate norm op would do
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
                for (int d = lanes >> 1; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
                if (rotate && nw != nullptr) {
                    const float inv = rsqrtf(ss / D + p.norm_eps);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        x[j] = __bfloat162float(__float2bfloat16(x[j] * inv * __bfloat162float(nw[sub * 8 + j])));
                }
            }
            float y[8];
            if (p.interleaved) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = sub * 4 + j;           // pair index: elements (2i, 2i + 1)
                    const float cs = s_cos[i], sn = s_sin[i];
                    y[2 * j] = rotate ? x[2 * j] * cs - x[2 * j + 1] * sn : x[2 * j];
                    y[2 * j + 1] = rotate ? x[2 * j + 1] * cs + x[2 * j] * sn : x[2 * j + 1];
                }
            } else {
                // rotate-half: element i pairs with i + D / 2, held by the lane lanes / 2 away
                const bool first = sub < (lanes >> 1);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float other = __shfl_xor_sync(0xffffffffu, x[j], lanes >> 1);
                    const int i = (sub * 8 + j) % half;
                    const float cs = s_cos[i], sn = s_sin[i];
                    y[j] = !rotate ? x[j] : (first ? x[j] * cs - other * sn : x[j] * cs + other * sn);
                }
            }
            if (on) {
                const int Hn = is_q ? p.Hq : p.Hkv;      // heads of this kind on this rank (before the exchange)
                const int hk = is_q ? h : (is_k ? h - p.Hq : h - p.Hq - p.Hkv);
                const int Hp = Hn / W;
                const int q = hk / Hp, hl = hk - q * Hp;
                const long long off = is_q ? p.q_off : (is_k ? p.k_off : p.v_off);
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(p.t.buf[q]) + off) +
                                     ((size_t)drow * Hp + hl) * D + sub * 8;
                *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]),
                                                            pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int old = atomicAdd(p.arrive, 1u);
        s_last = (old == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence_system();
        signal_and_wait_all(p.t, p.channel, s_epoch, p.status, p.wait_limit_ns, 6);
        *p.arrive = 0u;
        *p.epoch = s_epoch;
    }
}

// CFG-parallel combine: velocities of the branches live at `v_offset_bytes` in the data region of ranks
// cond_rank / uncond_rank / img_rank (img_rank < 0: two-branch guidance). Runs on the combine rank after the
// branch ranks have raised their flags on `channel`; reads the peers' tensors over NVLink.
struct CfgPeerParams {
    PeerTable t;
    long long v_offset_bytes;
    int cond_rank, uncond_rank, img_rank;
    const float* x;
    float* x_next;
    float* v_out;
    int rows, cols;
    float s_text, s_img, dt, renorm_min;
    int renorm;
    unsigned int* epoch;
    unsigned int* arrive;
    int channel;
    int wait_peers;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
};
__device__ __forceinline__ void cfg_publish_epoch(const CfgPeerParams& p, unsigned int e) {
    // the last CTA of the launch publishes the consumed epoch (every CTA has read the old value by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int old = atomicAdd(p.arrive, 1u);
        if (old == gridDim.x - 1) {
            *p.arrive = 0u;
            if (p.wait_peers) *p.epoch = e;
        }
    }
}
constexpr int CFG_STAGE_MAX_COLS = 8192;      // 32 KB of shared memory for the staged row
__global__ void __launch_bounds__(128) cfg_combine_peer_kernel(const __grid_constant__ CfgPeerParams p) {
    __shared__ float red[32];
    __shared__ int s_ok;
    __shared__ unsigned int s_e;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        s_ok = 1;
        s_e = *p.epoch + 1;
        if (p.wait_peers) {
            const unsigned int e = s_e;
            const int rk[3] = {p.cond_rank, p.uncond_rank, p.img_rank};
            for (int i = 0; i < 3; ++i) {
                if (rk[i] < 0 || rk[i] == p.t.rank) continue;
                if (!wait_flag(p.t.flags[p.t.rank] + (size_t)p.channel * MAX_RANKS + rk[i], e, p.wait_limit_ns)) {
                    report_status(p.status, KID_CFG, 1, rk[i], p.channel);
                    s_ok = 0;
                }
            }
        }
    }
    __syncthreads();
    if (!s_ok) { cfg_publish_epoch(p, s_e); return; }
    const int r = blockIdx.x;
    const size_t base = (size_t)r * p.cols;
    const float* vc = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.t.buf[p.cond_rank]) + p.v_offset_bytes);
    const float* vu = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.t.buf[p.uncond_rank]) + p.v_offset_bytes);
    const float* vi = p.img_rank >= 0
        ? reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.t.buf[p.img_rank]) + p.v_offset_bytes) : nullptr;
    // One pass over the peers' rows: 16-byte loads (a peer load is an NVLink round trip; the first version read
    // every value twice with 4-byte loads and reached 0.27 of the link rate), the combined velocity parked in
    // shared memory for the second pass that applies the row's renormalisation.
    extern __shared__ float vrow[];          // [cols] when it fits (host passes the size), else the row is re-read
    const bool staged = p.cols <= CFG_STAGE_MAX_COLS;
    const bool vec = (p.cols & 3) == 0 && (p.v_offset_bytes & 15) == 0;
    float nc = 0.f, nv = 0.f;
    if (vec) {
        const float4* vc4 = reinterpret_cast<const float4*>(vc + base);
        const float4* vu4 = reinterpret_cast<const float4*>(vu + base);
        const float4* vi4 = vi ? reinterpret_cast<const float4*>(vi + base) : nullptr;
        for (int i = threadIdx.x; i < (p.cols >> 2); i += blockDim.x) {
            const float4 c = vc4[i], u = vu4[i];
            float4 v = make_float4(u.x + p.s_text * (c.x - u.x), u.y + p.s_text * (c.y - u.y),
                                   u.z + p.s_text * (c.z - u.z), u.w + p.s_text * (c.w - u.w));
            if (vi4) {
                const float4 im = vi4[i];
                v = make_float4(im.x + p.s_img * (v.x - im.x), im.y + p.s_img * (v.y - im.y),
                                im.z + p.s_img * (v.z - im.z), im.w + p.s_img * (v.w - im.w));
            }
            nc += c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w;
            nv += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            if (staged) reinterpret_cast<float4*>(vrow)[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
            const float c = vc[base + i], u = vu[base + i];
            float v = u + p.s_text * (c - u);
            if (vi) { const float im = vi[base + i]; v = im + p.s_img * (v - im); }
            nc += c * c; nv += v * v;
            if (staged) vrow[i] = v;
        }
    }
    float scale = 1.f;
    if (p.renorm) {
        nc = warp_sum(nc); nv = warp_sum(nv);
        if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = nc; red[4 + (threadIdx.x >> 5)] = nv; }
        __syncthreads();
        nc = red[0] + red[1] + red[2] + red[3];
        nv = red[4] + red[5] + red[6] + red[7];
        scale = fminf(fmaxf(sqrtf(nc) / (sqrtf(nv) + 1e-8f), p.renorm_min), 1.f);
    }
    // each thread re-reads exactly the elements it wrote, so no barrier is needed for the staged row
    if (staged && vec) {
        for (int i = threadIdx.x; i < (p.cols >> 2); i += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(vrow)[i];
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
            if (p.v_out) reinterpret_cast<float4*>(p.v_out + base)[i] = v;
            if (p.x_next) {
                const float4 x = reinterpret_cast<const float4*>(p.x + base)[i];
                reinterpret_cast<float4*>(p.x_next + base)[i] =
                    make_float4(x.x + p.dt * v.x, x.y + p.dt * v.y, x.z + p.dt * v.z, x.w + p.dt * v.w);
            }
        }
    } else {
        for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
            float v;
            if (staged) {
                v = vrow[i];
            } else {
                const float c = vc[base + i], u = vu[base + i];
                v = u + p.s_text * (c - u);
                if (vi) { const float im = vi[base + i]; v = im + p.s_img * (v - im); }
            }
            v *= scale;
            if (p.v_out) p.v_out[base + i] = v;
            if (p.x_next) p.x_next[base + i] = p.x[base + i] + p.dt * v;
        }
    }
    cfg_publish_epoch(p, s_e);
}

// Raise this rank's flag on `channel` at rank `dst` (after earlier kernels' stores to the heap): one thread.
struct SignalParams { PeerTable t; unsigned int* epoch; int channel; int dst; int bump_epoch; };
__global__ void peer_signal_kernel(const __grid_constant__ SignalParams p) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        const unsigned int e = *p.epoch + 1;
        __threadfence_system();
        st_release_sys(p.t.flags[p.dst] + (size_t)p.channel * MAX_RANKS + p.t.rank, e);
        if (p.bump_epoch) *p.epoch = e;
    }
}

}  // namespace mstar

#include "comm_host.inc"
