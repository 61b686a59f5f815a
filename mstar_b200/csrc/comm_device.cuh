// Device-side pieces shared by the collective kernels and the fused GEMM epilogue: the table of peer heap
// pointers, system-scope release/acquire flag accesses, and the bounded signal/wait protocol.
#pragma once
#include "common.cuh"

namespace mstar {

constexpr int MAX_RANKS = 8;

struct PeerTable {
    void* buf[MAX_RANKS];            // base of each rank's data region
    unsigned int* flags[MAX_RANKS];  // base of each rank's flag region: [channel][MAX_RANKS]
    int world, rank;
};

// The multicast view of the same heaps (null pointers when the group has no NVLS multicast object: kernels then
// take their plain peer load / store path).
struct McastTable {
    char* data;                      // multicast address of the data region (offset 0 = offset 0 of every heap)
    unsigned int* flags;             // multicast address of the flag region
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ---------------------------------------------------------------------------------------------
// NVLS: loads, stores and reductions through a MULTICAST address. The symmetric heap of every rank is bound to one
// multicast object; an access to offset X of the multicast mapping reaches offset X of every rank's heap inside the
// NVSwitch: a load-reduce returns the sum of all ranks' values with one request, a store or reduction lands on every
// rank. These are not TMA operations and use no cluster multicast.
// ---------------------------------------------------------------------------------------------
// Sum over all ranks of 8 bf16 values at the same heap offset, accumulated in fp32 inside the switch.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
// Store 16 bytes to the same heap offset on every rank.
__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}
// Release-store of one flag word on every rank (this rank's own copy included).
__device__ __forceinline__ void multimem_st_release_u32(unsigned int* mc, unsigned int v) {
    asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// Wait until *flag >= target (epochs only grow; wrap-around after 2^31 steps is handled by the signed compare).
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int target, unsigned long long limit_ns) {
    if ((int)(ld_acquire_sys(flag) - target) >= 0) return true;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int it = 0;
    while ((int)(ld_acquire_sys(flag) - target) < 0) {
        if ((++it & 0xffu) == 0u) {
            if (globaltimer_ns() - t0 > limit_ns) return false;
            __nanosleep(64);
        }
    }
    return true;
}

// Signal every rank (one multicast store when available, else one store per peer) on `channel` with `epoch`.
__device__ __forceinline__ void signal_all(const PeerTable& t, const McastTable& mc, int channel, unsigned int epoch) {
    if (mc.flags != nullptr) {
        multimem_st_release_u32(mc.flags + (size_t)channel * MAX_RANKS + t.rank, epoch);
    } else {
        for (int p = 0; p < t.world; ++p)
            if (p != t.rank) st_release_sys(t.flags[p] + (size_t)channel * MAX_RANKS + t.rank, epoch);
    }
}
// Wait (bounded) until every peer has signalled `epoch` on `channel`.
__device__ __forceinline__ bool wait_all(const PeerTable& t, int channel, unsigned int epoch, KernelStatus* status,
                                         unsigned long long limit_ns, int phase) {
    bool ok = true;
    for (int p = 0; p < t.world; ++p) {
        if (p == t.rank) continue;
        if (!wait_flag(t.flags[t.rank] + (size_t)channel * MAX_RANKS + p, epoch, limit_ns)) {
            report_status(status, KID_COMM, phase, p, channel);
            ok = false;
        }
    }
    return ok;
}

// Signal every peer on `channel` with `epoch`, then wait for every peer's signal on the same channel.
// Called by ONE thread of a CTA after the CTA's data stores were fenced (__threadfence_system by the writers).
__device__ __forceinline__ bool signal_and_wait_all(const PeerTable& t, int channel, unsigned int epoch,
                                                    KernelStatus* status, unsigned long long limit_ns, int phase) {
    for (int p = 0; p < t.world; ++p)
        if (p != t.rank) st_release_sys(t.flags[p] + (size_t)channel * MAX_RANKS + t.rank, epoch);
    bool ok = true;
    for (int p = 0; p < t.world; ++p) {
        if (p == t.rank) continue;
        if (!wait_flag(t.flags[t.rank] + (size_t)channel * MAX_RANKS + p, epoch, limit_ns)) {
            report_status(status, KID_COMM, phase, p, channel);
            ok = false;
        }
    }
    return ok;
}

// ---- bf16 x 8 vector helpers and the plain peer-load / peer-store share reduction ----
__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4 v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
    return make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
}


// Sum vectors v, v + blockDim, ... of [.., b) over the ranks' regions and store the sum to every rank; UP vectors per
// thread and trip, all of their WW loads in flight together. Returns the first vector left for the tail loop.
template <int WW, int UP>
__device__ __forceinline__ long long p2p_share(const PeerTable& t, long long off, long long v, long long b) {
    const int W = t.world;
    for (; v + (long long)(UP - 1) * blockDim.x < b; v += (long long)UP * blockDim.x) {
        uint4 raw[UP][WW];
#pragma unroll
        for (int u = 0; u < UP; ++u)
#pragma unroll
            for (int q = 0; q < WW; ++q)
                if (q < W)
                    raw[u][q] = __ldcg(reinterpret_cast<const uint4*>(
                        reinterpret_cast<const char*>(t.buf[q]) + off + (v + (long long)u * blockDim.x) * 16));
#pragma unroll
        for (int u = 0; u < UP; ++u) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
            for (int q = 0; q < WW; ++q)
                if (q < W) add_bf16x8(acc, raw[u][q]);
            const uint4 o = pack8(acc);
#pragma unroll
            for (int q = 0; q < WW; ++q)
                if (q < W)
                    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.buf[q]) + off +
                                              (v + (long long)u * blockDim.x) * 16) = o;
        }
    }
    return v;
}


}  // namespace mstar
