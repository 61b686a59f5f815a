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

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
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

}  // namespace mstar
