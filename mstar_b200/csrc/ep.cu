// Expert-parallel dispatch / combine over the symmetric heap. Every rank of the EP group owns E / P whole experts.
//   dispatch : each (token, k) pair's hidden row is stored straight into the owner rank's receive buffer (peer
//              store over NVLink) together with {local expert, pair index, routing weight}; per-destination
//              counts are published once all rows are out.
//   prepare  : the owner turns what it received into the inputs of the grouped GEMM (flat expert ids, weights)
//              and a per-row table of destination pointers into the SOURCE ranks' combine buffers.
//   combine  : is the epilogue of the second grouped GEMM (row_dst / row_scale of csrc/gemm_tcgen05.cu): each
//              output row, scaled by its routing weight, is stored straight into its source rank's
//              [T, top_k, H] combine buffer; the source sums over k.
// The reference has no expert parallelism (EP was stripped from its vendored kernels,
// mstar/utils/fused_moe/kernels.py:4-7); this path serves the EP8 configuration.
#include "common.cuh"
#include "host_common.h"
#include "comm_device.cuh"

namespace mstar {

struct EpMeta { int e_local; int pair; float weight; int pad; };

struct EpDispatchParams {
    PeerTable t;
    const __nv_bfloat16* x;       // [T, H]
    const int* topk_ids;          // [T * top_k] global expert ids
    const float* topk_w;
    int n_pairs, top_k, H, E_local, cap;      // cap: receive slots per source rank
    long long recv_x_off, recv_meta_off;      // byte offsets inside every rank's heap
    int* send_counters;           // local [world], zero on entry
};

__global__ void __launch_bounds__(128) ep_dispatch_kernel(const __grid_constant__ EpDispatchParams p) {
    __shared__ int s_dst, s_slot;
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    if (i >= p.n_pairs) return;
    if (threadIdx.x == 0) {
        const int e = p.topk_ids[i];
        s_dst = e / p.E_local;
        s_slot = atomicAdd(&p.send_counters[s_dst], 1);
    }
    __syncthreads();
    const int dst = s_dst, slot = s_slot;
    if (slot >= p.cap) return;   // cannot happen when cap >= T * top_k
    char* base = reinterpret_cast<char*>(p.t.buf[dst]);
    const size_t row = (size_t)p.t.rank * p.cap + slot;
    uint4* d = reinterpret_cast<uint4*>(base + p.recv_x_off + row * p.H * 2);
    const uint4* s = reinterpret_cast<const uint4*>(p.x + (size_t)(i / p.top_k) * p.H);
    for (int v = threadIdx.x; v < (p.H >> 3); v += blockDim.x) d[v] = s[v];
    if (threadIdx.x == 0) {
        EpMeta m{p.topk_ids[i] - dst * p.E_local, i, p.topk_w[i], 0};
        reinterpret_cast<EpMeta*>(base + p.recv_meta_off)[row] = m;
    }
}

// one block: publish how many rows this rank sent to every peer, reset the counters
__global__ void ep_publish_counts_kernel(PeerTable t, int* send_counters, long long recv_count_off) {
    pdl_launch_dependents();
    pdl_wait();
    const int d = threadIdx.x;
    if (d < t.world) {
        reinterpret_cast<int*>(reinterpret_cast<char*>(t.buf[d]) + recv_count_off)[t.rank] = send_counters[d];
        send_counters[d] = 0;
    }
    __threadfence_system();
}

struct EpPrepareParams {
    PeerTable t;
    int cap, H, top_k;
    long long recv_meta_off, recv_count_off, combine_off;
    int* ids_flat;        // [world * cap]
    float* w_flat;
    void** dst_flat;      // [world * cap] destination row pointers (source ranks' combine buffers)
};
__global__ void ep_prepare_kernel(const __grid_constant__ EpPrepareParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.t.world * p.cap) return;
    const int src = i / p.cap, slot = i - src * p.cap;
    const char* mine = reinterpret_cast<const char*>(p.t.buf[p.t.rank]);
    const int n = reinterpret_cast<const int*>(mine + p.recv_count_off)[src];
    if (slot < n) {
        const EpMeta m = reinterpret_cast<const EpMeta*>(mine + p.recv_meta_off)[i];
        p.ids_flat[i] = m.e_local;
        p.w_flat[i] = m.weight;
        p.dst_flat[i] = reinterpret_cast<char*>(p.t.buf[src]) + p.combine_off + (size_t)m.pair * p.H * 2;
    } else {
        p.ids_flat[i] = -1;
        p.w_flat[i] = 0.f;
        p.dst_flat[i] = nullptr;
    }
}

__global__ void gather_ptrs_kernel(void* const* table, const int* index, int n, void** out) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = index[i] >= 0 ? table[index[i]] : nullptr;
}

}  // namespace mstar

using namespace mstar;

static int ep_table(PeerTable* t, void* const* bufs, void* const* flags, int world, int rank) {
    if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return set_error("ep: bad group", cudaSuccess);
    for (int i = 0; i < MAX_RANKS; ++i) {
        t->buf[i] = i < world ? bufs[i] : nullptr;
        t->flags[i] = i < world ? reinterpret_cast<unsigned int*>(flags[i]) : nullptr;
    }
    t->world = world; t->rank = rank;
    return 0;
}

MSTAR_API int mstar_ep_dispatch(void* const* bufs, void* const* flags, int world, int rank, const void* x,
                                const int* topk_ids, const float* topk_w, int n_pairs, int top_k, int H, int E_local,
                                int cap, long long recv_x_off, long long recv_meta_off, long long recv_count_off,
                                int* send_counters, void* stream_) {
    EpDispatchParams p;
    if (ep_table(&p.t, bufs, flags, world, rank)) return -1;
    if (H % 8) return set_error("ep_dispatch: H must be a multiple of 8", cudaSuccess);
    p.x = (const __nv_bfloat16*)x; p.topk_ids = topk_ids; p.topk_w = topk_w;
    p.n_pairs = n_pairs; p.top_k = top_k; p.H = H; p.E_local = E_local; p.cap = cap;
    p.recv_x_off = recv_x_off; p.recv_meta_off = recv_meta_off; p.send_counters = send_counters;
    cudaStream_t s = (cudaStream_t)stream_;
    if (n_pairs > 0) {
        cudaError_t e = launch_pdl(ep_dispatch_kernel, dim3(n_pairs), dim3(128), 0, s, p);
        if (e != cudaSuccess) return set_error("ep_dispatch launch", e);
    }
    cudaError_t e = launch_pdl(ep_publish_counts_kernel, dim3(1), dim3(32), 0, s, p.t, send_counters, recv_count_off);
    return e == cudaSuccess ? 0 : set_error("ep_publish_counts launch", e);
}

MSTAR_API int mstar_ep_prepare(void* const* bufs, void* const* flags, int world, int rank, int cap, int H, int top_k,
                               long long recv_meta_off, long long recv_count_off, long long combine_off, int* ids_flat,
                               float* w_flat, void** dst_flat, void* stream_) {
    EpPrepareParams p;
    if (ep_table(&p.t, bufs, flags, world, rank)) return -1;
    p.cap = cap; p.H = H; p.top_k = top_k;
    p.recv_meta_off = recv_meta_off; p.recv_count_off = recv_count_off; p.combine_off = combine_off;
    p.ids_flat = ids_flat; p.w_flat = w_flat; p.dst_flat = dst_flat;
    const int n = world * cap;
    cudaError_t e = launch_pdl(ep_prepare_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream_, p);
    return e == cudaSuccess ? 0 : set_error("ep_prepare launch", e);
}

MSTAR_API int mstar_gather_ptrs(void* const* table, const int* index, int n, void** out, void* stream_) {
    if (n <= 0) return 0;
    cudaError_t e = launch_pdl(gather_ptrs_kernel, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t)stream_, table, index, n, out);
    return e == cudaSuccess ? 0 : set_error("gather_ptrs launch", e);
}
