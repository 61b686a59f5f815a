// Mixture-of-experts routing and data movement around the grouped tcgen05 GEMM:
//   moe_topk         router logits -> softmax -> top-k (+ renormalisation) per token
//   moe_align        (token, k) pairs -> expert-sorted, block-padded order: sorted_pair[], block_expert[],
//                    num_blocks, inverse map pos_of_pair[], and per-row routing weight in sorted order
//   moe_permute      gather hidden rows into the sorted buffer (pads are zero rows); with a peer pointer table
//                    this is the expert-parallel DISPATCH: rows are stored straight into the owner GPU's buffer
//   moe_unpermute    out[t] = sum_j w[t,j] * y[pos(t,j)]  (or plain sum when the weights were applied already)
//
// Reference counterparts: moe_align_block_size.cu kernels (mstar/utils/fused_moe/csrc/moe_align_block_size.cu:
// 30-282), TopKRouter softmax/top-k/renorm (mstar/model/components/moe.py:85-140), Triton act_and_mul /
// moe_sum_reduce (mstar/utils/fused_moe/kernels.py:244-393). Expert parallelism does not exist in the reference.
#include "common.cuh"
#include "host_common.h"

namespace mstar {

// one warp per token; E <= 256 (8 values per lane)
__global__ void __launch_bounds__(256) moe_topk_kernel(const float* logits, int T, int E, int top_k, int renorm,
                                                       int* topk_ids, float* topk_w) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T) return;
    const float* row = logits + (size_t)warp * E;
    float v[8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? row[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f;
        sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    float wsum = 0.f;
    float picked_w = 0.f;
    int picked_e = -1;
    for (int k = 0; k < top_k; ++k) {
        float best = -1.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            if (v[i] > best || (v[i] == best && e < be)) { best = v[i]; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
        }
        if ((be & 31) == lane) v[be >> 5] = -1.f;     // remove the winner
        if (lane == k) { picked_w = best * inv; picked_e = be; }
        wsum += best * inv;
    }
    if (lane < top_k) {
        topk_ids[(size_t)warp * top_k + lane] = picked_e;
        topk_w[(size_t)warp * top_k + lane] = renorm ? picked_w / wsum : picked_w;
    }
}

// single CTA: counts -> block-padded offsets -> scatter. n_pairs = T * top_k.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* topk_ids, const float* topk_w, int n_pairs, int E,
                                                         int block_rows, int capacity_rows, int expert_begin,
                                                         int expert_end, int* sorted_pair, float* sorted_w,
                                                         int* pos_of_pair, int* block_expert, int* num_blocks) {
    __shared__ int cnt[1025];
    __shared__ int off[1025];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = topk_ids[i];
        if (e >= expert_begin && e < expert_end) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, nb = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = o;
            const int blocks = (cnt[e] + block_rows - 1) / block_rows;
            for (int b = 0; b < blocks && nb < capacity_rows / block_rows; ++b) block_expert[nb++] = e - expert_begin;
            o += blocks * block_rows;
        }
        off[E] = o;
        *num_blocks = nb;
    }
    __syncthreads();
    const int total = off[E] < capacity_rows ? off[E] : capacity_rows;
    for (int i = threadIdx.x; i < capacity_rows; i += blockDim.x) {
        if (i < total || true) { sorted_pair[i] = -1; sorted_w[i] = 0.f; }
    }
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;     // reuse as cursors
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
        const int e = topk_ids[i];
        int pos = -1;
        if (e >= expert_begin && e < expert_end) {
            pos = off[e] + atomicAdd(&cnt[e], 1);
            if (pos < capacity_rows) {
                sorted_pair[pos] = i;
                sorted_w[pos] = topk_w[i];
            } else {
                pos = -1;
            }
        }
        pos_of_pair[i] = pos;
    }
}

// dst[pos] = src[pair / top_k] for every sorted position; pads (pair < 0) become zero rows.
// dst_rows: optional per-position destination pointers (dispatch to peers); else dst + pos * H.
__global__ void moe_permute_kernel(const __nv_bfloat16* src, const int* sorted_pair, int capacity_rows, int H,
                                   int top_k, __nv_bfloat16* dst, void* const* dst_rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int pos = blockIdx.x;
    if (pos >= capacity_rows) return;
    const int pair = sorted_pair[pos];
    uint4* d = dst_rows ? reinterpret_cast<uint4*>(dst_rows[pos]) : reinterpret_cast<uint4*>(dst + (size_t)pos * H);
    if (d == nullptr) return;
    const uint4* s = pair >= 0 ? reinterpret_cast<const uint4*>(src + (size_t)(pair / top_k) * H) : nullptr;
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) d[v] = s ? s[v] : make_uint4(0, 0, 0, 0);
}

// out[t] = sum_j (w ? w[t,j] : 1) * y[pos_of_pair[t*k+j]]   (pairs with pos < 0 contribute nothing)
__global__ void moe_unpermute_kernel(const __nv_bfloat16* y, const int* pos_of_pair, const float* w, int T, int top_k,
                                     int H, long long ld_y, __nv_bfloat16* out, const __nv_bfloat16* add) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= T) return;
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int k = 0; k < top_k; ++k) {
            const int pos = pos_of_pair[(size_t)t * top_k + k];
            if (pos < 0) continue;
            const float wk = w ? w[(size_t)t * top_k + k] : 1.f;
            const uint4 x = reinterpret_cast<const uint4*>(y + (size_t)pos * ld_y)[v];
            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = unpack_bf16x2(xw[j]);
                acc[2 * j] += wk * f.x; acc[2 * j + 1] += wk * f.y;
            }
        }
        if (add) {
            const uint4 x = reinterpret_cast<const uint4*>(add + (size_t)t * H)[v];
            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = unpack_bf16x2(xw[j]);
                acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
            }
        }
        reinterpret_cast<uint4*>(out + (size_t)t * H)[v] =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                       pack_bf16x2(acc[6], acc[7]));
    }
}

}  // namespace mstar

using namespace mstar;

MSTAR_API int mstar_moe_topk(const float* logits, int T, int E, int top_k, int renorm, int* topk_ids, float* topk_w,
                             void* stream_) {
    if (T <= 0) return 0;
    if (E > 256 || top_k > 32 || top_k > E) return set_error("moe_topk: needs E <= 256 and top_k <= min(32, E)", cudaSuccess);
    cudaError_t e = launch_pdl(moe_topk_kernel, dim3((T * 32 + 255) / 256), dim3(256), 0, (cudaStream_t)stream_, logits,
                               T, E, top_k, renorm, topk_ids, topk_w);
    return e == cudaSuccess ? 0 : set_error("moe_topk launch", e);
}

MSTAR_API int mstar_moe_align(const int* topk_ids, const float* topk_w, int n_pairs, int E, int block_rows,
                              int capacity_rows, int expert_begin, int expert_end, int* sorted_pair, float* sorted_w,
                              int* pos_of_pair, int* block_expert, int* num_blocks, void* stream_) {
    if (E > 1024) return set_error("moe_align: E > 1024", cudaSuccess);
    cudaError_t e = launch_pdl(moe_align_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream_, topk_ids, topk_w,
                               n_pairs, E, block_rows, capacity_rows, expert_begin, expert_end, sorted_pair, sorted_w,
                               pos_of_pair, block_expert, num_blocks);
    return e == cudaSuccess ? 0 : set_error("moe_align launch", e);
}

MSTAR_API int mstar_moe_permute(const void* src, const int* sorted_pair, int capacity_rows, int H, int top_k, void* dst,
                                void* const* dst_rows, void* stream_) {
    if (capacity_rows <= 0) return 0;
    if (H % 8) return set_error("moe_permute: H must be a multiple of 8", cudaSuccess);
    cudaError_t e = launch_pdl(moe_permute_kernel, dim3(capacity_rows), dim3(128), 0, (cudaStream_t)stream_,
                               (const __nv_bfloat16*)src, sorted_pair, capacity_rows, H, top_k, (__nv_bfloat16*)dst, dst_rows);
    return e == cudaSuccess ? 0 : set_error("moe_permute launch", e);
}

MSTAR_API int mstar_moe_unpermute(const void* y, const int* pos_of_pair, const float* w, int T, int top_k, int H,
                                  long long ld_y, void* out, const void* add, void* stream_) {
    if (T <= 0) return 0;
    if (H % 8) return set_error("moe_unpermute: H must be a multiple of 8", cudaSuccess);
    cudaError_t e = launch_pdl(moe_unpermute_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream_,
                               (const __nv_bfloat16*)y, pos_of_pair, w, T, top_k, H, ld_y, (__nv_bfloat16*)out,
                               (const __nv_bfloat16*)add);
    return e == cudaSuccess ? 0 : set_error("moe_unpermute launch", e);
}
