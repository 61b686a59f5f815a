// Token sampling in one kernel per step: repetition penalty over the seen-token mask, temperature, top-k,
// top-p, one Philox draw per row, and the seen-mask update. One CTA per row, vocabulary up to a few 100k.
//
// Selection of the nucleus without a sort: three 8-bit radix passes over the float bit pattern of the
// probabilities (monotone for positive floats) give a 24-bit threshold key; the kept set is
// {p : key(p) >= threshold}, the smallest such set whose mass reaches top_p and whose size respects top_k
// (ties at the threshold are kept). The draw walks the kept probabilities in vocabulary order.
//
// Greedy rows (temperature == 0) take the first index of the maximum.
//
// Reference counterparts: Triton _fused_sampling_prep_kernel (mstar/utils/sampling.py:32-161) followed by
// FlashInfer top_p / top_k_top_p sampling from probs (mstar/utils/sampling.py:581-682).
#include "common.cuh"
#include "host_common.h"

namespace mstar {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t* out) {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct SampleParams {
    const void* logits;          // [B, ld] bf16 or fp32
    long long ld;
    int is_f32;
    int B, V;
    const float* temperature;    // [B]
    const int* top_k;            // [B] (<= 0: off)
    const float* top_p;          // [B] (>= 1: off)
    const float* rep_penalty;    // [B] (1: off)
    const unsigned long long* seed;    // [B]
    const unsigned long long* offset;  // [B] draw counter (step index)
    unsigned char* seen;         // [B, V] or null
    const int* row_slot;         // [B] row of seen/params for each logits row, or null (identity)
    long long* out;              // [B]
    float* out_prob;             // [B] probability of the sampled token (optional)
    float* u_override;           // [B] uniform draws supplied by the caller (tests), or null
};

constexpr int SP_NT = 1024;

template <bool F32>
__device__ __forceinline__ float load_logit(const void* base, long long i) {
    if constexpr (F32) return reinterpret_cast<const float*>(base)[i];
    else return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}

template <bool F32>
__global__ void __launch_bounds__(SP_NT) sample_kernel(const SampleParams p) {
    extern __shared__ unsigned long long sp_dyn[];                 // per-warp radix histograms (fixed-point mass)
    unsigned long long* hist_mass = sp_dyn;                                        // [32 warps][256]
    unsigned int* hist_cnt = reinterpret_cast<unsigned int*>(sp_dyn + (SP_NT / 32) * 256);   // [32 warps][256]
    __shared__ float merged_mass[256];
    __shared__ int merged_cnt[256];
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    __shared__ float sh_f[4];
    __shared__ int sh_i[4];
    const int row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const int slot = p.row_slot ? p.row_slot[row] : row;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const void* lg = reinterpret_cast<const char*>(p.logits) + (size_t)row * p.ld * (F32 ? 4 : 2);
    const float temp = p.temperature[slot];
    const float pen = p.rep_penalty ? p.rep_penalty[slot] : 1.0f;
    const unsigned char* seen = p.seen ? p.seen + (size_t)slot * p.V : nullptr;
    const bool greedy = temp <= 0.f;
    const float inv_t = greedy ? 1.f : 1.f / temp;

    auto logit_at = [&](int i) -> float {
        float x = load_logit<F32>(lg, i);
        if (seen && pen != 1.0f && seen[i]) x = x > 0.f ? x / pen : x * pen;
        return x * inv_t;
    };

    // ---- pass 1: max (and argmax for greedy rows) ----
    float mx = -INFINITY;
    int amx = 0x7fffffff;
    for (int i = tid; i < p.V; i += SP_NT) {
        const float x = logit_at(i);
        if (x > mx) { mx = x; amx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oi = __shfl_xor_sync(0xffffffffu, amx, o);
        if (om > mx || (om == mx && oi < amx)) { mx = om; amx = oi; }
    }
    if (lane == 0) { red_f[warp] = mx; red_i[warp] = amx; }
    __syncthreads();
    if (warp == 0) {
        mx = red_f[lane]; amx = red_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, mx, o);
            const int oi = __shfl_xor_sync(0xffffffffu, amx, o);
            if (om > mx || (om == mx && oi < amx)) { mx = om; amx = oi; }
        }
        if (lane == 0) { sh_f[0] = mx; sh_i[0] = amx; }
    }
    __syncthreads();
    mx = sh_f[0];
    if (greedy) {
        if (tid == 0) {
            const int tok = sh_i[0];
            p.out[row] = tok;
            if (p.out_prob) p.out_prob[row] = 1.0f;
            if (p.seen) p.seen[(size_t)slot * p.V + tok] = 1;
        }
        return;
    }

    // ---- pass 2: partition function ----
    float z = 0.f;
    for (int i = tid; i < p.V; i += SP_NT) z += __expf(logit_at(i) - mx);
    z = warp_sum(z);
    if (lane == 0) red_f[warp] = z;
    __syncthreads();
    if (warp == 0) {
        float t = red_f[lane];
        t = warp_sum(t);
        if (lane == 0) sh_f[1] = t;
    }
    __syncthreads();
    z = sh_f[1];
    const float top_p = p.top_p ? p.top_p[slot] : 1.0f;
    int top_k = p.top_k ? p.top_k[slot] : 0;
    if (top_k <= 0 || top_k > p.V) top_k = p.V;
    const bool filter = (top_p < 1.0f) || (top_k < p.V);
    uint32_t thr_key = 0;          // keep keys >= thr_key
    if (filter) {
        // Three radix levels of 8 bits over the 24-bit key. Every warp owns a private 256-bin histogram
        // (fixed-point mass, 2^-24 units, and count); lanes that hit the same bin are merged with
        // match_any + reduce_add before ONE lane updates the bin, so no atomics and no contention, whatever
        // the shape of the distribution.
        const float need = top_p * z;
        unsigned long long* wmass = hist_mass + warp * 256;
        unsigned int* wcnt = hist_cnt + warp * 256;
        uint32_t prefix = 0;            // key bits decided so far (aligned to the top)
        float acc_mass = 0.f;           // mass / count of keys strictly above the undecided range
        int acc_cnt = 0;
        const int iters = (p.V + SP_NT - 1) / SP_NT;
#pragma unroll 1
        for (int level = 0; level < 3; ++level) {
            const int shift = 16 - 8 * level;
            for (int i = lane; i < 256; i += 32) { wmass[i] = 0ull; wcnt[i] = 0u; }
            __syncwarp();
            for (int it = 0; it < iters; ++it) {
                const int i = tid + it * SP_NT;
                uint32_t bin = 0xffffffffu;
                unsigned int fx = 0;
                if (i < p.V) {
                    const float e = __expf(logit_at(i) - mx);
                    const uint32_t key = __float_as_uint(e) >> 8;
                    const bool in_range = level == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8));
                    if (in_range) { bin = (key >> shift) & 0xffu; fx = (unsigned int)(e * 16777216.0f); }
                }
                const unsigned int peers = __match_any_sync(0xffffffffu, bin);
                const unsigned int sum = __reduce_add_sync(peers, fx);
                if (bin != 0xffffffffu && lane == __ffs(peers) - 1) {
                    wmass[bin] += sum;
                    wcnt[bin] += __popc(peers);
                }
                __syncwarp();
            }
            __syncthreads();
            // merge the 32 warp histograms: thread t < 256 owns bin t (results into warp 0's arrays)
            if (tid < 256) {
                unsigned long long m = 0ull; unsigned int c = 0u;
                for (int w = 0; w < SP_NT / 32; ++w) { m += hist_mass[w * 256 + tid]; c += hist_cnt[w * 256 + tid]; }
                merged_mass[tid] = (float)m * (1.0f / 16777216.0f);
                merged_cnt[tid] = (int)c;
            }
            __syncthreads();
            if (tid == 0) {
                float acc = acc_mass; int cnt = acc_cnt; int bsel = 255;
                for (; bsel >= 0; --bsel) {
                    const float mb = merged_mass[bsel]; const int cb = merged_cnt[bsel];
                    if (cb == 0) continue;
                    if (acc + mb >= need || cnt + cb >= top_k) break;     // the threshold lies inside this bin
                    acc += mb; cnt += cb;
                }
                if (bsel < 0) bsel = 0;
                sh_i[1] = bsel; sh_f[2] = acc; sh_i[2] = cnt;
            }
            __syncthreads();
            prefix |= (uint32_t)sh_i[1] << shift;
            acc_mass = sh_f[2];
            acc_cnt = sh_i[2];
            __syncthreads();
        }
        thr_key = prefix;
    }

    // ---- draw ----
    float u;
    if (p.u_override) u = p.u_override[row];
    else {
        uint32_t r[4];
        const unsigned long long sd = p.seed[slot], off = p.offset ? p.offset[slot] : 0ull;
        philox4x32_10((uint32_t)off, (uint32_t)(off >> 32), 0u, 0u, (uint32_t)sd, (uint32_t)(sd >> 32), r);
        u = ((r[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    }
    // mass of the kept set, summed in walk order
    const int chunk = (p.V + SP_NT - 1) / SP_NT;
    const int i0 = tid * chunk, i1 = min(p.V, i0 + chunk);
    float local = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float e = __expf(logit_at(i) - mx);
        if ((__float_as_uint(e) >> 8) >= thr_key) local += e;
    }
    // block exclusive scan of `local`
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) red_f[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = red_f[lane];
        float wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        red_f[lane] = wi - w;            // exclusive warp offsets
        if (lane == 31) sh_f[0] = wi;    // total
    }
    __syncthreads();
    const float total = sh_f[0];
    const float excl = red_f[warp] + incl - local;
    const float target = u * total;
    if (tid == 0) sh_i[0] = -1;
    __syncthreads();
    if (local > 0.f && target >= excl && target < excl + local) {
        float acc = excl;
        int pick = -1, last = -1;
        for (int i = i0; i < i1; ++i) {
            const float e = __expf(logit_at(i) - mx);
            if ((__float_as_uint(e) >> 8) >= thr_key) {
                last = i;
                acc += e;
                if (acc > target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last;
        atomicMax(&sh_i[0], pick);
    }
    __syncthreads();
    if (tid == 0) {
        int tok = sh_i[0];
        if (tok < 0) tok = sh_i[0] = -2;   // rounding left the target outside every chunk: fall back below
    }
    __syncthreads();
    if (sh_i[0] == -2) {
        // fallback: last kept index (target == total up to rounding)
        int last = -1;
        for (int i = i0; i < i1; ++i) {
            const float e = __expf(logit_at(i) - mx);
            if ((__float_as_uint(e) >> 8) >= thr_key) last = i;
        }
        __syncthreads();
        if (tid == 0) sh_i[0] = -1;
        __syncthreads();
        if (last >= 0) atomicMax(&sh_i[0], last);
        __syncthreads();
    }
    if (tid == 0) {
        int tok = sh_i[0];
        if (tok < 0) tok = 0;
        p.out[row] = tok;
        if (p.out_prob) p.out_prob[row] = __expf(logit_at(tok) - mx) / total;
        if (p.seen) p.seen[(size_t)slot * p.V + tok] = 1;
    }
}

}  // namespace mstar

using namespace mstar;

MSTAR_API int mstar_sample(const void* logits, long long ld, int is_f32, int B, int V, const float* temperature,
                           const int* top_k, const float* top_p, const float* rep_penalty,
                           const unsigned long long* seed, const unsigned long long* offset, unsigned char* seen,
                           const int* row_slot, long long* out, float* out_prob, float* u_override, void* stream_) {
    if (B <= 0) return 0;
    SampleParams p{logits, ld, is_f32, B, V, temperature, top_k, top_p, rep_penalty, seed, offset, seen, row_slot,
                   out, out_prob, u_override};
    cudaStream_t s = (cudaStream_t)stream_;
    constexpr int smem = (SP_NT / 32) * 256 * 12;
    static bool configured = false;
    if (!configured) {
        cudaError_t e1 = cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaError_t e2 = cudaFuncSetAttribute(sample_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e1 != cudaSuccess || e2 != cudaSuccess) return set_error("sample: cudaFuncSetAttribute failed", e1 != cudaSuccess ? e1 : e2);
        configured = true;
    }
    cudaError_t e = is_f32 ? launch_pdl(sample_kernel<true>, dim3(B), dim3(SP_NT), smem, s, p)
                           : launch_pdl(sample_kernel<false>, dim3(B), dim3(SP_NT), smem, s, p);
    return e == cudaSuccess ? 0 : set_error("sample launch", e);
}
