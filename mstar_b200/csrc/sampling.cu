// Token sampling in one kernel per step: repetition penalty over the seen-token mask, temperature, top-k,
// top-p, one Philox draw per row, and the seen-mask update. One CTA per row, vocabulary up to a few 100k.
//
// Selection of the nucleus without a sort: two 4096-bin histograms over the float bit pattern of the
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
constexpr int SP_BINS = 4096;

template <bool F32>
__device__ __forceinline__ float load_logit(const void* base, long long i) {
    if constexpr (F32) return reinterpret_cast<const float*>(base)[i];
    else return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}

template <bool F32>
__global__ void __launch_bounds__(SP_NT) sample_kernel(const SampleParams p) {
    __shared__ float hist_mass[SP_BINS];
    __shared__ int hist_cnt[SP_BINS];
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

    // ---- pass 2: partition function + first-level histogram of e = exp(x - max) in (0, 1] ----
    for (int i = tid; i < SP_BINS; i += SP_NT) { hist_mass[i] = 0.f; hist_cnt[i] = 0; }
    __syncthreads();
    float z = 0.f;
    {
        // run-length aggregation: neighbouring elements often fall into the same bin (flat distributions put most
        // of the vocabulary into a handful of bins), so a thread flushes to shared memory only when the bin changes
        int cur = -1, ccnt = 0;
        float cmass = 0.f;
        for (int i = tid; i < p.V; i += SP_NT) {
            const float e = __expf(logit_at(i) - mx);
            z += e;
            const int bin = (int)((__float_as_uint(e) >> 8) >> 12);     // top 12 of a 24-bit monotone key
            if (bin != cur) {
                if (ccnt) { atomicAdd(&hist_mass[cur], cmass); atomicAdd(&hist_cnt[cur], ccnt); }
                cur = bin; cmass = 0.f; ccnt = 0;
            }
            cmass += e; ++ccnt;
        }
        if (ccnt) { atomicAdd(&hist_mass[cur], cmass); atomicAdd(&hist_cnt[cur], ccnt); }
    }
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
    float kept_mass = z;
    if (filter) {
        const float need = top_p * z;
        // walk the bins from the top: thread 0 only (4096 steps at most, usually a few hundred)
        if (tid == 0) {
            float acc = 0.f; int cnt = 0; int b = SP_BINS - 1;
            for (; b >= 0; --b) {
                const float mb = hist_mass[b]; const int cb = hist_cnt[b];
                if (cb == 0) continue;
                if (acc + mb >= need || cnt + cb >= top_k) break;
                acc += mb; cnt += cb;
            }
            if (b < 0) b = 0;
            sh_i[1] = b; sh_f[2] = acc; sh_i[2] = cnt;
        }
        __syncthreads();
        const int b1 = sh_i[1];
        const float acc1 = sh_f[2];
        const int cnt1 = sh_i[2];
        __syncthreads();
        // second level inside bin b1
        for (int i = tid; i < SP_BINS; i += SP_NT) { hist_mass[i] = 0.f; hist_cnt[i] = 0; }
        __syncthreads();
        {
            int cur = -1, ccnt = 0;
            float cmass = 0.f;
            for (int i = tid; i < p.V; i += SP_NT) {
                const float e = __expf(logit_at(i) - mx);
                const uint32_t key = __float_as_uint(e) >> 8;
                if ((int)(key >> 12) == b1) {
                    const int bin = (int)(key & 0xfff);
                    if (bin != cur) {
                        if (ccnt) { atomicAdd(&hist_mass[cur], cmass); atomicAdd(&hist_cnt[cur], ccnt); }
                        cur = bin; cmass = 0.f; ccnt = 0;
                    }
                    cmass += e; ++ccnt;
                }
            }
            if (ccnt) { atomicAdd(&hist_mass[cur], cmass); atomicAdd(&hist_cnt[cur], ccnt); }
        }
        __syncthreads();
        if (tid == 0) {
            float acc = acc1; int cnt = cnt1; int b = SP_BINS - 1;
            for (; b >= 0; --b) {
                const float mb = hist_mass[b]; const int cb = hist_cnt[b];
                if (cb == 0) continue;
                acc += mb; cnt += cb;
                if (acc >= need || cnt >= top_k) break;
            }
            if (b < 0) b = 0;
            sh_i[3] = b; sh_f[3] = acc;
        }
        __syncthreads();
        thr_key = ((uint32_t)b1 << 12) | (uint32_t)sh_i[3];
        kept_mass = sh_f[3];
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
    // kept_mass from the histograms is summed in a different order than below; recompute it in walk order
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
    (void)kept_mass;
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
    cudaError_t e = is_f32 ? launch_pdl(sample_kernel<true>, dim3(B), dim3(SP_NT), 0, s, p)
                           : launch_pdl(sample_kernel<false>, dim3(B), dim3(SP_NT), 0, s, p);
    return e == cudaSuccess ? 0 : set_error("sample launch", e);
}
