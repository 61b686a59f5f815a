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
#include <cooperative_groups.h>

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
    float* escratch;             // [B, V] fp32 scratch or null: exp(logit - max) of every element, written by the first
                                 // radix level and read by every later pass (the penalty, temperature and exponential
                                 // are then evaluated twice per element instead of six times)
};

constexpr int SP_NT = 256;        // threads per CTA: 64 rows x 8 CTAs fit in ONE wave at four CTAs per SM (512 threads ran two)
constexpr int SP_NW = SP_NT / 32;
constexpr int SP_CL = 8;          // CTAs per row (one thread-block cluster) for large vocabularies

template <bool F32>
__device__ __forceinline__ float load_logit(const void* base, long long i) {
    if constexpr (F32) return reinterpret_cast<const float*>(base)[i];
    else return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
}

// One thread-block CLUSTER per row: CTA c of the cluster owns the contiguous vocabulary slice
// [c * slice, (c + 1) * slice). Row-wide quantities (max, partition function, radix histograms, kept mass) are
// combined by every CTA reading its peers' partial results from distributed shared memory after a cluster barrier;
// every CTA then takes the same decision, so nothing has to be sent back.
template <bool F32>
__global__ void __launch_bounds__(SP_NT, 4) sample_kernel(const __grid_constant__ SampleParams p, const int cl) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ unsigned long long sp_dyn[];                 // per-warp radix histograms (fixed-point mass)
    unsigned long long* hist_mass = sp_dyn;                                        // [SP_NW][256]
    unsigned int* hist_cnt = reinterpret_cast<unsigned int*>(sp_dyn + SP_NW * 256);   // [SP_NW][256]
    __shared__ float merged_mass[256];      // this CTA's histogram of the current level (read by the peers)
    __shared__ int merged_cnt[256];
    __shared__ float tot_mass[256];         // cluster totals
    __shared__ int tot_cnt[256];
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    __shared__ float xf[4];                 // exchanged partials: [0] max, [1] sum, [2] kept mass
    __shared__ int xi[4];                   // [0] argmax, [1] picked token (-1: none)
    __shared__ float sh_f[4];
    __shared__ int sh_i[4];
    const int crank = cl > 1 ? (int)cluster.block_rank() : 0;
    const int row = blockIdx.x / cl;
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
    const int slice = ((p.V + cl - 1) / cl + 3) & ~3;      // multiples of four: 16-byte reads of the scratch below
    const int v0 = crank * slice, v1 = min(p.V, v0 + slice);      // this CTA's slice of the vocabulary

    auto logit_at = [&](int i) -> float {
        float x = load_logit<F32>(lg, i);
        if (seen && pen != 1.0f && seen[i]) x = x > 0.f ? x / pen : x * pen;
        return x * inv_t;
    };
    float* es = p.escratch ? p.escratch + (size_t)row * p.V : nullptr;
    auto csync = [&]() { if (cl > 1) cluster.sync(); else __syncthreads(); };
    auto peer_f = [&](float* ptr, int r) -> float { return cl > 1 ? *cluster.map_shared_rank(ptr, r) : *ptr; };
    auto peer_i = [&](int* ptr, int r) -> int { return cl > 1 ? *cluster.map_shared_rank(ptr, r) : *ptr; };

    // ---- pass 1: max (and argmax for greedy rows) ----
    float mx = -INFINITY;
    int amx = 0x7fffffff;
    for (int i = v0 + tid; i < v1; i += SP_NT) {
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
        mx = lane < SP_NW ? red_f[lane] : -INFINITY;
        amx = lane < SP_NW ? red_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, mx, o);
            const int oi = __shfl_xor_sync(0xffffffffu, amx, o);
            if (om > mx || (om == mx && oi < amx)) { mx = om; amx = oi; }
        }
        if (lane == 0) { xf[0] = mx; xi[0] = amx; }
    }
    csync();
    mx = -INFINITY; amx = 0x7fffffff;
    for (int r = 0; r < cl; ++r) {
        const float om = peer_f(&xf[0], r);
        const int oi = peer_i(&xi[0], r);
        if (om > mx || (om == mx && oi < amx)) { mx = om; amx = oi; }
    }
    if (greedy) {
        if (crank == 0 && tid == 0) {
            p.out[row] = amx;
            if (p.out_prob) p.out_prob[row] = 1.0f;
            if (p.seen) p.seen[(size_t)slot * p.V + amx] = 1;
        }
        csync();                  // peers may still be reading this CTA's shared memory
        return;
    }

    const float top_p = p.top_p ? p.top_p[slot] : 1.0f;
    int top_k = p.top_k ? p.top_k[slot] : 0;
    if (top_k <= 0 || top_k > p.V) top_k = p.V;
    const bool filter = (top_p < 1.0f) || (top_k < p.V);
    uint32_t thr_key = 0;          // keep keys >= thr_key
    float z = 0.f;
    // Three radix levels of 8 bits over the 24-bit key of e = exp(logit - max). Every warp owns a private 256-bin
    // histogram (fixed-point mass, 2^-24 units, and count); lanes that hit the same bin are merged with
    // match_any + reduce_add before ONE lane updates the bin, so no atomics and no contention, whatever the shape
    // of the distribution. The first level also yields the partition function (the sum of all bins).
    {
        unsigned long long* wmass = hist_mass + warp * 256;
        unsigned int* wcnt = hist_cnt + warp * 256;
        uint2* lane_hist = reinterpret_cast<uint2*>(sp_dyn);     // [256 bins][16 half-warp positions] {low, high} mass
        const bool need_counts = top_k < p.V;                    // a top-k cut needs exact element counts per bin
        uint32_t prefix = 0;            // key bits decided so far (aligned to the top)
        float acc_mass = 0.f;           // mass / count of keys strictly above the undecided range
        int acc_cnt = 0;
        float need = 0.f;
        const int iters = (v1 - v0 + SP_NT - 1) / SP_NT;
        const int levels = filter ? 3 : 1;
#pragma unroll 1
        for (int level = 0; level < levels; ++level) {
            const int shift = 16 - 8 * level;
            if (need_counts) {
                for (int i = lane; i < 256; i += 32) { wmass[i] = 0ull; wcnt[i] = 0u; }
                __syncwarp();
            } else {
                for (int i = tid; i < 256 * 16; i += SP_NT) lane_hist[i] = make_uint2(0u, 0u);
                __syncthreads();
            }
            // Eight elements are loaded before the first warp-wide match: the match / syncwarp pair keeps the compiler
            // from moving the next trip's loads above it, so one element per trip paid a memory round trip each
            // (a row took 270 us however few rows there were).
            constexpr int PF = 8;
            for (int it0 = 0; it0 < iters; it0 += PF) {
                float ev[PF];
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    const int i = v0 + tid + (it0 + u) * SP_NT;
                    if (it0 + u < iters && i < v1) {
                        if (es != nullptr && level > 0) {
                            ev[u] = es[i];
                        } else {
                            ev[u] = __expf(logit_at(i) - mx);
                            if (es != nullptr) es[i] = ev[u];
                        }
                    } else {
                        ev[u] = -1.f;
                    }
                }
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    uint32_t bin = 0xffffffffu;
                    unsigned int fx = 0;
                    if (ev[u] >= 0.f) {
                        const uint32_t key = __float_as_uint(ev[u]) >> 8;
                        const bool in_range = level == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8));
                        if (in_range) { bin = (key >> shift) & 0xffu; fx = (unsigned int)(ev[u] * 16777216.0f); }
                    }
                    if (!need_counts) {
                        // nucleus only: no element counts are needed, so the bin update is two native 32-bit
                        // shared-memory additions (the fixed-point mass split in two 12-bit halves, exact and
                        // order-independent) into a slot private to the lane's half-warp position: ~8 instructions
                        // per element instead of the ~50 of the warp-wide match below
                        if (bin != 0xffffffffu) {
                            uint2* slot = lane_hist + bin * 16 + (lane & 15);
                            atomicAdd(&slot->x, fx & 0xfffu);
                            atomicAdd(&slot->y, fx >> 12);
                        }
                        continue;
                    }
                    // below the first level almost no element lies in the undecided range: skip the warp-wide match
                    if (__any_sync(0xffffffffu, bin != 0xffffffffu)) {
                        const unsigned int peers = __match_any_sync(0xffffffffu, bin);
                        const unsigned int sum = __reduce_add_sync(peers, fx);
                        if (bin != 0xffffffffu && lane == __ffs(peers) - 1) {
                            wmass[bin] += sum;
                            wcnt[bin] += __popc(peers);
                        }
                        __syncwarp();
                    }
                }
            }
            __syncthreads();
            if (tid < 256) {          // this CTA's histogram: thread t owns bin t
                unsigned long long m = 0ull; unsigned int c = 0u;
                if (need_counts) {
                    for (int w = 0; w < SP_NW; ++w) { m += hist_mass[w * 256 + tid]; c += hist_cnt[w * 256 + tid]; }
                } else {
                    unsigned long long lo = 0ull, hi = 0ull;
                    for (int l = 0; l < 16; ++l) { const uint2 v = lane_hist[tid * 16 + ((l + tid) & 15)]; lo += v.x; hi += v.y; }
                    m = lo + (hi << 12);
                    c = m != 0ull ? 1u : 0u;          // only "is the bin empty" is read from the count on this path
                }
                merged_mass[tid] = (float)m * (1.0f / 16777216.0f);
                merged_cnt[tid] = (int)c;
            }
            csync();
            if (tid < 256) {          // cluster totals, computed redundantly by every CTA
                float m = 0.f; int c = 0;
                for (int r = 0; r < cl; ++r) { m += peer_f(&merged_mass[tid], r); c += peer_i(&merged_cnt[tid], r); }
                tot_mass[tid] = m; tot_cnt[tid] = c;
            }
            __syncthreads();
            if (level == 0) {
                if (warp == 0) {
                    float t = 0.f;
                    for (int i = lane; i < 256; i += 32) t += tot_mass[i];
                    t = warp_sum(t);
                    if (lane == 0) sh_f[1] = t;
                }
                __syncthreads();
                z = sh_f[1];
                need = top_p * z;
            }
            if (tid == 0) {
                float acc = acc_mass; int cnt = acc_cnt; int bsel = 255;
                for (; bsel >= 0; --bsel) {
                    const float mb = tot_mass[bsel]; const int cb = tot_cnt[bsel];
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
            csync();                  // every peer has read merged_* before the next level rewrites them
        }
        if (filter) thr_key = prefix;
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
    // mass of the kept set, summed in walk (vocabulary) order: thread t owns a contiguous piece of the CTA's slice
    const int chunk = ((v1 - v0 + SP_NT - 1) / SP_NT + 3) & ~3;
    const int i0 = min(v1, v0 + tid * chunk), i1 = min(v1, i0 + chunk);
    float local = 0.f;
    auto e_at = [&](int i) -> float { return es != nullptr ? es[i] : __expf(logit_at(i) - mx); };
    {
        int i = i0;
        if (es != nullptr && (p.V & 3) == 0) {      // rows, slices and chunks all start on 16-byte boundaries
            for (; i + 4 <= i1; i += 4) {
                const float4 e4 = *reinterpret_cast<const float4*>(es + i);
                const float ee[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if ((__float_as_uint(ee[j]) >> 8) >= thr_key) local += ee[j];
            }
        }
        for (; i < i1; ++i) {
            const float e = e_at(i);
            if ((__float_as_uint(e) >> 8) >= thr_key) local += e;
        }
    }
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) red_f[warp] = incl;
    if (tid == 0) xi[1] = -1;
    __syncthreads();
    if (warp == 0) {
        float w = lane < SP_NW ? red_f[lane] : 0.f;
        float wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        if (lane < SP_NW) red_f[lane] = wi - w;     // exclusive warp offsets
        if (lane == 31) xf[2] = wi;                 // kept mass of this CTA's slice
    }
    csync();
    float before = 0.f, total = 0.f;                // kept mass of the lower slices / of the whole row
    for (int r = 0; r < cl; ++r) {
        const float m = peer_f(&xf[2], r);
        if (r < crank) before += m;
        total += m;
    }
    const float excl = before + red_f[warp] + incl - local;
    const float target = u * total;
    if (local > 0.f && target >= excl && target < excl + local) {
        float acc = excl;
        int pick = -1, last = -1;
        for (int i = i0; i < i1; ++i) {
            const float e = e_at(i);
            if ((__float_as_uint(e) >> 8) >= thr_key) {
                last = i;
                acc += e;
                if (acc > target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last;
        atomicMax(&xi[1], pick);
    }
    // rounding can leave the target outside every piece: remember the last kept index as the fallback
    {
        int last = -1;
        if (local > 0.f)
            for (int i = i1 - 1; i >= i0; --i) {
                const float e = e_at(i);
                if ((__float_as_uint(e) >> 8) >= thr_key) { last = i; break; }
            }
        last = warp_max_i(last);
        if (lane == 0) red_i[warp] = last;
        __syncthreads();
        if (tid == 0) {
            int l = -1;
            for (int w = 0; w < SP_NW; ++w) l = max(l, red_i[w]);
            xi[2] = l;
        }
    }
    csync();
    if (crank == 0 && tid == 0) {
        int tok = -1, last = -1;
        for (int r = 0; r < cl; ++r) { tok = max(tok, peer_i(&xi[1], r)); last = max(last, peer_i(&xi[2], r)); }
        if (tok < 0) tok = last;
        if (tok < 0) tok = 0;
        p.out[row] = tok;
        if (p.out_prob) p.out_prob[row] = __expf(logit_at(tok) - mx) / total;
        if (p.seen) p.seen[(size_t)slot * p.V + tok] = 1;
    }
    csync();                          // keep shared memory alive until rank 0 has read it
}

}  // namespace mstar

using namespace mstar;

MSTAR_API int mstar_sample(const void* logits, long long ld, int is_f32, int B, int V, const float* temperature,
                           const int* top_k, const float* top_p, const float* rep_penalty,
                           const unsigned long long* seed, const unsigned long long* offset, unsigned char* seen,
                           const int* row_slot, long long* out, float* out_prob, float* u_override, float* escratch,
                           void* stream_) {
    if (B <= 0) return 0;
    SampleParams p{logits, ld, is_f32, B, V, temperature, top_k, top_p, rep_penalty, seed, offset, seen, row_slot,
                   out, out_prob, u_override, escratch};
    cudaStream_t s = (cudaStream_t)stream_;
    constexpr int smem = (SP_NW * 256 * 12) > (256 * 16 * 8) ? (SP_NW * 256 * 12) : (256 * 16 * 8);
    static PerDeviceFlag configured;
    if (!configured()) {
        cudaError_t e1 = cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        cudaError_t e2 = cudaFuncSetAttribute(sample_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e1 != cudaSuccess || e2 != cudaSuccess) return set_error("sample: cudaFuncSetAttribute failed", e1 != cudaSuccess ? e1 : e2);
        configured() = true;
    }
    const int cl = V >= 16384 ? SP_CL : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(B * cl);
    cfg.blockDim = dim3(SP_NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = is_f32 ? cudaLaunchKernelEx(&cfg, sample_kernel<true>, p, cl)
                           : cudaLaunchKernelEx(&cfg, sample_kernel<false>, p, cl);
    return e == cudaSuccess ? 0 : set_error("sample launch", e);
}
