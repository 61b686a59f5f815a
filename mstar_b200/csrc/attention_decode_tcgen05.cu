// Paged-KV decode attention with the roles of keys and queries swapped on the tensor core.
//
// A decode step has only G = Hq/Hkv query rows per (request, kv head) — far too few to fill the 128-row UMMA M
// dimension. Here the 128 KEYS of a tile take the M dimension instead:
//     S^T[key, col] = K_tile[128 x D] * Q^T[D x 16]          (A = K tile, K-major; B = Q rows, N = 16)
//     O^T[d,  col] += V_tile^T[D x 128] * P^T[128 x 16]       (A = V tile as MN-major operand; B = P^T, N = 16)
// so every TMEM lane / softmax thread owns one key (then one head-dim row d) and handles only <= 16 values per
// tile instead of a 128-wide score row. Columns are (token, head-in-group) pairs; up to 16 / G new tokens per
// request are supported (plain decode uses one).
//
// Per tile: TMA brings K and V pages (3-stage ring), UMMA 1 -> the 4 softmax warps read S^T (16 columns), reduce
// the column maxima across the 128 keys (warp shuffles + one named barrier), write P^T as bf16 into the swizzled
// K-major B tile, UMMA 2 -> fold O^T tile into 16 fp32 registers per thread with the running rescale. Row sums
// stay thread-private until the end. Split-KV partials are merged by the last CTA of a (request, kv head).
//
// Reference counterparts: FlashInfer BatchDecodeWithPagedKVCacheWrapper (mstar/utils/flashinfer_utils.py:293-489),
// Triton dense-KV decode kernel (mstar/utils/attention.py:6-134).
#include <cuda.h>
#include <stdlib.h>
#include "common.cuh"
#include "host_common.h"

namespace mstar {

struct DecAttnParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    long long q_tok_stride, o_tok_stride;
    const int* q_indptr;
    const int* kv_lens;
    const int* page_indptr;
    const int* page_indices;
    int B, Hq, Hkv, G, page_size, causal, window, splits;
    float scale_log2;
    float* ws_o;              // [splits, T*Hq, D]
    float* ws_ml;             // [splits, T*Hq, 2]
    unsigned int* counters;   // [B * Hkv]
    long long ws_rows;
    KernelStatus* status;
    unsigned long long wait_limit_ns;
    // while the K/V pages stream through (marked evict-first with l2_hints), the L2 fetches the weights of the
    // projections that follow this kernel
    const void* pf_ptr = nullptr;
    unsigned long long pf_bytes = 0;
    int l2_hints = 0;
};

constexpr int DA_KEYS = 128;
constexpr int DA_COLS = 16;
constexpr int DA_HD = 128;
constexpr int DA_K_BYTES = DA_KEYS * DA_HD * 2;     // 32 KB (one K or V tile)
constexpr int DA_Q_BYTES = DA_COLS * DA_HD * 2;     // 4 KB
constexpr int DA_P_BYTES = DA_COLS * DA_KEYS * 2;   // 4 KB
__host__ __device__ constexpr int da_smem_bytes(int ks, int vs) {
    return DA_Q_BYTES + DA_P_BYTES + (ks + vs) * DA_K_BYTES + 1024 + 1024;
}

// KS / VS: depth of the K and V tile rings. <1,1> keeps a CTA at 74 KB so that three CTAs share an SM and hide
// each other's per-tile latency chain (the regime of batched decode); deeper rings serve small grids, where one
// CTA per SM must prefetch for itself. NC: number of accumulator columns kept in registers (>= q_len * G).
template <int KS, int VS, int NC, int MINB>
__global__ void __launch_bounds__(192, MINB)
attn_decode_tcgen05_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                           const __grid_constant__ DecAttnParams p) {
    constexpr int TMEM_S0 = 0, TMEM_S1 = 16, TMEM_O = 32, TMEM_COLS = 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                         // [2 atoms][16 rows][128 B]
    uint8_t* sP = smem + DA_Q_BYTES;            // [2 atoms][16 rows][128 B]  (P^T: rows = columns c, K = keys)
    uint8_t* sK = sP + DA_P_BYTES;              // K ring
    uint8_t* sV = sK + KS * DA_K_BYTES;         // V ring
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + VS * DA_K_BYTES);
    uint64_t* k_full = bars;                    // [KS] (<= 4)
    uint64_t* v_full = bars + 4;                // [VS]
    uint64_t* k_empty = bars + 8;               // [KS]
    uint64_t* v_empty = bars + 12;              // [VS]
    uint64_t* s_full = bars + 16;               // [2]
    uint64_t* s_empty = bars + 18;              // [2]
    uint64_t* p_full = bars + 20;
    uint64_t* o_full = bars + 21;
    uint64_t* o_empty = bars + 22;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
    volatile int* sh = reinterpret_cast<volatile int*>(tmem_slot + 1);   // [0] abort [1] last-split flag
    float* red = reinterpret_cast<float*>(const_cast<int*>(sh) + 4);     // [2][4 warps][16] max exchange, then sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();     // the plan arrays, q and the KV pages all come from earlier kernels of the step
    // Longest context first: CTAs are handed out in linear order, and a long request that starts late sets the
    // kernel's length (contexts of one batch differ by 10x). CTA number lin works on the (lin / Hkv)-th longest
    // request; every CTA finds it by ranking the batch's kv_lens itself (B values), so the host plan is unchanged.
    __shared__ int sh_req;
    __shared__ __align__(16) int sh_len[256];
    {
        const int lin = blockIdx.y * gridDim.x + blockIdx.x;
        const int target = lin / p.Hkv;
        if (p.B <= 256) {
            const int Bp = (p.B + 3) & ~3;
            for (int t = threadIdx.x; t < Bp; t += blockDim.x) sh_len[t] = t < p.B ? p.kv_lens[t] : -1;
            __syncthreads();
            for (int t = threadIdx.x; t < p.B; t += blockDim.x) {
                const int mine = sh_len[t];
                int rank = 0;
                for (int o = 0; o < Bp; o += 4) {          // 16-byte broadcast reads; padding entries (-1) never outrank
                    const int4 v = *reinterpret_cast<const int4*>(&sh_len[o]);
                    rank += (v.x > mine || (v.x == mine && o < t)) ? 1 : 0;
                    rank += (v.y > mine || (v.y == mine && o + 1 < t)) ? 1 : 0;
                    rank += (v.z > mine || (v.z == mine && o + 2 < t)) ? 1 : 0;
                    rank += (v.w > mine || (v.w == mine && o + 3 < t)) ? 1 : 0;
                }
                if (rank == target) sh_req = t;
            }
        } else if (threadIdx.x == 0) {
            sh_req = target;          // larger batches keep the natural order
        }
        __syncthreads();
    }
    const int req = sh_req, kvh = (int)((blockIdx.y * gridDim.x + blockIdx.x) % p.Hkv);
    const int q_begin = p.q_indptr[req];
    const int q_len = p.q_indptr[req + 1] - q_begin;
    int ncols = q_len * p.G;
    if (ncols > NC) ncols = NC;                 // host picks NC >= q_len * G
    int kv_len = p.kv_lens[req];
    const int npages = p.page_indptr[req + 1] - p.page_indptr[req];
    if (kv_len > npages * p.page_size) kv_len = npages * p.page_size;
    const int qpos0 = kv_len - q_len;
    int key_begin = 0;
    if (p.window > 0) { key_begin = qpos0 - p.window + 1; if (key_begin < 0) key_begin = 0; }
    const int tile_first = key_begin / DA_KEYS;
    const int tile_last = kv_len > 0 ? (kv_len - 1) / DA_KEYS : -1;
    int nt_all = tile_last - tile_first + 1;
    if (nt_all < 0 || q_len <= 0) nt_all = 0;
    const int per = (nt_all + p.splits - 1) / p.splits;
    const int jt0 = tile_first + split * per;
    int jt1 = jt0 + per;
    if (jt1 > tile_last + 1) jt1 = tile_last + 1;
    const int ntiles = jt1 > jt0 ? jt1 - jt0 : 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 16; ++i) mbar_init(&bars[i], 1);
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&s_empty[0], 128); mbar_init(&s_empty[1], 128);
        mbar_init(p_full, 128);
        mbar_init(o_full, 1);
        mbar_init(o_empty, 128);
        sh[0] = 0; sh[1] = 0;
        mbar_fence_init();
    }
    // K / V tile i of this CTA -> ring slot (thread 0 only). The first tile is requested right after the barriers
    // exist, before the Q rows are staged and TMEM is allocated: the page-table reads and the first DRAM round trip
    // then run under the rest of the prologue (a CTA of a short context has only ~5 tiles to amortise its start).
    const int ppt = DA_KEYS / p.page_size;
    const int* pages = p.page_indices + p.page_indptr[req];
    const bool kv_hint = p.l2_hints != 0;
    const uint64_t pol_kv = kv_hint ? l2_policy_evict_first() : 0ull;
    auto load_kv = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int x, int kvh_, int page) {
        if (kv_hint) tma_load_4d_hint(dst, tm, bar, x, 0, kvh_, page, pol_kv);
        else tma_load_4d(dst, tm, bar, x, 0, kvh_, page);
    };
    auto issue_k = [&](int i) {
        const int jt = jt0 + i, s = i % KS;
        uint8_t* dst = sK + s * DA_K_BYTES;
        mbar_expect_tx(&k_full[s], DA_K_BYTES);
        for (int pg = 0; pg < ppt; ++pg) {
            int pi = jt * ppt + pg;
            if (pi >= npages) pi = npages - 1;
            const int page = pages[pi];
            const int row_off = pg * p.page_size * 128;
            load_kv(dst + row_off, &tmK, &k_full[s], 0, kvh, page);
            load_kv(dst + DA_KEYS * 128 + row_off, &tmK, &k_full[s], 64, kvh, page);
        }
    };
    auto issue_v = [&](int i) {
        const int jt = jt0 + i, s = i % VS;
        uint8_t* dst = sV + s * DA_K_BYTES;
        mbar_expect_tx(&v_full[s], DA_K_BYTES);
        for (int pg = 0; pg < ppt; ++pg) {
            int pi = jt * ppt + pg;
            if (pi >= npages) pi = npages - 1;
            const int page = pages[pi];
            const int row_off = pg * p.page_size * 128;
            load_kv(dst + row_off, &tmV, &v_full[s], 0, kvh, page);
            load_kv(dst + DA_KEYS * 128 + row_off, &tmV, &v_full[s], 64, kvh, page);
        }
    };
    if (threadIdx.x == 0 && ntiles > 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        issue_k(0);
        issue_v(0);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    if (warp == 2) {
        // Q rows -> swizzled K-major B tile: lane c < 16 copies row c (zero rows beyond ncols)
        if (lane < DA_COLS) {
            const int c = lane, tl = c / p.G, g = c - tl * p.G;
            const bool valid = c < ncols;
            const uint4* src = reinterpret_cast<const uint4*>(
                p.q + (size_t)(q_begin + (valid ? tl : 0)) * p.q_tok_stride + (size_t)(kvh * p.G + (valid ? g : 0)) * DA_HD);
#pragma unroll
            for (int ch = 0; ch < DA_HD / 8; ++ch) {
                const uint4 v = valid ? src[ch] : make_uint4(0, 0, 0, 0);
                const int atom = ch >> 3, cc = ch & 7;
                *reinterpret_cast<uint4*>(sQ + atom * (DA_COLS * 128) + c * 128 + ((cc ^ (c & 7)) << 4)) = v;
            }
        }
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (p.pf_bytes != 0 && threadIdx.x == 33)       // second lane of the MMA warp: idle
        l2_prefetch_slice(p.pf_ptr, p.pf_bytes, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                          gridDim.x * gridDim.y * gridDim.z, p.l2_hints != 0);

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0 && ntiles > 0) {
            int issued_k = 1, issued_v = 1;          // tile 0 went out in the prologue
            for (int i = 1; i < ntiles; ++i) {
                {
                    const int s = i % KS;
                    if (!mbar_wait(&k_empty[s], ((i / KS) & 1) ^ 1, p.wait_limit_ns)) {
                        report_status(p.status, KID_ATTN_DECODE, 1, i, s);
                        sh[0] = 1;
                        break;
                    }
                    if (sh[0]) break;
                    issue_k(i);
                    issued_k = i + 1;
                }
                {
                    const int s = i % VS;
                    if (!mbar_wait(&v_empty[s], ((i / VS) & 1) ^ 1, p.wait_limit_ns)) {
                        report_status(p.status, KID_ATTN_DECODE, 9, i, s);
                        sh[0] = 1;
                        break;
                    }
                    if (sh[0]) break;
                    issue_v(i);
                    issued_v = i + 1;
                }
            }
            if (sh[0]) {
                // error path: let copies already in flight land before the CTA leaves
                for (int i = (issued_k > KS ? issued_k - KS : 0); i < issued_k; ++i)
                    mbar_wait(&k_full[i % KS], (i / KS) & 1, 1000000ull);
                for (int i = (issued_v > VS ? issued_v - VS : 0); i < issued_v; ++i)
                    mbar_wait(&v_full[i % VS], (i / VS) & 1, 1000000ull);
            }
        }
    } else if (warp == 1) {
        // =========================== UMMA issuer ===========================
        if (lane == 0 && ntiles > 0) {
            constexpr uint32_t idesc_s = umma_idesc(DA_KEYS, DA_COLS, 1, 1);                  // K tile x Q^T
            constexpr uint32_t idesc_o = umma_idesc(DA_HD, DA_COLS, 1, 1) | (1u << 15);       // A (V^T) MN-major
            const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
            bool ok = true;
            auto issue_s = [&](int i) -> bool {
                const int s = i % KS;
                if (!mbar_wait(&k_full[s], (i / KS) & 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_ATTN_DECODE, 2, i, s);
                    return false;
                }
                if (i >= 2 && !mbar_wait(&s_empty[i & 1], ((i >> 1) - 1) & 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_ATTN_DECODE, 3, i, 0);
                    return false;
                }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sK + s * DA_K_BYTES);
                const uint32_t d = tmem_base + ((i & 1) ? TMEM_S1 : TMEM_S0);
#pragma unroll
                for (int k = 0; k < DA_HD / 16; ++k) {
                    const uint32_t aoff = (k >> 2) * (DA_KEYS * 128) + (k & 3) * 32;
                    const uint32_t boff = (k >> 2) * (DA_COLS * 128) + (k & 3) * 32;
                    umma_f16_ss(d, umma_smem_desc_sw128(k_addr + aoff), umma_smem_desc_sw128(q_addr + boff), idesc_s,
                                k != 0 ? 1u : 0u);
                }
                umma_commit(&s_full[i & 1]);
                umma_commit(&k_empty[s]);
                return true;
            };
            ok = issue_s(0);
            for (int i = 0; ok && i < ntiles; ++i) {
                const int s = i % VS;
                if (i + 1 < ntiles) ok = issue_s(i + 1);
                if (!ok) break;
                if (!mbar_wait(p_full, i & 1, p.wait_limit_ns)) { report_status(p.status, KID_ATTN_DECODE, 4, i, 0); ok = false; break; }
                if (!mbar_wait(&v_full[s], (i / VS) & 1, p.wait_limit_ns)) { report_status(p.status, KID_ATTN_DECODE, 5, i, 0); ok = false; break; }
                if (i >= 1 && !mbar_wait(o_empty, (i - 1) & 1, p.wait_limit_ns)) { report_status(p.status, KID_ATTN_DECODE, 6, i, 0); ok = false; break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sV + s * DA_K_BYTES);
#pragma unroll
                for (int k = 0; k < DA_KEYS / 16; ++k) {
                    // A = V^T: M (= d) is the contiguous dimension. LBO = distance of the two 64-wide d atoms,
                    // SBO = distance of 8-key groups; one K step = 16 keys = 2048 bytes.
                    uint64_t da = umma_smem_desc_sw128(v_addr + k * 2048);
                    da = (da & ~(uint64_t(0x3fff) << 16)) | (uint64_t((DA_KEYS * 128) >> 4) << 16);
                    const uint32_t boff = (k >> 2) * (DA_COLS * 128) + (k & 3) * 32;
                    umma_f16_ss(tmem_base + TMEM_O, da, umma_smem_desc_sw128(p_addr + boff), idesc_o, k != 0 ? 1u : 0u);
                }
                umma_commit(o_full);
                umma_commit(&v_empty[s]);
            }
            if (!ok) sh[0] = 1;
        }
    } else {
#include "attention_decode_softmax.inc"
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace mstar

using namespace mstar;

MSTAR_API int mstar_attention_decode(const void* q, void* out, long long q_tok_stride, long long o_tok_stride,
                                     const int* q_indptr, const int* kv_lens, int B, int T_q, int Hq, int Hkv, int D,
                                     const void* kcache, int num_pages, int page_size, const int* page_indptr,
                                     const int* page_indices, int causal, int window, float scale, int splits,
                                     int max_q_len, float* ws_o, float* ws_ml, void* counters, void* stream_) {
    if (B <= 0) return 0;
    if (D != DA_HD) return set_error("attention_decode: head_dim must be 128", cudaSuccess);
    if (Hq % Hkv || max_q_len < 1 || max_q_len * (Hq / Hkv) > DA_COLS)
        return set_error("attention_decode: q_len * (Hq / Hkv) must be in [1, 16]", cudaSuccess);
    if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1)))
        return set_error("attention_decode: page_size must be a power of two in [8, 128]", cudaSuccess);
    DecAttnParams p;
    { const PrefetchHint h = take_prefetch_hint(); p.pf_ptr = h.ptr; p.pf_bytes = h.bytes; p.l2_hints = h.l2_hints; }
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
    p.q_tok_stride = q_tok_stride; p.o_tok_stride = o_tok_stride;
    p.q_indptr = q_indptr; p.kv_lens = kv_lens; p.page_indptr = page_indptr; p.page_indices = page_indices;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.page_size = page_size;
    p.causal = causal; p.window = window; p.splits = splits < 1 ? 1 : splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.ws_o = ws_o; p.ws_ml = ws_ml; p.counters = (unsigned int*)counters;
    p.ws_rows = (long long)T_q * Hq;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    if (p.splits > 1 && (!ws_o || !ws_ml || !counters)) return set_error("attention_decode: split-KV needs scratch", cudaSuccess);
    unsigned long long dims[4] = {(unsigned long long)D, (unsigned long long)page_size, (unsigned long long)Hkv,
                                  (unsigned long long)num_pages};
    unsigned long long strides[4] = {2ull, (unsigned long long)D * 2, (unsigned long long)page_size * D * 2,
                                     2ull * Hkv * page_size * D * 2};
    unsigned int box[4] = {64u, (unsigned int)page_size, 1u, 1u};
    CUtensorMap tmK, tmV;
    const __nv_bfloat16* kc = (const __nv_bfloat16*)kcache;
    if (make_tmap(&tmK, kc, 2, 4, dims, strides, box, 1)) return -1;
    if (make_tmap(&tmV, kc + (size_t)Hkv * page_size * D, 2, 4, dims, strides, box, 1)) return -1;
    dim3 grid(B, Hkv, p.splits);
    const long long ctas = (long long)B * Hkv * p.splits;
    const int ncols_max = max_q_len * p.G;
    const bool many = ctas > 2LL * device_sm_count();
    cudaStream_t stream = (cudaStream_t)stream_;
#define MSTAR_DA_LAUNCH(KS, VS, NC, MINB)                                                                        \
    do {                                                                                                          \
        static PerDeviceFlag configured;                                                                           \
        constexpr int smem = da_smem_bytes(KS, VS);                                                               \
        if (!configured()) {                                                                                        \
            cudaError_t e_ = cudaFuncSetAttribute(attn_decode_tcgen05_kernel<KS, VS, NC, MINB>,                   \
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, smem);             \
            if (e_ != cudaSuccess) return set_error("attention_decode: cudaFuncSetAttribute failed", e_);         \
            configured() = true;                                                                                    \
        }                                                                                                         \
        cudaError_t le_ = launch_pdl(attn_decode_tcgen05_kernel<KS, VS, NC, MINB>, grid, dim3(192), smem, stream,  \
                                     tmK, tmV, p);                                                                \
        if (le_ != cudaSuccess) return set_error("attention_decode: launch failed", le_);                         \
    } while (0)
    // MSTAR_DA_RING (tuning aid): 21 = two K tiles + one V tile, two CTAs per SM; 22 = two of each, one CTA per SM
    static int ring = -1;
    if (ring < 0) {
        const char* e = getenv("MSTAR_DA_RING");
        ring = e ? atoi(e) : 0;
    }
    if (many && ring == 21 && ncols_max <= 4) {
        MSTAR_DA_LAUNCH(2, 1, 4, 2);
    } else if (many && ring == 22 && ncols_max <= 4) {
        MSTAR_DA_LAUNCH(2, 2, 4, 1);
    } else if (many && ring == 33 && ncols_max <= 4) {
        MSTAR_DA_LAUNCH(3, 3, 4, 1);
    } else if (many) {
        if (ncols_max <= 4) MSTAR_DA_LAUNCH(1, 1, 4, 3);
        else if (ncols_max <= 8) MSTAR_DA_LAUNCH(1, 1, 8, 3);
        else MSTAR_DA_LAUNCH(1, 1, 16, 2);
    } else {
        if (ncols_max <= 4) MSTAR_DA_LAUNCH(3, 3, 4, 1);
        else if (ncols_max <= 8) MSTAR_DA_LAUNCH(3, 3, 8, 1);
        else MSTAR_DA_LAUNCH(3, 3, 16, 1);
    }
#undef MSTAR_DA_LAUNCH
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("attention_decode: launch failed", e);
}
