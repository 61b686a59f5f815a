// One attention kernel family for serving: paged-KV prefill, paged-KV decode (split-KV), dense varlen
// (DiT / encoder towers), with causal, full and sliding-window masks and GQA.
//
// Mapping to the hardware: a CTA owns a 128-row query tile of ONE kv head. The rows are (token, q-head-in-group)
// pairs, group index fastest, so the G = Hq/Hkv query heads that share a kv head are packed into the UMMA M
// dimension: a decode step with one token per request fills G rows, a prefill tile holds 128/G tokens.
// Per 128-key tile:  S = Q K^T  (tcgen05, K-major operands, fp32 in TMEM)  ->  online softmax by 4 warps that
// read S from TMEM, write P (bf16) to shared memory in the swizzled K-major layout  ->  O_tile = P V
// (tcgen05, V as MN-major operand straight from the page layout)  ->  the softmax warps fold O_tile into
// their register accumulator with the running rescale. K/V tiles arrive by non-multicast TMA from the page
// pool ([pages, 2, Hkv, page_size, D], one box per page) or from dense [tokens, Hkv, D] tensors through a
// 2-stage mbarrier ring; QK^T of tile j+1 is issued while the softmax of tile j runs (S is double-buffered
// in TMEM).
//
// The plan is read from device arrays (q_indptr, kv_lens, page tables), so a step can be captured in a CUDA
// graph and replayed after the host has only rewritten those arrays.
//
// Split-KV (decode with few requests): every split writes (m, l, O) partials to a scratch workspace; the last
// CTA of a (tile, kv head) merges them in split order and writes the output.
//
// Reference counterparts: FlashInfer BatchPrefill/BatchDecodeWithPagedKVCacheWrapper
// (mstar/utils/flashinfer_utils.py:70-489), FA3 varlen (mstar/engine/cache_manager.py:1455-1485),
// sliding-window Triton kernel (mstar/utils/attention.py:297-437), F.scaled_dot_product_attention call sites.
#include <cuda.h>
#include "common.cuh"
#include "host_common.h"

namespace mstar {

struct AttnParams {
    const __nv_bfloat16* q;   // [T, Hq, D] with token stride q_tok_stride (elements)
    __nv_bfloat16* out;       // [T, Hq, D] with token stride o_tok_stride
    long long q_tok_stride, o_tok_stride;
    const int* q_indptr;      // [B+1] token offsets of each request in q/out
    const int* kv_lens;       // [B] keys visible to the request (cache length including the new tokens)
    const int* kv_indptr;     // dense mode: [B+1] token offsets in k/v
    const int* page_indptr;   // paged mode: [B+1]
    const int* page_indices;  // paged mode
    int B, Hq, Hkv, G;
    int paged, page_size;
    int causal, window;       // window <= 0: none. key visible iff qpos - window < kpos <= qpos (causal)
    int toks_per_tile;        // 128 / G
    int splits;
    float scale_log2;         // softmax scale * log2(e)
    float* ws_o;              // [splits, T*Hq, D]
    float* ws_ml;             // [splits, T*Hq, 2]
    unsigned int* counters;   // [num_q_tiles * Hkv]
    long long ws_rows;        // T*Hq
    KernelStatus* status;
    unsigned long long wait_limit_ns;
    float* lse_out;           // optional [T, Hq] log-sum-exp (natural log), may be null
};

constexpr int AT_BM = 128;   // query rows per tile
constexpr int AT_BN = 128;   // keys per tile
constexpr int AT_STAGES = 2;

template <int HD>
struct AttnSmem {
    static constexpr int Q_BYTES = AT_BM * HD * 2;
    static constexpr int K_BYTES = AT_BN * HD * 2;
    static constexpr int V_BYTES = AT_BN * HD * 2;
    static constexpr int P_BYTES = AT_BM * AT_BN * 2;
    static constexpr int STAGE = K_BYTES + V_BYTES;
    static constexpr int XCH_BYTES = 2 * AT_BM * 4;   // per-row exchange between the two threads of a row
    static constexpr int TOTAL = Q_BYTES + AT_STAGES * STAGE + P_BYTES + 1024 + 256 + XCH_BYTES;
};

// swizzled K-major byte offset of (row, 16-byte chunk c) in a [atoms][rows][128 B] operand tile
__device__ __forceinline__ uint32_t sw128_offset(int rows, int row, int chunk) {
    const int atom = chunk >> 3, cc = chunk & 7;
    return (uint32_t)(atom * rows * 128 + row * 128 + ((cc ^ (row & 7)) << 4));
}

// 10 warps: TMA producer, UMMA issuer, and EIGHT softmax warps. A query row is shared by two threads (warps w and
// w + 4 reach the same TMEM lane quarter): one takes key columns 0-63 of every S tile and output dims 0-63, the
// other the upper halves. With one softmax warp per scheduler the kernel was bound by the issue latency of that
// single warp's dependent instructions (tensor pipe 14-22 % busy); two warps per scheduler overlap each other.
constexpr int AT_THREADS = 320;

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_tcgen05_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ AttnParams p) {
    using SM = AttnSmem<HD>;
    constexpr int KATOMS = HD / 64;           // 64-element (128-byte) atoms along the head dim
    constexpr int TMEM_S0 = 0, TMEM_S1 = 128, TMEM_O = 256;
    constexpr int TMEM_COLS = 512;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sKV = smem + SM::Q_BYTES;
    uint8_t* sP = sKV + AT_STAGES * SM::STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + SM::P_BYTES);
    uint64_t* k_full = bars;                  // [2]
    uint64_t* v_full = bars + 2;              // [2]
    uint64_t* kv_empty = bars + 4;            // [2]
    uint64_t* s_full = bars + 6;              // [2]
    uint64_t* s_empty = bars + 8;             // [2]
    uint64_t* p_full = bars + 10;
    uint64_t* o_full = bars + 11;
    uint64_t* o_empty = bars + 12;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    volatile int* sh = reinterpret_cast<volatile int*>(tmem_slot + 1);  // [0] abort [1] req [2] tile-in-req [3] last
    float* xch = reinterpret_cast<float*>(sP + SM::P_BYTES + 256);       // [2 halves][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();     // plan arrays, q and K/V all come from earlier kernels

    // ---- locate this CTA's (request, q tile): tiles are numbered request by request ----
    if (threadIdx.x == 0) {
        int t = blockIdx.x, req = -1, tin = 0;
        for (int b = 0; b < p.B; ++b) {
            const int ql = p.q_indptr[b + 1] - p.q_indptr[b];
            const int nt = (ql + p.toks_per_tile - 1) / p.toks_per_tile;
            if (t < nt) { req = b; tin = t; break; }
            t -= nt;
        }
        sh[0] = 0; sh[1] = req; sh[2] = tin; sh[3] = 0;
        for (int i = 0; i < 6; ++i) mbar_init(&bars[i], 1);     // k_full, v_full, kv_empty
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&s_empty[0], 256); mbar_init(&s_empty[1], 256);
        mbar_init(p_full, 256);
        mbar_init(o_full, 1);
        mbar_init(o_empty, 128);
        mbar_fence_init();
    }
    __syncthreads();
    const int req = sh[1];
    if (req < 0) return;  // grid is an upper bound on the tile count
    const int tin = sh[2];
    const int q_begin = p.q_indptr[req];
    const int q_len = p.q_indptr[req + 1] - q_begin;
    int kv_len = p.kv_lens[req];
    if (p.paged) {
        // never read past the pages the request owns, whatever the length array says
        const int cap = (p.page_indptr[req + 1] - p.page_indptr[req]) * p.page_size;
        if (kv_len > cap) kv_len = cap;
    }
    const int tok0 = tin * p.toks_per_tile;                      // first token of the tile inside the request
    int ntok = q_len - tok0;
    if (ntok > p.toks_per_tile) ntok = p.toks_per_tile;
    const int nrows = ntok * p.G;                                // valid rows of this tile
    const int qpos0 = kv_len - q_len + tok0;                     // sequence position of the tile's first token
    // key range visible to this tile
    int key_end = p.causal ? (qpos0 + ntok) : kv_len;
    if (key_end > kv_len) key_end = kv_len;
    int key_begin = 0;
    if (p.window > 0) {
        key_begin = qpos0 - p.window + 1;
        if (key_begin < 0) key_begin = 0;
    }
    const int tile_first = key_begin / AT_BN;
    const int tile_last = key_end > 0 ? (key_end - 1) / AT_BN : -1;   // inclusive
    int ntiles_all = tile_last - tile_first + 1;
    if (ntiles_all < 0) ntiles_all = 0;
    // split-KV: contiguous ranges of key tiles
    const int per = (ntiles_all + p.splits - 1) / p.splits;
    int jt0 = tile_first + split * per;
    int jt1 = jt0 + per;
    if (jt1 > tile_last + 1) jt1 = tile_last + 1;
    const int ntiles = jt1 > jt0 ? jt1 - jt0 : 0;

    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    // ---- Q tile -> swizzled smem (softmax warps; each thread owns one row) ----
    if (warp >= 2) {
        const int r = (warp & 3) * 32 + lane;
        const int half = (warp - 2) >> 2;
        const int tl = r / p.G, g = r - tl * p.G;
        const bool valid = r < nrows;
        const uint4* src = reinterpret_cast<const uint4*>(
            p.q + (size_t)(q_begin + tok0 + (valid ? tl : 0)) * p.q_tok_stride + (size_t)(kvh * p.G + g) * HD);
#pragma unroll
        for (int c = half * (HD / 16); c < (half + 1) * (HD / 16); ++c) {
            uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(sQ + sw128_offset(AT_BM, r, c)) = v;
        }
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // =========================== TMA producer ===========================
        if (lane == 0 && ntiles > 0) {
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            const int ppt = p.paged ? (AT_BN / p.page_size) : 1;
            const int npages = p.paged ? (p.page_indptr[req + 1] - p.page_indptr[req]) : 0;
            const int* pages = p.paged ? p.page_indices + p.page_indptr[req] : nullptr;
            const int kv_tok0 = p.paged ? 0 : p.kv_indptr[req];
            int issued = 0;
            for (int i = 0; i < ntiles; ++i) {
                const int s = i % AT_STAGES;
                const uint32_t ph = (i / AT_STAGES) & 1;
                if (!mbar_wait(&kv_empty[s], ph ^ 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_ATTN_DENSE, 1, i, s);
                    sh[0] = 1;
                    break;
                }
                if (sh[0]) break;
                uint8_t* sK = sKV + s * SM::STAGE;
                uint8_t* sV = sK + SM::K_BYTES;
                const int jt = jt0 + i;
                mbar_expect_tx(&k_full[s], SM::K_BYTES);
                mbar_expect_tx(&v_full[s], SM::V_BYTES);
                if (p.paged) {
                    for (int pg = 0; pg < ppt; ++pg) {
                        int pi = jt * ppt + pg;
                        if (pi >= npages) pi = npages - 1;   // masked keys; any finite data will do
                        const int page = pages[pi];
                        const int row_off = pg * p.page_size * 128;
#pragma unroll
                        for (int a = 0; a < KATOMS; ++a) {
                            tma_load_4d(sK + a * (AT_BN * 128) + row_off, &tmK, &k_full[s], a * 64, 0, kvh, page);
                        }
#pragma unroll
                        for (int a = 0; a < KATOMS; ++a) {
                            tma_load_4d(sV + a * (AT_BN * 128) + row_off, &tmV, &v_full[s], a * 64, 0, kvh, page);
                        }
                    }
                } else {
                    const int t0 = kv_tok0 + jt * AT_BN;
#pragma unroll
                    for (int a = 0; a < KATOMS; ++a) tma_load_3d(sK + a * (AT_BN * 128), &tmK, &k_full[s], a * 64, kvh, t0);
#pragma unroll
                    for (int a = 0; a < KATOMS; ++a) tma_load_3d(sV + a * (AT_BN * 128), &tmV, &v_full[s], a * 64, kvh, t0);
                }
                issued = i + 1;
            }
            if (sh[0]) {
                for (int i = (issued > AT_STAGES ? issued - AT_STAGES : 0); i < issued; ++i) {
                    mbar_wait(&k_full[i % AT_STAGES], (i / AT_STAGES) & 1, 1000000ull);
                    mbar_wait(&v_full[i % AT_STAGES], (i / AT_STAGES) & 1, 1000000ull);
                }
            }
        }
    } else if (warp == 1) {
        // =========================== UMMA issuer ===========================
        if (lane == 0 && ntiles > 0) {
            constexpr uint32_t idesc_qk = umma_idesc(AT_BM, AT_BN, 1, 1);                 // K-major x K-major
            constexpr uint32_t idesc_pv = umma_idesc(AT_BM, HD, 1, 1) | (1u << 16);       // B (V) is MN-major
            const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
            bool ok = true;
            auto issue_qk = [&](int i) -> bool {
                const int s = i % AT_STAGES;
                if (!mbar_wait(&k_full[s], (i / AT_STAGES) & 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_ATTN_DENSE, 2, i, s);
                    return false;
                }
                if (i >= 2 && !mbar_wait(&s_empty[i & 1], ((i >> 1) - 1) & 1, p.wait_limit_ns)) {
                    report_status(p.status, KID_ATTN_DENSE, 3, i, 0);
                    return false;
                }
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sKV + s * SM::STAGE);
                const uint32_t d = tmem_base + ((i & 1) ? TMEM_S1 : TMEM_S0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * (AT_BM * 128) + (k & 3) * 32;
                    umma_f16_ss(d, umma_smem_desc_sw128(q_addr + off), umma_smem_desc_sw128(k_addr + off), idesc_qk,
                                k != 0 ? 1u : 0u);
                }
                umma_commit(&s_full[i & 1]);
                return true;
            };
            ok = issue_qk(0);
            for (int i = 0; ok && i < ntiles; ++i) {
                const int s = i % AT_STAGES;
                if (i + 1 < ntiles) ok = issue_qk(i + 1);
                if (!ok) break;
                if (!mbar_wait(p_full, i & 1, p.wait_limit_ns)) { report_status(p.status, KID_ATTN_DENSE, 4, i, 0); ok = false; break; }
                if (!mbar_wait(&v_full[s], (i / AT_STAGES) & 1, p.wait_limit_ns)) { report_status(p.status, KID_ATTN_DENSE, 5, i, 0); ok = false; break; }
                // (the softmax warps finished any rescaling of O before they arrived on p_full)
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sKV + s * SM::STAGE + SM::K_BYTES);
                // V tile: [d atoms][keys][64 d] rows of 128 B. MN-major descriptor: LBO = distance between the
                // 64-wide d atoms, SBO = distance between 8-key groups (1024 B); one UMMA K step = 16 keys = 2048 B.
#pragma unroll
                for (int k = 0; k < AT_BN / 16; ++k) {
                    uint64_t db = umma_smem_desc_sw128(v_addr + k * 2048);
                    db = (db & ~(uint64_t(0x3fff) << 16)) | (uint64_t((AT_BN * 128) >> 4) << 16);
                    const uint32_t poff = (k >> 2) * (AT_BM * 128) + (k & 3) * 32;
                    // O accumulates in TMEM over all KV tiles of the CTA
                    umma_f16_ss(tmem_base + TMEM_O, umma_smem_desc_sw128(p_addr + poff), db, idesc_pv, (i | k) != 0 ? 1u : 0u);
                }
                umma_commit(o_full);
                umma_commit(&kv_empty[s]);
            }
            if (!ok) sh[0] = 1;
        }
    } else {
        // =========================== softmax (256 threads, two per row) ===========================
        const int q4 = warp & 3;
        const int half = (warp - 2) >> 2;            // which 64 key columns / 64 output dims this thread owns
        constexpr int HB = AT_BN / 2;                // key columns per thread
        constexpr int HO = HD / 2;                   // output dims per thread
        const int r = q4 * 32 + lane;
        const bool row_valid = r < nrows;
        const bool warp_valid = q4 * 32 < nrows;
        const int tl = r / p.G, g = r - tl * p.G;
        const int qpos = qpos0 + tl;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const int pair_bar = 2 + q4;                 // named barrier of the two warps that share these rows
        // The running maximum m is the reference of the exponentials; it is only moved (and O, which accumulates in
        // TMEM, rescaled) when a tile's maximum exceeds it by more than RESCALE_T in log2 units. Until then the
        // probabilities may grow up to 2^RESCALE_T, which bf16 and the fp32 accumulators hold without loss, and a
        // tile costs one TMEM read of S instead of two reads of S plus a read-modify of O.
        constexpr float RESCALE_T = 8.0f;
        float m = -INFINITY, l = 0.f;                // l: this thread's half of the row sum
        bool ok = true;
        for (int i = 0; i < ntiles && ok; ++i) {
            if (!mbar_wait(&s_full[i & 1], (i >> 1) & 1, p.wait_limit_ns)) {
                report_status(p.status, KID_ATTN_DENSE, 7, i, 0);
                sh[0] = 1; ok = false; break;
            }
            tc_fence_after();
            const uint32_t s_addr = lane_addr + ((i & 1) ? TMEM_S1 : TMEM_S0) + half * HB;
            const int k0 = (jt0 + i) * AT_BN + half * HB;       // first key of this thread's columns
            // visible keys for this row: [lo, hi)
            int hi = p.causal ? (qpos + 1) : kv_len;
            if (hi > kv_len) hi = kv_len;
            int lo = p.window > 0 ? qpos - p.window + 1 : 0;
            const bool need_mask = (k0 + HB > hi) || (k0 < lo);
            uint32_t sv[HB];                          // this thread's half row of S, read from TMEM once
            float alpha = 1.f;
            if (warp_valid) {
#pragma unroll
                for (int c0 = 0; c0 < HB; c0 += 32) tmem_ld32(s_addr + c0, sv + c0);
                tmem_ld_wait();
            }
            tc_fence_before();
            mbar_arrive(&s_empty[i & 1]);             // the S buffer may be overwritten by QK of tile i + 2
            float mx = -INFINITY;
            if (warp_valid) {
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < HB; ++c) {
                        const int kp = k0 + c;
                        if (kp < hi && kp >= lo) mx = fmaxf(mx, __uint_as_float(sv[c]));
                    }
                } else {
                    // four independent chains instead of one long dependent chain
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int c = 0; c < HB; c += 4) {
                        m0 = fmaxf(m0, __uint_as_float(sv[c]));
                        m1 = fmaxf(m1, __uint_as_float(sv[c + 1]));
                        m2 = fmaxf(m2, __uint_as_float(sv[c + 2]));
                        m3 = fmaxf(m3, __uint_as_float(sv[c + 3]));
                    }
                    mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                }
                mx *= p.scale_log2;   // scale > 0, so max commutes with the scaling
            }
            // the row maximum over both halves
            xch[half * AT_BM + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            mx = fmaxf(mx, xch[(half ^ 1) * AT_BM + r]);
            const bool move = warp_valid && (mx > m + RESCALE_T || (m == -INFINITY && mx != -INFINITY));
            if (move) {
                alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - mx);
                m = mx;
            }
            // PV of the previous tile must have finished before O is rescaled or P is overwritten in shared memory
            if (i >= 1 && !mbar_wait(o_full, (i - 1) & 1, p.wait_limit_ns)) {
                report_status(p.status, KID_ATTN_DENSE, 8, i, 0);
                sh[0] = 1; ok = false; break;
            }
            tc_fence_after();
            if (i >= 1 && warp_valid && __any_sync(0xffffffffu, move)) {
#pragma unroll 1
                for (int c0 = 0; c0 < HO; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + TMEM_O + half * HO + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * alpha);
                    tmem_st32(lane_addr + TMEM_O + half * HO + c0, v);
                }
                tmem_st_wait();
            }
            if (warp_valid) {
                const float neg_m = (m == -INFINITY) ? 0.f : -m;
                const float sc = p.scale_log2;
                float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
                for (int c0 = 0; c0 < HB; c0 += 32) {
                    uint32_t w[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        float p0 = ex2_approx(fmaf(__uint_as_float(sv[c0 + c]), sc, neg_m));
                        float p1 = ex2_approx(fmaf(__uint_as_float(sv[c0 + c + 1]), sc, neg_m));
                        if (need_mask) {
                            const int kp = k0 + c0 + c;
                            if (!(kp < hi && kp >= lo)) p0 = 0.f;
                            if (!(kp + 1 < hi && kp + 1 >= lo)) p1 = 0.f;
                        }
                        w[c >> 1] = pack_bf16x2(p0, p1);
                        rs0 += p0;
                        rs1 += p1;
                    }
                    if (row_valid) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            *reinterpret_cast<uint4*>(sP + sw128_offset(AT_BM, r, ((half * HB + c0) >> 3) + q)) =
                                make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    }
                }
                l = l * alpha + (rs0 + rs1);
            }
            tc_fence_before();
            fence_proxy_async_smem();
            mbar_arrive(p_full);
            // the exchange slots are rewritten in the next iteration: both readers must be done with them
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        }
        // the row sum over both halves
        xch[half * AT_BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        l += xch[(half ^ 1) * AT_BM + r];
        // the accumulator: wait for the last PV, then read this thread's half of O from TMEM once
        float o[HO];
#pragma unroll
        for (int i = 0; i < HO; ++i) o[i] = 0.f;
        if (ok && ntiles > 0) {
            if (!mbar_wait(o_full, (ntiles - 1) & 1, p.wait_limit_ns)) {
                report_status(p.status, KID_ATTN_DENSE, 9, ntiles, 0);
                sh[0] = 1; ok = false;
            }
            tc_fence_after();
            if (ok && warp_valid) {
#pragma unroll
                for (int c0 = 0; c0 < HO; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + TMEM_O + half * HO + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c0 + c] = __uint_as_float(v[c]);
                }
            }
            tc_fence_before();
        }

        // ---- epilogue: every thread handles its HO output dims ----
        const size_t tok = (size_t)(q_begin + tok0 + tl);
        const int head = kvh * p.G + g;
        bool do_final = ok;
        if (ok && p.splits > 1) {
            if (row_valid) {
                const size_t wrow = tok * p.Hq + head;
                float* wo = p.ws_o + ((size_t)split * p.ws_rows + wrow) * HD + half * HO;
#pragma unroll
                for (int c = 0; c < HO; c += 4) __stcg(reinterpret_cast<float4*>(wo + c), make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]));
                if (half == 0) {
                    float* wm = p.ws_ml + ((size_t)split * p.ws_rows + wrow) * 2;
                    __stcg(wm, m);
                    __stcg(wm + 1, l);
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const int cidx = blockIdx.x * p.Hkv + kvh;
            if (threadIdx.x == 64) {
                unsigned int old = atomicAdd(&p.counters[cidx], 1u);
                sh[3] = (old == (unsigned int)(p.splits - 1)) ? 1 : 0;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            do_final = sh[3] != 0;
            if (do_final) {
                __threadfence();
                if (row_valid) {
                    const size_t wrow = tok * p.Hq + head;
                    float mg = -INFINITY;
                    for (int z = 0; z < p.splits; ++z) mg = fmaxf(mg, __ldcg(p.ws_ml + ((size_t)z * p.ws_rows + wrow) * 2));
                    const float mg_use = (mg == -INFINITY) ? 0.f : mg;
#pragma unroll
                    for (int c = 0; c < HO; ++c) o[c] = 0.f;
                    l = 0.f;
                    for (int z = 0; z < p.splits; ++z) {
                        const float* wm = p.ws_ml + ((size_t)z * p.ws_rows + wrow) * 2;
                        const float mz = __ldcg(wm), lz = __ldcg(wm + 1);
                        const float wgt = (mz == -INFINITY) ? 0.f : exp2f(mz - mg_use);
                        l += lz * wgt;
                        const float* wo = p.ws_o + ((size_t)z * p.ws_rows + wrow) * HD + half * HO;
#pragma unroll
                        for (int c = 0; c < HO; c += 4) {
                            float4 t = __ldcg(reinterpret_cast<const float4*>(wo + c));
                            o[c] += t.x * wgt; o[c + 1] += t.y * wgt; o[c + 2] += t.z * wgt; o[c + 3] += t.w * wgt;
                        }
                    }
                    m = mg;
                }
                if (threadIdx.x == 64) p.counters[cidx] = 0u;
            }
        }
        if (do_final && row_valid) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(p.out + tok * p.o_tok_stride + (size_t)head * HD + half * HO);
#pragma unroll
            for (int c = 0; c < HO; c += 8) {
                dst[c >> 3] = make_uint4(pack_bf16x2(o[c] * inv, o[c + 1] * inv), pack_bf16x2(o[c + 2] * inv, o[c + 3] * inv),
                                         pack_bf16x2(o[c + 4] * inv, o[c + 5] * inv), pack_bf16x2(o[c + 6] * inv, o[c + 7] * inv));
            }
            if (p.lse_out && half == 0) p.lse_out[tok * p.Hq + head] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int HD>
static int launch_attn(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, dim3 grid,
                       cudaStream_t stream) {
    constexpr int smem = AttnSmem<HD>::TOTAL;
    static PerDeviceFlag configured;
    if (!configured()) {
        cudaError_t e = cudaFuncSetAttribute(attn_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error("attention: cudaFuncSetAttribute failed", e);
        configured() = true;
    }
    cudaError_t e = launch_pdl(attn_tcgen05_kernel<HD>, grid, dim3(AT_THREADS), smem, stream, tmK, tmV, p);
    return e == cudaSuccess ? 0 : set_error("attention: launch failed", e);
}

}  // namespace mstar

using namespace mstar;

// Attention over paged or dense KV.
//   q/out: [T, Hq, D] bf16 (token strides in elements);  q_indptr [B+1];  kv_lens [B]
//   paged: kcache = this layer's pool [num_pages, 2, Hkv, page_size, D]; page_indptr/page_indices give each
//          request's pages in order;  dense: k, v = [T_kv, Hkv, D] with token stride kv_tok_stride, kv_indptr [B+1]
//   num_q_tiles: upper bound of sum_b ceil(q_len_b / (128 / G)) (grid size; surplus CTAs exit at once)
//   splits > 1 needs ws_o (splits * T*Hq * D floats), ws_ml (splits * T*Hq * 2 floats), counters (zeroed once)
MSTAR_API int mstar_attention(const void* q, void* out, long long q_tok_stride, long long o_tok_stride,
                              const int* q_indptr, const int* kv_lens, int B, int T_q, int Hq, int Hkv, int D,
                              int paged, const void* k, const void* v, long long kv_tok_stride, long long T_kv,
                              const int* kv_indptr, int num_pages, int page_size, const int* page_indptr,
                              const int* page_indices, int causal, int window, float scale, int num_q_tiles,
                              int splits, float* ws_o, float* ws_ml, void* counters, float* lse_out, void* stream_) {
    if (B <= 0 || num_q_tiles <= 0) return 0;
    if (D != 64 && D != 128) return set_error("attention: head_dim must be 64 or 128", cudaSuccess);
    if (Hq % Hkv) return set_error("attention: Hq must be a multiple of Hkv", cudaSuccess);
    const int G = Hq / Hkv;
    if (G > 128) return set_error("attention: GQA group too large", cudaSuccess);
    AttnParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
    p.q_tok_stride = q_tok_stride; p.o_tok_stride = o_tok_stride;
    p.q_indptr = q_indptr; p.kv_lens = kv_lens; p.kv_indptr = kv_indptr;
    p.page_indptr = page_indptr; p.page_indices = page_indices;
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
    p.paged = paged; p.page_size = page_size;
    p.causal = causal; p.window = window;
    p.toks_per_tile = AT_BM / G;
    p.splits = splits < 1 ? 1 : splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.ws_o = ws_o; p.ws_ml = ws_ml; p.counters = (unsigned int*)counters;
    p.ws_rows = (long long)T_q * Hq;
    p.status = status_ptr();
    p.wait_limit_ns = wait_limit_ns();
    p.lse_out = lse_out;
    if (p.splits > 1 && (!ws_o || !ws_ml || !counters)) return set_error("attention: split-KV needs scratch", cudaSuccess);

    CUtensorMap tmK, tmV;
    if (paged) {
        if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1)))
            return set_error("attention: page_size must be a power of two in [8, 128]", cudaSuccess);
        unsigned long long dims[4] = {(unsigned long long)D, (unsigned long long)page_size, (unsigned long long)Hkv,
                                      (unsigned long long)num_pages};
        unsigned long long strides[4] = {2ull, (unsigned long long)D * 2, (unsigned long long)page_size * D * 2,
                                         2ull * Hkv * page_size * D * 2};
        unsigned int box[4] = {64u, (unsigned int)page_size, 1u, 1u};
        const __nv_bfloat16* kc = (const __nv_bfloat16*)k;
        if (make_tmap(&tmK, kc, 2, 4, dims, strides, box, 1)) return -1;
        if (make_tmap(&tmV, kc + (size_t)Hkv * page_size * D, 2, 4, dims, strides, box, 1)) return -1;
    } else {
        unsigned long long dims[3] = {(unsigned long long)D, (unsigned long long)Hkv, (unsigned long long)T_kv};
        unsigned long long strides[3] = {2ull, (unsigned long long)D * 2, (unsigned long long)kv_tok_stride * 2};
        unsigned int box[3] = {64u, 1u, (unsigned int)AT_BN};
        if (make_tmap(&tmK, k, 2, 3, dims, strides, box, 1)) return -1;
        if (make_tmap(&tmV, v, 2, 3, dims, strides, box, 1)) return -1;
    }
    dim3 grid(num_q_tiles, Hkv, p.splits);
    cudaStream_t stream = (cudaStream_t)stream_;
    if (D == 64) return launch_attn<64>(tmK, tmV, p, grid, stream);
    return launch_attn<128>(tmK, tmV, p, grid, stream);
}
