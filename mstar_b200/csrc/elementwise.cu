// Memory-bound helper kernels: RMSNorm / LayerNorm (+residual, +AdaLN modulation), QK-norm + RoPE + paged-KV
// write, SiLU-mul, embedding gather, gated residual, CFG combine + Euler step, image normalise, decode-state
// advance. All are single-pass over their operands with 16-byte accesses where alignment allows.
//
// Reference counterparts (Triton / FlashInfer / torch elementwise): mstar/utils/attention.py:137-286,447-501
// (qk-norm+rope, rope, rms_norm), mstar/utils/adarms_norm.py:31-77, mstar/utils/flashinfer_utils.py:25-50,273-290,
// mstar/model/pi05/kernels/image_normalize.py:39, mstar/model/bagel/submodules.py:1005-1100 (CFG combine).
#include <cuda_fp8.h>
#include "common.cuh"
#include "host_common.h"

namespace mstar {

// ------------------------------------------------------------------------------------------------------------
// block reduce
// ------------------------------------------------------------------------------------------------------------
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = (l < NT / 32) ? red[l] : 0.0f;
    t = warp_sum(t);
    return t;
}

// ------------------------------------------------------------------------------------------------------------
// RMSNorm / LayerNorm with optional residual add and optional (1 + scale) * y + shift modulation.
//   h = x (+ residual);  if residual_out: residual_out = h (bf16)
//   y = h * rsqrt(mean(h^2) + eps) [or (h - mean) * rsqrt(var + eps)] * (weight [+1 if gemma]) (+ bias)
//   if scale: y = y * (1 + scale[b]) + shift[b]   (scale/shift rows are picked by row / rows_per_mod)
// ------------------------------------------------------------------------------------------------------------
struct NormParams {
    const __nv_bfloat16* x;
    const __nv_bfloat16* residual;
    __nv_bfloat16* residual_out;
    const __nv_bfloat16* weight;  // may be null (no affine)
    const __nv_bfloat16* bias;    // may be null
    const __nv_bfloat16* scale;   // may be null; [rows / rows_per_mod, mod_stride]
    const __nv_bfloat16* shift;
    __nv_bfloat16* out;
    int rows, hidden;
    long long ld_x, ld_res, ld_out;
    int rows_per_mod;
    long long mod_stride;
    float eps;
    int layernorm;   // 1: subtract mean
    int gemma;       // 1: weight + 1
};

template <int NT, int MAXV>
__global__ void __launch_bounds__(NT) norm_kernel(const __grid_constant__ NormParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const int row = blockIdx.x;
    if (row >= p.rows) return;
    const int nvec = p.hidden >> 3;  // 8 bf16 per 16 bytes
    const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)row * p.ld_x);
    const uint4* rr = p.residual ? reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ld_res) : nullptr;
    uint4* ro = p.residual_out ? reinterpret_cast<uint4*>(p.residual_out + (size_t)row * p.ld_res) : nullptr;
    float h[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * NT;
        if (v < nvec) {
            uint4 a = xr[v];
            uint32_t aw[4] = {a.x, a.y, a.z, a.w};
            if (rr) {
                uint4 b = rr[v];
                uint32_t bw[4] = {b.x, b.y, b.z, b.w};
                uint32_t ow[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 fa = unpack_bf16x2(aw[j]), fb = unpack_bf16x2(bw[j]);
                    // the stored residual is the bf16 rounding of the sum; the norm sees that rounded value
                    ow[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
                    float2 fo = unpack_bf16x2(ow[j]);
                    h[i][2 * j] = fo.x;
                    h[i][2 * j + 1] = fo.y;
                }
                if (ro) ro[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 fa = unpack_bf16x2(aw[j]);
                    h[i][2 * j] = fa.x;
                    h[i][2 * j + 1] = fa.y;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s1 += h[i][j];
                s2 += h[i][j] * h[i][j];
            }
        }
    }
    float mean = 0.f;
    float inv;
    if (p.layernorm) {
        mean = block_sum<NT>(s1, red) / p.hidden;
        float var = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int v = threadIdx.x + i * NT;
            if (v < nvec) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float d = h[i][j] - mean;
                    var += d * d;
                }
            }
        }
        var = block_sum<NT>(var, red) / p.hidden;
        inv = rsqrtf(var + p.eps);
    } else {
        s2 = block_sum<NT>(s2, red);
        inv = rsqrtf(s2 / p.hidden + p.eps);
    }
    const int mrow = p.scale ? row / p.rows_per_mod : 0;
    uint4* outr = reinterpret_cast<uint4*>(p.out + (size_t)row * p.ld_out);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * NT;
        if (v < nvec) {
            float w[8], b[8], sc[8], sh[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { w[j] = 1.f; b[j] = 0.f; sc[j] = 0.f; sh[j] = 0.f; }
            if (p.weight) {
                uint4 t = reinterpret_cast<const uint4*>(p.weight)[v];
                uint32_t tw[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = unpack_bf16x2(tw[j]);
                    w[2 * j] = f.x + (p.gemma ? 1.f : 0.f);
                    w[2 * j + 1] = f.y + (p.gemma ? 1.f : 0.f);
                }
            }
            if (p.bias) {
                uint4 t = reinterpret_cast<const uint4*>(p.bias)[v];
                uint32_t tw[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = unpack_bf16x2(tw[j]);
                    b[2 * j] = f.x; b[2 * j + 1] = f.y;
                }
            }
            if (p.scale) {
                uint4 t = reinterpret_cast<const uint4*>(p.scale + (size_t)mrow * p.mod_stride)[v];
                uint4 u = reinterpret_cast<const uint4*>(p.shift + (size_t)mrow * p.mod_stride)[v];
                uint32_t tw[4] = {t.x, t.y, t.z, t.w};
                uint32_t uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = unpack_bf16x2(tw[j]), g = unpack_bf16x2(uw[j]);
                    sc[2 * j] = f.x; sc[2 * j + 1] = f.y;
                    sh[2 * j] = g.x; sh[2 * j + 1] = g.y;
                }
            }
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float y0 = (h[i][2 * j] - mean) * inv * w[2 * j] + b[2 * j];
                float y1 = (h[i][2 * j + 1] - mean) * inv * w[2 * j + 1] + b[2 * j + 1];
                if (p.scale) {
                    y0 = y0 * (1.f + sc[2 * j]) + sh[2 * j];
                    y1 = y1 * (1.f + sc[2 * j + 1]) + sh[2 * j + 1];
                }
                ow[j] = pack_bf16x2(y0, y1);
            }
            outr[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// QK-norm + RoPE + KV write.  One CTA per token, one warp per head (looping).
//   qkv: [T, (Hq + 2*Hkv) * D] (q heads, then k heads, then v heads)
//   q_out: [T, Hq, D];  K/V go to the paged cache [pages, 2, Hkv, page_size, D] and/or dense k_out/v_out
//   rotation: split-half ("neox") or interleaved pairs; angle = pos[axis_of_freq[i]][t] * inv_freq[i]
// ------------------------------------------------------------------------------------------------------------
struct RopeParams {
    const __nv_bfloat16* qkv;
    long long ld_qkv;
    __nv_bfloat16* q_out;
    __nv_bfloat16* k_out;  // dense [T, Hkv, D] or null
    __nv_bfloat16* v_out;
    __nv_bfloat16* cache;  // paged cache of this layer or null
    const int* positions;  // [n_axes, pos_stride], first T entries of each axis used
    long long pos_stride;
    const float* inv_freq;  // [rot_dim/2]
    const signed char* axis_of_freq;  // [rot_dim/2] or null (axis 0)
    const __nv_bfloat16* q_norm_w;  // [D] or null
    const __nv_bfloat16* k_norm_w;
    const int* token_req;    // [T] request index of each token (cache write)
    const int* cache_pos;    // [T] position of the token inside its sequence (cache write)
    const int* page_indptr;  // [B+1]
    const int* page_indices;
    int T, Hq, Hkv, D, rot_dim, page_size, interleaved, gemma_norm;
    float norm_eps;
    float attn_scale_q;  // multiplies q after rope (1.0 = off)
};

__global__ void __launch_bounds__(256) rope_kv_kernel(const __grid_constant__ RopeParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= p.T) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int D = p.D, half = p.rot_dim >> 1;
    const int nheads = p.Hq + 2 * p.Hkv;
    const __nv_bfloat16* row = p.qkv + (size_t)t * p.ld_qkv;
    // destination of K/V for this token
    size_t cache_tok = 0;
    bool write_cache = p.cache != nullptr;
    int page = 0, off = 0;
    if (write_cache) {
        const int b = p.token_req[t];
        const int cp = p.cache_pos[t];
        if (b < 0 || cp < 0) write_cache = false;
        else {
            page = p.page_indices[p.page_indptr[b] + cp / p.page_size];
            off = cp % p.page_size;
        }
    }
    (void)cache_tok;
    // the rotation angles depend on the token only: compute cos/sin once, every head reuses them
    __shared__ float s_cos[256], s_sin[256];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int axis = p.axis_of_freq ? p.axis_of_freq[i] : 0;
        const float ang = (float)p.positions[(size_t)axis * p.pos_stride + t] * p.inv_freq[i];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        s_cos[i] = cs;
        s_sin[i] = sn;
    }
    __syncthreads();
    for (int hidx = blockIdx.y * nwarps + warp; hidx < nheads; hidx += nwarps * gridDim.y) {
        const bool is_q = hidx < p.Hq;
        const bool is_k = !is_q && hidx < p.Hq + p.Hkv;
        const __nv_bfloat16* src = row + (size_t)hidx * D;
        __nv_bfloat16* dst;
        __nv_bfloat16* dst2 = nullptr;
        if (is_q) dst = p.q_out + ((size_t)t * p.Hq + hidx) * D;
        else {
            const int kvh = is_k ? hidx - p.Hq : hidx - p.Hq - p.Hkv;
            __nv_bfloat16* dense = is_k ? p.k_out : p.v_out;
            dst = dense ? dense + ((size_t)t * p.Hkv + kvh) * D : nullptr;
            if (write_cache)
                dst2 = p.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * p.Hkv + kvh) * p.page_size + off) * D;
        }
        if (!is_q && !is_k) {  // V: plain copy
            for (int i = lane * 2; i < D; i += 64) {
                uint32_t v = *reinterpret_cast<const uint32_t*>(src + i);
                if (dst) *reinterpret_cast<uint32_t*>(dst + i) = v;
                if (dst2) *reinterpret_cast<uint32_t*>(dst2 + i) = v;
            }
            continue;
        }
        const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
        float inv = 1.0f;
        if (nw) {
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) {
                float x = __bfloat162float(src[i]);
                ss += x * x;
            }
            ss = warp_sum(ss);
            inv = rsqrtf(ss / D + p.norm_eps);
        }
        const float qs = is_q ? p.attn_scale_q : 1.0f;
        // rotated part
        for (int i = lane; i < half; i += 32) {
            const int i0 = p.interleaved ? 2 * i : i;
            const int i1 = p.interleaved ? 2 * i + 1 : i + half;
            float x0 = __bfloat162float(src[i0]), x1 = __bfloat162float(src[i1]);
            if (nw) {
                // norm output is rounded to bf16 before the rotation, as a separate norm op would do
                float w0 = __bfloat162float(nw[i0]) + (p.gemma_norm ? 1.f : 0.f);
                float w1 = __bfloat162float(nw[i1]) + (p.gemma_norm ? 1.f : 0.f);
                x0 = __bfloat162float(__float2bfloat16(x0 * inv * w0));
                x1 = __bfloat162float(__float2bfloat16(x1 * inv * w1));
            }
            const float sn = s_sin[i], cs = s_cos[i];
            const float y0 = (x0 * cs - x1 * sn) * qs, y1 = (x1 * cs + x0 * sn) * qs;
            const __nv_bfloat16 b0 = __float2bfloat16(y0), b1 = __float2bfloat16(y1);
            if (dst) { dst[i0] = b0; dst[i1] = b1; }
            if (dst2) { dst2[i0] = b0; dst2[i1] = b1; }
        }
        // pass-through part (partial rotary)
        for (int i = p.rot_dim + lane; i < D; i += 32) {
            float x = __bfloat162float(src[i]);
            if (nw) x = __bfloat162float(__float2bfloat16(x * inv * (__bfloat162float(nw[i]) + (p.gemma_norm ? 1.f : 0.f))));
            const __nv_bfloat16 b = __float2bfloat16(x * qs);
            if (dst) dst[i] = b;
            if (dst2) dst2[i] = b;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// small elementwise kernels
// ------------------------------------------------------------------------------------------------------------
// out[r, i] = act(x[r, i]) * x[r, I + i]   (x: [rows, 2I] halves layout)  act: 0 silu, 1 gelu-tanh
__global__ void act_mul_kernel(const __nv_bfloat16* x, __nv_bfloat16* out, long long rows, int I, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const long long n = rows * (long long)I;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / I;
        const int i = (int)(idx - r * I);
        const float g = __bfloat162float(x[r * 2 * I + i]), u = __bfloat162float(x[r * 2 * I + I + i]);
        out[idx] = __float2bfloat16((act == 0 ? silu_f(g) : gelu_tanh_f(g)) * u);
    }
}

// out[t, :] = table[ids[t] - vocab_start, :] if the id falls in [vocab_start, vocab_end), else 0
__global__ void embed_gather_kernel(const long long* ids, const __nv_bfloat16* table, __nv_bfloat16* out, int T,
                                    int hidden, long long vocab_start, long long vocab_end, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= T) return;
    const long long id = ids[t];
    const bool ok = id >= vocab_start && id < vocab_end;
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id - vocab_start : 0) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * hidden);
    for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x) {
        uint4 a = ok ? src[v] : make_uint4(0, 0, 0, 0);
        if (scale != 1.0f && ok) {
            uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16x2(w[j]);
                w[j] = pack_bf16x2(f.x * scale, f.y * scale);
            }
            a = make_uint4(w[0], w[1], w[2], w[3]);
        }
        dst[v] = a;
    }
}

// out = x + gate[row / rows_per_mod] * y      (gated residual of AdaLN blocks); gate may be null (plain add).
// Eight bf16 per thread (16-byte loads and stores); hidden must be a multiple of 8.
__global__ void gated_residual_kernel(const __nv_bfloat16* x, const __nv_bfloat16* y, const __nv_bfloat16* gate,
                                      __nv_bfloat16* out, long long rows, int hidden, int rows_per_mod,
                                      long long gate_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int hv = hidden >> 3;
    const long long n = rows * (long long)hv;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / hv;
        const int i = (int)(idx - r * hv) << 3;
        const uint4 xv = *reinterpret_cast<const uint4*>(x + r * hidden + i);
        const uint4 yv = *reinterpret_cast<const uint4*>(y + r * hidden + i);
        uint4 gv = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);   // bf16 ones
        if (gate) gv = *reinterpret_cast<const uint4*>(gate + (r / rows_per_mod) * gate_stride + i);
        const uint32_t* xa = &xv.x; const uint32_t* ya = &yv.x; const uint32_t* ga = &gv.x;
        uint4 ov; uint32_t* oa = &ov.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 xf = unpack_bf16x2(xa[j]), yf = unpack_bf16x2(ya[j]), gf = unpack_bf16x2(ga[j]);
            oa[j] = pack_bf16x2(xf.x + gf.x * yf.x, xf.y + gf.y * yf.y);
        }
        *reinterpret_cast<uint4*>(out + r * hidden + i) = ov;
    }
}

// Merge two partial attention results over disjoint key sets (a cached prefix and the fresh tokens):
//   w_i = exp(lse_i - max) / sum, out = w_a * o_a + w_b * o_b.  lse = -inf marks an empty key set.
// o_*: [rows = tokens * heads, D] bf16 with row stride D, lse_*: [rows] fp32. Optionally writes the merged lse.
__global__ void attn_merge_kernel(const __nv_bfloat16* oa, const float* la, const __nv_bfloat16* ob, const float* lb,
                                  __nv_bfloat16* out, float* lse_out, long long rows, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int dv = D >> 3;
    const long long n = rows * (long long)dv;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / dv;
        const int i = (int)(idx - r * dv) << 3;
        const float a = la[r], b = lb[r];
        const float m = fmaxf(a, b);
        float wa = 0.f, wb = 0.f;
        if (m > -INFINITY) {
            const float ea = __expf(a - m), eb = __expf(b - m);
            const float inv = 1.0f / (ea + eb);
            wa = ea * inv; wb = eb * inv;
            if (lse_out && i == 0) lse_out[r] = m + __logf(ea + eb);
        } else if (lse_out && i == 0) {
            lse_out[r] = -INFINITY;
        }
        const uint4 av = *reinterpret_cast<const uint4*>(oa + r * D + i);
        const uint4 bv = *reinterpret_cast<const uint4*>(ob + r * D + i);
        const uint32_t* aa = &av.x; const uint32_t* ba = &bv.x;
        uint4 ov; uint32_t* o = &ov.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 af = unpack_bf16x2(aa[j]), bf = unpack_bf16x2(ba[j]);
            o[j] = pack_bf16x2(wa * af.x + wb * bf.x, wa * af.y + wb * bf.y);
        }
        *reinterpret_cast<uint4*>(out + r * D + i) = ov;
    }
}

// Snake activation of neural audio codecs: y = x + sin^2(alpha_c * x) / alpha_c, alpha per channel, x: [B, C, T].
// One pass over the tensor instead of the five elementwise kernels of the composed expression.
template <typename T>
__global__ void snake_kernel(const T* x, const float* alpha, T* out, long long n, int C, long long Tlen) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)((i / Tlen) % C);
        const float a = alpha[c];
        float v;
        if constexpr (sizeof(T) == 4) v = x[i]; else v = __bfloat162float(x[i]);
        const float sn = __sinf(a * v);
        const float y = v + sn * sn / (a + 1e-9f);
        if constexpr (sizeof(T) == 4) out[i] = y; else out[i] = __float2bfloat16(y);
    }
}

// Classifier-free guidance combine + optional per-token renorm + Euler step, fp32 latents.
//   v = v_uncond + s_text * (v_cond - v_uncond) [+ s_img * (v_cond_img - v_uncond_img) when given]
//   renorm (mode 1, per row): v *= min(1, |v_cond| / |v|) with clamp [renorm_min, 1]
//   x_next = x + dt * v
struct CfgParams {
    const float* v_cond; const float* v_uncond; const float* v_img;  // v_img may be null
    const float* x; float* x_next; float* v_out;
    int rows, cols;
    float s_text, s_img, dt, renorm_min;
    int renorm;
};
__global__ void __launch_bounds__(128) cfg_combine_kernel(const __grid_constant__ CfgParams p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    if (r >= p.rows) return;
    const size_t base = (size_t)r * p.cols;
    float nc = 0.f, nv = 0.f;
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
        const float c = p.v_cond[base + i], u = p.v_uncond[base + i];
        float v;
        if (p.v_img) {
            // two-level guidance: text guidance on top of the image-conditioned branch
            const float t = u + p.s_text * (c - u);
            const float im = p.v_img[base + i];
            v = im + p.s_img * (t - im);
        } else {
            v = u + p.s_text * (c - u);
        }
        nc += c * c;
        nv += v * v;
    }
    float scale = 1.0f;
    if (p.renorm) {
        nc = block_sum<128>(nc, red);
        nv = block_sum<128>(nv, red);
        scale = sqrtf(nc) / (sqrtf(nv) + 1e-8f);
        scale = fminf(fmaxf(scale, p.renorm_min), 1.0f);
    }
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
        const float c = p.v_cond[base + i], u = p.v_uncond[base + i];
        float v;
        if (p.v_img) {
            const float t = u + p.s_text * (c - u);
            const float im = p.v_img[base + i];
            v = im + p.s_img * (t - im);
        } else {
            v = u + p.s_text * (c - u);
        }
        v *= scale;
        if (p.v_out) p.v_out[base + i] = v;
        if (p.x_next) p.x_next[base + i] = p.x[base + i] + p.dt * v;
    }
}

// uint8 / float image -> [-1, 1] (or any affine): out = x * a + b
__global__ void affine_kernel(const float* x, __nv_bfloat16* out_bf16, float* out_f32, long long n, float a,
                              float b) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float y = x[i] * a + b;
        if (out_bf16) out_bf16[i] = __float2bfloat16(y);
        if (out_f32) out_f32[i] = y;
    }
}

// Decode-loop state advance, on device so that a captured step can be replayed without host planning:
//   kv_lens[b] += 1; positions[:, b] += 1; cache_pos[b] += 1; input_ids[b] = sampled[b]
//   Entries with kv_lens == 0 are padding of a captured batch and never advance.
__global__ void advance_decode_kernel(int* kv_lens, int* positions, int* cache_pos, long long* input_ids,
                                      const long long* sampled, const int* active, int B, int n_axes,
                                      int pos_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    if (input_ids && sampled) input_ids[b] = sampled[b];
    if (active && !active[b]) return;
    if (kv_lens[b] <= 0) return;
    kv_lens[b] += 1;
    for (int a = 0; a < n_axes; ++a) positions[(size_t)a * pos_stride + b] += 1;
    if (cache_pos) cache_pos[b] += 1;
}

}  // namespace mstar

using namespace mstar;

MSTAR_API int mstar_norm(const void* x, const void* residual, void* residual_out, const void* weight,
                         const void* bias, const void* scale, const void* shift, void* out, int rows, int hidden,
                         long long ld_x, long long ld_res, long long ld_out, int rows_per_mod, long long mod_stride,
                         float eps, int layernorm, int gemma, void* stream_) {
    if (rows <= 0) return 0;
    if (hidden % 8) return set_error("norm: hidden must be a multiple of 8", cudaSuccess);
    if (hidden > 16384) return set_error("norm: hidden > 16384 not supported", cudaSuccess);
    NormParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (__nv_bfloat16*)residual_out,
                 (const __nv_bfloat16*)weight, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)scale,
                 (const __nv_bfloat16*)shift, (__nv_bfloat16*)out, rows, hidden, ld_x, ld_res, ld_out,
                 rows_per_mod > 0 ? rows_per_mod : 1, mod_stride, eps, layernorm, gemma};
    cudaStream_t s = (cudaStream_t)stream_;
    const int nvec = hidden / 8;
    cudaError_t e;
    if (nvec <= 128) e = launch_pdl(norm_kernel<128, 1>, dim3(rows), dim3(128), 0, s, p);
    else if (nvec <= 256) e = launch_pdl(norm_kernel<128, 2>, dim3(rows), dim3(128), 0, s, p);
    else if (nvec <= 512) e = launch_pdl(norm_kernel<256, 2>, dim3(rows), dim3(256), 0, s, p);
    else if (nvec <= 1024) e = launch_pdl(norm_kernel<256, 4>, dim3(rows), dim3(256), 0, s, p);
    else e = launch_pdl(norm_kernel<256, 8>, dim3(rows), dim3(256), 0, s, p);
    return e == cudaSuccess ? 0 : set_error("norm launch", e);
}

MSTAR_API int mstar_rope_kv(const void* qkv, long long ld_qkv, void* q_out, void* k_out, void* v_out, void* cache,
                            const int* positions, long long pos_stride, const float* inv_freq,
                            const signed char* axis_of_freq, const void* q_norm_w, const void* k_norm_w, const int* token_req, const int* cache_pos,
                            const int* page_indptr, const int* page_indices, int T, int Hq, int Hkv, int D,
                            int rot_dim, int page_size, int interleaved, int gemma_norm, float norm_eps,
                            float q_scale, void* stream_) {
    if (T <= 0) return 0;
    RopeParams p{(const __nv_bfloat16*)qkv, ld_qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out,
                 (__nv_bfloat16*)v_out, (__nv_bfloat16*)cache, positions, pos_stride, inv_freq, axis_of_freq,
                 (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, token_req, cache_pos, page_indptr,
                 page_indices, T, Hq, Hkv, D, rot_dim, page_size, interleaved, gemma_norm, norm_eps, q_scale};
    const int nheads = Hq + 2 * Hkv;
    const int gy = T >= 1024 ? 1 : (nheads + 7) / 8;   // few tokens: one warp per head across several CTAs
    cudaError_t e = launch_pdl(rope_kv_kernel, dim3(T, gy), dim3(256), 0, (cudaStream_t)stream_, p);
    return e == cudaSuccess ? 0 : set_error("rope_kv launch", e);
}

static inline int grid_for(long long n, int bs) {
    long long g = (n + bs - 1) / bs;
    const long long cap = 148LL * 16;
    return (int)(g > cap ? cap : (g < 1 ? 1 : g));
}

MSTAR_API int mstar_act_mul(const void* x, void* out, long long rows, int I, int act, void* stream_) {
    if (rows <= 0) return 0;
    act_mul_kernel<<<grid_for(rows * I, 256), 256, 0, (cudaStream_t)stream_>>>((const __nv_bfloat16*)x,
                                                                               (__nv_bfloat16*)out, rows, I, act);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("act_mul launch", e);
}

MSTAR_API int mstar_embed_gather(const long long* ids, const void* table, void* out, int T, int hidden,
                                 long long vocab_start, long long vocab_end, float scale, void* stream_) {
    if (T <= 0) return 0;
    if (hidden % 8) return set_error("embed: hidden must be a multiple of 8", cudaSuccess);
    cudaError_t e = launch_pdl(embed_gather_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream_, ids,
                               (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, hidden, vocab_start, vocab_end, scale);
    return e == cudaSuccess ? 0 : set_error("embed launch", e);
}

MSTAR_API int mstar_gated_residual(const void* x, const void* y, const void* gate, void* out, long long rows,
                                   int hidden, int rows_per_mod, long long gate_stride, void* stream_) {
    if (rows <= 0) return 0;
    if (hidden % 8) return set_error("gated_residual: hidden must be a multiple of 8", cudaSuccess);
    gated_residual_kernel<<<grid_for(rows * (hidden / 8), 256), 256, 0, (cudaStream_t)stream_>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, rows,
        hidden, rows_per_mod > 0 ? rows_per_mod : 1, gate_stride);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("gated_residual launch", e);
}

// Activation quantisation for the block-scaled fp8 GEMM: one scale per token row and 128-wide K block
// (scale = max|x| / 448), e4m3 bytes out, scales written transposed ([K block][token]) as the GEMM reads them.
// One warp per (row, K block): four elements per lane. Optional row gather (src_row[r], negative = zero row) serves
// the mixture-of-experts path, which quantises the token copies in expert order.
namespace mstar {
__global__ void quant_fp8_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ src_row,
                                       int src_div, unsigned char* __restrict__ out, long long ldo,
                                       float* __restrict__ scale_t, int ld_s, int rows, int K) {
    const int kblocks = (K + 127) / 128;
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)rows * kblocks) return;
    const int r = (int)(w / kblocks), kb = (int)(w - (long long)r * kblocks);
    long long sr = r;
    if (src_row != nullptr) {
        const int q = src_row[r];
        sr = q < 0 ? -1 : q / src_div;
    }
    const int k0 = kb * 128 + lane * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (sr >= 0 && k0 < K) {       // K is a multiple of 4
        const uint2 raw = *reinterpret_cast<const uint2*>(x + sr * ldx + k0);
        const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-12f) * (1.0f / 448.0f);
    const float inv = 1.0f / scale;
    if (k0 < K) {
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            packed |= (uint32_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        *reinterpret_cast<uint32_t*>(out + (long long)r * ldo + k0) = packed;
    }
    if (lane == 0) scale_t[(long long)kb * ld_s + r] = scale;
}
}  // namespace mstar

MSTAR_API int mstar_quant_fp8_1x128(const void* x, long long ldx, const int* src_row, int src_div, void* out,
                                    long long ldo, float* scale_t, int ld_s, int rows, int K, void* stream_) {
    if (rows <= 0) return 0;
    if (K % 4 || ldx % 4 || ldo % 4) return set_error("quant_fp8: K and the leading dimensions must be multiples of 4", cudaSuccess);
    const long long warps = (long long)rows * ((K + 127) / 128);
    const long long blocks = (warps * 32 + 255) / 256;
    quant_fp8_1x128_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream_>>>(
        (const __nv_bfloat16*)x, ldx, src_row, src_div < 1 ? 1 : src_div, (unsigned char*)out, ldo, scale_t, ld_s, rows, K);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("quant_fp8 launch", e);
}

MSTAR_API int mstar_snake(const void* x, const float* alpha, void* out, long long n, int C, long long Tlen, int is_f32,
                          void* stream_) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream_;
    if (is_f32) snake_kernel<float><<<grid_for(n, 256), 256, 0, s>>>((const float*)x, alpha, (float*)out, n, C, Tlen);
    else snake_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, s>>>((const __nv_bfloat16*)x, alpha, (__nv_bfloat16*)out, n, C, Tlen);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("snake launch", e);
}

MSTAR_API int mstar_attn_merge(const void* oa, const float* la, const void* ob, const float* lb, void* out,
                               float* lse_out, long long rows, int D, void* stream_) {
    if (rows <= 0) return 0;
    if (D % 8) return set_error("attn_merge: head dim must be a multiple of 8", cudaSuccess);
    attn_merge_kernel<<<grid_for(rows * (D / 8), 256), 256, 0, (cudaStream_t)stream_>>>(
        (const __nv_bfloat16*)oa, la, (const __nv_bfloat16*)ob, lb, (__nv_bfloat16*)out, lse_out, rows, D);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("attn_merge launch", e);
}

MSTAR_API int mstar_cfg_combine(const float* v_cond, const float* v_uncond, const float* v_img, const float* x,
                                float* x_next, float* v_out, int rows, int cols, float s_text, float s_img, float dt,
                                int renorm, float renorm_min, void* stream_) {
    if (rows <= 0) return 0;
    CfgParams p{v_cond, v_uncond, v_img, x, x_next, v_out, rows, cols, s_text, s_img, dt, renorm_min, renorm};
    cfg_combine_kernel<<<rows, 128, 0, (cudaStream_t)stream_>>>(p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("cfg_combine launch", e);
}

MSTAR_API int mstar_affine(const float* x, void* out_bf16, float* out_f32, long long n, float a, float b,
                           void* stream_) {
    if (n <= 0) return 0;
    affine_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream_>>>(x, (__nv_bfloat16*)out_bf16, out_f32, n, a, b);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("affine launch", e);
}

MSTAR_API int mstar_advance_decode(int* kv_lens, int* positions, int* cache_pos, long long* input_ids,
                                   const long long* sampled, const int* active, int B, int n_axes, int pos_stride,
                                   void* stream_) {
    if (B <= 0) return 0;
    advance_decode_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream_>>>(kv_lens, positions, cache_pos,
                                                                             input_ids, sampled, active, B, n_axes, pos_stride);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : set_error("advance launch", e);
}
