// Library-wide host state: error text, status word, wait limit, TMA descriptor encoding.
#include <string.h>
#include <stdlib.h>
#include <stdio.h>
#include <mutex>
#include <cstdlib>
#include "host_common.h"

namespace mstar {

static char g_err[512] = "";
static KernelStatus* g_status[kMaxDevices] = {};
// Limit of every bounded device wait. 2 s suits decode-sized steps; deployments whose steps take seconds (video DiTs
// on a tensor- / sequence-parallel mesh: the ranks' first steps differ by allocator growth alone) raise it with
// MSTAR_WAIT_LIMIT_MS or mstar_set_wait_limit_ns.
static unsigned long long initial_wait_limit() {
    const char* e = getenv("MSTAR_WAIT_LIMIT_MS");
    const long long ms = e != nullptr ? atoll(e) : 0;
    return ms > 0 ? (unsigned long long)ms * 1000000ull : MSTAR_WAIT_LIMIT_NS_DEFAULT;
}
static unsigned long long g_wait_limit = initial_wait_limit();
static int g_sms[kMaxDevices] = {};
static std::mutex g_mu;

int set_error(const char* msg, cudaError_t e) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (e != cudaSuccess)
        snprintf(g_err, sizeof(g_err), "%s: %s", msg, cudaGetErrorString(e));
    else
        snprintf(g_err, sizeof(g_err), "%s", msg);
    return -1;
}

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
    return dev < kMaxDevices ? dev : kMaxDevices - 1;
}

KernelStatus* status_ptr() {
    const int dev = current_device();
    if (g_status[dev] == nullptr) {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_status[dev] == nullptr) {
            KernelStatus* p = nullptr;
            if (cudaMalloc(&p, sizeof(KernelStatus)) == cudaSuccess) {      // lands on the current device
                cudaMemset(p, 0, sizeof(KernelStatus));
                g_status[dev] = p;
            }
        }
    }
    return g_status[dev];
}

unsigned long long wait_limit_ns() { return g_wait_limit; }

static int g_pdl = -1;
bool pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("MSTAR_PDL");
        // on unless MSTAR_PDL=0: with cluster split-K and the short prologues the decode step of the 3B model runs
        // 4.29 ms with it against 4.83 ms without (it used to be slower, when every kernel's prologue was long)
        g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return g_pdl == 1;
}

int device_sm_count() {
    const int dev = current_device();
    if (g_sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            g_sms[dev] = n;
        else
            g_sms[dev] = 148;
    }
    return g_sms[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static EncodeTiledFn get_encode() {
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || fn == nullptr) {
            set_error("cuTensorMapEncodeTiled entry point not found", e);
            return nullptr;
        }
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    return g_encode;
}

int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const unsigned long long* dims,
              const unsigned long long* strides_bytes, const unsigned int* box, int swizzle_128b) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return -1;
    cuuint64_t gdim[5];
    cuuint64_t gstr[5];
    cuuint32_t bx[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i];
    }
    CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                             : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[160];
        snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed (CUresult %d) rank=%d dim0=%llu dim1=%llu", (int)r,
                 rank, dims[0], rank > 1 ? dims[1] : 0ull);
        return set_error(buf, cudaSuccess);
    }
    return 0;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, int rows, int cols, int ld, int box_rows, int box_cols) {
    unsigned long long dims[2] = {(unsigned long long)cols, (unsigned long long)rows};
    unsigned long long strides[2] = {2ull, (unsigned long long)ld * 2ull};
    unsigned int box[2] = {(unsigned int)box_cols, (unsigned int)box_rows};
    return make_tmap(out, base, 2, 2, dims, strides, box, 1);
}

}  // namespace mstar

using namespace mstar;

MSTAR_API const char* mstar_last_error() { return g_err; }

// Copies the status word to the host and clears it when `clear` is non-zero. Returns the code (0 = ok).
MSTAR_API unsigned int mstar_read_status(unsigned int* out4, int clear) {
    KernelStatus* p = status_ptr();
    KernelStatus h = {0, 0, 0, 0};
    if (p == nullptr) return 0xffffffffu;
    cudaMemcpy(&h, p, sizeof(h), cudaMemcpyDeviceToHost);
    if (out4) {
        out4[0] = h.code; out4[1] = h.block; out4[2] = h.aux0; out4[3] = h.aux1;
    }
    if (clear && h.code != 0) cudaMemset(p, 0, sizeof(h));
    return h.code;
}

// Queues a copy of the current device's status word (16 bytes) into `host_dst16` (pinned host memory) on `stream`:
// a serving loop reads the word with the batch's results, after the event it already waits for, instead of paying
// a synchronous copy per batch. The word is not cleared; mstar_read_status(.., 1) does that once a code was seen.
namespace mstar {
static PrefetchHint g_prefetch[kMaxDevices];

PrefetchHint take_prefetch_hint() {
    PrefetchHint& h = g_prefetch[current_device()];
    PrefetchHint out = h;
    h = PrefetchHint{};
    return out;
}
}  // namespace mstar
using mstar::g_prefetch;
using mstar::PrefetchHint;

// The next GEMM / decode-attention launch on the current device prefetches [ptr, ptr + bytes) into the L2 while it
// runs (bytes 0: only the evict-first marking of its own operand, when l2_hints is set). The hint is used once.
MSTAR_API void mstar_prefetch_hint(const void* ptr, unsigned long long bytes, int l2_hints) {
    PrefetchHint& h = g_prefetch[current_device()];
    const unsigned long long mis = reinterpret_cast<unsigned long long>(ptr) & 15ull;
    if (ptr != nullptr && mis && bytes > 16) { ptr = static_cast<const char*>(ptr) + (16 - mis); bytes -= 16 - mis; }
    h.ptr = ptr;
    h.bytes = ptr != nullptr ? bytes : 0;
    h.l2_hints = l2_hints;
}

MSTAR_API int mstar_status_copy_async(void* host_dst16, void* stream) {
    KernelStatus* p = status_ptr();
    if (p == nullptr) return set_error("status word could not be allocated", cudaSuccess);
    cudaError_t e = cudaMemcpyAsync(host_dst16, p, sizeof(KernelStatus), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : set_error("status copy failed", e);
}

MSTAR_API void mstar_set_wait_limit_ns(unsigned long long ns) { g_wait_limit = ns; }
MSTAR_API unsigned long long mstar_get_wait_limit_ns() { return g_wait_limit; }
MSTAR_API int mstar_sm_count() { return device_sm_count(); }
MSTAR_API void mstar_set_pdl(int on) { g_pdl = on ? 1 : 0; }
