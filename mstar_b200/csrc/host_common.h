// Host-side helpers shared by all kernel launchers of the library: last-error text, the device status word,
// the wait limit for device-side waits, and TMA tensor-map encoding through the driver entry point (looked up
// at run time, so the library links against cudart only).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "common.cuh"

namespace mstar {

// CUDA state is per device while a process may drive several GPUs (one worker thread per GPU): everything the
// launchers cache (status word, kernel attributes already set, SM count, cluster occupancy) is indexed by device.
constexpr int kMaxDevices = 64;
int current_device();                               // index of the current CUDA device, clamped to [0, kMaxDevices)

// "Has this been done on the current device yet?" flag for one-time per-device set-up such as
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize), which applies to the function on ONE device only.
struct PerDeviceFlag {
    bool done[kMaxDevices] = {};
    bool& operator()() { return done[current_device()]; }
};

// What the NEXT weight-streaming kernel launched on the current device should ask the L2 to fetch while it runs
// (the weights of the kernel after it). Set by mstar_prefetch_hint, taken (and cleared) by the next launcher that
// supports it; l2_hints also makes that kernel mark its own streamed operand evict-first.
struct PrefetchHint {
    const void* ptr = nullptr;
    unsigned long long bytes = 0;
    int l2_hints = 0;
};
PrefetchHint take_prefetch_hint();

int set_error(const char* msg, cudaError_t e);      // stores the message, returns -1
KernelStatus* status_ptr();                         // status word of the CURRENT device (lazily made, one per device)
unsigned long long wait_limit_ns();
int device_sm_count();                              // SM count of the current device

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements); box =
// box_rows x box_cols, SWIZZLE_128B (box_cols * 2 bytes must be 128).
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, int rows, int cols, int ld, int box_rows, int box_cols);
// Generic form: up to 5 dims, sizes/strides innermost first, strides in bytes (stride[0] implied by elem size).
int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const unsigned long long* dims,
              const unsigned long long* strides_bytes, const unsigned int* box, int swizzle_128b);

bool pdl_enabled();

// Launch with the programmatic-stream-serialization attribute (when enabled), so that the kernel's prologue and
// its independent prefetches overlap the tail of the previous kernel in the stream.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, as thread-block clusters of `cluster_z` CTAs along grid z (grid.z must be a multiple of cluster_z).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster_z(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, unsigned cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = cluster_z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace mstar
