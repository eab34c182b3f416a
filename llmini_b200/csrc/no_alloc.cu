// b2_materialize_master_static: requantise one FP32 master tensor to NVFP4 without taking any
// scratch from the caller and without allocating.
//
// Who needs this: code that is handed only the master tensor and the destination NVFP4 triple
// and owns no scratch arena of its own — a checkpoint-export or evaluation hook running beside
// the trainer, or an embedder whose device-memory budget is frozen before the first step.  For
// such a caller cudaMalloc is either unavailable (all of HBM is already reserved by the
// trainer's pools) or harmful (it synchronises the whole device, stalling the training stream),
// and the regular entry point b2_materialize_master wants two scratch buffers (the per-chunk
// maxima and the tensor maximum) that it has nowhere to take from.
//
// The scratch therefore lives in this library image: one file-scope __device__ array (128 KiB +
// 256 B) that every GPU carries, from the moment this module is loaded onto it until the process
// exits.  Its size bounds the tensor: at most B2_STATIC_MAX_ELEMENTS values per call.
//
// First call on a device: the CUDA runtime loads modules lazily by default, so the module holding the
// array is created on a device by the first cudaGetSymbolAddress there, and that is when the driver sets
// the 128 KiB aside.  A caller whose device memory is about to be fully reserved therefore makes one
// warm-up call per device (len = 0 is enough) at start-up, before the reservation and outside any
// stream capture; from the second call on nothing is looked up, loaded or reserved.  The address is
// cached for the life of the process and is stale after cudaDeviceReset.
#include <cuda_runtime.h>

#include <mutex>

#include "internal.h"

namespace {

constexpr uint32_t kMaxElements = B2_STATIC_MAX_ELEMENTS;
constexpr uint32_t kMaxChunks = kMaxElements / 2048;  // one maximum per 2048-value chunk
constexpr uint32_t kAmaxSlot = kMaxChunks;            // the tensor maximum sits after the chunk maxima

// Host code must never hand this name to a kernel: on the host it is only a stand-in for the
// symbol.  The device address is looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[kMaxChunks + 64];

struct PerDevice {
    float *scratch = nullptr;
    int grid_cap = 0;
};

// First use on a device resolves the array's device address and the SM count, with that device
// current.  Later calls on the same device reuse both.
cudaError_t per_device(PerDevice &out) {
    static std::mutex mu;
    static PerDevice cache[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev].scratch == nullptr) {
        float *p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_scratch);
        if (e != cudaSuccess) return e;
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        cache[dev].scratch = p;
        cache[dev].grid_cap = sms * 8;
    }
    out = cache[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int b2_materialize_master_static(uint8_t *d_bytes, uint8_t *d_scales, float *d_global_scale,
                                            const float *d_master, uint32_t len, uint32_t scale_layout,
                                            void *stream) {
    if (!d_bytes || !d_scales || !d_global_scale || !d_master) return B2_ERROR_INVALID_VALUE;
    if (len % 16 != 0 || scale_layout > B2_SCALES_RAW) return B2_ERROR_INVALID_VALUE;
    if (scale_layout == B2_SCALES_CSF && len % 128 != 0) return B2_ERROR_INVALID_VALUE;
    // larger tensors do not fit the built-in scratch: use b2_materialize_master with caller scratch
    if (len > kMaxElements) return B2_ERROR_INVALID_VALUE;
    PerDevice dev;
    cudaError_t e = per_device(dev);
    if (e != cudaSuccess) return (int)e;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    float *chunk_amax = dev.scratch;
    float *amax = dev.scratch + kAmaxSlot;
    // Nothing in the scratch has to start at zero: the chunk pass overwrites entries
    // [0, ceil(len / 2048)) and the reduction overwrites the tensor maximum before the encode
    // pass reads it; entries left over from a longer earlier call are never read.
    e = b2::launch_tensor_chunk_amax(d_master, chunk_amax, len, s);
    if (e == cudaSuccess) e = b2::launch_tensor_amax_from_chunks(chunk_amax, amax, (len + 2047) / 2048, s);
    if (e == cudaSuccess)
        e = b2::launch_quantize_flat(d_master, nullptr, nullptr, 0.f, 0, amax, d_bytes, d_scales, d_global_scale,
                                     len / 16, (int)scale_layout, dev.grid_cap, s);
    return (int)e;
}
