// Host-I/O NVFP4 quantize that never allocates: the device-side staging of the
// input rows, the codes and the block scales lives in a fixed array that is
// part of the library image instead of buffers obtained from the allocator.
//
// For callers that must not allocate once they are running — the memory of the
// device is fully budgeted, the allocator is frozen, or the implicit device-wide
// synchronisation of an allocation is not acceptable where the call is made.
// The price is a fixed ceiling (kStaticScratchBytes for input + codes + scales
// of one call) and one array per device shared by every call: two calls that
// overlap in time on the same device overwrite each other's staging.
#include "runtime.hpp"

namespace axb {
namespace {

constexpr uint64_t kStaticScratchBytes = 8ull << 20;  // 8 MiB: 639 rows of 5120 BF16 values with their codes and scales

static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];

inline uint64_t align256(uint64_t v) { return (v + 255u) & ~255ull; }

// Address of the array on the current device, looked up once per device.  With CUDA's lazy module loading that
// first lookup is also the moment the driver loads the module holding the array and reserves its 8 MiB on the
// device (it may synchronise the device while doing so, and it fails when the device has no room left): the
// first call per device belongs to start-up, before the caller freezes its memory budget and before any capture.
uint8_t *static_scratch() {
    static uint8_t *base[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!base[dev]) {
        uint8_t *ptr = nullptr;
        if (cudaGetSymbolAddress((void **)&ptr, g_static_scratch) != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            return nullptr;
        }
        base[dev] = ptr;
    }
    return base[dev];
}

}  // namespace
}  // namespace axb

using namespace axb;

extern "C" uint64_t axiom_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int axiom_b200_nvfp4_quantize_bf16_host_static(
        int device, const void *input_bf16_host, uint32_t rows, uint32_t cols, float global_scale,
        uint32_t scale_layout, uint8_t *out_codes_host, uint8_t *out_scales_host, void *stream) {
    if (!input_bf16_host || !out_codes_host || !out_scales_host || rows == 0u || cols == 0u ||
        (cols % kGroup) != 0u || !valid_scale(global_scale) || scale_layout > AXIOM_SCALE_LAYOUT_TILED ||
        (uint64_t)rows * (cols / 8u) > 0xffffffffull) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    const uint64_t in_bytes = (uint64_t)rows * cols * 2u, code_bytes = (uint64_t)rows * cols / 2u;
    const uint64_t scale_bytes = axiom_nvfp4_scale_plane_bytes(rows, cols / kGroup, scale_layout);
    const uint64_t off_codes = align256(in_bytes), off_scales = off_codes + align256(code_bytes);
    if (off_scales + scale_bytes > kStaticScratchBytes) return AXIOM_ERR_BUDGET;  // beyond the fixed ceiling
    int rc = select_device(device);
    if (rc != AXIOM_OK) return rc;
    uint8_t *dev = static_scratch();
    if (!dev) return AXIOM_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;
    // Once anything has been enqueued, every way out synchronises the stream first: the caller's host buffers
    // and the shared array must be idle when the call returns, also when a later step fails.
    auto fail_after_enqueue = [&]() {
        (void)cudaStreamSynchronize(s);
        (void)cudaGetLastError();
        return (int)AXIOM_ERR_CUDA;
    };
    if (cudaMemcpyAsync(dev, input_bf16_host, (size_t)in_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) return fail_after_enqueue();
    // The tiled plane pads rows to 128 and groups to 4; the kernel writes real cells only and the
    // pad cells must read as zero, so the plane starts from zero on every call (a previous call
    // of another shape left its bytes here).
    if (scale_layout == AXIOM_SCALE_LAYOUT_TILED &&
        cudaMemsetAsync(dev + off_scales, 0, (size_t)scale_bytes, s) != cudaSuccess) {
        return fail_after_enqueue();
    }
    launch_nvfp4_quantize_bf16(dev, rows, cols, global_scale, dev + off_codes, dev + off_scales, scale_layout, s);
    if (cudaGetLastError() != cudaSuccess) return fail_after_enqueue();
    if (cudaMemcpyAsync(out_codes_host, dev + off_codes, (size_t)code_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(out_scales_host, dev + off_scales, (size_t)scale_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess) {
        return fail_after_enqueue();
    }
    return cudaStreamSynchronize(s) == cudaSuccess ? AXIOM_OK : AXIOM_ERR_CUDA;
}
