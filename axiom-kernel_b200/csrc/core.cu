// Host core of libaxiom_b200: ABI identity, runtime and device-buffer handles,
// completion convention, scale-plane arithmetic.  Mirrors the behaviour of the
// reference runtime wrappers for the hot-path subset
// (src/axiom_runtime.cpp:3037-3340) without sharing their structure.
#include "runtime.hpp"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <new>

namespace axb {

namespace {
std::atomic<uint64_t> g_launches{0};

bool env_truthy(const char *name) {
    const char *v = std::getenv(name);
    if (!v || !v[0]) return false;
    return std::strcmp(v, "0") != 0 && std::strcmp(v, "false") != 0 &&
           std::strcmp(v, "False") != 0 && std::strcmp(v, "FALSE") != 0;
}

bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone;
}
}  // namespace

void note_launch(uint32_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int select_device(int device) {
    if (device < 0) return AXIOM_ERR_INVALID_ARGUMENT;
    return cudaSetDevice(device) == cudaSuccess ? AXIOM_OK : AXIOM_ERR_CUDA;
}

int launch_status() { return cudaGetLastError() == cudaSuccess ? AXIOM_OK : AXIOM_ERR_CUDA; }

int finish_after_launch(cudaStream_t stream) {
    if (cudaGetLastError() != cudaSuccess) return AXIOM_ERR_CUDA;
    // The environment is read on every call, as the reference's generic ops do
    // (src/axiom_cuda.cu:162-164), so a host can flip it between phases.
    if (env_truthy("AXIOM_CUDA_LAUNCH_ASYNC") || capturing(stream)) return AXIOM_OK;
    return cuda_to_status(cudaStreamSynchronize(stream));
}

bool span_ok(const axiom_device_buffer *buffer, uint64_t offset, uint64_t bytes) {
    return buffer && offset <= buffer->bytes && bytes <= buffer->bytes - offset;
}

bool mul_ok(uint64_t a, uint64_t b, uint64_t *out) {
    if (a != 0 && b > UINT64_MAX / a) return false;
    *out = a * b;
    return true;
}

bool ranges_overlap(const axiom_device_buffer *a, uint64_t a_off, uint64_t a_bytes,
                    const axiom_device_buffer *b, uint64_t b_off, uint64_t b_bytes) {
    if (a != b || a_bytes == 0 || b_bytes == 0) return false;
    return a_off < b_off + b_bytes && b_off < a_off + a_bytes;
}

}  // namespace axb

using namespace axb;

extern "C" {

uint32_t axiom_abi_version(void) { return AXIOM_ABI_VERSION; }

const char *axiom_version(void) { return "axiom-b200-fused 0.1.0 abi=1 cuda sm_100a"; }

int axiom_abi_info_get(axiom_abi_info *out) {
    if (!out || out->abi_version != AXIOM_ABI_VERSION) return AXIOM_ERR_INVALID_ARGUMENT;
    std::memset(out, 0, sizeof(*out));
    out->abi_version = AXIOM_ABI_VERSION;
    out->header_abi_version = AXIOM_ABI_VERSION;
    out->runtime_abi_version = AXIOM_ABI_VERSION;
    out->struct_size = (uint32_t)sizeof(*out);
    out->version = axiom_version();
    out->backend = "cuda";
    out->build_target = "sm_100a";
    return AXIOM_OK;
}

int axiom_abi_check(uint32_t header_abi_version) {
    return header_abi_version == AXIOM_ABI_VERSION ? AXIOM_OK : AXIOM_ERR_INVALID_ARGUMENT;
}

const char *axiom_status_string(int status) {
    switch (status) {
    case AXIOM_OK: return "ok";
    case AXIOM_ERR_INVALID_ARGUMENT: return "invalid argument";
    case AXIOM_ERR_UNSUPPORTED_BACKEND: return "unsupported backend";
    case AXIOM_ERR_CUDA: return "cuda error";
    case AXIOM_ERR_RUNTIME: return "runtime error";
    case AXIOM_ERR_NOT_IMPLEMENTED: return "not implemented";
    case AXIOM_ERR_IO: return "io error";
    case AXIOM_ERR_BUDGET: return "budget exceeded";
    default: return "unknown error";
    }
}

uint64_t axiom_b200_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int axiom_runtime_device_count(uint32_t *out_count) {
    if (!out_count) return AXIOM_ERR_INVALID_ARGUMENT;
    *out_count = 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return AXIOM_ERR_CUDA;
    *out_count = n > 0 ? (uint32_t)n : 0u;
    return AXIOM_OK;
}

int axiom_runtime_create(axiom_runtime **out, const axiom_config *config) {
    if (!out || !config || config->abi_version != AXIOM_ABI_VERSION) return AXIOM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (config->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) return AXIOM_ERR_CUDA;
    if (config->device >= (uint32_t)count) return AXIOM_ERR_INVALID_ARGUMENT;
    if (cudaSetDevice((int)config->device) != cudaSuccess) return AXIOM_ERR_CUDA;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, (int)config->device) != cudaSuccess) return AXIOM_ERR_CUDA;
    // The library carries sm_100a code only; any other device cannot run it.
    if (prop.major != 10) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    axiom_runtime *rt = new (std::nothrow) axiom_runtime();
    if (!rt) return AXIOM_ERR_RUNTIME;
    rt->backend = config->backend;
    rt->device = config->device;
    rt->sm_count = (uint32_t)prop.multiProcessorCount;
    *out = rt;
    return AXIOM_OK;
}

void axiom_runtime_destroy(axiom_runtime *runtime) {
    if (!runtime) return;
    (void)cudaSetDevice((int)runtime->device);
    runtime->staging.release();
    delete runtime;
}

int axiom_runtime_device_id(const axiom_runtime *runtime, uint32_t *out_device) {
    if (!runtime || !out_device) return AXIOM_ERR_INVALID_ARGUMENT;
    *out_device = runtime->device;
    return AXIOM_OK;
}

int axiom_device_buffer_create(axiom_runtime *runtime, axiom_device_buffer **out, uint64_t bytes) {
    if (!runtime || !out || bytes == 0) return AXIOM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (runtime->backend != AXIOM_BACKEND_CUDA) return AXIOM_ERR_UNSUPPORTED_BACKEND;
    if (cudaSetDevice((int)runtime->device) != cudaSuccess) return AXIOM_ERR_CUDA;
    axiom_device_buffer *buf = new (std::nothrow) axiom_device_buffer();
    if (!buf) return AXIOM_ERR_RUNTIME;
    const cudaError_t err = cudaMalloc(&buf->ptr, (size_t)bytes);
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        delete buf;
        return cuda_to_status(err);
    }
    buf->runtime = runtime;
    buf->device = runtime->device;
    buf->bytes = bytes;
    *out = buf;
    return AXIOM_OK;
}

void axiom_device_buffer_destroy(axiom_device_buffer *buffer) {
    if (!buffer) return;
    if (buffer->ptr) {
        (void)cudaSetDevice((int)buffer->device);
        (void)cudaFree(buffer->ptr);
    }
    delete buffer;
}

int axiom_device_buffer_upload(axiom_device_buffer *buffer, uint64_t offset, const void *src_host, uint64_t bytes) {
    if (!buffer || !src_host || bytes == 0 || !span_ok(buffer, offset, bytes)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (cudaSetDevice((int)buffer->device) != cudaSuccess) return AXIOM_ERR_CUDA;
    return cuda_to_status(cudaMemcpy((uint8_t *)buffer->ptr + offset, src_host, (size_t)bytes, cudaMemcpyHostToDevice));
}

int axiom_device_buffer_download(axiom_device_buffer *buffer, uint64_t offset, void *dst_host, uint64_t bytes) {
    if (!buffer || !dst_host || bytes == 0 || !span_ok(buffer, offset, bytes)) return AXIOM_ERR_INVALID_ARGUMENT;
    if (cudaSetDevice((int)buffer->device) != cudaSuccess) return AXIOM_ERR_CUDA;
    return cuda_to_status(cudaMemcpy(dst_host, (const uint8_t *)buffer->ptr + offset, (size_t)bytes, cudaMemcpyDeviceToHost));
}

int axiom_device_buffer_copy(axiom_device_buffer *dst, uint64_t dst_offset, const axiom_device_buffer *src, uint64_t src_offset, uint64_t bytes) {
    if (!dst || !src || bytes == 0 || !span_ok(dst, dst_offset, bytes) || !span_ok(src, src_offset, bytes)) {
        return AXIOM_ERR_INVALID_ARGUMENT;
    }
    if (!dst->runtime || !src->runtime) return AXIOM_ERR_INVALID_ARGUMENT;
    if (cudaSetDevice((int)dst->device) != cudaSuccess) return AXIOM_ERR_CUDA;
    return cuda_to_status(cudaMemcpy((uint8_t *)dst->ptr + dst_offset, (const uint8_t *)src->ptr + src_offset,
                                     (size_t)bytes, cudaMemcpyDeviceToDevice));
}

int axiom_device_buffer_device_id(const axiom_device_buffer *buffer, uint32_t *out_device) {
    if (!buffer || !out_device) return AXIOM_ERR_INVALID_ARGUMENT;
    *out_device = buffer->device;
    return AXIOM_OK;
}

int axiom_device_buffer_cuda_pointer(const axiom_device_buffer *buffer, void **out_pointer) {
    if (out_pointer) *out_pointer = nullptr;
    if (!buffer || !out_pointer || !buffer->runtime || !buffer->ptr) return AXIOM_ERR_INVALID_ARGUMENT;
    *out_pointer = buffer->ptr;
    return AXIOM_OK;
}

uint64_t axiom_nvfp4_scale_plane_bytes(uint32_t rows, uint32_t groups, uint32_t scale_layout) {
    if (scale_layout == AXIOM_SCALE_LAYOUT_CANONICAL) return (uint64_t)rows * groups;
    return (((uint64_t)rows + 127u) / 128u) * (((uint64_t)groups + 3u) / 4u) * 512u;
}

uint64_t axiom_nvfp4_scale_plane_offset(uint32_t row, uint32_t group, uint32_t groups, uint32_t scale_layout) {
    if (scale_layout == AXIOM_SCALE_LAYOUT_CANONICAL) return (uint64_t)row * groups + group;
    const uint32_t inner_tiles = (groups + 3u) / 4u;
    const uint32_t in_tile = row % 128u;
    return ((uint64_t)(row / 128u) * inner_tiles + group / 4u) * 512u + (in_tile % 32u) * 16u +
           (in_tile / 32u) * 4u + group % 4u;
}

}  // extern "C"
