// ribn_gemv_noalloc: the quantized GEMV for callers that must not allocate.
//
// Who needs it: code that runs where device-memory allocation is off limits --
// a serving loop that has handed all of HBM to its KV cache and weight pools and
// forbids cudaMalloc after start-up, a host thread inside a latency-critical
// section where the implicit synchronisation of cudaMalloc/cudaFree is not
// acceptable, or a plug-in loaded into a process whose allocator it may not
// touch.  Such callers cannot use ribn_create (which allocates a status word and
// a workspace), so this entry point takes no context at all.
//
// The integer-dot GEMV needs scratch for the packed activations (two int8
// planes + block scales + block sums, 2.25 bytes per activation).  Here that
// scratch is a file-scope device array of fixed size, part of the library image:
// every GPU that loads the library holds it until the process exits, whether or
// not this entry point is ever called.  The price of "no allocation" is the
// stated size limit below and one shared buffer: two calls whose kernels may
// overlap on the GPU (different streams, or different host threads) race on it
// and must be serialised by the caller.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "../../include/ribn_b200.h"
#include "internal.h"

namespace {

// Limit: members * K (K rounded up to a multiple of 256) activations per call.
constexpr unsigned long long kMaxActivations = RIBN_NOALLOC_MAX_ACTIVATIONS;
constexpr unsigned long long kStatusBytes = 256;   // first 256 bytes: the device status word
constexpr unsigned long long kScratchBytes = kStatusBytes + kMaxActivations * 2 + (kMaxActivations / 32) * 8;

// In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a device address,
// and a kernel handed `g_scratch` directly would fault (or quietly use host memory).
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
// Per device, filled by the first call on that device.  The address is published last (release) and read first
// (acquire), so a thread that sees it also sees the SM count; two threads racing through the set-up write the same values.
std::atomic<unsigned char*> g_scratch_address[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

// Every buffer must be device (or managed) memory of `device`: a host pointer handed to the kernels would fault.
// cudaPointerGetAttributes allocates nothing.
bool on_device(const void* p, int device) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) && attr.device == device;
}


}  // namespace

extern "C" {

int ribn_gemv_noalloc(int device, void* cuda_stream, const ribn_qweight* weight, const void* x_device, int x_dtype,
                      uint64_t x_len, void* y_device, int y_dtype, uint64_t y_len, uint32_t members, int wait,
                      char* error_message, uint64_t error_capacity) {
    char unused[8];
    char* g_message = error_message != nullptr && error_capacity > 0 ? error_message : unused;
    const size_t g_capacity = error_message != nullptr && error_capacity > 0 ? static_cast<size_t>(error_capacity) : sizeof unused;
    g_message[0] = 0;
    auto fail = [&](int status, const char* message) {
        snprintf(g_message, g_capacity, "%s", message);
        return status;
    };
    if (device < 0 || device >= kMaxDevices) return fail(RIBN_E_INVALID_ARGUMENT, "device index out of range");
    if ((x_dtype != RIBN_F32 && x_dtype != RIBN_BF16) || (y_dtype != RIBN_F32 && y_dtype != RIBN_BF16))
        return fail(RIBN_E_INVALID_ARGUMENT, "unknown activation dtype");
    if (members == 0) return fail(RIBN_E_INPUT_LENGTH, "quantized GEMV input has 0 values, expected 1");
    if (members > 4) return fail(RIBN_E_INVALID_WEIGHT, "invalid quantized weight: ribn_gemv_noalloc supports at most 4 members");
    uint64_t k = 0, n = 0;
    const int geometry = ribn_validate_quantized_geometry(weight, 0, &k, &n);
    if (geometry != RIBN_OK) return fail(geometry, ribn_status_string(geometry));
    if (x_len != k * members) return fail(RIBN_E_INPUT_LENGTH, "quantized GEMV input length does not match members * K");
    if (y_len != n * members) return fail(RIBN_E_OUTPUT_LENGTH, "quantized GEMV output length does not match members * N");
    const unsigned long long kpad = static_cast<unsigned long long>(ribn::padded_k(static_cast<int>(k)));
    if (kpad * members > kMaxActivations) {
        snprintf(g_message, g_capacity,
                 "ribn_gemv_noalloc: members * K = %llu exceeds the fixed scratch of %llu activations; use ribn_gemv",
                 kpad * members, kMaxActivations);
        return RIBN_E_SHAPE_OVERFLOW;
    }
    if (!ribn::gemv_dp4a_fits(weight->value_type, static_cast<int>(k), static_cast<int>(members)))
        return fail(RIBN_E_SHAPE_OVERFLOW, "ribn_gemv_noalloc: activations do not fit the kernel's shared memory; use ribn_gemv");
    if (weight->data == nullptr || x_device == nullptr || y_device == nullptr ||
        reinterpret_cast<uintptr_t>(weight->data) % 16 || reinterpret_cast<uintptr_t>(x_device) % 16 ||
        reinterpret_cast<uintptr_t>(y_device) % 16)
        return fail(RIBN_E_INVALID_ARGUMENT, "pointers must be non-null and 16-byte aligned");

    int previous = -1;
    cudaGetDevice(&previous);
    if (previous != device && cudaSetDevice(device) != cudaSuccess) return fail(RIBN_E_DRIVER, "cannot select the device");
    if (!on_device(weight->data, device) || !on_device(x_device, device) || !on_device(y_device, device)) {
        if (previous >= 0 && previous != device) cudaSetDevice(previous);
        return fail(RIBN_E_CONTEXT_MISMATCH, "quantized GEMV buffers and stream belong to different CUDA contexts");
    }
    int status = RIBN_OK;
    // Set-up, once per device, with that device current: resolve the device address of the array.
    if (g_scratch_address[device].load(std::memory_order_acquire) == nullptr) {
        unsigned char* address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_scratch);
        int sm_count = 0;
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || address == nullptr) {
            snprintf(g_message, g_capacity, "CUDA driver error: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            status = RIBN_E_DRIVER;
        } else {
            g_sm_count[device] = sm_count;
            g_scratch_address[device].store(address, std::memory_order_release);
        }
    }
    if (status == RIBN_OK) {
        cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
        unsigned char* scratch = g_scratch_address[device].load(std::memory_order_acquire);
        int* device_status = reinterpret_cast<int*>(scratch);
        unsigned char* packed = scratch + kStatusBytes;
        // The array keeps the previous call's contents.  The packed rows are fully rewritten below;
        // the status word must start at zero.
        cudaError_t e = cudaMemsetAsync(device_status, 0, sizeof(int), stream);
        if (e == cudaSuccess)
            e = ribn::launch_quantize_activations(x_device, x_dtype == RIBN_BF16, nullptr, 0.0f, packed,
                                                  static_cast<int>(members), static_cast<int>(k), stream);
        bool handled = false;
        if (e == cudaSuccess) {
            ribn::GemvArgs a{};
            a.weights = static_cast<const uint8_t*>(weight->data);
            a.weight_bytes = weight->encoded_bytes;
            a.value_type = weight->value_type;
            a.k = static_cast<int>(k);
            a.n = static_cast<int>(n);
            a.x = packed;
            a.x_bf16 = false;
            a.y = y_device;
            a.y_bf16 = y_dtype == RIBN_BF16;
            a.members = static_cast<int>(members);
            a.device_status = device_status;
            a.sm_count = g_sm_count[device];
            a.variant = 0;
            a.stream = stream;
            e = ribn::launch_gemv_dp4a(a, &handled);
        }
        if (e != cudaSuccess) {
            snprintf(g_message, g_capacity, "CUDA driver error: %s", cudaGetErrorString(e));
            status = RIBN_E_DRIVER;
        } else if (!handled) {
            status = fail(RIBN_E_SHAPE_OVERFLOW, "ribn_gemv_noalloc: shape refused by the kernel; use ribn_gemv");
        } else if (wait != 0) {
            int flag = 0;
            e = cudaStreamSynchronize(stream);
            if (e == cudaSuccess) e = cudaMemcpy(&flag, device_status, sizeof flag, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) {
                snprintf(g_message, g_capacity, "CUDA driver error: %s", cudaGetErrorString(e));
                status = RIBN_E_DRIVER;
            } else if (flag != ribn::kDeviceOk) {
                status = fail(RIBN_E_TIMEOUT, "a bounded device-side wait ran out; the output is invalid");
            }
        }
    }
    if (previous >= 0 && previous != device) cudaSetDevice(previous);
    return status;
}

int ribn_noalloc_status(int device, void* cuda_stream) {
    if (device < 0 || device >= kMaxDevices) return RIBN_E_INVALID_ARGUMENT;
    unsigned char* scratch = g_scratch_address[device].load(std::memory_order_acquire);
    if (scratch == nullptr) return RIBN_OK;   // no call was ever made on this device
    int previous = -1;
    cudaGetDevice(&previous);
    if (previous != device && cudaSetDevice(device) != cudaSuccess) return RIBN_E_DRIVER;
    int flag = 0;
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream));
    if (e == cudaSuccess) e = cudaMemcpy(&flag, scratch, sizeof flag, cudaMemcpyDeviceToHost);
    if (previous >= 0 && previous != device) cudaSetDevice(previous);
    if (e != cudaSuccess) return RIBN_E_DRIVER;
    return flag == ribn::kDeviceOk ? RIBN_OK : RIBN_E_TIMEOUT;
}

}  // extern "C"
