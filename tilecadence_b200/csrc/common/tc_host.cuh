// Host-side plumbing shared by the C-ABI translation units: thread-local error text, CUDA error
// checks that turn into status codes (never exceptions across the C boundary), tensor-map
// encoding through the driver entry point (no link-time libcuda dependency), and the small
// per-device scratch block (split tickets + kernel status word) the library owns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "tilecadence_b200.h"

namespace tc {

inline std::string& error_slot() {
    thread_local std::string message;
    return message;
}

inline int fail(int code, const char* format, ...) {
    char buffer[1024];
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(buffer, sizeof(buffer), format, arguments);
    va_end(arguments);
    error_slot() = buffer;
    return code;
}

#define TC_REQUIRE(condition, ...)                                   \
    do {                                                             \
        if (!(condition)) return ::tc::fail(TC_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define TC_CUDA(call)                                                                                   \
    do {                                                                                                \
        cudaError_t tc_status_ = (call);                                                                \
        if (tc_status_ != cudaSuccess)                                                                  \
            return ::tc::fail(TC_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(tc_status_));     \
    } while (0)

// Restores the caller's current device on scope exit.
struct DeviceGuard {
    int previous = -1;
    bool switched = false;
    cudaError_t status = cudaSuccess;
    explicit DeviceGuard(int device) {
        status = cudaGetDevice(&previous);
        if (status == cudaSuccess && previous != device) {
            status = cudaSetDevice(device);
            switched = status == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(previous);
    }
};

struct DeviceInfo {
    int sms = 0, major = 0, minor = 0, smem_optin = 0;
};

inline int device_info(int device, DeviceInfo* info) {
    static std::mutex lock;
    static std::unordered_map<int, DeviceInfo> cache;
    std::lock_guard<std::mutex> guard(lock);
    auto found = cache.find(device);
    if (found == cache.end()) {
        DeviceInfo fresh;
        TC_CUDA(cudaDeviceGetAttribute(&fresh.sms, cudaDevAttrMultiProcessorCount, device));
        TC_CUDA(cudaDeviceGetAttribute(&fresh.major, cudaDevAttrComputeCapabilityMajor, device));
        TC_CUDA(cudaDeviceGetAttribute(&fresh.minor, cudaDevAttrComputeCapabilityMinor, device));
        TC_CUDA(cudaDeviceGetAttribute(&fresh.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        found = cache.emplace(device, fresh).first;
    }
    *info = found->second;
    return TC_OK;
}

// Refuses to run anywhere but a compute-capability 10.x device: there is no other code path.
inline int require_sm100(int device, DeviceInfo* info) {
    int status = device_info(device, info);
    if (status != TC_OK) return status;
    if (info->major != 10)
        return fail(TC_ERR_DEVICE, "device %d is sm_%d%d; these kernels are built for sm_100a only", device,
                    info->major, info->minor);
    return TC_OK;
}

// ----------------------------------------------------------------------------- tensor maps
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int encode_entry(EncodeTiled* out) {
    static std::mutex lock;
    static EncodeTiled cached = nullptr;
    std::lock_guard<std::mutex> guard(lock);
    if (!cached) {
        void* pointer = nullptr;
        cudaDriverEntryPointQueryResult query;
        TC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &query));
        if (query != cudaDriverEntryPointSuccess || !pointer)
            return fail(TC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        cached = reinterpret_cast<EncodeTiled>(pointer);
    }
    *out = cached;
    return TC_OK;
}

// 4-D map over a [d3, d2, d1, d0=128] 16-bit tensor whose innermost dimension is contiguous.
// The box is {64 elements, 1, box_rows, 1} with the 128-byte swizzle, so one copy lands as
// box_rows rows of 128 bytes in shared memory (the layout tcgen05 descriptors and the swizzled
// ldmatrix addressing expect). Strides are in elements.
inline int make_rows_map(CUtensorMap* map, const void* base, bool is_fp16, int64_t d1, int64_t d2, int64_t d3,
                         int64_t stride1, int64_t stride2, int64_t stride3, int box_rows, int row_dim) {
    EncodeTiled encode = nullptr;
    int status = encode_entry(&encode);
    if (status != TC_OK) return status;
    cuuint64_t dims[4] = {128, cuuint64_t(d1), cuuint64_t(d2), cuuint64_t(d3)};
    // A size-1 dimension may carry any stride; keep the encoder's "multiple of 16 bytes" rule happy.
    auto bytes = [](int64_t elements) { return cuuint64_t(elements > 0 ? elements : 128) * 2; };
    cuuint64_t strides[3] = {bytes(stride1), bytes(stride2), bytes(stride3)};
    cuuint32_t box[4] = {64, 1, 1, 1};
    box[row_dim] = cuuint32_t(box_rows);
    cuuint32_t element_strides[4] = {1, 1, 1, 1};
    CUresult result = encode(map, is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                             const_cast<void*>(base), dims, strides, box, element_strides,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) return fail(TC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(result));
    return TC_OK;
}

// ----------------------------------------------------------------------------- per-device scratch
// tickets[0 .. kTicketSlots): split-completion counters, zero between launches (the last CTA of
// each (batch, kv head) resets its slot). status: first non-zero kernel error code since the
// last tc_device_status() call.
constexpr int kTicketSlots = 8192;
struct DeviceScratch {
    int32_t* tickets = nullptr;
    int32_t* status = nullptr;
};

struct ScratchRegistry {
    std::mutex lock;
    std::unordered_map<int, DeviceScratch> blocks;               // allocated on a device's first decode call
    std::unordered_multimap<int, int32_t*> extra_status_words;   // status words that live elsewhere
};
inline ScratchRegistry& scratch_registry() {
    static ScratchRegistry registry;
    return registry;
}

inline int device_scratch(int device, DeviceScratch* out) {
    ScratchRegistry& registry = scratch_registry();
    std::lock_guard<std::mutex> guard(registry.lock);
    auto found = registry.blocks.find(device);
    if (found == registry.blocks.end()) {
        int32_t* block = nullptr;
        TC_CUDA(cudaMalloc(&block, sizeof(int32_t) * (kTicketSlots + 64)));
        TC_CUDA(cudaMemset(block, 0, sizeof(int32_t) * (kTicketSlots + 64)));
        TC_CUDA(cudaDeviceSynchronize());
        DeviceScratch fresh;
        fresh.tickets = block;
        fresh.status = block + kTicketSlots;
        found = registry.blocks.emplace(device, fresh).first;
    }
    *out = found->second;
    return TC_OK;
}

// A translation unit whose kernels report into a status word outside the per-device block (a word
// inside a file-scope device array, for one) announces its device address here once per device, so
// that tc_device_status finds it. Nothing is allocated on the device.
inline void register_status_word(int device, int32_t* word) {
    ScratchRegistry& registry = scratch_registry();
    std::lock_guard<std::mutex> guard(registry.lock);
    auto range = registry.extra_status_words.equal_range(device);
    for (auto it = range.first; it != range.second; ++it)
        if (it->second == word) return;
    registry.extra_status_words.emplace(device, word);
}

// Device addresses of every status word that exists for `device` right now; never creates the block.
inline int known_status_words(int device, int32_t** words, int capacity) {
    ScratchRegistry& registry = scratch_registry();
    std::lock_guard<std::mutex> guard(registry.lock);
    int count = 0;
    auto block = registry.blocks.find(device);
    if (block != registry.blocks.end() && count < capacity) words[count++] = block->second.status;
    auto range = registry.extra_status_words.equal_range(device);
    for (auto it = range.first; it != range.second && count < capacity; ++it) words[count++] = it->second;
    return count;
}

inline bool ranges_overlap(const void* a, size_t a_bytes, const void* b, size_t b_bytes) {
    if (!a_bytes || !b_bytes) return false;
    const auto x = reinterpret_cast<uintptr_t>(a), y = reinterpret_cast<uintptr_t>(b);
    return x < y + b_bytes && y < x + a_bytes;
}

template <typename Kernel>
inline int kernel_resources(Kernel kernel, int threads, int shared, int64_t* out8) {
    if (shared >= 48 * 1024)
        TC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared));
    cudaFuncAttributes attributes{};
    TC_CUDA(cudaFuncGetAttributes(&attributes, kernel));
    int active = 0;
    TC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&active, kernel, threads, shared));
    out8[0] = threads;
    out8[1] = shared;
    out8[2] = int64_t(attributes.sharedSizeBytes);
    out8[3] = attributes.numRegs;
    out8[4] = int64_t(attributes.localSizeBytes);
    out8[5] = attributes.binaryVersion;
    out8[6] = attributes.ptxVersion;
    out8[7] = active;
    return TC_OK;
}

}  // namespace tc
