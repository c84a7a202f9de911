// Entry points every phase library carries: error text, ABI version, kernel status word.
#include "tc_host.cuh"

extern "C" {

const char* tc_last_error(void) { return tc::error_slot().c_str(); }

int tc_abi_version(void) { return TC_ABI_VERSION; }

int tc_device_status(int device, int32_t* status) {
    TC_REQUIRE(status, "null status");
    tc::DeviceInfo info;
    int result = tc::require_sm100(device, &info);
    if (result != TC_OK) return result;
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    tc::DeviceScratch scratch;
    result = tc::device_scratch(device, &scratch);
    if (result != TC_OK) return result;
    TC_CUDA(cudaDeviceSynchronize());
    TC_CUDA(cudaMemcpy(status, scratch.status, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (*status != 0) TC_CUDA(cudaMemset(scratch.status, 0, sizeof(int32_t)));
    return TC_OK;
}

}  // extern "C"
