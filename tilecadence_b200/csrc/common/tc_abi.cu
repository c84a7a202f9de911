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
    // Every status word that exists for this device: the per-device block's (if a decode call ever created
    // the block; reading the status never allocates it) and words registered by allocation-free entries.
    int32_t* words[8];
    const int count = tc::known_status_words(device, words, 8);
    *status = 0;
    if (count == 0) return TC_OK;
    TC_CUDA(cudaDeviceSynchronize());
    for (int i = 0; i < count; ++i) {
        int32_t value = 0;
        TC_CUDA(cudaMemcpy(&value, words[i], sizeof(int32_t), cudaMemcpyDeviceToHost));
        if (value != 0) {
            TC_CUDA(cudaMemset(words[i], 0, sizeof(int32_t)));
            if (*status == 0) *status = value;
        }
    }
    return TC_OK;
}

}  // extern "C"
