// Version / status strings of the C ABI, and the cached device query.
#include "common.cuh"

namespace mfar {

int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace mfar

extern "C" int mfar_version(void) { return 100; }

extern "C" const char* mfar_status_string(int status) {
    switch (status) {
        case MFAR_OK: return "ok";
        case MFAR_ERR_ARG: return "bad argument (size, null pointer or unsupported shape)";
        case MFAR_ERR_ALIGN: return "pointer or stride not aligned as the header requires";
        case MFAR_ERR_WORKSPACE: return "scratch / workspace too small or misaligned";
        case MFAR_ERR_LAUNCH: return "CUDA launch failed";
        case MFAR_ERR_DEVICE: return "kernel reported an error in dev_status";
        case MFAR_ERR_LIMIT: return "size beyond a fixed limit of this entry point";
        default: return "unknown status";
    }
}
