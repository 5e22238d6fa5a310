// Library-level entry points: error text, version, device status word.
#include "common.cuh"

namespace qt {

char* last_error_buffer() {
    static thread_local char buf[kErrBufSize] = {0};
    return buf;
}

// Written by kernels whose bounded waits run out; read and cleared by qt_device_status().
__device__ int g_device_status = 0;

int device_status_ptr(int** out) {
    static int* cached[64] = {nullptr};
    int dev = 0;
    QT_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && cached[dev]) {
        *out = cached[dev];
        return QT_OK;
    }
    void* p = nullptr;
    QT_CUDA_CHECK(cudaGetSymbolAddress(&p, g_device_status));
    *out = reinterpret_cast<int*>(p);
    if (dev >= 0 && dev < 64) cached[dev] = *out;
    return QT_OK;
}

}  // namespace qt

extern "C" const char* qt_last_error(void) { return qt::last_error_buffer(); }

extern "C" const char* qt_version(void) { return "qt_b200 0.1 sm_100a"; }

extern "C" int qt_device_status(int* status_out) {
    QT_REQUIRE(status_out, "device_status: null output");
    int* dptr = nullptr;
    if (int rc = qt::device_status_ptr(&dptr)) return rc;
    QT_CUDA_CHECK(cudaDeviceSynchronize());
    QT_CUDA_CHECK(cudaMemcpy(status_out, dptr, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_out != 0) QT_CUDA_CHECK(cudaMemset(dptr, 0, sizeof(int)));
    return QT_OK;
}
