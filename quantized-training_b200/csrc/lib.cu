// Library-level entry points: error text, version, device status word.
#include "common.cuh"

namespace qt {

char* last_error_buffer() {
    static thread_local char buf[kErrBufSize] = {0};
    return buf;
}

// Status block of a device: word 0 is written (first code wins) by kernels whose bounded waits run out;
// bytes 8..15 hold the device-visible address of a pinned host word that receives a copy of the code, so
// the host can notice a failure without synchronising (qt_device_status_peek).
__device__ __align__(16) unsigned long long g_device_status[2] = {0ull, 0ull};

namespace {
int* g_status_dev[64] = {nullptr};
volatile int* g_status_host[64] = {nullptr};

int status_setup(int dev) {
    void* p = nullptr;
    QT_CUDA_CHECK(cudaGetSymbolAddress(&p, g_device_status));
    int* host = nullptr;
    QT_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
    *host = 0;
    void* host_dev = nullptr;
    QT_CUDA_CHECK(cudaHostGetDevicePointer(&host_dev, host, 0));
    const unsigned long long mirror = reinterpret_cast<unsigned long long>(host_dev);
    QT_CUDA_CHECK(cudaMemcpy(reinterpret_cast<unsigned long long*>(p) + 1, &mirror, sizeof(mirror), cudaMemcpyHostToDevice));
    g_status_host[dev] = host;
    g_status_dev[dev] = reinterpret_cast<int*>(p);
    return QT_OK;
}
}  // namespace

// Device address of the current device's status block (set up on first use: one pinned host word and
// one small copy, so the first kernel launch of a process should not sit inside a stream capture).
int device_status_ptr(int** out) {
    int dev = 0;
    QT_CUDA_CHECK(cudaGetDevice(&dev));
    QT_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (!g_status_dev[dev])
        if (int rc = status_setup(dev)) return rc;
    *out = g_status_dev[dev];
    return QT_OK;
}

volatile int* device_status_host_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return g_status_host[dev];
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
    if (volatile int* h = qt::device_status_host_word()) *h = 0;
    return QT_OK;
}

extern "C" int qt_device_status_peek(int* status_out) {
    QT_REQUIRE(status_out, "device_status_peek: null output");
    volatile int* h = qt::device_status_host_word();
    *status_out = h ? *h : 0;
    return QT_OK;
}
