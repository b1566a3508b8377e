// Process-wide pieces of the kernel library: the error text buffer and a probe that the
// Python loader calls to make sure the library was built for the device it runs on.
#include "common.cuh"

static char g_error[512] = "";

char* llm_error_buffer() { return g_error; }

static int g_pdl = 1;

bool llm_pdl_enabled() { return g_pdl != 0; }

// Switch programmatic dependent launch on (default) or off for all later launches; returns the old value.
LLM_API int llm_set_pdl(int on) {
    const int old = g_pdl;
    g_pdl = on ? 1 : 0;
    return old;
}

LLM_API const char* llm_last_error() { return g_error; }

LLM_API int llm_abi_version() { return 1; }

// 0 if the current device can run sm_100a code, else a negative code and a message.
LLM_API int llm_check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) LLM_FAIL(-2, "cudaGetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) LLM_FAIL(-2, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (p.major != 10)
        LLM_FAIL(-3, "device %d is sm_%d%d; this library holds sm_100a code only", dev, p.major, p.minor);
    return 0;
}

LLM_TRACE_EXPORT(runtime)
