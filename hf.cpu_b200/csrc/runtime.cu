// Status reporting and the device error word.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

namespace hfb {

static thread_local char g_msg[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof g_msg, fmt, ap);
    va_end(ap);
    return code;
}

bool pdl_enabled()
{
    static int on = -1;
    if (on < 0) {
        const char *v = getenv("HFB_PDL");
        on = !(v && v[0] == '0');
    }
    return on != 0;
}

__device__ int g_error_word = 0;

// Device address of the error word on the current device (looked up once per device).
int *error_word()
{
    static int *ptr[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_error_word) != cudaSuccess) return nullptr;
        ptr[dev] = (int *)p;
    }
    return ptr[dev];
}

}  // namespace hfb

extern "C" const char *hfb_last_error(void) { return hfb::g_msg; }
extern "C" int hfb_version(void) { return 1; }

extern "C" int hfb_error_word_take(int32_t *word, hfb_stream s)
{
    int *p = hfb::error_word();
    if (!p) return hfb::fail(HFB_ECUDA, "cannot locate the device error word");
    int v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, p, sizeof v, cudaMemcpyDeviceToHost, (cudaStream_t)s);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)s);
    if (e == cudaSuccess && v) e = cudaMemsetAsync(p, 0, sizeof v, (cudaStream_t)s);
    if (e != cudaSuccess) return hfb::fail(HFB_ECUDA, "reading the device error word: %s", cudaGetErrorString(e));
    *word = v;
    return HFB_OK;
}
