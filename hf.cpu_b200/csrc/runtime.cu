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

#ifdef HFB_TRACE
static void (*g_trace_setters[32])(void *);
static int g_trace_setter_n = 0;
static unsigned long long *g_trace_buf = nullptr;
void trace_register(void (*setter)(void *)) { if (g_trace_setter_n < 32) g_trace_setters[g_trace_setter_n++] = setter; }
#endif

}  // namespace hfb

// Kernel timeline of a -DHFB_TRACE build: start (or restart) logging; copy out up to `max` (tag, nanoseconds) pairs.
extern "C" int hfb_trace_start(void)
{
#ifdef HFB_TRACE
    using namespace hfb;
    const size_t bytes = (2 + 2 * HFB_TRACE_CAP) * sizeof(unsigned long long);
    if (!g_trace_buf && cudaMalloc(&g_trace_buf, bytes) != cudaSuccess) return fail(HFB_ECUDA, "trace: cannot allocate the log");
    cudaDeviceSynchronize();
    cudaMemset(g_trace_buf, 0, bytes);
    for (int i = 0; i < g_trace_setter_n; i++) g_trace_setters[i](g_trace_buf);
    return HFB_OK;
#else
    return hfb::fail(HFB_ENOTSUP, "trace: this library was built without -DHFB_TRACE");
#endif
}

extern "C" long long hfb_trace_take(unsigned long long *pairs, long long max)
{
#ifdef HFB_TRACE
    using namespace hfb;
    if (!g_trace_buf) return 0;
    cudaDeviceSynchronize();
    unsigned long long n = 0;
    cudaMemcpy(&n, g_trace_buf, sizeof n, cudaMemcpyDeviceToHost);
    if (n > HFB_TRACE_CAP) n = HFB_TRACE_CAP;
    if ((long long)n > max) n = (unsigned long long)max;
    cudaMemcpy(pairs, g_trace_buf + 2, n * 2 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
    cudaMemset(g_trace_buf, 0, sizeof(unsigned long long));
    return (long long)n;
#else
    (void)pairs; (void)max;
    return 0;
#endif
}

extern "C" const char *hfb_last_error(void) { return hfb::g_msg; }
extern "C" int hfb_version(void) { return 1; }

// Queues a copy of the error word into `host_word` (pinned host memory) on the stream and returns at once: the
// caller reads it after an event or synchronisation of its own, beside the results it is waiting for anyway.
extern "C" int hfb_error_word_peek_async(int32_t *host_word, hfb_stream s)
{
    int *p = hfb::error_word();
    if (!p) return hfb::fail(HFB_ECUDA, "cannot locate the device error word");
    cudaError_t e = cudaMemcpyAsync(host_word, p, sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)s);
    if (e != cudaSuccess) return hfb::fail(HFB_ECUDA, "copying the device error word: %s", cudaGetErrorString(e));
    return HFB_OK;
}

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
