// Library-wide entry points: version, the per-thread error message, the device status word.
#include <stdarg.h>

#include "cgnn_plan.h"

namespace cgnn {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

}  // namespace cgnn

extern "C" {

int cgnn_version(void) { return 100; }

const char *cgnn_last_error(void) { return cgnn::g_error; }

int cgnn_device_status(int *status_out) {
    CGNN_REQUIRE(status_out != nullptr, "device_status: null output");
    int a = 0, b = 0, c = 0;
    CGNN_CUDA(cudaDeviceSynchronize());
    int rc = cgnn::segreduce_status(&a);
    if (rc == CGNN_OK) rc = cgnn::gather_status(&b);
    if (rc == CGNN_OK) rc = cgnn::cluster_status(&c);
    *status_out = a | b | c;
    return rc;
}

}  // extern "C"
