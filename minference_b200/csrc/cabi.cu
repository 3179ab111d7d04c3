// Library-wide entry points of the C ABI: version string, per-thread error text, options.
#include "common.h"

namespace minf {
char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}
}  // namespace minf

extern "C" const char* minf_version(void) { return "minfer_b200 0.1 (sm_100a)"; }
extern "C" const char* minf_last_error(void) { return minf::last_error_buffer(); }
