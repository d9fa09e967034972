// Last-error text and version of the C-ABI library.
#include "common.h"
#include <cstring>

namespace et {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
}  // namespace et

extern "C" const char* et_last_error(void) { return et::g_err; }
extern "C" int et_version(void) { return ET_B200_VERSION; }
