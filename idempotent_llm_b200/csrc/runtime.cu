// Error reporting and identification of the compiled library.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[1024] = "";

int idm_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

extern "C" const char* idm_last_error() { return g_error; }
extern "C" const char* idm_dtype_name() { return IDM_DTYPE_NAME; }
extern "C" int idm_page_tokens() { return IDM_PAGE; }
