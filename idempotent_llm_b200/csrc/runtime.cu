// Error reporting and identification of the compiled library.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

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

static int g_pdl = -1;
int idm_pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("IDM_PDL");
        g_pdl = (e && strcmp(e, "0") == 0) ? 0 : 1;
    }
    return g_pdl;
}
extern "C" void idm_set_pdl(int on) { g_pdl = on ? 1 : 0; }

int idm_pdl_flag(const char* name, int dflt) {
    const char* e = getenv(name);
    if (!e) return dflt;
    return strcmp(e, "0") != 0;
}
