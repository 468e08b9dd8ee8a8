// The library's last error text and its version, readable from any binding.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void bc_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// Whether launches ask for programmatic dependent launch (see common.cuh).
int g_bc_pdl = 1;
extern "C" void bc_set_pdl(int on) { g_bc_pdl = on ? 1 : 0; }
extern "C" int bc_get_pdl() { return g_bc_pdl; }

extern "C" const char* bc_last_error() { return g_error; }

// Bumped when an exported signature changes, so a stale build is never called.
extern "C" int bc_abi_version() { return 1; }

extern "C" int bc_page_size() { return BC_PAGE; }
