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

// Streaming multiprocessors of the current device (asked once a device; 1 if it cannot be had).
extern "C" int bc_sm_count() {
    static int counts[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (counts[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        counts[dev] = n;
    }
    return counts[dev];
}

// ------------------------------------------------------------- status words the host can see
// Every kernel unit with bounded waits keeps a status word on the device.  Here each unit is
// given, once a device, a word of mapped host memory as well: the first wait that gives up
// writes its code there, and the host reads it after any synchronisation of its own (a copy
// of token ids, say) at no cost.  Word 0: the tensor-core product; word 1: the tcgen05
// prompt attention.
extern "C" int bc_gemm_tc_bind_host_word(int*);
extern "C" int bc_attention_prefill_tc_bind_host_word(int*);
extern "C" int bc_attention_decode_bind_host_word(int*);
extern "C" int bc_gemm_tc_status(int);
extern "C" int bc_attention_prefill_tc_status(int);
extern "C" int bc_attention_decode_status(int);

#define BC_STATUS_UNITS 3
static int* g_status_words[64];   // per device: BC_STATUS_UNITS ints of mapped host memory

extern "C" int bc_status_bind() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        bc_set_error("status_bind: no usable current device (%s)", cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : BC_ERR_ARG;
    }
    if (g_status_words[dev]) return BC_OK;
    int* host = nullptr;
    int* seen_by_device = nullptr;
    if ((e = cudaHostAlloc((void**)&host, 64, cudaHostAllocMapped)) != cudaSuccess ||
        (e = cudaHostGetDevicePointer((void**)&seen_by_device, host, 0)) != cudaSuccess) {
        bc_set_error("status_bind: no mapped host memory: %s", cudaGetErrorString(e));
        return (int)e;
    }
    for (int i = 0; i < 16; i++) host[i] = 0;
    int st = bc_gemm_tc_bind_host_word(seen_by_device + 0);
    if (st == 0) st = bc_attention_prefill_tc_bind_host_word(seen_by_device + 1);
    if (st == 0) st = bc_attention_decode_bind_host_word(seen_by_device + 2);
    if (st != 0) {
        bc_set_error("status_bind: cannot hand the status words to the kernels: %s", cudaGetErrorString((cudaError_t)st));
        return st;
    }
    g_status_words[dev] = host;
    return BC_OK;
}

// The status word of `unit` on the current device as the host sees it, without waiting for the
// device: 0 while all is well (or if bc_status_bind was never called).  `reset` clears a word
// that is set, on both sides.
extern "C" int bc_status_peek(int unit, int reset) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_status_words[dev] || unit < 0 || unit >= BC_STATUS_UNITS) return 0;
    const int v = *reinterpret_cast<volatile int*>(g_status_words[dev] + unit);
    if (v != 0 && reset) {
        g_status_words[dev][unit] = 0;
        if (unit == 0) bc_gemm_tc_status(1);
        else if (unit == 1) bc_attention_prefill_tc_status(1);
        else bc_attention_decode_status(1);
    }
    return v;
}
