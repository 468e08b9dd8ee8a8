// Causal grouped-query attention over the paged cache, one warp a (row, head).
//
// For the new row at position p of the sequence in `slot`, head h reads kv head
// g = h / (H / G) and sees cached positions lo..p, lo = 0 or p + 1 - window:
//   s_t = (q . k_t) / sqrt(D);  out = sum_t softmax(s)_t v_t
// (crates/bc-infer/src/model.rs:448-481).  Like the reference's kernel
// (crates/bc-infer/src/gpu/kernels.h:271-324) it keeps a running maximum m, a running sum
// l and a running weighted sum of values, rescaled by e^(m - m') when a tile of positions
// raises the maximum; scores go lanes-over-positions, values lanes-over-dimensions.  The
// order of every sum depends only on the position index, so a row's result is the same
// bits whether it came in a prompt, alone, or beside other sequences.  This kernel serves
// the true 32-bit path for prompts and decoding alike, and stands as the checked twin of
// the faster bf16 kernels.
//
// Cache layout of one layer: [page][kv_head][BC_PAGE][D]; page_table[slot][i] names the
// page of positions 64 i .. 64 i + 63.  Rows whose slot is negative are padding: their
// output is zero.
#include "common.cuh"

#define WARPS 4
#define MAX_D 256

template <class T> struct KeyDot;
template <> struct KeyDot<float> {
    static __device__ __forceinline__ float dot(const float* k, const float* q, int D) {
        float s = 0.0f;
        for (int d = 0; d < D; d += 4) {
            const float4 kv = *reinterpret_cast<const float4*>(k + d);
            const float4 qv = *reinterpret_cast<const float4*>(q + d);
            s = fmaf(kv.x, qv.x, s); s = fmaf(kv.y, qv.y, s); s = fmaf(kv.z, qv.z, s); s = fmaf(kv.w, qv.w, s);
        }
        return s;
    }
};
template <> struct KeyDot<bf16> {
    static __device__ __forceinline__ float dot(const bf16* k, const float* q, int D) {
        float s = 0.0f;
        for (int d = 0; d < D; d += 8) {
            const uint4 kv = *reinterpret_cast<const uint4*>(k + d);
            const float4 q0 = *reinterpret_cast<const float4*>(q + d);
            const float4 q1 = *reinterpret_cast<const float4*>(q + d + 4);
            s = fmaf(__uint_as_float(kv.x << 16), q0.x, s); s = fmaf(__uint_as_float(kv.x & 0xffff0000u), q0.y, s);
            s = fmaf(__uint_as_float(kv.y << 16), q0.z, s); s = fmaf(__uint_as_float(kv.y & 0xffff0000u), q0.w, s);
            s = fmaf(__uint_as_float(kv.z << 16), q1.x, s); s = fmaf(__uint_as_float(kv.z & 0xffff0000u), q1.y, s);
            s = fmaf(__uint_as_float(kv.w << 16), q1.z, s); s = fmaf(__uint_as_float(kv.w & 0xffff0000u), q1.w, s);
        }
        return s;
    }
};

template <class T>
__global__ void __launch_bounds__(WARPS * 32) attention_rows_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                                                                   const T* __restrict__ v_cache, const int* __restrict__ page_table,
                                                                   const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                                                                   T* __restrict__ out, int H, int G, int D, int max_pages, int n_pages,
                                                                   int window, float scale) {
    __shared__ __align__(16) float qs[WARPS][MAX_D];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x, h = blockIdx.y * WARPS + warp;
    if (h >= H) return;
    T* o = out + ((size_t)r * H + h) * D;
    const int slot = row_slot[r];
    const int nd = (D + 31) / 32;
    if (slot < 0) {
        for (int j = 0; j < nd; j++)
            if (lane + 32 * j < D) o[lane + 32 * j] = from_f32<T>(0.0f);
        return;
    }
    const int pos = row_pos[r];
    const int g = h / (H / G);
    const T* qh = q + (size_t)r * q_stride + (size_t)h * D;
    for (int d = lane; d < D; d += 32) qs[warp][d] = to_f32(qh[d]);
    __syncwarp();

    const int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    const int* pages = page_table + (size_t)slot * max_pages;
    float acc[MAX_D / 32];
#pragma unroll
    for (int j = 0; j < MAX_D / 32; j++) acc[j] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    for (int t0 = lo & ~31; t0 <= pos; t0 += 32) {
        // A tile of 32 positions starts at a multiple of 32, so it lies in one page.
        const int pi = t0 / BC_PAGE;
        int page = pi < max_pages ? pages[pi] : -1;
        if (page < 0 || page >= n_pages) page = -1;
        const size_t base = (((size_t)(page < 0 ? 0 : page) * G + g) * BC_PAGE + (t0 % BC_PAGE)) * D;
        const int t = t0 + lane;
        const bool seen = page >= 0 && t >= lo && t <= pos;
        float s = -INFINITY;
        if (seen) s = KeyDot<T>::dot(k_cache + base + (size_t)lane * D, qs[warp], D) * scale;
        const float mn = fmaxf(m, warp_max(s));
        const float corr = mn == -INFINITY ? 1.0f : expf(m - mn);
        const float p = seen ? expf(s - mn) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int j = 0; j < MAX_D / 32; j++) acc[j] *= corr;
        const int count = page < 0 ? 0 : min(32, pos + 1 - t0);
        const T* vt = v_cache + base;
        for (int i = 0; i < count; i++) {
            const float pi_ = __shfl_sync(0xffffffffu, p, i);
#pragma unroll
            for (int j = 0; j < MAX_D / 32; j++) {
                const int d = lane + 32 * j;
                if (j < nd && d < D) acc[j] = fmaf(pi_, to_f32(vt[(size_t)i * D + d]), acc[j]);
            }
        }
        m = mn;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < MAX_D / 32; j++) {
        const int d = lane + 32 * j;
        if (j < nd && d < D) o[d] = from_f32<T>(acc[j] * inv);
    }
}

template <class T>
static int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table, const int* row_pos,
                  const int* row_slot, void* out, int rows, int H, int G, int D, int max_pages, int n_pages, int window, float scale,
                  cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && G > 0 && H % G == 0, "attention_rows: bad sizes rows=%d H=%d G=%d", rows, H, G);
    BC_CHECK_ARG(D > 0 && D % 16 == 0 && D <= MAX_D, "attention_rows: head size %d is not a multiple of 16 up to %d", D, MAX_D);
    BC_CHECK_ARG(rows <= 2147483647 && (H + WARPS - 1) / WARPS <= 65535, "attention_rows: too many heads (%d)", H);
    if (rows == 0) return BC_OK;
    dim3 grid(rows, (H + WARPS - 1) / WARPS);
    bc_launch(attention_rows_kernel<T>, grid, dim3(WARPS * 32), 0, s, (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, page_table,
              row_pos, row_slot, (T*)out, H, G, D, max_pages, n_pages, window, scale);
    BC_LAUNCH_STATUS();
}

// q: row r's head h at q + r * q_stride + h * D (so q may live inside a fused projection).
extern "C" int bc_attention_rows_f32(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                     const int* row_pos, const int* row_slot, void* out, int rows, int H, int G, int D, int max_pages,
                                     int n_pages, int window, float scale, cudaStream_t s) {
    return launch<float>(q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, rows, H, G, D, max_pages, n_pages, window, scale, s);
}
extern "C" int bc_attention_rows_bf16(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                      const int* row_pos, const int* row_slot, void* out, int rows, int H, int G, int D, int max_pages,
                                      int n_pages, int window, float scale, cudaStream_t s) {
    return launch<bf16>(q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, rows, H, G, D, max_pages, n_pages, window, scale, s);
}
