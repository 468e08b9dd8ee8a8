// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, and rotary encoding fused with the
// append of new keys and values to the paged cache.  Each is templated on the activation
// type (float for the true 32-bit path, bf16 for serving); statistics, angles and the
// residual stream are float in both.
#include "common.cuh"

// ------------------------------------------------------------------------------ embedding
// out[r, :] = table[tokens[r], :] widened to float (the residual stream is float).
// Reference: Part::embed, crates/bc-infer/src/model.rs:270-280.  A token outside the
// table (the host rejects those before launch) yields a row of zeros, never a wild read.
template <class T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ out, int E, int V) {
    const int r = blockIdx.x;
    const int t = tokens[r];
    const bool ok = t >= 0 && t < V;
    const T* src = table + (size_t)(ok ? t : 0) * E;
    float* dst = out + (size_t)r * E;
    for (int c = threadIdx.x; c < E; c += blockDim.x) dst[c] = ok ? to_f32(src[c]) : 0.0f;
}

// -------------------------------------------------------------------------------- RMSNorm
// out[i, c] = x[row(i), c] * rsqrt(mean_c(x^2) + eps) * w[c]; eps inside the root, the
// weight applied after the scale (model.rs:381-389; gpu/kernels.h:226-233).  `gather`
// (may be null) picks the rows to normalise, so the head runs on wanted rows only.
template <class T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                               const int* __restrict__ gather, int E, float eps) {
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int r = gather ? gather[i] : i;
    const float* xr = x + (size_t)r * E;
    float s = 0.0f;
    for (int c = threadIdx.x; c < E; c += blockDim.x) {
        float v = xr[c];
        s += v * v;
    }
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)E + eps);
    T* o = out + (size_t)i * E;
    for (int c = threadIdx.x; c < E; c += blockDim.x) o[c] = from_f32<T>(xr[c] * scale * w[c]);
}

// --------------------------------------------------------------------------------- SwiGLU
// out[r, j] = silu(gu[r, j]) * gu[r, F + j], silu(g) = g / (1 + e^-g) (model.rs:343;
// kernels.h:330).  The stand-alone form; the serving GEMM fuses it into its epilogue.
template <class T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t r = i / F;
    int j = (int)(i - r * F);
    float g = to_f32(gu[r * 2 * F + j]);
    float u = to_f32(gu[r * 2 * F + F + j]);
    out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// ----------------------------------------------------------------- rotary + cache append
// For every row r of the fused projection qkv[r] = [q heads | k heads | v heads]:
//   q and k pairs (a, b) rotate by the angle of (row_pos[r], pair i):
//     x_a' = x_a cos - x_b sin,  x_b' = x_a sin + x_b cos          (model.rs:391-403)
//   with (a, b) = (i, i + D/2) for pairing 0 and (2i, 2i + 1) for pairing 1 (kernels.h:243-244).
//   q is rotated in place; rotated k and plain v go to the cache page of (row_slot[r],
//   row_pos[r]) (the reference appends with k_copy, gpu/mod.rs:473-475).
// cos_sin[pos][i] = (cos, sin) of the float product pos * inv_freq[i], tabulated by the host.
// A null table leaves q and k unrotated.  Rows whose slot is negative are padding: they
// touch nothing.  Cache layout of one layer: [page][kv_head][BC_PAGE][D].
template <class T>
__global__ void rope_append_kernel(T* __restrict__ qkv, const float2* __restrict__ cos_sin, const int* __restrict__ row_pos,
                                   const int* __restrict__ row_slot, const int* __restrict__ page_table, T* __restrict__ k_cache,
                                   T* __restrict__ v_cache, int H, int G, int D, int pairing, int max_pages, int n_pages, int write_cache) {
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = row_pos[r];
    const int half = D / 2;
    T* row = qkv + (size_t)r * (H + 2 * G) * D;
    int page = -1;
    if (write_cache && pos / BC_PAGE < max_pages) page = page_table[(size_t)slot * max_pages + pos / BC_PAGE];
    const bool can_write = page >= 0 && page < n_pages;
    const int in_page = pos % BC_PAGE;
    const float2* cs = cos_sin ? cos_sin + (size_t)pos * half : nullptr;

    const int rot_pairs = (H + G) * half;
    for (int idx = threadIdx.x; idx < rot_pairs; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const int a = pairing ? 2 * i : i, b = pairing ? 2 * i + 1 : i + half;
        T* head = row + (size_t)h * D;
        float x0 = to_f32(head[a]), x1 = to_f32(head[b]);
        float y0 = x0, y1 = x1;
        if (cs) {
            const float2 c = cs[i];
            y0 = x0 * c.x - x1 * c.y;
            y1 = x0 * c.y + x1 * c.x;
        }
        if (h < H) {
            head[a] = from_f32<T>(y0);
            head[b] = from_f32<T>(y1);
        } else if (can_write) {
            T* dst = k_cache + (((size_t)page * G + (h - H)) * BC_PAGE + in_page) * D;
            dst[a] = from_f32<T>(y0);
            dst[b] = from_f32<T>(y1);
        }
    }
    if (can_write) {
        const T* v = row + (size_t)(H + G) * D;
        for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
            const int g = idx / D, d = idx - g * D;
            v_cache[(((size_t)page * G + g) * BC_PAGE + in_page) * D + d] = v[idx];
        }
    }
}

// ------------------------------------------------------------------------------ launchers
static int pick_threads(int n) {
    int t = 32;
    while (t < n && t < 256) t <<= 1;
    return t;
}

#define ROWWISE_LAUNCHERS(SUFFIX, T)                                                                                             \
    extern "C" int bc_embed_##SUFFIX(const void* table, const int* tokens, float* out, int rows, int E, int V, cudaStream_t s) { \
        BC_CHECK_ARG(rows >= 0 && E > 0 && V > 0, "embed: bad sizes rows=%d E=%d V=%d", rows, E, V);                             \
        if (rows == 0) return BC_OK;                                                                                             \
        embed_kernel<T><<<rows, pick_threads(E), 0, s>>>((const T*)table, tokens, out, E, V);                                    \
        BC_LAUNCH_STATUS();                                                                                                      \
    }                                                                                                                            \
    extern "C" int bc_rmsnorm_##SUFFIX(const float* x, const float* w, void* out, const int* gather, int rows, int E, float eps, \
                                       cudaStream_t s) {                                                                         \
        BC_CHECK_ARG(rows >= 0 && E > 0 && eps > 0.0f, "rmsnorm: bad sizes rows=%d E=%d eps=%g", rows, E, (double)eps);          \
        if (rows == 0) return BC_OK;                                                                                             \
        rmsnorm_kernel<T><<<rows, pick_threads(E), 0, s>>>(x, w, (T*)out, gather, E, eps);                                       \
        BC_LAUNCH_STATUS();                                                                                                      \
    }                                                                                                                            \
    extern "C" int bc_swiglu_##SUFFIX(const void* gu, void* out, int rows, int F, cudaStream_t s) {                              \
        BC_CHECK_ARG(rows >= 0 && F > 0, "swiglu: bad sizes rows=%d F=%d", rows, F);                                             \
        size_t total = (size_t)rows * F;                                                                                         \
        if (total == 0) return BC_OK;                                                                                            \
        swiglu_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, s>>>((const T*)gu, (T*)out, F, total);                       \
        BC_LAUNCH_STATUS();                                                                                                      \
    }                                                                                                                            \
    extern "C" int bc_rope_append_##SUFFIX(void* qkv, const float* cos_sin, const int* row_pos, const int* row_slot,             \
                                           const int* page_table, void* k_cache, void* v_cache, int rows, int H, int G, int D,   \
                                           int pairing, int max_pages, int n_pages, int write_cache, cudaStream_t s) {           \
        BC_CHECK_ARG(rows >= 0 && H > 0 && G > 0 && D > 0 && D % 2 == 0, "rope_append: bad sizes rows=%d H=%d G=%d D=%d", rows, \
                     H, G, D);                                                                                                   \
        BC_CHECK_ARG(pairing == 0 || pairing == 1, "rope_append: pairing %d is neither 0 (half) nor 1 (adjacent)", pairing);     \
        if (rows == 0) return BC_OK;                                                                                             \
        rope_append_kernel<T><<<rows, 256, 0, s>>>((T*)qkv, (const float2*)cos_sin, row_pos, row_slot, page_table, (T*)k_cache,  \
                                                   (T*)v_cache, H, G, D, pairing, max_pages, n_pages, write_cache);              \
        BC_LAUNCH_STATUS();                                                                                                      \
    }

ROWWISE_LAUNCHERS(f32, float)
ROWWISE_LAUNCHERS(bf16, bf16)
