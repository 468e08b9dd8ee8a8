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
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int t = tokens[r];
    const bool ok = t >= 0 && t < V;
    const T* src = table + (size_t)(ok ? t : 0) * E;
    float* dst = out + (size_t)r * E;
    if (E % 4 == 0) {
        // Four elements a thread a turn: rows start 16-byte aligned when E is a multiple of 4 (float) or 8 (bf16).
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (ok) {
                if (sizeof(T) == 4) {
                    v = *reinterpret_cast<const float4*>(src + c);
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2*>(src + c);
                    v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                                    __uint_as_float(raw.y & 0xffff0000u));
                }
            }
            *reinterpret_cast<float4*>(dst + c) = v;
        }
        return;
    }
    for (int c = threadIdx.x; c < E; c += blockDim.x) dst[c] = ok ? to_f32(src[c]) : 0.0f;
}

// -------------------------------------------------------------------------------- RMSNorm
// out[i, c] = x[row(i), c] * rsqrt(mean_c(x^2) + eps) * w[c]; eps inside the root, the
// weight applied after the scale (model.rs:381-389; gpu/kernels.h:226-233).  `gather`
// (may be null) picks the rows to normalise, so the head runs on wanted rows only.
template <class T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// A thread's share of the sum of squares is taken in ascending column order and the
// shares are added in a fixed tree, so a row's statistic is the same bits in any batch.
template <class T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                               const int* __restrict__ gather, int E, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int i = blockIdx.x;
    if (E % 4 == 0 && E <= 4 * (int)blockDim.x) {
        // A thread holds at most one float4 of the row: the row is read once, and the norm's
        // weights (written by no kernel) are fetched before the wait for the preceding kernel.
        // The sums are the same as below, in the same order.
        const int c = 4 * threadIdx.x;
        const bool mine = c < E;
        const float4 g = mine ? *reinterpret_cast<const float4*>(w + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        pdl_wait();
        const int r = gather ? gather[i] : i;
        const float4 v = mine ? *reinterpret_cast<const float4*>(x + (size_t)r * E + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float s = 0.0f;
        if (mine) s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        s = block_sum(s, scratch);
        const float scale = 1.0f / sqrtf(s / (float)E + eps);
        if (mine) store4<T>(out + (size_t)i * E + c, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        return;
    }
    pdl_wait();
    const int r = gather ? gather[i] : i;
    const float* xr = x + (size_t)r * E;
    T* o = out + (size_t)i * E;
    float s = 0.0f;
    if (E % 4 == 0) {
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(xr + c);
            s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        s = block_sum(s, scratch);
        const float scale = 1.0f / sqrtf(s / (float)E + eps);
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(xr + c);
            const float4 g = *reinterpret_cast<const float4*>(w + c);
            store4<T>(o + c, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
        return;
    }
    for (int c = threadIdx.x; c < E; c += blockDim.x) {
        float v = xr[c];
        s += v * v;
    }
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)E + eps);
    for (int c = threadIdx.x; c < E; c += blockDim.x) o[c] = from_f32<T>(xr[c] * scale * w[c]);
}

// The same for many rows (prompts): 256 threads a row, each keeping its share of the row in
// registers, so that the row is read once.  Takes E a multiple of 4 up to 8192.
template <class T>
__global__ void __launch_bounds__(256) rmsnorm_wide_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                                                           const int* __restrict__ gather, int E, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int r = gather ? gather[i] : i;
    const float* xr = x + (size_t)r * E;
    T* o = out + (size_t)i * E;
    float4 v[8];
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int c = 4 * (threadIdx.x + 256 * k);
        v[k] = c < E ? *reinterpret_cast<const float4*>(xr + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        s += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
    s = block_sum(s, scratch);
    const float scale = 1.0f / sqrtf(s / (float)E + eps);
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int c = 4 * (threadIdx.x + 256 * k);
        if (c < E) {
            const float4 g = *reinterpret_cast<const float4*>(w + c);
            store4<T>(o + c, v[k].x * scale * g.x, v[k].y * scale * g.y, v[k].z * scale * g.z, v[k].w * scale * g.w);
        }
    }
}

// --------------------------------------------------------------------------------- SwiGLU
// out[r, j] = silu(gu[r, j]) * gu[r, F + j], silu(g) = g / (1 + e^-g) (model.rs:343;
// kernels.h:330).  The stand-alone form; the serving GEMM fuses it into its epilogue.
template <class T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t r = i / F;
    int j = (int)(i - r * F);
    float g = to_f32(gu[r * 2 * F + j]);
    float u = to_f32(gu[r * 2 * F + F + j]);
    out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// Four or eight consecutive elements moved as one aligned piece (heads are multiples of 16
// elements and pairs are taken four at a time, so the alignment holds).
template <class T> struct __align__(4 * sizeof(T)) Wide4 { T v[4]; };
template <class T> struct __align__(8 * sizeof(T)) Wide8 { T v[8]; };

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
    // threadIdx.y picks one (row, head of the fused projection) of the block's: q heads, then
    // k heads, then v heads.  Nothing below synchronises, so threads may leave early.
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y * blockDim.y + threadIdx.y;
    if (h >= H + 2 * G) return;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = row_pos[r];
    const int half = D / 2;
    T* head = qkv + ((size_t)r * (H + 2 * G) + h) * D;
    int page = -1;
    if (h >= H && write_cache && pos / BC_PAGE < max_pages) page = page_table[(size_t)slot * max_pages + pos / BC_PAGE];
    const bool can_write = page >= 0 && page < n_pages;
    const int in_page = pos % BC_PAGE;
    if (h >= H + G) {
        if (!can_write) return;
        T* dst = v_cache + (((size_t)page * G + (h - H - G)) * BC_PAGE + in_page) * D;
        // D is a multiple of 16, so a head is whole 16-byte pieces in either type.
        constexpr int PER = 16 / sizeof(T);
        for (int d = threadIdx.x * PER; d < D; d += blockDim.x * PER)
            *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(head + d);
        return;
    }
    const float2* cs = cos_sin ? cos_sin + (size_t)pos * half : nullptr;
    T* dst = h < H ? head : (can_write ? k_cache + (((size_t)page * G + (h - H)) * BC_PAGE + in_page) * D : nullptr);
    if (!dst) return;
    // Four pairs a thread a turn (D/2 is a multiple of 8): both pairings then read and write
    // whole 8- or 16-byte pieces.  Each product and sum is rounded on its own (no fused
    // multiply-add): the decode attention kernel rotates with the same four roundings and
    // must give the same bits.
    for (int i = 4 * threadIdx.x; i < half; i += 4 * blockDim.x) {
        float x0[4], x1[4], y0[4], y1[4];
        T in[8], res[8];   // the 8 values of 4 pairs: one wide read or two, by pairing
        if (pairing) {
            *reinterpret_cast<Wide8<T>*>(in) = *reinterpret_cast<const Wide8<T>*>(head + 2 * i);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                x0[j] = to_f32(in[2 * j]);
                x1[j] = to_f32(in[2 * j + 1]);
            }
        } else {
            *reinterpret_cast<Wide4<T>*>(in) = *reinterpret_cast<const Wide4<T>*>(head + i);
            *reinterpret_cast<Wide4<T>*>(in + 4) = *reinterpret_cast<const Wide4<T>*>(head + i + half);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                x0[j] = to_f32(in[j]);
                x1[j] = to_f32(in[4 + j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            y0[j] = x0[j];
            y1[j] = x1[j];
            if (cs) {
                const float2 c = cs[i + j];
                y0[j] = __fsub_rn(__fmul_rn(x0[j], c.x), __fmul_rn(x1[j], c.y));
                y1[j] = __fadd_rn(__fmul_rn(x0[j], c.y), __fmul_rn(x1[j], c.x));
            }
        }
        if (pairing) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                res[2 * j] = from_f32<T>(y0[j]);
                res[2 * j + 1] = from_f32<T>(y1[j]);
            }
            *reinterpret_cast<Wide8<T>*>(dst + 2 * i) = *reinterpret_cast<const Wide8<T>*>(res);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                res[j] = from_f32<T>(y0[j]);
                res[4 + j] = from_f32<T>(y1[j]);
            }
            *reinterpret_cast<Wide4<T>*>(dst + i) = *reinterpret_cast<const Wide4<T>*>(res);
            *reinterpret_cast<Wide4<T>*>(dst + i + half) = *reinterpret_cast<const Wide4<T>*>(res + 4);
        }
    }
}

// The same for many rows of bf16 (prompts) with a head size that is a multiple of 16: eight
// pairs a thread, 16-byte reads and writes, 32 heads of a row a block.  The same products,
// sums and roundings as above.
__global__ void __launch_bounds__(256)
rope_append_wide_kernel(bf16* __restrict__ qkv, const float2* __restrict__ cos_sin, const int* __restrict__ row_pos,
                        const int* __restrict__ row_slot, const int* __restrict__ page_table, bf16* __restrict__ k_cache,
                        bf16* __restrict__ v_cache, int H, int G, int D, int pairing, int max_pages, int n_pages, int write_cache) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, h = blockIdx.y * blockDim.y + threadIdx.y;
    if (h >= H + 2 * G) return;
    const int slot = row_slot[r];
    if (slot < 0) return;
    const int pos = row_pos[r];
    const int half = D / 2;
    bf16* head = qkv + ((size_t)r * (H + 2 * G) + h) * D;
    int page = -1;
    if (h >= H && write_cache && pos / BC_PAGE < max_pages) page = page_table[(size_t)slot * max_pages + pos / BC_PAGE];
    const bool can_write = page >= 0 && page < n_pages;
    const int in_page = pos % BC_PAGE;
    if (h >= H + G) {
        if (!can_write) return;
        bf16* dst = v_cache + (((size_t)page * G + (h - H - G)) * BC_PAGE + in_page) * D;
        for (int d = threadIdx.x * 8; d < D; d += blockDim.x * 8) *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(head + d);
        return;
    }
    const float2* cs = cos_sin ? cos_sin + (size_t)pos * half : nullptr;
    bf16* dst = h < H ? head : (can_write ? k_cache + (((size_t)page * G + (h - H)) * BC_PAGE + in_page) * D : nullptr);
    if (!dst) return;
    for (int i = 8 * threadIdx.x; i < half; i += 8 * blockDim.x) {   // pairs i .. i + 7
        bf16 lo[8], hi[8];   // pairing 0: elements i.. and i + half..; pairing 1: elements 2 i .. 2 i + 15, even and odd taken apart below
        if (pairing) {
            *reinterpret_cast<uint4*>(lo) = *reinterpret_cast<const uint4*>(head + 2 * i);
            *reinterpret_cast<uint4*>(hi) = *reinterpret_cast<const uint4*>(head + 2 * i + 8);
        } else {
            *reinterpret_cast<uint4*>(lo) = *reinterpret_cast<const uint4*>(head + i);
            *reinterpret_cast<uint4*>(hi) = *reinterpret_cast<const uint4*>(head + i + half);
        }
        float2 c[8];
        if (cs) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float4 two = *reinterpret_cast<const float4*>(cs + i + j);
                c[j] = make_float2(two.x, two.y);
                c[j + 1] = make_float2(two.z, two.w);
            }
        }
        bf16 out_lo[8], out_hi[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // pair j of this thread: (lo[j], hi[j]), or for adjacent pairs elements 2 j and 2 j + 1 of the 16 read
            const bf16 a = pairing ? (j < 4 ? lo[2 * j] : hi[2 * j - 8]) : lo[j];
            const bf16 b = pairing ? (j < 4 ? lo[2 * j + 1] : hi[2 * j - 7]) : hi[j];
            const float x0 = __bfloat162float(a), x1 = __bfloat162float(b);
            float y0 = x0, y1 = x1;
            if (cs) {
                y0 = __fsub_rn(__fmul_rn(x0, c[j].x), __fmul_rn(x1, c[j].y));
                y1 = __fadd_rn(__fmul_rn(x0, c[j].y), __fmul_rn(x1, c[j].x));
            }
            if (pairing) {
                bf16* o = j < 4 ? out_lo : out_hi;
                o[(2 * j) & 7] = __float2bfloat16_rn(y0);
                o[(2 * j + 1) & 7] = __float2bfloat16_rn(y1);
            } else {
                out_lo[j] = __float2bfloat16_rn(y0);
                out_hi[j] = __float2bfloat16_rn(y1);
            }
        }
        if (pairing) {
            *reinterpret_cast<uint4*>(dst + 2 * i) = *reinterpret_cast<const uint4*>(out_lo);
            *reinterpret_cast<uint4*>(dst + 2 * i + 8) = *reinterpret_cast<const uint4*>(out_hi);
        } else {
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(out_lo);
            *reinterpret_cast<uint4*>(dst + i + half) = *reinterpret_cast<const uint4*>(out_hi);
        }
    }
}

// ------------------------------------------------------------------------------ launchers
static int pick_threads(int n, int cap = 256) {
    int t = 32;
    while (t < n && t < cap) t <<= 1;
    return t;
}

#define ROWWISE_LAUNCHERS(SUFFIX, T)                                                                                             \
    extern "C" int bc_embed_##SUFFIX(const void* table, const int* tokens, float* out, int rows, int E, int V, cudaStream_t s) { \
        BC_CHECK_ARG(rows >= 0 && E > 0 && V > 0, "embed: bad sizes rows=%d E=%d V=%d", rows, E, V);                             \
        if (rows == 0) return BC_OK;                                                                                             \
        bc_launch(embed_kernel<T>, dim3(rows), dim3(pick_threads(E % 4 == 0 ? E / 4 : E, 1024)), 0, s, (const T*)table, tokens, out, E, V);                                    \
        BC_LAUNCH_STATUS();                                                                                                      \
    }                                                                                                                            \
    extern "C" int bc_rmsnorm_##SUFFIX(const float* x, const float* w, void* out, const int* gather, int rows, int E, float eps, \
                                       cudaStream_t s) {                                                                         \
        BC_CHECK_ARG(rows >= 0 && E > 0 && eps > 0.0f, "rmsnorm: bad sizes rows=%d E=%d eps=%g", rows, E, (double)eps);          \
        if (rows == 0) return BC_OK;                                                                                             \
        /* The two kernels add a row's squares in different orders.  The 32-bit path promises the same bits for a row */      \
        /* however it is batched, so it keeps one kernel; serving takes the single-pass one for prompts.                */      \
        if (sizeof(T) == 2 && rows > 64 && E % 4 == 0 && E <= 8192)                                                             \
            bc_launch(rmsnorm_wide_kernel<T>, dim3(rows), dim3(256), 0, s, x, w, (T*)out, gather, E, eps);                       \
        else                                                                                                                     \
            bc_launch(rmsnorm_kernel<T>, dim3(rows), dim3(pick_threads(E % 4 == 0 ? E / 4 : E, 1024)), 0, s, x, w, (T*)out,      \
                      gather, E, eps);                                                                                           \
        BC_LAUNCH_STATUS();                                                                                                      \
    }                                                                                                                            \
    extern "C" int bc_swiglu_##SUFFIX(const void* gu, void* out, int rows, int F, cudaStream_t s) {                              \
        BC_CHECK_ARG(rows >= 0 && F > 0, "swiglu: bad sizes rows=%d F=%d", rows, F);                                             \
        size_t total = (size_t)rows * F;                                                                                         \
        if (total == 0) return BC_OK;                                                                                            \
        bc_launch(swiglu_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, (const T*)gu, (T*)out, F, total);                       \
        BC_LAUNCH_STATUS();                                                                                                      \
    }                                                                                                                            \
    extern "C" int bc_rope_append_##SUFFIX(void* qkv, const float* cos_sin, const int* row_pos, const int* row_slot,             \
                                           const int* page_table, void* k_cache, void* v_cache, int rows, int H, int G, int D,   \
                                           int pairing, int max_pages, int n_pages, int write_cache, cudaStream_t s) {           \
        BC_CHECK_ARG(rows >= 0 && H > 0 && G > 0 && D > 0 && D % 2 == 0, "rope_append: bad sizes rows=%d H=%d G=%d D=%d", rows, \
                     H, G, D);                                                                                                   \
        BC_CHECK_ARG(pairing == 0 || pairing == 1, "rope_append: pairing %d is neither 0 (half) nor 1 (adjacent)", pairing);     \
        if (rows == 0) return BC_OK;                                                                                             \
        BC_CHECK_ARG(H + 2 * G <= 65535, "rope_append: too many heads (%d)", H + 2 * G);                                          \
        if (sizeof(T) == 2 && rows > 64 && D % 16 == 0) {                                                                        \
            /* many rows (prompts): eight pairs a thread, 32 heads of a row a block */                                           \
            const int wx = D / 16 < 32 ? D / 16 : 32, wy = 256 / wx < H + 2 * G ? 256 / wx : H + 2 * G;                          \
            bc_launch(rope_append_wide_kernel, dim3(rows, (H + 2 * G + wy - 1) / wy), dim3(wx, wy), 0, s, (bf16*)qkv,              \
                      (const float2*)cos_sin, row_pos, row_slot, page_table, (bf16*)k_cache, (bf16*)v_cache, H, G, D, pairing,     \
                      max_pages, n_pages, write_cache);                                                                          \
            BC_LAUNCH_STATUS();                                                                                                  \
        }                                                                                                                        \
        /* few rows (decoding): a block a head, for the shortest critical path; many rows: eight heads a block */                \
        const int tx = pick_threads(D / 8, 32), ty = rows <= 64 ? 1 : 8;                                         \
        bc_launch(rope_append_kernel<T>, dim3(rows, (H + 2 * G + ty - 1) / ty), dim3(tx, ty), 0, s, (T*)qkv,                       \
                  (const float2*)cos_sin, row_pos, row_slot, page_table, (T*)k_cache, (T*)v_cache, H, G, D, pairing, max_pages,  \
                  n_pages, write_cache);                                                                                         \
        BC_LAUNCH_STATUS();                                                                                                      \
    }

ROWWISE_LAUNCHERS(f32, float)
ROWWISE_LAUNCHERS(bf16, bf16)
