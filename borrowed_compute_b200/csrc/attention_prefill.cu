// Prompt attention for bf16: many new rows a sequence against the paged cache (which by
// then holds their own keys and values too), causal, grouped-query, in one pass.
//
// What is computed is the reference's attention (crates/bc-infer/src/model.rs:448-481),
// with the running maximum / sum / weighted values of its kernel
// (crates/bc-infer/src/gpu/kernels.h:271-324).  How: a block takes (tile of query rows,
// kv head, sequence).  A tile is 64 rows = (tokens) x (the heads that share the kv head),
// token-major, so every 64-position page of keys and values read from the cache serves
// all of those heads; four warps take 16 rows each.  Per page: S = Q K^T on m16n8k16
// tensor-core tiles, scores masked to the positions each row may see (0 .. its own, or the
// last `window`), softmax statistics in float, P rounded to bf16, O += P V in float.
// Pages stream through shared memory by cp.async, one ahead (two stages, so that three
// blocks fit an SM).  Rows are found through
// per-sequence row ranges and start positions, so sequences of any lengths, with or
// without earlier cached positions, share one launch.
#include "common.cuh"
#include "mma_tiles.cuh"

#define AP_THREADS 128
#define AP_STAGES 2
#define AP_ROWS 64

template <int D>
__global__ void __launch_bounds__(AP_THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                         const int* __restrict__ page_table, const int* __restrict__ seq_rows, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_start, bf16* __restrict__ out, int H, int G, int max_pages, int n_pages, int window,
                         float scale_log2) {
    constexpr int CHUNKS = D / 8;
    constexpr int TILE_BYTES = 64 * D * 2;
    constexpr int KD = D / 16;
    constexpr int ND = D / 8;
    extern __shared__ __align__(128) uint8_t smem[];

    pdl_launch_dependents();
    pdl_wait();
    const int g = blockIdx.x, sq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int group = H / G;
    const int tokens_per_tile = AP_ROWS / group;          // rows past tokens_per_tile * group are padding
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    const int n_tiles_q = (n_new + tokens_per_tile - 1) / tokens_per_tile;
    // The last query tiles see the most keys: they go first, for all kv heads (x runs fastest),
    // so that the blocks start in the order of their work.
    const int q_tile = n_tiles_q - 1 - (int)blockIdx.y;
    if (slot < 0 || q_tile < 0) return;
    const int start = seq_start[sq];
    const int tok0 = q_tile * tokens_per_tile;            // first token (within the step) of this tile
    const int tok_end = min(n_new, tok0 + tokens_per_tile);
    const int* pages = page_table + (size_t)slot * max_pages;

    // This thread's two rows of the warp's 16: which token and head they are, and what they see.
    int tok[2], head[2], pos[2], lo[2];
    bool live[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int row = 16 * warp + gq + 8 * i;
        tok[i] = tok0 + row / group;
        head[i] = g * group + row % group;
        live[i] = row / group < tokens_per_tile && tok[i] < n_new;
        pos[i] = start + tok[i];
        lo[i] = window > 0 && pos[i] + 1 > window ? pos[i] + 1 - window : 0;
    }
    uint32_t qf[KD][4];
#pragma unroll
    for (int kd = 0; kd < KD; kd++) {
        const int d0 = kd * 16 + 2 * tq;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const bf16* qr = q + (size_t)(row0 + tok[i]) * q_stride + (size_t)head[i] * D;
            qf[kd][i] = live[i] ? *reinterpret_cast<const uint32_t*>(qr + d0) : 0u;
            qf[kd][i + 2] = live[i] ? *reinterpret_cast<const uint32_t*>(qr + d0 + 8) : 0u;
        }
    }

    // Pages this tile reads: from the first position its first token sees to its last token's own.
    const int first_pos = window > 0 && start + tok0 + 1 > window ? start + tok0 + 1 - window : 0;
    const int t_begin = first_pos / BC_PAGE, t_end = (start + tok_end - 1) / BC_PAGE + 1;
    const int n_tiles = t_end - t_begin;
    const int last_pos = start + n_new - 1;               // the last position the sequence holds after this step

    // A tile without a page is neither fetched nor multiplied: what another sequence left in
    // some page never meets these rows.
    auto load_tile = [&](int tile, int stage) {
        const int page = tile < max_pages ? pages[tile] : -1;
        if (page < 0 || page >= n_pages) return;
        const bf16* ks = k_cache + ((size_t)page * G + g) * BC_PAGE * D;
        const bf16* vs = v_cache + ((size_t)page * G + g) * BC_PAGE * D;
        const uint32_t kb = ad_smem(smem + (size_t)stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        for (int i = threadIdx.x; i < 64 * CHUNKS; i += AP_THREADS) {
            const int row = i / CHUNKS, c = i - row * CHUNKS;
            cp_async16(kb + tile_offset<D>(row, c), ks + (size_t)row * D + c * 8);
            cp_async16(vb + tile_offset<D>(row, c), vs + (size_t)row * D + c * 8);
        }
    };

    float o[ND][4];
#pragma unroll
    for (int i = 0; i < ND; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

#pragma unroll
    for (int s = 0; s < AP_STAGES - 1; s++) {
        if (s < n_tiles) load_tile(t_begin + s, s);
        cp_async_commit();
    }
    const int j4 = lane >> 3, r8 = lane & 7;
    for (int it = 0; it < n_tiles; it++) {
        cp_async_wait<AP_STAGES - 2>();
        __syncthreads();
        if (it + AP_STAGES - 1 < n_tiles) load_tile(t_begin + it + AP_STAGES - 1, (it + AP_STAGES - 1) % AP_STAGES);
        cp_async_commit();
        const int tile = t_begin + it;
        const bool page_ok = tile < max_pages && pages[tile] >= 0 && pages[tile] < n_pages;
        if (!page_ok) continue;
        const uint32_t kb = ad_smem(smem + (size_t)(it % AP_STAGES) * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        if (tile == last_pos / BC_PAGE && last_pos % BC_PAGE != BC_PAGE - 1) {
            // The sequence's last page: what lies past its last position belongs to nobody (a
            // sequence that held the page before may have left not-a-numbers there, and 0 x NaN
            // is NaN in the product with the values): those value rows are cleared in the copy.
            uint8_t* vt = smem + (size_t)(it % AP_STAGES) * 2 * TILE_BYTES + TILE_BYTES;
            const int first = last_pos % BC_PAGE + 1;
            for (int i = threadIdx.x; i < (BC_PAGE - first) * CHUNKS; i += AP_THREADS)
                *reinterpret_cast<uint4*>(vt + tile_offset<D>(first + i / CHUNKS, i % CHUNKS)) = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
        }

        // S = Q K^T for this warp's 16 rows against the page's 64 positions.
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; nb++) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
        for (int kd = 0; kd < KD; kd++) {
#pragma unroll
            for (int np = 0; np < 4; np++) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kb + tile_offset<D>(np * 16 + (j4 >> 1) * 8 + r8, kd * 2 + (j4 & 1)), b0, b1, b2, b3);
                mma_16816(s[2 * np], qf[kd], b0, b1);
                mma_16816(s[2 * np + 1], qf[kd], b2, b3);
            }
        }
        float tmax[2] = {-INFINITY, -INFINITY};
        // A page that ends at or before the position of this warp's first row is seen whole by
        // all sixteen rows (padding rows' results are never written): no mask to work out.
        const bool whole = window == 0 && page_ok && tile * BC_PAGE + BC_PAGE - 1 <= start + tok0 + (16 * warp) / group;
        if (whole) {
#pragma unroll
            for (int nb = 0; nb < 8; nb++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s[nb][e] *= scale_log2;
                    tmax[e >> 1] = fmaxf(tmax[e >> 1], s[nb][e]);
                }
        } else {
#pragma unroll
            for (int nb = 0; nb < 8; nb++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int i = e >> 1;
                    const int t = tile * BC_PAGE + nb * 8 + 2 * tq + (e & 1);
                    const bool seen = page_ok && live[i] && t >= lo[i] && t <= pos[i];
                    s[nb][e] = seen ? s[nb][e] * scale_log2 : -INFINITY;
                    tmax[i] = fmaxf(tmax[i], s[nb][e]);
                }
        }
        float corr[2], base[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            const float mn = fmaxf(m[i], tmax[i]);
            corr[i] = mn == -INFINITY ? 1.0f : fast_exp2(m[i] - mn);
            base[i] = mn == -INFINITY ? 0.0f : mn;
            m[i] = mn;
        }
        float psum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int nb = 0; nb < 8; nb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                s[nb][e] = fast_exp2(s[nb][e] - base[e >> 1]);
                psum[e >> 1] += s[nb][e];
            }
        l[0] = l[0] * corr[0] + psum[0];
        l[1] = l[1] * corr[1] + psum[1];
#pragma unroll
        for (int nd = 0; nd < ND; nd++) {
            o[nd][0] *= corr[0]; o[nd][1] *= corr[0]; o[nd][2] *= corr[1]; o[nd][3] *= corr[1];
        }
        // O += P V, 16 positions a step.
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const uint32_t pf[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                    pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vb + tile_offset<D>(kk * 16 + (j4 & 1) * 8 + r8, nd + (j4 >> 1)), b0, b1, b2, b3);
                mma_16816(o[nd], pf, b0, b1);
                mma_16816(o[nd + 1], pf, b2, b3);
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (!live[i]) continue;
        const float inv = l[i] > 0.0f ? 1.0f / l[i] : 0.0f;
        bf16* dst = out + ((size_t)(row0 + tok[i]) * H + head[i]) * D + 2 * tq;
#pragma unroll
        for (int nd = 0; nd < ND; nd++)
            *reinterpret_cast<uint32_t*>(dst + nd * 8) = pack_bf16(o[nd][2 * i] * inv, o[nd][2 * i + 1] * inv);
    }
}

template <int D>
static int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table, const int* seq_rows,
                  const int* seq_slot, const int* seq_start, void* out, int seqs, int max_new, int H, int G, int max_pages, int n_pages,
                  int window, float scale, cudaStream_t s) {
    constexpr int SMEM = AP_STAGES * 2 * 64 * D * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) {
            bc_set_error("attention_prefill: cannot set shared memory to %d: %s", SMEM, cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    const int tokens_per_tile = AP_ROWS / (H / G);
    dim3 grid(G, (max_new + tokens_per_tile - 1) / tokens_per_tile, seqs);
    bc_launch(attention_prefill_kernel<D>, grid, dim3(AP_THREADS), (size_t)SMEM, s, (const bf16*)q, q_stride, (const bf16*)k_cache,
              (const bf16*)v_cache, page_table, seq_rows, seq_slot, seq_start, (bf16*)out, H, G, max_pages, n_pages, window,
              scale * 1.4426950408889634f);
    BC_LAUNCH_STATUS();
}

// Whether this kernel takes the sizes (else the caller uses the one-warp-a-row kernel).
extern "C" int bc_attention_prefill_accepts(int H, int G, int D) {
    return G > 0 && H % G == 0 && H / G <= AP_ROWS && D % 16 == 0 && D >= 16 && D <= 128;
}

// Sequence s owns rows seq_rows[s] .. seq_rows[s + 1] of q and out (row r's head h at
// q + r * q_stride + h * D), lives in slot seq_slot[s] (negative: skipped, its rows of
// `out` are left untouched) and held seq_start[s] positions before this step; the cache
// already holds this step's keys and values.  max_new: the most rows any sequence brings.
extern "C" int bc_attention_prefill_bf16(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                         const int* seq_rows, const int* seq_slot, const int* seq_start, void* out, int seqs, int max_new,
                                         int H, int G, int D, int max_pages, int n_pages, int window, float scale, cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 65535 && max_new >= 0 && max_new < 65535, "attention_prefill: bad sizes seqs=%d max_new=%d", seqs, max_new);
    BC_CHECK_ARG(bc_attention_prefill_accepts(H, G, D), "attention_prefill: H=%d G=%d D=%d is outside what this kernel takes "
                 "(at most %d heads a kv head, head size a multiple of 16 up to 128)", H, G, D, AP_ROWS);
    BC_CHECK_ARG(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0) && ((uintptr_t)out % 4 == 0), "attention_prefill: q and out must be 4-byte aligned");
    if (seqs == 0 || max_new == 0) return BC_OK;
#define AP_CASE(DD) \
    case DD: return launch<DD>(q, q_stride, k_cache, v_cache, page_table, seq_rows, seq_slot, seq_start, out, seqs, max_new, H, G, max_pages, n_pages, window, scale, s);
    switch (D) {
        AP_CASE(16) AP_CASE(32) AP_CASE(48) AP_CASE(64) AP_CASE(80) AP_CASE(96) AP_CASE(112) AP_CASE(128)
    }
#undef AP_CASE
    bc_set_error("attention_prefill: no kernel for head size %d", D);
    return BC_ERR_ARG;
}
