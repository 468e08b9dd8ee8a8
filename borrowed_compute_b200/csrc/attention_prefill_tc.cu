// Prompt attention on the 5th-generation tensor cores (bf16, head size 64 or 128).
//
// What is computed is the reference's attention (crates/bc-infer/src/model.rs:448-481) with
// the running maximum / sum of its kernel (crates/bc-infer/src/gpu/kernels.h:271-324); how
// it is laid out is Blackwell's own:
//
//   - A block takes one or two tiles of 128 query rows = (tokens) x (the heads that share one
//     kv head), token major, of one sequence.  Q comes by one 3-d TMA box per 64 elements
//     of the head size straight out of the fused projection [row][head][d]; every
//     64-position page of keys and values comes by 2-d TMA boxes from the paged cache into
//     a ring of stages.  All tiles are 128-byte-swizzled blocks of [rows][64 elements].
//   - S = Q K^T is one chain of tcgen05.mma (M 128 rows, N 64 positions, K the head size),
//     accumulated in TMEM, two buffers, so the scores of the next page are computed while
//     the softmax warps work on this one.  Keys are the k-major B operand as they lie.
//   - Four softmax warps a query tile own 32 rows each, one row a thread (TMEM lane = row), so row
//     maxima and sums need no shuffles: tcgen05.ld the scores, mask what the row may not
//     see (positions after its own, before its window), exponentiate against the running
//     maximum (scaled two at a time, fma.rn.f32x2), round to bf16 and write P back into tensor
//     memory (tcgen05.st), two to a column, over the first half of the scores it came from.
//   - O += P V is a second chain of tcgen05.mma (N = head size, K = 64 positions) whose A
//     operand is read out of tensor memory, into a TMEM accumulator that stays there for the
//     whole block.  Values are the n-major B operand ([position][d] with d contiguous),
//     exactly as TMA wrote the page.  Shared memory holds Q and the ring of pages, nothing else.
//   - The running maximum is only raised when the new maximum exceeds it by more than 8 (in
//     log2 units), so P stays below 2^8 and the accumulator is rescaled (TMEM load, multiply,
//     store) a few times a block instead of once a page.  Sums and outputs use the same
//     maximum, so the result is the softmax all the same.
//
// Warp roles: warp 0 issues TMA, warp 1 owns TMEM and issues the MMAs, warps 2-5 (and 6-9 for
// the second query tile) are the softmax and write the output.  Every wait is bounded
// (about a second); a wait that gives up records where in a status word, and the block
// frees its TMEM and returns.
#include "mma_tiles.cuh"
#include "tc_ptx.cuh"
#include "tma_host.cuh"

#define APT_ROWS 128        // query rows of one tile: the M of the MMAs, the lanes of TMEM
#define APT_PAGES_KEPT 256
// Where P (the exponentials, bf16) goes between the softmax and the product with the values:
// into tensor memory, over the first half of the scores it came from (1, the default: the
// product then reads its A operand out of TMEM and shared memory carries 72 KB a page less for
// two query tiles of head size 128), or into shared memory (0, for comparison).
#ifndef APT_P_TMEM
#define APT_P_TMEM 1
#endif
#define APT_SMEM_LIMIT 232448
#define APT_Q_BYTES(D, NT) (((D) / 64) * (NT) * APT_ROWS * 128)
#define APT_STAGE_BYTES(D) (2 * ((D) / 64) * 64 * 128)
#define APT_PB(D, NT) (APT_P_TMEM ? 0 : ((D) == 128 && (NT) == 2) ? 1 : 2)
#define APT_STAGES_FIT(D, NT) ((APT_SMEM_LIMIT - 1024 - APT_Q_BYTES(D, NT)) / APT_STAGE_BYTES(D))
#define APT_STAGES(D, NT) (!APT_P_TMEM ? 4 : APT_STAGES_FIT(D, NT) > 6 ? 6 : APT_STAGES_FIT(D, NT))
#define APT_RAISE 8.0f      // the running maximum follows the true one at this distance at most

// Time stamps of one block's life, for measurement builds only (-DBC_APT_TRACE; compiled out
// otherwise): the block (0, trace_y, 0) writes clock64() values, [page][what], what 0-7 by the
// MMA thread (0 P of tile 0 seen, 1 its product issued, 2 P of tile 1 seen, 3 its product issued,
// 4 the page after next seen, 5 its scores issued), 8-15 by the first softmax warp of tile 0
// (8 scores seen, 9 read out of TMEM, 10 maximum known, 11 the product before seen, 12 P written
// and handed over).
#ifdef BC_APT_TRACE
__device__ long long* g_apt_trace = nullptr;
__device__ int g_apt_trace_y = 0;
extern "C" int bc_attention_prefill_tc_set_trace(long long* buf, int y) {
    cudaError_t e = cudaMemcpyToSymbol(g_apt_trace, &buf, sizeof(buf));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_apt_trace_y, &y, sizeof(y));
    return (int)e;
}
#define APT_STAMP(page, what) do { if (g_apt_trace && blockIdx.x == 0 && (int)blockIdx.y == g_apt_trace_y && blockIdx.z == 0 && (page) < 64) g_apt_trace[(page) * 16 + (what)] = clock64(); } while (0)
#else
#define APT_STAMP(page, what)
#endif

// NT query tiles a block (1 or 2).  Two tiles share every page of keys and values, and their
// two groups of softmax warps give every SM sub-partition two warps to switch between while
// one waits for TMEM, a fence or a barrier: with one tile the softmax warps, one a
// sub-partition, are the kernel's limit.  One tile serves steps with few new rows.
template <int D, int NT>
__global__ void __launch_bounds__(64 + NT * 128, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table, const int* __restrict__ seq_rows,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_start, bf16* __restrict__ out, int H, int G,
                            int max_pages, int n_pages, int window, float scale_log2) {
    constexpr int THREADS = 64 + NT * 128;
    constexpr int STAGES = APT_STAGES(D, NT);
    // P in shared memory only (APT_P_TMEM 0): two P tiles a query tile let the softmax of page
    // j + 1 write while the product of page j reads; with two query tiles of head size 128 shared
    // memory has room for one only, and the softmax then waits for that product.
    constexpr int PB = APT_PB(D, NT);
    constexpr int DB = D / 64;                         // 64-element blocks of the head size
    constexpr int ROW_BLOCK = APT_ROWS * 128;          // bytes of a [128 rows][64 elements] block
    constexpr int KV_BLOCK = BC_PAGE * 128;            // bytes of a [64 positions][64 elements] block
    constexpr int Q_BYTES = DB * NT * ROW_BLOCK;       // per 64 elements: the rows of all tiles, one after another
    constexpr int STAGE_BYTES = 2 * DB * KV_BLOCK;     // keys, then values, of one page
    constexpr int O_COL = NT * 128;                    // TMEM columns: scores of (tile t, buffer b) from (2 t + b) 64, outputs from O_COL + t D
    constexpr int TMEM_COLS = NT == 1 ? 256 : 512;
    static_assert(D == 64 || D == 128, "head size 64 or 128");
    static_assert(NT == 1 || NT == 2, "one or two query tiles");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* p_smem = q_smem + Q_BYTES;                // P of (tile t, buffer b) at (PB t + b) ROW_BLOCK
    uint8_t* kv_smem = p_smem + NT * PB * ROW_BLOCK;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1 + 6 * NT];
    __shared__ uint32_t tmem_slot;
    __shared__ int page_of[APT_PAGES_KEPT];   // the first pages this block reads, fetched once (-1: none)

    pdl_launch_dependents();
    pdl_wait();
    const int g = blockIdx.x, sq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = H / G;
    const int tokens_per_block = NT * APT_ROWS / group;   // rows past tokens_per_block * group are padding
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    const int n_blocks_q = (n_new + tokens_per_block - 1) / tokens_per_block;
    // The last query rows see the most keys: they go first, for all kv heads (x runs fastest),
    // so that the blocks start in the order of their work.
    const int q_block = n_blocks_q - 1 - (int)blockIdx.y;
    if (slot < 0 || q_block < 0) return;                  // the whole block, before anything is set up
    const int start = seq_start[sq];
    const int tok0 = q_block * tokens_per_block;
    const int tok_end = min(n_new, tok0 + tokens_per_block);
    const int* pages = page_table + (size_t)slot * max_pages;
    // Pages this block reads: from the first position its first token sees to its last token's own.
    const int first_pos = window > 0 && start + tok0 + 1 > window ? start + tok0 + 1 - window : 0;
    const int t_begin = first_pos / BC_PAGE, t_end = (start + tok_end - 1) / BC_PAGE + 1;
    const int n_tiles = t_end - t_begin;
    const int last_pos = start + n_new - 1;               // the last position the sequence holds after this step

    const uint32_t kv_full0 = smem_u32(&bars[0]), kv_empty0 = smem_u32(&bars[STAGES]), q_full = smem_u32(&bars[2 * STAGES]);
    // Per query tile t and buffer b: scores ready, P written, product done.
    auto s_full = [&](int t, int b) { return smem_u32(&bars[2 * STAGES + 1 + 6 * t + b]); };
    auto p_full = [&](int t, int b) { return smem_u32(&bars[2 * STAGES + 1 + 6 * t + 2 + b]); };
    auto o_done = [&](int t, int b) { return smem_u32(&bars[2 * STAGES + 1 + 6 * t + 4 + b]); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(kv_full0 + 8 * s, 1);
            mbar_init(kv_empty0 + 8 * s, 1);
        }
        mbar_init(q_full, 1);
        for (int t = 0; t < NT; t++)
            for (int b = 0; b < 2; b++) {
                mbar_init(s_full(t, b), 1);
                mbar_init(p_full(t, b), 128);
                // The products of even pages arrive on the first, of odd pages on the second: a
                // waiter is then never more than one phase behind either of them.
                mbar_init(o_done(t, b), 1);
            }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    for (int i = threadIdx.x; i < min(n_tiles, APT_PAGES_KEPT); i += THREADS) {
        const int tile = t_begin + i;
        const int page = tile < max_pages ? pages[tile] : -1;
        page_of[i] = page >= 0 && page < n_pages ? page : -1;
    }
    auto page_at = [&](int j) {   // the page of this block's j-th tile, or -1
        if (j < APT_PAGES_KEPT) return page_of[j];
        const int tile = t_begin + j;
        const int page = tile < max_pages ? pages[tile] : -1;
        return page >= 0 && page < n_pages ? page : -1;
    };
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // Q: one box [tokens][heads of the group][64 elements] per 64 elements of the head size.
            mbar_expect_tx(q_full, (uint32_t)(DB * tokens_per_block * group * 128));
            for (int b = 0; b < DB; b++) tma_load_3d(smem_u32(q_smem + b * NT * ROW_BLOCK), &map_q, q_full, b * 64, g * group, row0 + tok0);
            for (int j = 0; j < n_tiles; j++) {
                const int s = j % STAGES;
                if (j >= STAGES && !mbar_wait(kv_empty0 + 8 * s, ((j / STAGES) & 1) ^ 1, 1)) break;
                const int page = page_at(j);
                if (page < 0) {
                    // No page: nothing is fetched (what another sequence left in some page never
                    // meets these rows); the stage's phase ends at once, the scores of whatever the
                    // stage still holds are masked, and its values are cleared before they are used.
                    mbar_arrive(kv_full0 + 8 * s);
                    continue;
                }
                const int y = (page * G + g) * BC_PAGE;
                const uint32_t dst = smem_u32(kv_smem + (size_t)s * STAGE_BYTES);
                mbar_expect_tx(kv_full0 + 8 * s, STAGE_BYTES);
                for (int b = 0; b < DB; b++) {
                    tma_load_2d(dst + b * KV_BLOCK, &map_k, kv_full0 + 8 * s, b * 64, y);
                    tma_load_2d(dst + (DB + b) * KV_BLOCK, &map_v, kv_full0 + 8 * s, b * 64, y);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc_b(BC_PAGE, false);   // S: N = 64 positions, keys k-major
            constexpr uint32_t idesc_o = instr_desc_b(D, true);          // O: N = head size, values n-major
            // The operand descriptors are worked out once; an address further on is the descriptor
            // plus that many 16-byte units, so that a product costs its issuing thread an addition
            // or two (this one thread issues every product of the block: what it spends between
            // two of them, the tensor core waits).
            const uint64_t q_desc0 = smem_desc(smem_u32(q_smem));
            const uint64_t k_desc0 = smem_desc(smem_u32(kv_smem));
            const uint64_t v_desc0 = smem_desc_mn(smem_u32(kv_smem) + DB * KV_BLOCK, KV_BLOCK);
            auto scores = [&](int j) {   // S[t][j & 1] = Q_t K(j)^T for every query tile t
                const uint64_t k_desc = k_desc0 + (uint64_t)((j % STAGES) * (STAGE_BYTES >> 4));
#pragma unroll
                for (int t = 0; t < NT; t++) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++)
                        mma_bf16(tmem + (2 * t + (j & 1)) * BC_PAGE, q_desc0 + (uint64_t)((((kk >> 2) * NT + t) * ROW_BLOCK >> 4) + 2 * (kk & 3)),
                                 k_desc + (uint64_t)(((kk >> 2) * KV_BLOCK >> 4) + 2 * (kk & 3)), idesc_s, kk != 0);
                    mma_commit(s_full(t, j & 1));
                }
            };
            bool ok = mbar_wait(q_full, 0, 2);
            for (int j = 0; j < 2 && j < n_tiles && ok; j++) {
                ok = mbar_wait(kv_full0 + 8 * (j % STAGES), 0, 3);
                if (!ok) break;
                tc_fence_after();
                scores(j);
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                const uint64_t v_desc = v_desc0 + (uint64_t)((j % STAGES) * (STAGE_BYTES >> 4));   // 16 positions on: 2048 bytes
#pragma unroll
                for (int t = 0; t < NT; t++) {
                    ok = ok && mbar_wait(p_full(t, j & 1), (j >> 1) & 1, 4);
                    if (!ok) break;
                    APT_STAMP(j, 2 * t);
                    tc_fence_after();
#if APT_P_TMEM
                    // P lies over the first 32 columns of the scores it came from: 8 columns a k-step of 16 positions.
#pragma unroll
                    for (int kk = 0; kk < BC_PAGE / 16; kk++)
                        mma_bf16_a_tmem(tmem + O_COL + t * D, tmem + (2 * t + (j & 1)) * BC_PAGE + 8 * kk, v_desc + (uint64_t)(kk * (2048 >> 4)), idesc_o,
                                        (j | kk) != 0);
#else
                    const uint32_t p_addr = smem_u32(p_smem + (PB * t + (j & (PB - 1))) * ROW_BLOCK);
#pragma unroll
                    for (int kk = 0; kk < BC_PAGE / 16; kk++)
                        mma_bf16(tmem + O_COL + t * D, smem_desc(p_addr) + 2 * kk, v_desc + (uint64_t)(kk * (2048 >> 4)), idesc_o, (j | kk) != 0);
#endif
                    mma_commit(o_done(t, j & 1));
                    APT_STAMP(j, 2 * t + 1);
                }
                if (!ok) break;
                mma_commit(kv_empty0 + 8 * (j % STAGES));
                if (j + 2 < n_tiles) {
                    const int s = (j + 2) % STAGES;
                    ok = mbar_wait(kv_full0 + 8 * s, ((j + 2) / STAGES) & 1, 5);
                    if (!ok) break;
                    APT_STAMP(j, 4);
                    tc_fence_after();
                    scores(j + 2);
                    APT_STAMP(j, 5);
                }
            }
        }
    } else {
        // Softmax: warps 2-5 own query tile 0, warps 6-9 tile 1; this thread owns row 32 q + lane
        // of its tile, the TMEM lane of the same number.
        const int q = warp & 3, t = (warp - 2) >> 2;
        const int row = t * APT_ROWS + 32 * q + lane;                    // among the block's rows
        const int tok = tok0 + row / group, head = g * group + row % group;
        const bool live = row / group < tokens_per_block && tok < n_new;
        const int pos = start + tok;
        const int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
        const int warp_first_pos = start + tok0 + (t * APT_ROWS + 32 * q) / group;   // the smallest position a row of this warp has
        const uint32_t lane_base = tmem + ((uint32_t)(32 * q) << 16);
        const uint32_t o_addr = lane_base + O_COL + t * D;
        float m_used = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            if (lane == 0) ok = mbar_wait(s_full(t, j & 1), (j >> 1) & 1, 6);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (warp == 2 && lane == 0) APT_STAMP(j, 8);
            tc_fence_after();
            uint32_t sv[64];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_load16(lane_base + (2 * t + (j & 1)) * BC_PAGE + 16 * c, sv + 16 * c);
            tmem_load_wait();
            if (warp == 2 && lane == 0) APT_STAMP(j, 9);
            const int tile = t_begin + j;
            const bool page_ok = page_at(j) >= 0;
            // A page that ends at or before the position of this warp's first row is seen whole
            // by all of its rows (padding rows are never written): no mask to work out.
            const bool whole = window == 0 && page_ok && tile * BC_PAGE + BC_PAGE - 1 <= warp_first_pos;
            float tmax = -INFINITY;
            if (whole) {
                // Two chains of three-input maxima: 32 instructions, each chain 16 long.
                float ta = -INFINITY, tb = -INFINITY;
#pragma unroll
                for (int c = 0; c < 64; c += 4) {
                    ta = max3(ta, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
                    tb = max3(tb, __uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3]));
                }
                tmax = fmaxf(ta, tb);
            } else {
#pragma unroll
                for (int c = 0; c < 64; c++) {
                    const int kpos = tile * BC_PAGE + c;
                    const bool seen = page_ok && live && kpos >= lo && kpos <= pos;
                    const float v = seen ? __uint_as_float(sv[c]) : -INFINITY;
                    sv[c] = __float_as_uint(v);
                    tmax = fmaxf(tmax, v);
                }
            }
            const float m_true = fmaxf(m_used, tmax * scale_log2);
            const bool raise = m_true > m_used + APT_RAISE;     // also the first finite maximum: -inf + 8 = -inf
            float corr = 1.0f;
            if (raise) {
                corr = m_used == -INFINITY ? 0.0f : exp2f(m_used - m_true);
                m_used = m_true;
                l *= corr;
            }
            if (warp == 2 && lane == 0) APT_STAMP(j, 10);
            if (j >= (APT_P_TMEM ? 2 : PB)) {
                // The P tile written below was last read by the product of page j - PB (with two
                // P tiles: done long ago as a rule, the scores of page j were issued after it).
                // Waiting for every phase in order also keeps the parities apart: a parity tells
                // two phases apart, not more.
                constexpr int BACK = APT_P_TMEM ? 2 : PB;   // in TMEM, P lies over the scores of the page two before: that product is long done
                if (lane == 0) ok = mbar_wait(o_done(t, (j - BACK) & 1), ((j - BACK) >> 1) & 1, 7);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            if (warp == 2 && lane == 0) APT_STAMP(j, 11);
            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                // Rescale this warp's rows of the accumulator, once every product issued so far is in it.
                if (PB != 1) {
                    if (lane == 0) ok = mbar_wait(o_done(t, (j - 1) & 1), ((j - 1) >> 1) & 1, 9);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D; c += 16) {
                    uint32_t ov[16];
                    tmem_load16(o_addr + c, ov);
                    tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 16; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_store16(o_addr + c, ov);
                }
                tmem_store_wait();
            }
            const float base = m_used == -INFINITY ? 0.0f : m_used;
            // Scores scaled and shifted two at a time (fma.rn.f32x2: the same roundings as fmaf),
            // the exponentials' sums kept in four pairs, so that no chain of additions is longer than 8.
            const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2), shift2 = pack_f32x2(-base, -base);
            uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};
#if APT_P_TMEM
            // P goes back into tensor memory, two bf16 a column, over the scores just read (this
            // thread's own lane): the product reads it there as its A operand.
            const uint32_t p_addr = lane_base + (2 * t + (j & 1)) * BC_PAGE;
#pragma unroll
            for (int c16 = 0; c16 < 2; c16++) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    float a, b;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[c16 * 32 + 2 * i]), __uint_as_float(sv[c16 * 32 + 2 * i + 1])), scale2, shift2), a, b);
                    a = fast_exp2(a), b = fast_exp2(b);
                    sums[i & 3] = add_f32x2(sums[i & 3], pack_f32x2(a, b));
                    packed[i] = pack_bf16(a, b);
                }
                tmem_store16(p_addr + 16 * c16, packed);
            }
#else
            uint8_t* p_row = p_smem + (PB * t + (j & (PB - 1))) * ROW_BLOCK + (32 * q + lane) * 128;
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++) {
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float a, b;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[c8 * 8 + 2 * i]), __uint_as_float(sv[c8 * 8 + 2 * i + 1])), scale2, shift2), a, b);
                    a = fast_exp2(a), b = fast_exp2(b);
                    sums[i] = add_f32x2(sums[i], pack_f32x2(a, b));
                    packed[i] = pack_bf16(a, b);
                }
                *reinterpret_cast<uint4*>(p_row + ((c8 ^ (lane & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
#endif
            {
                float s0, s1, s2, s3;
                unpack_f32x2(add_f32x2(sums[0], sums[1]), s0, s1);
                unpack_f32x2(add_f32x2(sums[2], sums[3]), s2, s3);
                l += (s0 + s1) + (s2 + s3);
            }
            // Value rows that hold no position of this sequence: the whole page if there is none,
            // else what lies past the sequence's last position in its last page (a sequence that
            // held the page before may have left not-a-numbers there, and 0 x NaN is NaN in the
            // product).  The first query tile's threads clear them in the copy, before the
            // product of this page is let go.
            const int first_bad = !page_ok ? 0 : min(BC_PAGE, max(0, last_pos - tile * BC_PAGE + 1));
            if (t == 0 && first_bad < BC_PAGE) {
                uint8_t* v_tile = kv_smem + (size_t)(j % STAGES) * STAGE_BYTES + DB * KV_BLOCK;
                for (int c = 32 * q + lane; c < (BC_PAGE - first_bad) * DB * 8; c += 128) {
                    const int vrow = first_bad + c / (DB * 8), within = c % (DB * 8);
                    *reinterpret_cast<uint4*>(v_tile + (within >> 3) * KV_BLOCK + vrow * 128 + (within & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#if APT_P_TMEM
            if (t == 0 && first_bad < BC_PAGE) fence_proxy_async();   // the cleared value rows, for the tensor core's reads
            tmem_store_wait();
#else
            fence_proxy_async();
#endif
            tc_fence_before();
            mbar_arrive(p_full(t, j & 1));
            if (warp == 2 && lane == 0) APT_STAMP(j, 12);
        }
        // The output: the accumulator over this row's sum.
        if (ok) {
            if (lane == 0) ok = mbar_wait(o_done(t, (n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, 8);
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* dst = out + ((size_t)(row0 + tok) * H + head) * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 16) {
                uint32_t ov[16];
                tmem_load16(o_addr + c, ov);
                tmem_load_wait();
                if (live) {
                    uint32_t packed[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) packed[i] = pack_bf16(__uint_as_float(ov[2 * i]) * inv, __uint_as_float(ov[2 * i + 1]) * inv);
                    *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// -------------------------------------------------------------------------------- the host
// The queries as a tensor [rows][heads][D] inside the fused projection (a row is q_stride
// elements long), cut into boxes of [tokens][heads of a group][64].
static int query_map(CUtensorMap* map, const void* q, int q_stride, int total_rows, int H, int D, int group, int tokens_per_tile) {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)total_rows};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)tokens_per_tile};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = bc_encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        bc_set_error("attention_prefill_tc: cuTensorMapEncodeTiled failed (%d) for queries [%d, %d, %d], row stride %d", (int)r, total_rows, H, D,
                     q_stride);
        return BC_ERR_DRIVER;
    }
    return BC_OK;
}

template <int D, int NT>
static int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const int* page_table, const int* seq_rows,
                  const int* seq_slot, const int* seq_start, void* out, int seqs, int max_new, int H, int G, int max_pages, int n_pages,
                  int window, float scale, cudaStream_t s) {
    constexpr int DB = D / 64;
    constexpr int STAGES = APT_STAGES(D, NT), PB = APT_PB(D, NT);
    constexpr int SMEM = DB * NT * APT_ROWS * 128 + NT * PB * APT_ROWS * 128 + STAGES * 2 * DB * BC_PAGE * 128 + 1024;
    static_assert(SMEM <= APT_SMEM_LIMIT, "the ring does not fit");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) {
            bc_set_error("attention_prefill_tc: cannot set shared memory to %d: %s", SMEM, cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    const int tokens_per_block = NT * APT_ROWS / (H / G);
    dim3 grid(G, (max_new + tokens_per_block - 1) / tokens_per_block, seqs);
    cudaError_t e = bc_launch(attention_prefill_tc_kernel<D, NT>, grid, dim3(64 + NT * 128), (size_t)SMEM, s, mq, mk, mv, page_table, seq_rows,
                              seq_slot, seq_start, (bf16*)out, H, G, max_pages, n_pages, window, scale * 1.4426950408889634f);
    if (e != cudaSuccess) {
        bc_set_error("attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    BC_LAUNCH_STATUS();
}

// Query tiles a block: 0 lets the launcher choose, 1 or 2 force it (measurements and tests).
static int g_apt_tiles = 0;
extern "C" void bc_attention_prefill_tc_set_tiles(int n) { g_apt_tiles = n == 1 || n == 2 ? n : 0; }

static int g_apt_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = bc_sm_count();
    }
    return sms;
}

// Whether this kernel takes the sizes (else the caller uses the mma.sync kernel or the
// one-warp-a-row kernel): head size 64 or 128, at most 128 heads a kv head.
extern "C" int bc_attention_prefill_tc_accepts(int H, int G, int D) {
    return G > 0 && H % G == 0 && H / G <= APT_ROWS && (D == 64 || D == 128) && bc_encode_tiled_fn() != nullptr;
}

// The interface of bc_attention_prefill_bf16, plus total_rows: how many rows q has in all
// (TMA reads past them as zeros).  q and the caches 16-byte aligned, q_stride a multiple of 8.
extern "C" int bc_attention_prefill_tc_bf16(const void* q, int q_stride, int total_rows, const void* k_cache, const void* v_cache,
                                            const int* page_table, const int* seq_rows, const int* seq_slot, const int* seq_start, void* out,
                                            int seqs, int max_new, int H, int G, int D, int max_pages, int n_pages, int window, float scale,
                                            cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 65535 && max_new >= 0 && total_rows >= 0, "attention_prefill_tc: bad sizes seqs=%d max_new=%d rows=%d", seqs,
                 max_new, total_rows);
    BC_CHECK_ARG(bc_attention_prefill_tc_accepts(H, G, D), "attention_prefill_tc: H=%d G=%d D=%d is outside what this kernel takes "
                 "(at most %d heads a kv head, head size 64 or 128)", H, G, D, APT_ROWS);
    BC_CHECK_ARG(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0,
                 "attention_prefill_tc: q, out and the caches must be 16-byte aligned, the row stride a multiple of 8");
    BC_CHECK_ARG(n_pages > 0 && max_new / (APT_ROWS / (H / G)) < 65535, "attention_prefill_tc: bad pages %d or too many new rows %d", n_pages, max_new);
    if (seqs == 0 || max_new == 0 || total_rows == 0) return BC_OK;
    CUtensorMap mq, mk, mv;
    const int group = H / G;
    // Two query tiles a block when that still gives every SM a block (about: the host knows the
    // longest sequence's rows, not every one's); else one tile, twice as many blocks.
    const int per_two = 2 * APT_ROWS / group;
    const long long blocks_of_two = (long long)seqs * ((max_new + per_two - 1) / per_two) * G;
    const int nt = g_apt_tiles ? g_apt_tiles : (blocks_of_two >= g_apt_sms() ? 2 : 1);
    int st = query_map(&mq, q, q_stride, total_rows, H, D, group, nt * APT_ROWS / group);
    if (st != BC_OK) return st;
    const long long cache_rows = (long long)n_pages * G * BC_PAGE;
    if ((st = bc_cached_cache_map(&mk, k_cache, cache_rows, D, "attention_prefill_tc")) != BC_OK) return st;
    if ((st = bc_cached_cache_map(&mv, v_cache, cache_rows, D, "attention_prefill_tc")) != BC_OK) return st;
#define APT_GO(DD, NN) return launch<DD, NN>(mq, mk, mv, page_table, seq_rows, seq_slot, seq_start, out, seqs, max_new, H, G, max_pages, n_pages, window, scale, s)
    if (D == 64 && nt == 1) APT_GO(64, 1);
    if (D == 64) APT_GO(64, 2);
    if (nt == 1) APT_GO(128, 1);
    APT_GO(128, 2);
#undef APT_GO
}

// This unit's status word (0, or where a bounded wait gave up), its wait limit and its word
// of host memory: bc_attention_prefill_tc_status / _set_wait_cycles / _bind_host_word.
TC_STATUS_EXPORTS(attention_prefill_tc)
