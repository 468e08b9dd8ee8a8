// Decode attention for bf16: one new row a sequence against its paged cache, the cached
// positions split across blocks, the query heads of one kv head sharing every key and value
// read.
//
// What is computed is the reference's attention (crates/bc-infer/src/model.rs:448-481;
// online softmax as crates/bc-infer/src/gpu/kernels.h:271-324).  How: a block takes
// (row, kv head, split).  The heads that share the kv head (H / G of them, at most 16)
// are the 16 rows of an m16n8k16 tensor-core tile, so a 64-position page of keys is read
// once for all of them.  Pages stream through a ring of three stages of shared memory: for head
// sizes 64 and 128 as TMA boxes (cp.async.bulk.tensor out of the cache seen as a matrix, one
// thread asking, an mbarrier a stage counting the bytes), else by cp.async;
// each of the four warps takes 16 of a page's 64 positions: S = Q K^T, a running maximum
// and sum in float, P V accumulated in float.  The four warps' partial results are merged
// in a fixed order; with several splits each block leaves (sum, maximum, normaliser) in
// scratch memory and the last block to finish merges the splits, again in a fixed order,
// so the result is the same bits whatever the scheduling.  The launch does not depend on
// the sequence lengths (they are read on the device), so one captured graph serves every
// step of a batch.
#include <cooperative_groups.h>

#include <type_traits>

#include "common.cuh"
#include "mma_tiles.cuh"
#include "tc_ptx.cuh"
#include "tma_host.cuh"

namespace cg = cooperative_groups;

#define AD_THREADS 128            // the threads that compute: four warps, each 16 of a page's 64 positions
#define AD_THREADS_TMA 160        // with pages by TMA a fifth warp asks for them (one thread of it)
#ifndef AD_STAGES
#define AD_STAGES 3
#endif
#define AD_MAX_GROUP 16
#define AD_PAGES_KEPT 256   // page numbers a block keeps in shared memory (it looks up the rest one by one)
#define AD_MAX_CLUSTER 16    // splits that merge through one another's shared memory (more than 8: not portable, asked for per kernel)

// Byte offset of 16-byte chunk c of row r in a page as TMA writes it: blocks of [64 rows][64
// elements] with the 128-byte swizzle (chunk xor row within each 128-byte row).
__device__ __forceinline__ int tma_tile_offset(int r, int c) { return (c >> 3) * 8192 + r * 128 + (((c & 7) ^ (r & 7)) << 4); }

// Clock stamps of the block (0, 0, 0), for measurement builds only (-DBC_AD_TRACE; compiled out
// otherwise): [0..15] the block's life (0 entry, 1 first pages asked for, 2 the kernel before is
// done, 3 query rotated, 4 pages done, 5 warps merged, 6 after the cluster's first barrier, 7
// outputs written, 8 end), then six a page from [16] on (top, page there, next page asked for,
// scores, softmax, product).
#ifdef BC_AD_TRACE
__device__ long long* g_ad_trace = nullptr;
extern "C" int bc_attention_decode_set_trace(long long* buf) { return (int)cudaMemcpyToSymbol(g_ad_trace, &buf, sizeof(buf)); }
#define AD_STAMP(at) do { if (g_ad_trace && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (at) < 400) g_ad_trace[at] = clock64(); } while (0)
#else
#define AD_STAMP(at)
#endif

// The four computing warps among themselves (the fifth warp, where there is one, is not part of it).
__device__ __forceinline__ void ad_workers_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int D, bool TMA>
__global__ void __launch_bounds__(TMA ? AD_THREADS_TMA : AD_THREADS)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ page_table, const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                        bf16* __restrict__ out, float* __restrict__ scratch, int* __restrict__ counters, int H, int G, int max_pages,
                        int n_pages, int window, float scale_log2, const float2* __restrict__ cos_sin, int pairing, int fuse,
                        int k_off, int v_off, bf16* __restrict__ k_write, bf16* __restrict__ v_write, int use_cluster) {
    constexpr int CHUNKS = D / 8;              // 16-byte chunks a row
    constexpr int TILE_BYTES = 64 * D * 2;     // one page of one kv head
    constexpr int KD = D / 16;                 // k-steps of Q K^T
    constexpr int ND = D / 8;                  // 8-wide dimension blocks of the output
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // TMA's swizzle wants 1024-byte alignment
    __shared__ int is_last;
    __shared__ int page_ids[AD_PAGES_KEPT];   // the pages of this block's first tiles (-1: none)
    __shared__ __align__(8) uint64_t full_bars[AD_STAGES], empty_bars[AD_STAGES];
    auto offset = [](int r, int c) { return TMA ? tma_tile_offset(r, c) : tile_offset<D>(r, c); };
    const uint32_t full0 = smem_u32(&full_bars[0]), empty0 = smem_u32(&empty_bars[0]);
    if (TMA && threadIdx.x == 0) {
        for (int s = 0; s < AD_STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);    // the asking thread, with the bytes that are to come
            mbar_init(empty0 + 8 * s, 4);   // one thread of each computing warp: done with the stage
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    // Slots, positions and page tables are in place before the step starts, and the pages read
    // here were written by earlier steps: the first pages are asked for before the wait for
    // the preceding kernel (which makes this row's q, k and v).  Nothing is written before it.
    AD_STAMP(0);
    pdl_launch_dependents();
    const int split = blockIdx.x, n_splits = gridDim.x, g = blockIdx.y, r = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int group = H / G;
    const int slot = row_slot[r];
    const int pos = row_pos[r];   // asked for together with the slot: one trip to global memory instead of two in a row
    if (slot < 0) {
        pdl_wait();
        if (split == 0)
            for (int i = threadIdx.x; i < group * D; i += AD_THREADS) out[((size_t)r * H + (size_t)g * group) * D + i] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    const int first_tile = lo / BC_PAGE, end_tile = pos / BC_PAGE + 1;
    const int per_split = (end_tile - first_tile + n_splits - 1) / n_splits;
    const int t_begin = first_tile + split * per_split;
    const int t_end = min(end_tile, t_begin + per_split);
    const int n_tiles = max(0, t_end - t_begin);
    const int* pages = page_table + (size_t)slot * max_pages;

    // A tile without a page (behind a window, or past what the sequence holds) is neither
    // fetched nor multiplied: what another sequence left in some page never meets this row.
    // The block's page numbers are fetched once, all at a time, not one by one inside the page
    // loop, where each would cost a trip to global memory.
    for (int i = threadIdx.x; i < min(n_tiles, AD_PAGES_KEPT); i += blockDim.x) {
        const int tile = t_begin + i;
        const int page = tile < max_pages ? pages[tile] : -1;
        page_ids[i] = page >= 0 && page < n_pages ? page : -1;
    }
    __syncthreads();   // the page numbers, and the barriers set up above (every thread of the block, the asking warp too)
    auto page_of = [&](int tile) {   // of one of this block's tiles
        const int i = tile - t_begin;
        if (i < AD_PAGES_KEPT) return page_ids[i];
        const int page = tile < max_pages ? pages[tile] : -1;
        return page >= 0 && page < n_pages ? page : -1;
    };
    auto load_tile = [&](int tile, int stage) {
        const int page = page_of(tile);
        const uint32_t kb = ad_smem(smem + (size_t)stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        if (TMA) {   // called by the asking thread alone
            if (page < 0) {
                mbar_arrive(full0 + 8 * stage);   // nothing comes: the stage's phase ends at once
                return;
            }
            const int y = (page * G + g) * BC_PAGE;
            mbar_expect_tx(full0 + 8 * stage, 2 * TILE_BYTES);
#pragma unroll
            for (int b = 0; b < D / 64; b++) {
                tma_load_2d(kb + b * 8192, &map_k, full0 + 8 * stage, b * 64, y);
                tma_load_2d(vb + b * 8192, &map_v, full0 + 8 * stage, b * 64, y);
            }
            return;
        }
        if (page < 0) return;
        const bf16* ks = k_cache + ((size_t)page * G + g) * BC_PAGE * D;
        const bf16* vs = v_cache + ((size_t)page * G + g) * BC_PAGE * D;
        for (int i = threadIdx.x; i < 64 * CHUNKS; i += AD_THREADS) {
            const int row = i / CHUNKS, c = i - row * CHUNKS;
            cp_async16(kb + tile_offset<D>(row, c), ks + (size_t)row * D + c * 8);
            cp_async16(vb + tile_offset<D>(row, c), vs + (size_t)row * D + c * 8);
        }
    };

    // The first pages are asked for at once, before the wait and before the query is fetched
    // and rotated.  The row's own page (the last one of the last split) gets the row's key and
    // value in this step.  Where this block writes them itself (fuse 2) the page is fetched
    // early like the others, with whatever the row's place holds, and the row is then put into
    // the copy in shared memory by hand; where a kernel before this one wrote them, the page
    // is fetched after the wait for that kernel.
    const bool appends = fuse == 2 && n_tiles > 0 && t_end == end_tile;
    if (TMA && warp == 4) {
        // The asking warp: one thread of it asks for page after page, as far ahead as the ring has
        // stages, each as soon as the four computing warps have let go of the stage.  (Asked for
        // by a computing thread, a page costs that thread's warp some 450 clocks of the 1,750
        // that a page takes, and the other warps wait for it at the block's barrier: measured.)
        if (lane == 0) {
            for (int it = 0; it < n_tiles; it++) {
                const int stage = it % AD_STAGES;
                if (it >= AD_STAGES && !mbar_wait(empty0 + 8 * stage, ((it / AD_STAGES) & 1) ^ 1, 2)) break;
                if (fuse != 2 && t_begin + it == end_tile - 1) pdl_wait();   // the row's own page: written by the kernel before this one
                load_tile(t_begin + it, stage);
            }
        }
        __syncwarp();
        // It takes no part in the merges, but in the cluster's barriers it must (they count every thread).
        if (n_splits > 1 && use_cluster) {
            cg::cluster_group cl = cg::this_cluster();
            cl.sync();
            cl.sync();
        }
        return;
    }
    int asked = 0;   // by cp.async: stages of the first ring asked for so far, in order
    if (!TMA)
        for (; asked < AD_STAGES - 1; asked++) {
            if (fuse != 2 && t_begin + asked == end_tile - 1) break;
            if (asked < n_tiles) load_tile(t_begin + asked, asked);
            cp_async_commit();
        }
    AD_STAMP(1);
    pdl_wait();
    AD_STAMP(2);

    // Q fragments: row i of the tile is head g * group + i (zero past the group).
    uint32_t qf[KD][4];
    {
        const bf16* qr = q + (size_t)r * q_stride + (size_t)g * group * D;
#pragma unroll
        for (int kd = 0; kd < KD; kd++) {
            const int d0 = kd * 16 + 2 * tq;
            qf[kd][0] = gq < group ? *reinterpret_cast<const uint32_t*>(qr + (size_t)gq * D + d0) : 0u;
            qf[kd][1] = gq + 8 < group ? *reinterpret_cast<const uint32_t*>(qr + (size_t)(gq + 8) * D + d0) : 0u;
            qf[kd][2] = gq < group ? *reinterpret_cast<const uint32_t*>(qr + (size_t)gq * D + d0 + 8) : 0u;
            qf[kd][3] = gq + 8 < group ? *reinterpret_cast<const uint32_t*>(qr + (size_t)(gq + 8) * D + d0 + 8) : 0u;
        }
    }

    // Fused mode (fuse > 0): q arrives unrotated inside the fused projection
    // [q heads | k heads | v heads]; it is rotated here, in registers, by the row's position.
    // A thread's register (kd, hi) holds dimensions base, base + 1 with base = 16 kd + 8 hi +
    // 2 tq, and the partner of dimension d (d + D/2, or d + 1) sits in the same thread, so no
    // data moves between threads.  Same formulas and roundings as rope_append_kernel.
    if (fuse > 0 && cos_sin != nullptr) {
        const float2* cs = cos_sin + (size_t)pos * (D / 2);
        if (pairing == 1) {
#pragma unroll
            for (int kd = 0; kd < KD; kd++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int base = kd * 16 + 8 * (j >> 1) + 2 * tq;
                    const float2 c = cs[base / 2];
                    const __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&qf[kd][j]);
                    const float x0 = __low2float(x), x1 = __high2float(x);
                    qf[kd][j] = pack_bf16(__fsub_rn(__fmul_rn(x0, c.x), __fmul_rn(x1, c.y)), __fadd_rn(__fmul_rn(x0, c.y), __fmul_rn(x1, c.x)));
                }
        } else {
#pragma unroll
            for (int u = 0; u < D / 16; u++)      // units of 8 dimensions in the first half of the head
#pragma unroll
                for (int rs = 0; rs < 2; rs++) {
                    const int u2 = u + D / 16;
                    const int base = u * 8 + 2 * tq;
                    const float4 c = *reinterpret_cast<const float4*>(cs + base);   // (cos, sin) of pairs base and base + 1
                    uint32_t& lo_reg = qf[u >> 1][rs + 2 * (u & 1)];
                    uint32_t& hi_reg = qf[u2 >> 1][rs + 2 * (u2 & 1)];
                    const __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&lo_reg), b = *reinterpret_cast<__nv_bfloat162*>(&hi_reg);
                    const float a0 = __low2float(a), a1 = __high2float(a), b0 = __low2float(b), b1 = __high2float(b);
                    lo_reg = pack_bf16(__fsub_rn(__fmul_rn(a0, c.x), __fmul_rn(b0, c.y)), __fsub_rn(__fmul_rn(a1, c.z), __fmul_rn(b1, c.w)));
                    hi_reg = pack_bf16(__fadd_rn(__fmul_rn(a0, c.y), __fmul_rn(b0, c.x)), __fadd_rn(__fmul_rn(a1, c.w), __fmul_rn(b1, c.z)));
                }
        }
    }
    if (!TMA)
        for (; asked < AD_STAGES - 1; asked++) {
            if (asked < n_tiles) load_tile(t_begin + asked, asked);
            cp_async_commit();
        }

    AD_STAMP(3);
    float o[ND][4];
#pragma unroll
    for (int i = 0; i < ND; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // rows gq and gq + 8

    bool waits_ok = true;
    for (int it = 0; it < n_tiles; it++) {
        AD_STAMP(16 + 6 * it);
        if (TMA) {
            // Every thread sees the page arrive for itself; a warp goes on or gives up as one.  A
            // warp that has given up (its wait ran out: recorded) still walks through the pages
            // without working, so that the others find it at the barrier of the last page.
            if (waits_ok) waits_ok = mbar_wait(full0 + 8 * (it % AD_STAGES), (it / AD_STAGES) & 1, 1);
            waits_ok = __all_sync(0xffffffffu, waits_ok);
        } else {
            cp_async_wait<AD_STAGES - 2>();
            ad_workers_sync();
        }
        AD_STAMP(16 + 6 * it + 1);
        if (!TMA) {
            if (it + AD_STAGES - 1 < n_tiles) load_tile(t_begin + it + AD_STAGES - 1, (it + AD_STAGES - 1) % AD_STAGES);
            cp_async_commit();
        }
        AD_STAMP(16 + 6 * it + 2);
        const int tile = t_begin + it;
        const bool page_ok = page_of(tile) >= 0;
        // This warp is done with the stage once the page's products are issued and read (end of the iteration).
        auto let_go = [&]() {
            if (!TMA) return;
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * (it % AD_STAGES));
        };
        if (!page_ok || !waits_ok) {
            if (page_ok && tile == end_tile - 1) ad_workers_sync();   // the barrier of the row's own page, below
            let_go();
            continue;
        }
        const uint32_t kb = ad_smem(smem + (size_t)(it % AD_STAGES) * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        const int key0 = 16 * warp;   // this warp's 16 positions of the page
        if (tile == end_tile - 1) {
            // The row's own page.  What lies past the row's position in it belongs to nobody (a
            // sequence that held the page before may have left anything there, not-a-numbers
            // too, and 0 x NaN is NaN in the product with the values): those value rows are
            // cleared in the copy.  And the block that appends puts the row itself there: its
            // key, rotated with the same four roundings as everywhere, and its value; the same
            // go to the cache for the steps to come.
            uint8_t* kt = smem + (size_t)(it % AD_STAGES) * 2 * TILE_BYTES;
            uint8_t* vt = kt + TILE_BYTES;
            const int pr = pos % BC_PAGE;
            for (int i = threadIdx.x; i < (BC_PAGE - 1 - pr) * CHUNKS; i += AD_THREADS) {
                const int row = pr + 1 + i / CHUNKS, c = i % CHUNKS;
                *reinterpret_cast<uint4*>(vt + offset(row, c)) = make_uint4(0u, 0u, 0u, 0u);
            }
            if (appends) {
                const int page = page_of(tile);
                const bf16* kr = q + (size_t)r * q_stride + k_off + (size_t)g * D;
                const bf16* vr = q + (size_t)r * q_stride + v_off + (size_t)g * D;
                bf16* kd_ = k_write + (((size_t)page * G + g) * BC_PAGE + pr) * D;
                bf16* vd_ = v_write + (((size_t)page * G + g) * BC_PAGE + pr) * D;
                const float2* cs = cos_sin ? cos_sin + (size_t)pos * (D / 2) : nullptr;
                for (int i = threadIdx.x; i < D / 2; i += AD_THREADS) {
                    const int a = pairing ? 2 * i : i, b = pairing ? 2 * i + 1 : i + D / 2;
                    const float x0 = __bfloat162float(kr[a]), x1 = __bfloat162float(kr[b]);
                    float y0 = x0, y1 = x1;
                    if (cs) {
                        const float2 c = cs[i];
                        y0 = __fsub_rn(__fmul_rn(x0, c.x), __fmul_rn(x1, c.y));
                        y1 = __fadd_rn(__fmul_rn(x0, c.y), __fmul_rn(x1, c.x));
                    }
                    const bf16 ka = __float2bfloat16_rn(y0), kb_ = __float2bfloat16_rn(y1);
                    kd_[a] = ka;
                    kd_[b] = kb_;
                    *reinterpret_cast<bf16*>(kt + offset(pr, a >> 3) + (a & 7) * 2) = ka;
                    *reinterpret_cast<bf16*>(kt + offset(pr, b >> 3) + (b & 7) * 2) = kb_;
                }
                for (int d = threadIdx.x; d < D; d += AD_THREADS) {
                    const bf16 val = vr[d];
                    vd_[d] = val;
                    *reinterpret_cast<bf16*>(vt + offset(pr, d >> 3) + (d & 7) * 2) = val;
                }
            }
            ad_workers_sync();
        }

        float s[2][4] = {};
#pragma unroll
        for (int kd = 0; kd < KD; kd++) {
            uint32_t b0, b1, b2, b3;
            const int j = lane >> 3, rr = lane & 7;
            ldmatrix_x4(kb + offset(key0 + (j >> 1) * 8 + rr, kd * 2 + (j & 1)), b0, b1, b2, b3);
            mma_16816(s[0], qf[kd], b0, b1);
            mma_16816(s[1], qf[kd], b2, b3);
        }
        AD_STAMP(16 + 6 * it + 3);
        // Scores in the log2 domain; positions outside [lo, pos] do not exist for this row.
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int t = tile * BC_PAGE + key0 + nb * 8 + 2 * tq + (e & 1);
                const bool seen = page_ok && t >= lo && t <= pos;
                s[nb][e] = seen ? s[nb][e] * scale_log2 : -INFINITY;
                if (e < 2) tmax0 = fmaxf(tmax0, s[nb][e]);
                else tmax1 = fmaxf(tmax1, s[nb][e]);
            }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        const float mn0 = fmaxf(m0, tmax0), mn1 = fmaxf(m1, tmax1);
        const float c0 = mn0 == -INFINITY ? 1.0f : fast_exp2(m0 - mn0), c1 = mn1 == -INFINITY ? 1.0f : fast_exp2(m1 - mn1);
        const float base0 = mn0 == -INFINITY ? 0.0f : mn0, base1 = mn1 == -INFINITY ? 0.0f : mn1;
        float p[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; nb++) {
            p[nb][0] = fast_exp2(s[nb][0] - base0);
            p[nb][1] = fast_exp2(s[nb][1] - base0);
            p[nb][2] = fast_exp2(s[nb][2] - base1);
            p[nb][3] = fast_exp2(s[nb][3] - base1);
        }
        l0 = l0 * c0 + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
        l1 = l1 * c1 + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
        m0 = mn0;
        m1 = mn1;
        AD_STAMP(16 + 6 * it + 4);
        uint32_t pf[4] = {pack_bf16(p[0][0], p[0][1]), pack_bf16(p[0][2], p[0][3]), pack_bf16(p[1][0], p[1][1]), pack_bf16(p[1][2], p[1][3])};
#pragma unroll
        for (int nd = 0; nd < ND; nd += 2) {
            o[nd][0] *= c0; o[nd][1] *= c0; o[nd][2] *= c1; o[nd][3] *= c1;
            o[nd + 1][0] *= c0; o[nd + 1][1] *= c0; o[nd + 1][2] *= c1; o[nd + 1][3] *= c1;
            uint32_t b0, b1, b2, b3;
            const int j = lane >> 3, rr = lane & 7;
            ldmatrix_x4_trans(vb + offset(key0 + (j & 1) * 8 + rr, nd + (j >> 1)), b0, b1, b2, b3);
            mma_16816(o[nd], pf, b0, b1);
            mma_16816(o[nd + 1], pf, b2, b3);
        }
        let_go();
        AD_STAMP(16 + 6 * it + 5);
    }
    AD_STAMP(4);
    if (!TMA) cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    ad_workers_sync();

    // Merge the four warps (each saw other positions) in the order 0, 1, 2, 3.
    float* wm = reinterpret_cast<float*>(smem);              // [4][16] maxima
    float* wl = wm + 4 * 16;                                 // [4][16] sums
    float* wo = wl + 4 * 16;                                 // [4][16][D] weighted values
    float* po = wo + 4 * 16 * D;                             // [16][D] this block's merged sum, for its cluster peers
    float* pm = po + 16 * D;                                 // [16] its maximum
    float* pl = pm + 16;                                     // [16] its normaliser
    if (tq == 0) {
        wm[warp * 16 + gq] = m0;
        wm[warp * 16 + gq + 8] = m1;
        wl[warp * 16 + gq] = l0;
        wl[warp * 16 + gq + 8] = l1;
    }
    // Only the rows that are heads of the group are read below (4 of the tile's 16 with four heads a kv head): the others are not written.
#pragma unroll
    for (int nd = 0; nd < ND; nd++) {
        float* base = wo + (size_t)warp * 16 * D + nd * 8 + 2 * tq;
        if (gq < group) *reinterpret_cast<float2*>(base + (size_t)gq * D) = make_float2(o[nd][0], o[nd][1]);
        if (gq + 8 < group) *reinterpret_cast<float2*>(base + (size_t)(gq + 8) * D) = make_float2(o[nd][2], o[nd][3]);
    }
    ad_workers_sync();
    // scratch: [row][head][split][D + 2]: the un-normalised sum, then maximum and normaliser.
    const int stride = D + 2;
    for (int i = threadIdx.x; i < group * D; i += AD_THREADS) {
        const int hr = i / D, d = i - hr * D;
        float M = -INFINITY;
        for (int w = 0; w < 4; w++) M = fmaxf(M, wm[w * 16 + hr]);
        float L = 0.0f, O = 0.0f;
        for (int w = 0; w < 4; w++) {
            const float mw = wm[w * 16 + hr];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - M);
            L += wl[w * 16 + hr] * f;
            O += wo[((size_t)w * 16 + hr) * D + d] * f;
        }
        const int h = g * group + hr;
        if (n_splits == 1) {
            out[((size_t)r * H + h) * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
        } else if (use_cluster) {
            po[i] = O;
            if (d == 0) {
                pm[hr] = M;
                pl[hr] = L;
            }
        } else {
            float* dst = scratch + (((size_t)r * H + h) * n_splits + split) * stride;
            __stcg(dst + d, O);
            if (d == 0) {
                __stcg(dst + D, M);
                __stcg(dst + D + 1, L);
            }
        }
    }
    AD_STAMP(5);
    if (n_splits == 1) return;
    // With a cluster, up to eight neighbouring splits merge among themselves first; what is
    // left to merge through scratch memory are the clusters' results (`parts` of them).
    const int csize = use_cluster ? use_cluster : 1;   // the launcher's cluster size: the splits themselves, or 8, 4 or 2 dividing them
    const int parts = n_splits / csize, part = split / csize;
    if (use_cluster) {
        // The splits of this (row, kv head), or eight neighbours among them, are one thread-block
        // cluster: each block reads its peers' results out of their shared memory and finishes a
        // share of the outputs, adding the splits in order.  No scratch memory, no counters, no
        // round trip through the L2 (unless there are more splits than a cluster holds: then
        // the cluster's sum goes to scratch memory as one part).
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();
        AD_STAMP(6);
        const int crank = split - part * csize;
        const int total = group * D, share = (total + csize - 1) / csize;
        // All reads of the peers' shared memory (a good tenth of a microsecond each) are asked
        // for before any is used; the splits are added in their order as ever.
        auto merge = [&](auto cap) {
            constexpr int CAP = decltype(cap)::value;   // peers the unrolled loops are written for
            // (A peer's maxima and normalisers lie behind its sums, as here: one address a peer.)
            const float* ppo[CAP];
#pragma unroll
            for (int sp = 0; sp < CAP; sp++) ppo[sp] = cl.map_shared_rank(po, sp < csize ? sp : 0);
            for (int i = crank * share + threadIdx.x; i < min(total, (crank + 1) * share); i += AD_THREADS) {
                const int hr = i / D, d = i - hr * D;
                float ms[CAP], ls[CAP], os[CAP];
#pragma unroll
                for (int sp = 0; sp < CAP; sp++) {
                    const bool has = sp < csize;
                    ms[sp] = has ? ppo[sp][16 * D + hr] : -INFINITY;
                    ls[sp] = has ? ppo[sp][16 * D + 16 + hr] : 0.0f;
                    os[sp] = has ? ppo[sp][i] : 0.0f;
                }
                float M = -INFINITY;
#pragma unroll
                for (int sp = 0; sp < CAP; sp++) M = fmaxf(M, ms[sp]);
                float L = 0.0f, O = 0.0f;
#pragma unroll
                for (int sp = 0; sp < CAP; sp++) {
                    const float f = ms[sp] == -INFINITY ? 0.0f : exp2f(ms[sp] - M);
                    L += ls[sp] * f;
                    O += os[sp] * f;
                }
                if (parts == 1) {
                    out[((size_t)r * H + g * group + hr) * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
                } else {
                    float* dst = scratch + (((size_t)r * H + g * group + hr) * parts + part) * stride;
                    __stcg(dst + d, O);
                    if (d == 0) {
                        __stcg(dst + D, M);
                        __stcg(dst + D + 1, L);
                    }
                }
            }
        };
        if (csize > 8) merge(std::integral_constant<int, AD_MAX_CLUSTER>());
        else merge(std::integral_constant<int, 8>());
        AD_STAMP(7);
        cl.sync();   // no block may leave while a peer still reads its shared memory
        AD_STAMP(8);
        if (parts == 1) return;
    }

    // The last block of this (row, kv head) to arrive merges the parts in order (every block
    // arrives, also those of a cluster that wrote a share of its part each).
    __threadfence();
    ad_workers_sync();
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(&counters[r * G + g], 1);
        is_last = arrived == n_splits - 1;
        if (is_last) counters[r * G + g] = 0;   // ready for the next launch
    }
    ad_workers_sync();
    if (!is_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < group * D; i += AD_THREADS) {
        const int hr = i / D, d = i - hr * D;
        const int h = g * group + hr;
        const float* src = scratch + ((size_t)r * H + h) * parts * stride;
        float M = -INFINITY;
        for (int sp = 0; sp < parts; sp++) M = fmaxf(M, __ldcg(src + (size_t)sp * stride + D));
        float L = 0.0f, O = 0.0f;
        for (int sp = 0; sp < parts; sp++) {
            const float ms = __ldcg(src + (size_t)sp * stride + D);
            const float f = ms == -INFINITY ? 0.0f : exp2f(ms - M);
            L += __ldcg(src + (size_t)sp * stride + D + 1) * f;
            O += __ldcg(src + (size_t)sp * stride + d) * f;
        }
        out[((size_t)r * H + h) * D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    }
}

struct FusedRope {
    const float* cos_sin;   // null: no rotation
    int pairing;
    int fuse;               // 0: q is already rotated and the cache already holds the row; 1: rotate q; 2: rotate q and append k, v
    int k_off, v_off;       // where a row's k and v heads start inside the fused projection, in elements
    bool allow_cluster;     // splits may run as a thread-block cluster (else they go through scratch memory)
};

// Whether pages come by TMA where the head size allows (the default) or by cp.async
// everywhere; both give the same bits.  For measurements and tests.
static int g_ad_tma = 1;
extern "C" void bc_attention_decode_set_tma(int on) { g_ad_tma = on != 0; }
// Whether sixteen splits may run as one cluster of sixteen (else as two of eight).  For measurements and tests.
static int g_ad_cluster16 = 1;
extern "C" void bc_attention_decode_set_cluster16(int on) { g_ad_cluster16 = on != 0; }

template <int D, bool TMA>
static int launch_as(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_stride, const void* k_cache, const void* v_cache,
                     const int* page_table, const int* row_pos, const int* row_slot, void* out, float* scratch, int* counters, int rows, int H,
                     int G, int max_pages, int n_pages, int window, float scale, int n_splits, FusedRope fr, cudaStream_t s) {
    constexpr int TILE_BYTES = 64 * D * 2;
    constexpr int MERGE_BYTES = (2 * 4 * 16 + 4 * 16 * D + 16 * D + 32) * 4;
    constexpr int SMEM = (AD_STAGES * 2 * TILE_BYTES > MERGE_BYTES ? AD_STAGES * 2 * TILE_BYTES : MERGE_BYTES) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) {
            bc_set_error("attention_decode: cannot set shared memory to %d: %s", SMEM, cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    dim3 grid(n_splits, G, rows);
    // Up to eight splits (the portable cluster size) exchange their results through
    // distributed shared memory; more go through the caller's scratch memory.
    // More than eight: clusters of eight, four or two where that divides them, whose sums then go through scratch.
    int csize = n_splits <= 8 ? n_splits : n_splits % 8 == 0 ? 8 : n_splits % 4 == 0 ? 4 : n_splits % 2 == 0 ? 2 : 1;
    if (n_splits == 16 && fr.allow_cluster && g_ad_cluster16 && (long long)rows * G * 16 <= bc_sm_count()) {
        // One cluster of sixteen, where every block has an SM to itself (with more blocks than SMs two clusters of
        // eight place better: measured).  Sixteen blocks a cluster is more than every device must offer: asked for
        // once, and taken only if the device can place one.
        static int sixteen = -1;
        if (sixteen < 0) {
            sixteen = 0;
            if (cudaFuncSetAttribute(attention_decode_kernel<D, TMA>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(16, 1, 1);
                cfg.blockDim = dim3(TMA ? AD_THREADS_TMA : AD_THREADS);
                cfg.dynamicSmemBytes = SMEM;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 16;
                attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                int fit = 0;
                if (cudaOccupancyMaxActiveClusters(&fit, attention_decode_kernel<D, TMA>, &cfg) == cudaSuccess && fit > 0) sixteen = 1;
            }
            (void)cudaGetLastError();
        }
        if (sixteen == 1) csize = 16;
    }
    if (n_splits > 8 && csize < n_splits && !(scratch && counters)) csize = 1;
    const bool clustered = n_splits > 1 && fr.allow_cluster && csize > 1;
    if (clustered)
        bc_launch_clustered(attention_decode_kernel<D, TMA>, grid, dim3(TMA ? AD_THREADS_TMA : AD_THREADS), (size_t)SMEM, s, dim3(csize, 1, 1), mk, mv, (const bf16*)q,
                            q_stride, (const bf16*)k_cache, (const bf16*)v_cache, page_table, row_pos, row_slot, (bf16*)out, scratch, counters, H, G,
                            max_pages, n_pages, window, scale * 1.4426950408889634f, (const float2*)fr.cos_sin, fr.pairing, fr.fuse,
                            fr.k_off, fr.v_off, (bf16*)k_cache, (bf16*)v_cache, csize);
    else
        bc_launch(attention_decode_kernel<D, TMA>, grid, dim3(TMA ? AD_THREADS_TMA : AD_THREADS), (size_t)SMEM, s, mk, mv, (const bf16*)q, q_stride, (const bf16*)k_cache,
                  (const bf16*)v_cache, page_table, row_pos, row_slot, (bf16*)out, scratch, counters, H, G, max_pages, n_pages, window,
                  scale * 1.4426950408889634f, (const float2*)fr.cos_sin, fr.pairing, fr.fuse, fr.k_off, fr.v_off, (bf16*)k_cache,
                  (bf16*)v_cache, 0);
    BC_LAUNCH_STATUS();
}

template <int D>
static int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table, const int* row_pos,
                  const int* row_slot, void* out, float* scratch, int* counters, int rows, int H, int G, int max_pages, int n_pages,
                  int window, float scale, int n_splits, FusedRope fr, cudaStream_t s) {
    CUtensorMap mk = {}, mv = {};
    if constexpr (D == 64 || D == 128) {
        // Pages by TMA: the cache as a matrix of [pages * kv heads * 64 positions, D], boxes of 64 x 64.
        if (g_ad_tma && bc_encode_tiled_fn() && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0) {
            const long long cache_rows = (long long)n_pages * G * BC_PAGE;
            int st = bc_cached_cache_map(&mk, k_cache, cache_rows, D, "attention_decode");
            if (st == BC_OK) st = bc_cached_cache_map(&mv, v_cache, cache_rows, D, "attention_decode");
            if (st != BC_OK) return st;
            return launch_as<D, true>(mk, mv, q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, scratch, counters, rows, H, G,
                                      max_pages, n_pages, window, scale, n_splits, fr, s);
        }
    }
    return launch_as<D, false>(mk, mv, q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, scratch, counters, rows, H, G, max_pages,
                               n_pages, window, scale, n_splits, fr, s);
}

// Whether this kernel takes the sizes (else the caller uses the one-warp-a-row kernel).
extern "C" int bc_attention_decode_accepts(int H, int G, int D) {
    return G > 0 && H % G == 0 && H / G <= AD_MAX_GROUP && D % 16 == 0 && D >= 16 && D <= 128;
}

// Floats of scratch and ints of counters for `rows` rows cut into `n_splits`.
extern "C" int bc_attention_decode_workspace(int rows, int H, int G, int D, int n_splits, long long* floats, long long* ints) {
    *floats = n_splits > 1 ? (long long)rows * H * n_splits * (D + 2) : 0;
    *ints = n_splits > 1 ? (long long)rows * G : 0;
    return BC_OK;
}

// The same with rotary encoding and the cache append fused in (the reference does these as
// k_rope and k_copy launches, crates/bc-infer/src/gpu/mod.rs:464-475): `q` is then the
// fused projection [rows, (H + 2 G) D] as the product left it, unrotated; fuse = 1 rotates
// q on the fly, fuse = 2 also writes the row's rotated key and its value to the cache
// before attending; fuse = 0 is the plain kernel.  cos_sin [positions, D/2, 2] float, or
// null for no rotation.  Two to eight splits run as a thread-block cluster and need no
// scratch memory; adding 4 to fuse sends them through scratch memory like larger counts.
extern "C" int bc_attention_decode_fused_bf16(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                              const int* row_pos, const int* row_slot, void* out, float* scratch, int* counters, int rows,
                                              int H, int G, int D, int max_pages, int n_pages, int window, float scale, int n_splits,
                                              const float* cos_sin, int pairing, int fuse, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && rows <= 65535, "attention_decode: %d rows (at most 65535)", rows);
    BC_CHECK_ARG(bc_attention_decode_accepts(H, G, D), "attention_decode: H=%d G=%d D=%d is outside what this kernel takes "
                 "(at most %d heads a kv head, head size a multiple of 16 up to 128)", H, G, D, AD_MAX_GROUP);
    BC_CHECK_ARG(n_splits >= 1 && n_splits <= 65535 && G <= 65535, "attention_decode: bad split count %d", n_splits);
    BC_CHECK_ARG(n_splits == 1 || (n_splits <= 8 && (fuse & 4) == 0) || (scratch && counters), "attention_decode: these splits need scratch memory");
    BC_CHECK_ARG(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0), "attention_decode: q must be 4-byte aligned with an even stride");
    BC_CHECK_ARG(fuse >= 0 && (fuse & 3) <= 2 && fuse < 8 && (pairing == 0 || pairing == 1), "attention_decode: bad fuse %d or pairing %d", fuse, pairing);
    BC_CHECK_ARG((fuse & 3) == 0 || q_stride == (H + 2 * G) * D, "attention_decode: fused mode wants the fused projection, stride %d", (H + 2 * G) * D);
    BC_CHECK_ARG((fuse & 3) == 0 || cos_sin == nullptr || (uintptr_t)cos_sin % 16 == 0, "attention_decode: the rotary table must be 16-byte aligned");
    if (rows == 0) return BC_OK;
    FusedRope fr{cos_sin, pairing, fuse & 3, H * D, (H + G) * D, (fuse & 4) == 0};
#define AD_CASE(DD) \
    case DD: return launch<DD>(q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, scratch, counters, rows, H, G, max_pages, n_pages, window, scale, n_splits, fr, s);
    switch (D) {
        AD_CASE(16) AD_CASE(32) AD_CASE(48) AD_CASE(64) AD_CASE(80) AD_CASE(96) AD_CASE(112) AD_CASE(128)
    }
#undef AD_CASE
    bc_set_error("attention_decode: no kernel for head size %d", D);
    return BC_ERR_ARG;
}

// q: row r's head h at q + r * q_stride + h * D.  scratch / counters: see above; counters
// zero before the first launch (every launch leaves them zero).  Rows must be <= 65535.
extern "C" int bc_attention_decode_bf16(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                        const int* row_pos, const int* row_slot, void* out, float* scratch, int* counters, int rows, int H,
                                        int G, int D, int max_pages, int n_pages, int window, float scale, int n_splits, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && rows <= 65535, "attention_decode: %d rows (at most 65535)", rows);
    BC_CHECK_ARG(bc_attention_decode_accepts(H, G, D), "attention_decode: H=%d G=%d D=%d is outside what this kernel takes "
                 "(at most %d heads a kv head, head size a multiple of 16 up to 128)", H, G, D, AD_MAX_GROUP);
    BC_CHECK_ARG(n_splits >= 1 && n_splits <= 65535 && G <= 65535, "attention_decode: bad split count %d", n_splits);
    BC_CHECK_ARG(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0), "attention_decode: q must be 4-byte aligned with an even stride");
    if (rows == 0) return BC_OK;
    return bc_attention_decode_fused_bf16(q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, scratch, counters, rows, H, G,
                                          D, max_pages, n_pages, window, scale, n_splits, nullptr, 0, 0, s);
}

// ------------------------------------------------- the variant that brings its own scratch
// See attention_decode_static.h for who needs this and what it costs.  The array below is
// part of the library's device image: in host code its name is only a stand-in, so the
// device address is asked for once per device and handed to the kernel like any pointer.
#include <mutex>

#include "attention_decode_static.h"

static __device__ __align__(256) unsigned char g_static_scratch[BC_STATIC_SCRATCH_BYTES];

#define BC_STATIC_MAX_DEVICES 64
static void* g_static_scratch_addr[BC_STATIC_MAX_DEVICES];        // per device, null until looked up
static unsigned g_static_configured[BC_STATIC_MAX_DEVICES];       // per device, bit D / 16: that head size's kernel is set up
static std::mutex g_static_mutex;

template <int D>
static int launch_static(float* scratch, int* counters, const void* q, int q_stride, const void* k_cache, const void* v_cache,
                         const int* page_table, const int* row_pos, const int* row_slot, void* out, int rows, int H, int G, int max_pages,
                         int n_pages, int window, float scale, int n_splits, int device, cudaStream_t s) {
    constexpr int TILE_BYTES = 64 * D * 2;
    constexpr int MERGE_BYTES = (2 * 4 * 16 + 4 * 16 * D + 16 * D + 32) * 4;
    constexpr int SMEM = (AD_STAGES * 2 * TILE_BYTES > MERGE_BYTES ? AD_STAGES * 2 * TILE_BYTES : MERGE_BYTES) + 1024;
    const CUtensorMap none = {};   // this entry point fetches pages by cp.async: it needs no tensor maps
    {
        // First call for this head size on this device: let the kernel use the shared memory it needs.
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!(g_static_configured[device] & (1u << (D / 16)))) {
            cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
            if (e != cudaSuccess) {
                bc_set_error("attention_decode_static: cannot set shared memory to %d: %s", SMEM, cudaGetErrorString(e));
                return (int)e;
            }
            g_static_configured[device] |= 1u << (D / 16);
        }
    }
    bc_launch(attention_decode_kernel<D, false>, dim3(n_splits, G, rows), dim3(AD_THREADS), (size_t)SMEM, s, none, none, (const bf16*)q, q_stride,
              (const bf16*)k_cache, (const bf16*)v_cache, page_table, row_pos, row_slot, (bf16*)out, scratch, counters, H, G, max_pages,
              n_pages, window, scale * 1.4426950408889634f, (const float2*)nullptr, 0, 0, 0, 0, (bf16*)nullptr, (bf16*)nullptr, 0);
    BC_LAUNCH_STATUS();
}

extern "C" int bc_attention_decode_static_bf16(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                               const int* row_pos, const int* row_slot, void* out, int rows, int heads, int kv_heads,
                                               int head_dim, int max_pages, int n_pages, int window, float scale, int n_splits,
                                               cudaStream_t stream) {
    BC_CHECK_ARG(rows >= 0 && rows <= 65535, "attention_decode_static: %d rows (at most 65535)", rows);
    BC_CHECK_ARG(bc_attention_decode_accepts(heads, kv_heads, head_dim), "attention_decode_static: heads=%d kv_heads=%d head_dim=%d is "
                 "outside what the kernel takes (at most %d heads a kv head, head size a multiple of 16 up to 128)", heads, kv_heads,
                 head_dim, AD_MAX_GROUP);
    BC_CHECK_ARG(n_splits >= 1 && n_splits <= 65535 && kv_heads <= 65535, "attention_decode_static: bad split count %d", n_splits);
    BC_CHECK_ARG(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0), "attention_decode_static: q must be 4-byte aligned with an even stride");
    const long long floats = n_splits > 1 ? (long long)rows * heads * n_splits * (head_dim + 2) : 0;
    const long long ints = n_splits > 1 ? (long long)rows * kv_heads : 0;
    if (floats > BC_STATIC_SCRATCH_FLOATS || ints > BC_STATIC_SCRATCH_COUNTERS) {
        bc_set_error("attention_decode_static: rows=%d heads=%d splits=%d head_dim=%d needs %lld floats and %lld counters of scratch; the "
                     "built-in array holds %d and %d.  Use fewer splits or rows, or bc_attention_decode_bf16 with scratch of your own",
                     rows, heads, n_splits, head_dim, floats, ints, BC_STATIC_SCRATCH_FLOATS, BC_STATIC_SCRATCH_COUNTERS);
        return BC_ERR_LIMIT;
    }
    if (rows == 0) return BC_OK;

    // Once per device, with that device current: the array's address on this device.
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= BC_STATIC_MAX_DEVICES) {
        bc_set_error("attention_decode_static: no usable current device (%s)", cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : BC_ERR_ARG;
    }
    void* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_scratch_addr[device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p) {
                bc_set_error("attention_decode_static: cannot find the scratch array on device %d: %s", device, cudaGetErrorString(e));
                return e != cudaSuccess ? (int)e : BC_ERR_DRIVER;
            }
            g_static_scratch_addr[device] = p;
        }
        base = g_static_scratch_addr[device];
    }
    float* scratch = reinterpret_cast<float*>(base);
    int* counters = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + (size_t)BC_STATIC_SCRATCH_FLOATS * 4);
    if (ints > 0) {
        // The array keeps what the last call left; the counters of this launch start at zero.
        e = cudaMemsetAsync(counters, 0, (size_t)ints * sizeof(int), stream);
        if (e != cudaSuccess) {
            bc_set_error("attention_decode_static: clearing the counters failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
#define ADS_CASE(DD) \
    case DD: return launch_static<DD>(scratch, counters, q, q_stride, k_cache, v_cache, page_table, row_pos, row_slot, out, rows, heads, kv_heads, max_pages, n_pages, window, scale, n_splits, device, stream);
    switch (head_dim) {
        ADS_CASE(16) ADS_CASE(32) ADS_CASE(48) ADS_CASE(64) ADS_CASE(80) ADS_CASE(96) ADS_CASE(112) ADS_CASE(128)
    }
#undef ADS_CASE
    bc_set_error("attention_decode_static: no kernel for head size %d", head_dim);
    return BC_ERR_ARG;
}

// This unit's status word (0, or where a bounded wait for a page gave up), its wait limit and its
// word of host memory: bc_attention_decode_status / _set_wait_cycles / _bind_host_word.
TC_STATUS_EXPORTS(attention_decode)
