// bf16 matrix product on the 5th-generation tensor cores: Y[t, n] = sum_k X[t, k] * W[n, k].
//
// The reference multiplies with one warp a weight row on the CUDA cores
// (crates/bc-infer/src/gpu/kernels.h:204-223, launched seven times a layer,
// crates/bc-infer/src/gpu/mod.rs:456-489).  Here the product is laid out for Blackwell:
//
//   - The WEIGHT tile is the MMA's M operand: 128 weight rows by 64 k, and the activation
//     tile is the N operand: BN tokens by 64 k (BN = 16 .. 256).  Both matrices are stored
//     k-major already ([out, in] weights, [token, hidden] activations), so neither needs a
//     transpose, and a decode step of a few tokens still fills all 128 rows of the tensor
//     core while it streams the weights once.  The accumulator D[n, t] lives in TMEM:
//     lane = weight row, column = token.
//   - Operands come by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a
//     ring of shared-memory stages guarded by mbarriers; one thread issues tcgen05.mma
//     (kind::f16, bf16 in, float accumulate); tcgen05.commit releases a stage when the
//     MMAs that read it are done.  TMA zero-fills past the edges, so any K that is a
//     multiple of 8 and any N and T work; the epilogue writes only what exists.
//   - Warp roles: warp 0 loads, warp 1 owns TMEM and issues MMAs, warps 2..5 read the
//     accumulator back (tcgen05.ld; a warp may touch lanes 32 (w mod 4) ..) and apply the
//     epilogue: store bf16, store float (scores), add into the float residual stream, or
//     SwiGLU over a weight that stacks gate rows on up rows (two accumulators, one B tile).
//   - With split-K (grid z > 1, for products with few weight tiles and a long K) every
//     split leaves its partial tile in scratch memory and the block that arrives last adds
//     them in the order of the splits, so the sum's order never changes from run to run.
//     Two to eight splits of a product with few tokens skip the scratch memory: they are
//     launched as one thread-block cluster, keep their partial tiles in shared memory, and
//     every block adds up a share of the token columns out of its peers' shared memory,
//     in the same order.
//   - More than 128 tokens (prompts) take the second kernel of this file: persistent, on
//     pairs of SMs (cta_group::2); see there.
//
// Every wait is bounded: after about a second without progress a thread records where it
// gave up in a status word, stops waiting, and the block frees its TMEM and returns.
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include <cooperative_groups.h>

#include "tc_ptx.cuh"

namespace cg = cooperative_groups;

// ---------------------------------------------------------------------------------- kernel
struct TcParams {
    void* out;          // bf16 [T, N] (store, swiglu) or float [T, N] (store_f32, add_f32)
    float* partial;     // split-K: float [tiles, splits, BN, TC_BM] scratch (contents need not be zero)
    int* counters;      // split-K: four a tile, zero before the first launch (a launch leaves them zero)
    int T, N, K;
    int up_row_offset;  // SwiGLU: rows of the up half start here in W
    int stages;
    int k_iters_per_split;
    int clustered;      // split-K: the splits of a tile are one thread-block cluster and add up through shared memory
    int n_tiles, t_tiles;   // blocks along the weight rows and along the tokens
    int pair_tokens;        // the paired kernel: tokens a tile (64, 128, 192 or 256)
    int starve;             // test hook: the first stage expects 16 bytes that never come, so a bounded wait runs out
    long long* trace;       // measurement builds (-DBC_TC_TRACE): sixteen time stamps a block, else null
};

// Time stamps of a block's life, for measurement builds only (compiled out otherwise):
// 0 entry, 1 set up, 2 first ring of weights asked for, 3 the preceding kernel is done, 4 first
// stage full, 5 all MMAs issued, 6 accumulator seen, 7 end, 8 partial tile written, 9 after
// the first cluster barrier, 10 columns finished, 11 after the second cluster barrier.
#ifdef BC_TC_TRACE
__device__ __forceinline__ void tc_stamp(const TcParams& p, int what) {
    if (!p.trace) return;
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[((size_t)blockIdx.x + (size_t)gridDim.x * blockIdx.z) * 16 + what] = t;
}
#define TC_STAMP(what) tc_stamp(p, what)
#else
#define TC_STAMP(what)
#endif

// Blocks that run at the same time should share operands: the block index walks up to
// TC_RASTER token tiles first, then the weight tiles, then the next band of token tiles.
// A wave of 148 blocks then touches about 16 + 9 operand tiles instead of all the weight
// tiles of one or two token tiles, and each is fetched from HBM once, not once a token tile.
#define TC_RASTER 16

// Threads a block: warp 0 asks for tiles, warp 1 issues the products, then the epilogue warps: four, or eight from 64
// tokens a tile on.
__host__ __device__ constexpr int tc_threads(int bn) { return bn >= 64 ? TC_THREADS + 128 : TC_THREADS; }

template <int BN, int EPI, bool STACK>
__global__ void __launch_bounds__(tc_threads(BN), BN == 64 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    constexpr int A_BYTES = TC_BM * TC_BK * 2;
    constexpr int B_BYTES = BN * TC_BK * 2;
    // Two accumulators share one activation tile: gate and up rows for SwiGLU, or, with the
    // widest token tile, two stacked weight tiles (256 output rows a block), which cuts the
    // bytes an SM must fetch per multiply-accumulate by a third.
    constexpr bool TWO_TILES = EPI != EPI_SWIGLU && BN == 256 && STACK;
    constexpr int N_ACC = (EPI == EPI_SWIGLU || TWO_TILES) ? 2 : 1;
    constexpr int OUT_TILES = TWO_TILES ? 2 : 1;
    constexpr int STAGE_BYTES = N_ACC * A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = N_ACC * BN < 32 ? 32 : N_ACC * BN;
    // From 64 tokens a tile on, eight warps share the epilogue: the two warps that may read a
    // quarter of the TMEM lanes (a warp reads lanes 32 (warp % 4) ..) take half of the token
    // columns each.  What the epilogue costs grows with the tile; at few tokens four suffice.
    constexpr int HALVES = (tc_threads(BN) - 64) / 128;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // Tiles need 1024-byte alignment for the 128-byte swizzle.
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * 16 + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int gave_up;   // a wait of this block ran out: nothing is written, the block only tears down

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = p.stages;
    const int band_blocks = TC_RASTER * p.n_tiles;
    const int band = blockIdx.x / band_blocks, in_band = blockIdx.x - band * band_blocks;
    const int band_height = min(TC_RASTER, p.t_tiles - band * TC_RASTER);
    const int tile_n = in_band / band_height, tile_t = band * TC_RASTER + in_band - tile_n * band_height;
    const int n0 = tile_n * (OUT_TILES * TC_BM), t0 = tile_t * BN;
    const int second_row = EPI == EPI_SWIGLU ? p.up_row_offset + n0 : n0 + TC_BM;   // where the second accumulator's weight rows start
    const int total_k_iters = (p.K + TC_BK - 1) / TC_BK;
    const int k_first = blockIdx.z * p.k_iters_per_split;
    const int k_iters = min(p.k_iters_per_split, total_k_iters - k_first);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[16]), acc_bar = smem_u32(&bars[32]);

    if (threadIdx.x == 0) {
        TC_STAMP(0);
        gave_up = 0;
        for (int s = 0; s < stages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            TC_STAMP(1);
            // Weights are written by no kernel, so the first ring of weight tiles is asked
            // for before the wait on the preceding kernel; activations only after it.
            const int ahead = min(stages, k_iters);
            const uint64_t stream_once = l2_evict_first_policy();
            auto load_w = [&](uint32_t dst, uint32_t bar, int k, int row) {
                if (BN <= 64) tma_load_2d_hint(dst, &map_w, bar, k, row, stream_once);   // few tokens: every weight is used once
                else tma_load_2d(dst, &map_w, bar, k, row);                              // many: token tiles share it through the L2
            };
            for (int i = 0; i < ahead; i++) {
                const uint32_t a = smem_u32(smem + (size_t)i * STAGE_BYTES);
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES + (p.starve && i == 0 ? 16 : 0));
                const int k = (k_first + i) * TC_BK;
                load_w(a, full0 + 8 * i, k, n0);
                if (N_ACC == 2) load_w(a + A_BYTES, full0 + 8 * i, k, second_row);
            }
            TC_STAMP(2);
            pdl_wait();
            TC_STAMP(3);
            for (int i = 0; i < ahead; i++) {
                const uint32_t a = smem_u32(smem + (size_t)i * STAGE_BYTES);
                tma_load_2d(a + N_ACC * A_BYTES, &map_x, full0 + 8 * i, (k_first + i) * TC_BK, t0);
            }
            for (int i = ahead; i < k_iters; i++) {
                const int s = i % stages;
                if (!mbar_wait(empty0 + 8 * s, ((i / stages) & 1) ^ 1, 1)) {
                    *reinterpret_cast<volatile int*>(&gave_up) = 1;
                    break;
                }
                const uint32_t a = smem_u32(smem + (size_t)s * STAGE_BYTES);
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                const int k = (k_first + i) * TC_BK;
                load_w(a, full0 + 8 * s, k, n0);
                if (N_ACC == 2) load_w(a + A_BYTES, full0 + 8 * s, k, second_row);
                tma_load_2d(a + N_ACC * A_BYTES, &map_x, full0 + 8 * s, k, t0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            bool ok = true;
            for (int i = 0; i < k_iters && ok; i++) {
                const int s = i % stages;
                ok = mbar_wait(full0 + 8 * s, (i / stages) & 1, 2);
                if (!ok) break;
                if (i == 0) TC_STAMP(4);
                tc_fence_after();
                const uint32_t a = smem_u32(smem + (size_t)s * STAGE_BYTES);
                const uint64_t da = smem_desc(a), db = smem_desc(a + N_ACC * A_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; kk++) {
                    const uint32_t acc = (i | kk) != 0;
                    mma_bf16(tmem, da + 2 * kk, db + 2 * kk, idesc, acc);
                    if (N_ACC == 2) mma_bf16(tmem + BN, smem_desc(a + A_BYTES) + 2 * kk, db + 2 * kk, idesc, acc);
                }
                mma_commit(empty0 + 8 * s);
            }
            if (!ok) {
                *reinterpret_cast<volatile int*>(&gave_up) = 1;
                __threadfence_block();
            }
            TC_STAMP(5);
            mma_commit(acc_bar);   // also after a wait that ran out: the epilogue warps must not be left waiting
        }
    } else {
        // Epilogue: this warp reads TMEM lanes 32 q .. 32 q + 31, i.e. weight rows n0 + 32 q + lane.
        const int q = warp & 3, half = (warp - 2) >> 2;
        const int n_first = n0 + 32 * q + lane;
        const bool split = gridDim.z > 1;
        constexpr int ACC_COLS = N_ACC * BN / HALVES;        // accumulator columns this warp moves out of TMEM
        const int acc_first = half * ACC_COLS;
        const int tile = blockIdx.x;
        // Split-K: every split leaves its partial tile in scratch memory; the four row
        // quarters of a tile each have a counter, and the warp that arrives last adds the
        // splits' partials in the order 0, 1, 2 .., so the sum never depends on timing.
        // Scratch layout [tile][split][column][row]: a warp touches 32 consecutive floats.
        const size_t part_tile = (size_t)N_ACC * TC_BM * BN;   // [accumulator][column][row]
        float* part = split ? p.partial + ((size_t)tile * gridDim.z + blockIdx.z) * part_tile + 32 * q + lane : nullptr;
        int* counter = split ? p.counters + (size_t)tile * 4 + q : nullptr;
        bool ok = true;
        pdl_wait();   // the output, the scratch and the counters may still be in use by the preceding kernel
        if (lane == 0) ok = mbar_wait(acc_bar, 0, 3) && *reinterpret_cast<volatile int*>(&gave_up) == 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (warp == 2 && lane == 0) TC_STAMP(6);
        tc_fence_after();
        const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16);
        bool finish = !split;   // this warp writes the output
        if (split && p.clustered) {
            // The partial tile goes to this block's shared memory (the ring is drained: every
            // load was consumed before the accumulator barrier fired), [column][row].
            if (ok) {
                float* mine = reinterpret_cast<float*>(smem) + 32 * q + lane;
#pragma unroll 1
                for (int c0 = acc_first; c0 < acc_first + ACC_COLS; c0 += 16) {
                    uint32_t v[16];
                    tmem_load16(taddr + c0, v);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) mine[(size_t)(c0 + j) * TC_BM] = __uint_as_float(v[j]);
                }
            }
        } else if (split) {
            if (ok) {
#pragma unroll 1
                for (int c0 = acc_first; c0 < acc_first + ACC_COLS; c0 += 16) {   // the second accumulator follows the first in TMEM and in scratch
                    uint32_t v[16];
                    tmem_load16(taddr + c0, v);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) __stcg(part + (size_t)(c0 + j) * TC_BM, __uint_as_float(v[j]));
                }
            }
            __threadfence();
            __syncwarp();
            int arrived = 0;
            if (lane == 0) arrived = atomicAdd(counter, 1);
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            finish = arrived == HALVES * (int)gridDim.z - 1;   // every warp of the quarter, in every split, has left its columns
            if (finish) {
                __threadfence();
                if (lane == 0) *counter = 0;   // ready for the next launch
            }
        }
        if (finish && ok) {
            const float* all = split ? p.partial + (size_t)tile * gridDim.z * part_tile + 32 * q + lane : nullptr;
            // 16 token columns of one accumulator: apply the epilogue and write.
            // The sixteen results are worked out first, with nothing that branches between them,
            // so that their chains of exponential, reciprocal and rounding run side by side;
            // then they are stored (a loop that tests, computes and stores one column at a time
            // runs the chains one after another: measured 60 ns a column).
            auto emit = [&](const uint32_t* v, const uint32_t* u, int cc) {
                const int acc_i = cc / BN, c0 = cc - acc_i * BN;     // which accumulator (stacked weight tile), which token column
                const int n = n_first + TC_BM * acc_i;
                if (n >= p.N) return;
                float r[16];
#pragma unroll
                for (int j = 0; j < 16; j++) r[j] = EPI == EPI_SWIGLU ? silu_mul(__uint_as_float(v[j]), __uint_as_float(u[j])) : __uint_as_float(v[j]);
                const int t_first = t0 + c0;
                const size_t o = (size_t)t_first * p.N + n;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (t_first + j >= p.T) break;
                    const size_t at = o + (size_t)j * p.N;
                    if (EPI == EPI_STORE || EPI == EPI_SWIGLU) ((bf16*)p.out)[at] = __float2bfloat16_rn(r[j]);
                    if (EPI == EPI_STORE_F32) ((float*)p.out)[at] = r[j];
                    // One thread owns each element, so a fire-and-forget reduction gives the same
                    // sum as a load, add and store, without waiting for the load.
                    if (EPI == EPI_ADD_F32) atomicAdd(&((float*)p.out)[at], r[j]);
                }
            };
            constexpr int TOTAL = OUT_TILES * BN;
            if (!split) {
                constexpr int MINE = TOTAL / HALVES;             // output columns this warp writes
                const int first = half * MINE, end = first + MINE;
                // The accumulator comes out of TMEM 16 columns at a time, the next piece on its way
                // while this one is written, so the round trip to TMEM is paid once, not per piece.
                uint32_t va[16], vb[16], ua[16], ub[16];
                tmem_load16(taddr + first, va);
                if (EPI == EPI_SWIGLU) tmem_load16(taddr + BN + first, ua);
#pragma unroll 1
                for (int cc = first; cc < end; cc += 32) {
                    tmem_load_wait();
                    if (cc + 16 < end) {
                        tmem_load16(taddr + cc + 16, vb);
                        if (EPI == EPI_SWIGLU) tmem_load16(taddr + BN + cc + 16, ub);
                    }
                    emit(va, ua, cc);
                    if (cc + 16 < end) {
                        tmem_load_wait();
                        if (cc + 32 < end) {
                            tmem_load16(taddr + cc + 32, va);
                            if (EPI == EPI_SWIGLU) tmem_load16(taddr + BN + cc + 32, ua);
                        }
                        emit(vb, ub, cc + 16);
                    }
                }
            } else {
#pragma unroll 1
                for (int cc = 0; cc < TOTAL; cc += 16) {
                    uint32_t v[16], u[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = u[j] = 0u;
                    for (int z = 0; z < (int)gridDim.z; z++) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(all + (size_t)z * part_tile + (size_t)(cc + j) * TC_BM));
                            if (EPI == EPI_SWIGLU)   // the up half follows the gate half; the gate is applied to the full sums
                                u[j] = __float_as_uint(__uint_as_float(u[j]) + __ldcg(all + (size_t)z * part_tile + (size_t)(BN + cc + j) * TC_BM));
                        }
                    }
                    emit(v, u, cc);
                }
            }
        }
    }
    if (warp == 2 && lane == 0) TC_STAMP(8);
    if (p.clustered) {
        // Split-K inside a cluster: block z of the cluster finishes the token columns z, z + S,
        // ..: it adds the S partial tiles in the order 0, 1, 2 .. straight out of the blocks'
        // shared memory.  The same sums as through scratch memory, without the round trip.
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();
        if (warp == 2 && lane == 0) TC_STAMP(9);
        if (warp >= 2) {
            const int q = warp & 3, half = (warp - 2) >> 2, row = 32 * q + lane, n = n0 + row;
            const int S = (int)gridDim.z, rank = (int)blockIdx.z;
            const float* base = reinterpret_cast<const float*>(smem) + row;
            auto write = [&](int c, float v, float u) {
                if (n < p.N) {
                    const size_t o = (size_t)(t0 + c) * p.N + n;
                    if (EPI == EPI_STORE) ((bf16*)p.out)[o] = __float2bfloat16_rn(v);
                    if (EPI == EPI_STORE_F32) ((float*)p.out)[o] = v;
                    if (EPI == EPI_ADD_F32) ((float*)p.out)[o] += v;   // one owner an element: no reduction needed (and measured 0.4 % of a step faster than a fire-and-forget one)
                    if (EPI == EPI_SWIGLU) ((bf16*)p.out)[o] = __float2bfloat16_rn(silu_mul(v, u));
                }
            };
            // A read of a peer's shared memory takes up to half a microsecond when all blocks of
            // the cluster read at once, so the reads of several of this block's token columns (32
            // reads a thread) are asked for before any is used, and only then added up, in the order
            // of the splits as ever (a loop that adds each value as it comes waits for every
            // read in turn).
            auto finish = [&](auto splits) {
                constexpr int SS = decltype(splits)::value;
                constexpr int CB = EPI == EPI_SWIGLU ? 16 / SS : 32 / SS;   // columns a batch: 32 reads in flight a thread (64 cost the registers that let two blocks share an SM)
                const float* peer[SS];
#pragma unroll
                for (int z = 0; z < SS; z++) peer[z] = cl.map_shared_rank(base, z);
                const int last = min(BN, p.T - t0);
                for (int c = rank + half * CB * SS; c < last; c += HALVES * CB * SS) {   // batches in turn to the two warps of a quarter
                    float v[CB][SS], u[CB][SS];
#pragma unroll
                    for (int b = 0; b < CB; b++) {
                        const int cb = c + b * SS;
#pragma unroll
                        for (int z = 0; z < SS; z++) {
                            v[b][z] = cb < last ? peer[z][(size_t)cb * TC_BM] : 0.0f;
                            if (EPI == EPI_SWIGLU) u[b][z] = cb < last ? peer[z][(size_t)(BN + cb) * TC_BM] : 0.0f;
                        }
                    }
#pragma unroll
                    for (int b = 0; b < CB; b++) {
                        const int cb = c + b * SS;
                        if (cb >= last) break;
                        float a = 0.0f, ua = 0.0f;
#pragma unroll
                        for (int z = 0; z < SS; z++) {
                            a += v[b][z];
                            if (EPI == EPI_SWIGLU) ua += u[b][z];
                        }
                        write(cb, a, ua);
                    }
                }
            };
            if (S == 8) finish(std::integral_constant<int, 8>());
            else if (S == 4) finish(std::integral_constant<int, 4>());
            else if (S == 2) finish(std::integral_constant<int, 2>());
            else
                for (int c = rank + half * S; c < BN && t0 + c < p.T; c += HALVES * S) {
                    float v = 0.0f, u = 0.0f;
                    for (int z = 0; z < S; z++) {
                        const float* theirs = cl.map_shared_rank(base, z);
                        v += theirs[(size_t)c * TC_BM];
                        if (EPI == EPI_SWIGLU) u += theirs[(size_t)(BN + c) * TC_BM];
                    }
                    write(c, v, u);
                }
        }
        if (warp == 2 && lane == 0) TC_STAMP(10);
        cl.sync();   // no block may leave while a peer still reads its shared memory
        if (warp == 2 && lane == 0) TC_STAMP(11);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) TC_STAMP(7);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ------------------------------------------------------- the product on pairs of SMs
// Many tokens (prompts): a persistent kernel, one pair of blocks on the two SMs of every TPC
// (cta_group::2).  A pair walks over tiles of 256 tokens; each block holds two 128-row weight
// tiles (gate and up rows of its 128 outputs for SwiGLU, else 256 consecutive outputs) and
// HALF of the token tile, and the tensor cores of both SMs read both halves.
//
// What bounds the mainloop is shared-memory bandwidth (128 bytes a clock): every MMA reads
// its A slice (4 KB) and the whole B slice (8 KB, half of it out of the partner's memory)
// while TMA writes the next stages.  Two weight tiles a block share every token slice, and
// a pair's stage is 48 KB a block for 2 x 128 x 256 x 64 multiply-accumulates instead of the
// 64 KB of a block on its own: measured 1.56 against 1.46 PFLOP/s in the mainloop.  (One
// weight tile a block with two accumulator buffers would hide the epilogue, but re-reads B
// twice as often and measured 0.97 PFLOP/s.)
//
// The two accumulators (256 token columns each) fill TMEM, so the epilogue of a tile cannot
// overlap the next tile's MMAs; instead it is short (eight warps) and the loader runs ahead:
// while a tile is written out, the ring already holds the first stages of the next one.
//
// The even block's MMA thread issues for the pair; its commits arrive on the barriers of
// both blocks; every block's loads count their bytes on the even block's barrier; the
// epilogue warps of both blocks hand the accumulators back by arriving on the even block's
// barrier.  No load is multicast.
#define TCP_THREADS 320        // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
#define TCP_STAGES_MAX 8

template <int EPI>
__global__ void __launch_bounds__(TCP_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    constexpr int BN = 256;                               // token columns of an accumulator in TMEM; a pair's tile takes p.pair_tokens <= BN
    constexpr int TILE = TC_BM * TC_BK * 2;               // 16 KB: 128 rows of 64 k
    constexpr int STAGE_BYTES = 3 * TILE;                 // two weight tiles and this block's half of the tokens
    constexpr int TMEM_COLS = 512;                        // two accumulators of 256 token columns
    constexpr int OUT_ROWS = EPI == EPI_SWIGLU ? TC_BM : 2 * TC_BM;   // outputs a block
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * TCP_STAGES_MAX + 2];
    __shared__ uint32_t tmem_slot;

    cg::cluster_group cl = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();              // 0: the block that issues the MMAs
    const int stages = p.stages;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int total_tiles = p.n_tiles * p.t_tiles;
    const int k_iters = (p.K + TC_BK - 1) / TC_BK;
    const int bn = p.pair_tokens;                         // tokens a pair's tile: a multiple of 64 (each block loads a box of 128 and uses bn / 2)
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[TCP_STAGES_MAX]);
    const uint32_t acc_full = smem_u32(&bars[2 * TCP_STAGES_MAX]), acc_empty = smem_u32(&bars[2 * TCP_STAGES_MAX + 1]);

    // Tile number -> (weight tile, token tile), in bands of TC_RASTER token tiles.
    auto place = [&](int tile, int& tile_n, int& tile_t) {
        const int band_blocks = TC_RASTER * p.n_tiles;
        const int band = tile / band_blocks, in_band = tile - band * band_blocks;
        const int band_height = min(TC_RASTER, p.t_tiles - band * TC_RASTER);
        tile_n = in_band / band_height;
        tile_t = band * TC_RASTER + in_band - tile_n * band_height;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 16);                         // the eight epilogue warps of both blocks
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_slot), TMEM_COLS);
    tc_fence_before();
    cl.sync();   // both blocks' barriers and TMEM exist before either signals or writes the other's
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            const uint32_t pair_full0 = map_to_rank(full0, 0);   // the even block's barriers count both blocks' bytes
            // This pair's k-steps over all of its tiles, numbered through: step `it` belongs to
            // the pair's tile number it / k_iters.
            const int my_tiles = (total_tiles - pair + n_pairs - 1) / n_pairs;
            const int total_it = my_tiles * k_iters;
            auto where = [&](int it, int& k, int& n0, int& t_mine) {
                const int seq = it / k_iters;
                int tile_n, tile_t;
                place(pair + seq * n_pairs, tile_n, tile_t);
                k = (it - seq * k_iters) * TC_BK;
                n0 = tile_n * 2 * OUT_ROWS + (int)rank * OUT_ROWS;
                t_mine = tile_t * bn + (int)rank * (bn / 2);
            };
            auto load_w = [&](uint32_t dst, uint32_t bar, int k, int n0) {
                tma_load_2d_pair(dst, &map_w, bar, k, n0);
                tma_load_2d_pair(dst + TILE, &map_w, bar, k, EPI == EPI_SWIGLU ? p.up_row_offset + n0 : n0 + TC_BM);
            };
            // Weights are written by no kernel, activations by the preceding one: the first
            // ring's weight tiles are on their way before the wait for it.
            const int ahead = min(stages, total_it);
            for (int it = 0; it < ahead; it++) {
                int k, n0, t_mine;
                where(it, k, n0, t_mine);
                if (rank == 0) mbar_expect_tx(full0 + 8 * it, 2 * STAGE_BYTES);
                load_w(smem_u32(smem + (size_t)it * STAGE_BYTES), pair_full0 + 8 * it, k, n0);
            }
            pdl_wait();
            for (int it = 0; it < ahead; it++) {
                int k, n0, t_mine;
                where(it, k, n0, t_mine);
                tma_load_2d_pair(smem_u32(smem + (size_t)it * STAGE_BYTES) + 2 * TILE, &map_x, pair_full0 + 8 * it, k, t_mine);
            }
            for (int it = ahead; it < total_it; it++) {
                const int s = it % stages;
                if (!mbar_wait(empty0 + 8 * s, ((it / stages) & 1) ^ 1, 1)) break;
                int k, n0, t_mine;
                where(it, k, n0, t_mine);
                const uint32_t a = smem_u32(smem + (size_t)s * STAGE_BYTES);
                if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                load_w(a, pair_full0 + 8 * s, k, n0);
                tma_load_2d_pair(a + 2 * TILE, &map_x, pair_full0 + 8 * s, k, t_mine);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc_pair(bn);
            bool ok = true;
            int it = 0, n = 0;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, n++) {
                // The epilogue warps of both blocks must have read the previous tile out of TMEM.
                if (!(ok = mbar_wait(acc_empty, (n & 1) ^ 1, 4))) break;
                tc_fence_after();
                for (int i = 0; i < k_iters; i++, it++) {
                    const int s = it % stages;
                    if (!(ok = mbar_wait(full0 + 8 * s, (it / stages) & 1, 2))) break;
                    tc_fence_after();
                    const uint32_t a = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t da = smem_desc(a), du = smem_desc(a + TILE), db = smem_desc(a + 2 * TILE);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; kk++) {
                        const uint32_t acc = (i | kk) != 0;
                        mma_bf16_pair(tmem, da + 2 * kk, db + 2 * kk, idesc, acc);
                        mma_bf16_pair(tmem + BN, du + 2 * kk, db + 2 * kk, idesc, acc);
                    }
                    mma_commit_pair(empty0 + 8 * s, 3);
                }
                if (ok) mma_commit_pair(acc_full, 3);
            }
        }
    } else {
        // Epilogue, in both blocks: warps 2-5 and 6-9 read TMEM lanes 32 q .. 32 q + 31 of their
        // own SM.  The first four take the first weight tile's accumulator, the others the
        // second's; for SwiGLU (gate and up sums of one output lie in the two accumulators) the
        // first four take token columns 0-127 of both, the others 128-255.
        const int q = warp & 3, set = (warp - 2) >> 2;
        const uint32_t pair_acc_empty = map_to_rank(acc_empty, 0);
        bool ok = true;
        pdl_wait();   // the output may still be in use by the preceding kernel
        int n = 0;
        for (int tile = pair; tile < total_tiles; tile += n_pairs, n++) {
            int tile_n, tile_t;
            place(tile, tile_n, tile_t);
            const int t0 = tile_t * bn;
            if (lane == 0) ok = mbar_wait(acc_full, n & 1, 3);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            const int out_n = tile_n * 2 * OUT_ROWS + (int)rank * OUT_ROWS + 32 * q + lane + (EPI == EPI_SWIGLU ? 0 : TC_BM * set);
            const uint32_t lanes = tmem + ((uint32_t)(32 * q) << 16);
            // 16 token columns at a time, the next piece on its way while this one is written.
            // All sixteen results first, then the stores: see the one-block kernel's epilogue.
            auto emit = [&](const uint32_t* v, const uint32_t* u, int c0) {
                if (out_n >= p.N) return;
                float r[16];
#pragma unroll
                for (int j = 0; j < 16; j++) r[j] = EPI == EPI_SWIGLU ? silu_mul(__uint_as_float(v[j]), __uint_as_float(u[j])) : __uint_as_float(v[j]);
                const int t_first = t0 + c0;
                const size_t o = (size_t)t_first * p.N + out_n;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (t_first + j >= p.T) break;
                    const size_t at = o + (size_t)j * p.N;
                    if (EPI == EPI_STORE || EPI == EPI_SWIGLU) ((bf16*)p.out)[at] = __float2bfloat16_rn(r[j]);
                    if (EPI == EPI_STORE_F32) ((float*)p.out)[at] = r[j];
                    // One thread owns each element, so a fire-and-forget reduction gives the same
                    // sum as a load, add and store, without waiting for the load.
                    if (EPI == EPI_ADD_F32) atomicAdd(&((float*)p.out)[at], r[j]);
                }
            };
            const int COLS = EPI == EPI_SWIGLU ? bn / 2 : bn;              // token columns this warp writes (a multiple of 32)
            const int c_first = EPI == EPI_SWIGLU ? set * COLS : 0;
            const uint32_t src = lanes + (EPI == EPI_SWIGLU ? c_first : set * BN);   // SwiGLU: the gate accumulator; up is BN columns on
            uint32_t va[16], vb[16], ua[16], ub[16];
            tmem_load16(src, va);
            if (EPI == EPI_SWIGLU) tmem_load16(src + BN, ua);
#pragma unroll 1
            for (int cc = 0; cc < COLS; cc += 32) {
                tmem_load_wait();
                tmem_load16(src + cc + 16, vb);
                if (EPI == EPI_SWIGLU) tmem_load16(src + BN + cc + 16, ub);
                emit(va, ua, c_first + cc);
                tmem_load_wait();
                if (cc + 32 < COLS) {
                    tmem_load16(src + cc + 32, va);
                    if (EPI == EPI_SWIGLU) tmem_load16(src + BN + cc + 32, ua);
                }
                emit(vb, ub, c_first + cc + 16);
            }
            // This warp has read its share of the accumulators: tell the MMA thread of the even block.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(pair_acc_empty);
        }
    }
    tc_fence_before();
    cl.sync();   // neither block leaves, or frees TMEM, while the pair's MMAs or arrivals may still touch it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, TMEM_COLS);
    }
}

// -------------------------------------------------------------------------------- the host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// A k-major bf16 matrix [rows, K] cut into boxes of box_rows x 64, 128-byte swizzle, zero fill.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) {
        bc_set_error("gemm_tc: the driver gives no cuTensorMapEncodeTiled");
        return BC_ERR_DRIVER;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        bc_set_error("gemm_tc: cuTensorMapEncodeTiled failed (%d) for a [%d, %d] matrix, box %d x %d", (int)r, rows, K, box_rows, TC_BK);
        return BC_ERR_DRIVER;
    }
    return BC_OK;
}

// Weight maps are made once per (pointer, shape) and kept: weights do not move.
struct MapKey {
    const void* p;
    int rows, K, box;
    bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && K == o.K && box == o.box; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const { return std::hash<const void*>()(k.p) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K << 20) ^ (size_t)k.box; }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_weight_maps;
static std::mutex g_weight_maps_mutex;

static int weight_map(CUtensorMap* out, const void* base, int rows, int K) {
    std::lock_guard<std::mutex> lock(g_weight_maps_mutex);
    MapKey key{base, rows, K, TC_BM};
    auto it = g_weight_maps.find(key);
    if (it == g_weight_maps.end()) {
        CUtensorMap m;
        int st = make_map(&m, base, rows, K, TC_BM);
        if (st != BC_OK) return st;
        if (g_weight_maps.size() > 65536) g_weight_maps.clear();
        it = g_weight_maps.emplace(key, m).first;
    }
    *out = it->second;
    return BC_OK;
}

// A tuning knob for measurements: 0 lets the launcher choose the ring depth, n > 0 caps it.
static int g_tc_stage_cap = 0;
extern "C" void bc_gemm_tc_set_stage_cap(int n) { g_tc_stage_cap = n < 0 ? 0 : n; }

// Two to eight splits of a product with few tokens run as a thread-block cluster and add up
// through shared memory; 0 sends them through the scratch memory like every other split.
static int g_tc_cluster = 1;
extern "C" void bc_gemm_tc_set_cluster(int on) { g_tc_cluster = on != 0; }

template <int BN, int EPI, bool STACK>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, TcParams p, int splits, cudaStream_t s) {
    constexpr bool TWO_TILES = EPI != EPI_SWIGLU && BN == 256 && STACK;
    constexpr int N_ACC = (EPI == EPI_SWIGLU || TWO_TILES) ? 2 : 1;
    constexpr int STAGE_BYTES = N_ACC * TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    const int total_k_iters = (p.K + TC_BK - 1) / TC_BK;
    p.k_iters_per_split = (total_k_iters + splits - 1) / splits;
    splits = (total_k_iters + p.k_iters_per_split - 1) / p.k_iters_per_split;
    int stages = (TC_SMEM_LIMIT - 1024) / STAGE_BYTES;
    if (stages > 12) stages = 12;
    // Few tokens (decoding): the product streams weights and the next product's blocks should
    // be able to sit beside this one's on an SM, prefetching their weights while these drain.
    // Half the shared memory still keeps ~100 KB of loads in flight a block; where that would
    // leave fewer than four stages (SwiGLU's double weight tile, unsplit) the block takes the whole SM.
    const int half_stages = (TC_SMEM_LIMIT / 2 - 2048) / STAGE_BYTES;
    if (g_tc_stage_cap == 0 && BN <= 64 && (half_stages >= 4 || (splits > 1 && half_stages >= 3)) && stages > half_stages) stages = half_stages;
    if (g_tc_stage_cap > 0 && stages > g_tc_stage_cap) stages = g_tc_stage_cap;
    if (stages > p.k_iters_per_split) stages = p.k_iters_per_split < 2 ? 2 : p.k_iters_per_split;
    p.stages = stages;
    const int smem = stages * STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, STACK>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_LIMIT);
        if (e != cudaSuccess) {
            bc_set_error("gemm_tc: cannot raise the shared memory limit: %s", cudaGetErrorString(e));
            return (int)e;
        }
        configured = true;
    }
    constexpr int ROWS = TWO_TILES ? 2 * TC_BM : TC_BM;   // output rows a block
    p.n_tiles = (p.N + ROWS - 1) / ROWS;
    p.t_tiles = (p.T + BN - 1) / BN;
    dim3 grid(p.n_tiles * p.t_tiles, 1, splits);
    // The partial tile of a clustered split lies in the drained ring: N_ACC * 128 * BN floats.
    p.clustered = g_tc_cluster && splits > 1 && splits <= 8 && BN <= 64 && N_ACC * TC_BM * BN * 4 <= stages * STAGE_BYTES;
    if (!p.clustered && splits > 1 && !(p.partial && p.counters)) {
        bc_set_error("gemm_tc: this split-K needs a workspace");
        return BC_ERR_ARG;
    }
    cudaError_t e = p.clustered ? bc_launch_clustered(gemm_tc_kernel<BN, EPI, STACK>, grid, dim3(tc_threads(BN)), (size_t)smem, s, dim3(1, 1, splits), mw, mx, p)
                                : bc_launch(gemm_tc_kernel<BN, EPI, STACK>, grid, dim3(tc_threads(BN)), (size_t)smem, s, mw, mx, p);
    if (e != cudaSuccess) {
        bc_set_error("gemm_tc: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    BC_LAUNCH_STATUS();
}

// Whether prompts run on pairs of SMs (the default) or every block on its own; for measurements and tests.
static int g_tc_pair = 1;
static int g_tc_pair_tokens = 0;   // 0: the launcher chooses the tokens a paired tile takes; 64, 128, 192, 256 force it
extern "C" void bc_gemm_tc_set_pair_tokens(int n) { g_tc_pair_tokens = (n == 64 || n == 128 || n == 192 || n == 256) ? n : 0; }
extern "C" void bc_gemm_tc_set_pair(int on) { g_tc_pair = on != 0; }

template <int EPI>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, TcParams p, cudaStream_t s) {
    constexpr int STAGE_BYTES = 3 * TC_BM * TC_BK * 2;
    const int k_iters = (p.K + TC_BK - 1) / TC_BK;
    int stages = (TC_SMEM_LIMIT - 1024) / STAGE_BYTES;
    if (stages > TCP_STAGES_MAX) stages = TCP_STAGES_MAX;
    if (g_tc_stage_cap > 0 && stages > g_tc_stage_cap) stages = g_tc_stage_cap;
    if (stages < 2) stages = 2;
    p.stages = stages;
    p.clustered = 0;
    p.k_iters_per_split = k_iters;
    const int smem = stages * STAGE_BYTES + 1024;
    static bool configured = false;
    static int pairs_on_device = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_LIMIT);
        if (e != cudaSuccess) {
            bc_set_error("gemm_tc: cannot raise the shared memory limit: %s", cudaGetErrorString(e));
            return (int)e;
        }
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        pairs_on_device = sms / 2 > 0 ? sms / 2 : 1;
        configured = true;
    }
    const int rows = EPI == EPI_SWIGLU ? 2 * TC_BM : 4 * TC_BM;   // outputs a pair
    p.n_tiles = (p.N + rows - 1) / rows;
    // Tokens a tile: whole tiles are lost when the tile count is just over a multiple of the
    // pairs (96 tiles on 74 pairs take two rounds).  A narrower tile costs less than its share
    // (per k-step about 640 + 2 x tokens clocks of shared-memory traffic: the weight slices
    // and the TMA writes do not shrink), so it pays only when it saves a round.
    int best = 256;
    if (g_tc_pair_tokens > 0) best = g_tc_pair_tokens;
    else {
        double best_cost = 1e30;
        for (int bn = 256; bn >= 128; bn -= 64) {
            const long long tiles = (long long)p.n_tiles * ((p.T + bn - 1) / bn);
            const double cost = (double)((tiles + pairs_on_device - 1) / pairs_on_device) * (700.0 + 2.0 * bn);
            if (cost < best_cost * 0.97) best_cost = cost, best = bn;
        }
    }
    p.pair_tokens = best;
    p.t_tiles = (p.T + best - 1) / best;
    const long long tiles = (long long)p.n_tiles * p.t_tiles;
    const int pairs = tiles < pairs_on_device ? (int)tiles : pairs_on_device;   // persistent: a pair walks over tiles
    dim3 grid(2 * pairs, 1, 1);
    cudaError_t e = bc_launch_clustered(gemm_tc_pair_kernel<EPI>, grid, dim3(TCP_THREADS), (size_t)smem, s, dim3(2, 1, 1), mw, mx, p);
    if (e != cudaSuccess) {
        bc_set_error("gemm_tc: launch of the paired kernel failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    BC_LAUNCH_STATUS();
}

template <int EPI>
static int launch_bn(int bn, bool stack, const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, int splits, cudaStream_t s) {
    switch (bn) {
        case 16: return launch<16, EPI, false>(mw, mx, p, splits, s);
        case 32: return launch<32, EPI, false>(mw, mx, p, splits, s);
        case 64: return launch<64, EPI, false>(mw, mx, p, splits, s);
        case 128: return launch<128, EPI, false>(mw, mx, p, splits, s);
        case 256: return stack ? launch<256, EPI, true>(mw, mx, p, splits, s) : launch<256, EPI, false>(mw, mx, p, splits, s);
    }
    bc_set_error("gemm_tc: no kernel for a token tile of %d", bn);
    return BC_ERR_ARG;
}

// Token tile for T tokens: the smallest that covers them, up to 256.
extern "C" int bc_gemm_tc_token_tile(int T, int epilogue) {
    (void)epilogue;
    int bn = 16;
    while (bn < T && bn < 256) bn <<= 1;
    return bn;
}

// Output rows one block covers: 128, or 256 when, with the widest token tile, two weight
// tiles are stacked (SwiGLU's two accumulators are gate and up of the same 128 outputs
// instead).  Stacking cuts shared-memory traffic per multiply by a third but halves the
// number of blocks; it is used unless that leaves the last wave of blocks much emptier.
static int g_tc_stack = -1;   // tuning knob for measurements: -1 decide here, 0 never, 1 always
extern "C" void bc_gemm_tc_set_stack(int mode) { g_tc_stack = mode; }
static double wave_fill(long long blocks) {
    const long long sms = bc_sm_count();
    return (double)blocks / (double)(((blocks + sms - 1) / sms) * sms);
}
extern "C" int bc_gemm_tc_rows_per_block(int T, int N, int epilogue) {
    const int bn = bc_gemm_tc_token_tile(T, epilogue);
    if (bn != 256 || epilogue == EPI_SWIGLU || g_tc_stack == 0) return TC_BM;
    if (g_tc_stack == 1) return 2 * TC_BM;
    const long long t_tiles = (T + bn - 1) / bn;
    const long long stacked = (long long)((N + 2 * TC_BM - 1) / (2 * TC_BM)) * t_tiles, single = (long long)((N + TC_BM - 1) / TC_BM) * t_tiles;
    return wave_fill(stacked) >= 0.9 * wave_fill(single) ? 2 * TC_BM : TC_BM;
}

// Floats of workspace and ints of counters a split-K launch needs.  The counters are zero
// before the first launch and every launch leaves them zero; the floats may hold anything.
extern "C" int bc_gemm_tc_workspace(int T, int N, int epilogue, int splits, long long* floats, long long* ints) {
    const int bn = bc_gemm_tc_token_tile(T, epilogue);
    const int rows = bc_gemm_tc_rows_per_block(T, N, epilogue);
    const long long tiles = (long long)((N + rows - 1) / rows) * ((T + bn - 1) / bn);
    *floats = splits > 1 ? tiles * splits * (epilogue == EPI_SWIGLU ? 2 : 1) * rows * bn : 0;
    *ints = splits > 1 ? tiles * 4 : 0;
    return BC_OK;
}

// Test hook: the next launch of the one-block kernel (at most 128 tokens) arms its first
// stage for 16 bytes more than it loads, so that a bounded wait of that launch runs out,
// the blocks tear down, and the status word names the wait.  Nothing faults or hangs; with
// the wait limit set to a millisecond or so the launch returns at once.  The output of such
// a launch is left unwritten.
static int g_tc_starve = 0;
extern "C" void bc_gemm_tc_test_starve_next_launch() { g_tc_starve = 1; }

#ifdef BC_TC_TRACE
// Measurement builds: launch i of the one-block kernel stamps into buf + i * 1024 * 16.
static long long* g_tc_trace = nullptr;
static int g_tc_trace_launches = 0, g_tc_trace_next = 0;
extern "C" void bc_gemm_tc_set_trace(long long* buf, int launches) { g_tc_trace = buf, g_tc_trace_launches = launches, g_tc_trace_next = 0; }
#endif

// X [T, K] bf16, W [N, K] bf16 (SwiGLU: [2N, K], gate rows then up rows); out [T, N] bf16 or
// float by epilogue.  K must be a multiple of 8 (a TMA row stride is a multiple of 16
// bytes); pointers 16-byte aligned.  splits > 1 needs the workspace above.
extern "C" int bc_gemm_tc_bf16(const void* X, const void* W, void* out, int T, int N, int K, int epilogue, int splits, float* partial,
                               int* counters, cudaStream_t s) {
    BC_CHECK_ARG(T >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes T=%d N=%d K=%d", T, N, K);
    BC_CHECK_ARG(K % 8 == 0, "gemm_tc: K=%d is not a multiple of 8 (TMA needs 16-byte row strides); use the CUDA-core product", K);
    BC_CHECK_ARG(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
    BC_CHECK_ARG(epilogue >= 0 && epilogue <= 3, "gemm_tc: unknown epilogue %d", epilogue);
    BC_CHECK_ARG(splits >= 1, "gemm_tc: bad split count %d", splits);
    if (T == 0) return BC_OK;
    const int bn = bc_gemm_tc_token_tile(T, epilogue);
    BC_CHECK_ARG((T + bn - 1) / bn <= 65535, "gemm_tc: %d tokens are too many token tiles", T);
    const bool stack = bc_gemm_tc_rows_per_block(T, N, epilogue) == 2 * TC_BM;
    const int w_rows = epilogue == EPI_SWIGLU ? 2 * N : N;
    const bool paired = g_tc_pair && bn == 256 && splits == 1;   // prompts: pairs of SMs share tiles, each block loading half the tokens
    CUtensorMap mw, mx;
    int st = weight_map(&mw, W, w_rows, K);
    if (st != BC_OK) return st;
    st = make_map(&mx, X, T, K, paired ? 128 : bn);
    if (st != BC_OK) return st;
    TcParams p;
    p.out = out;
    p.partial = partial;
    p.counters = counters;
    p.T = T;
    p.N = N;
    p.K = K;
    p.up_row_offset = N;
    p.stages = 0;
    p.k_iters_per_split = 0;
    p.n_tiles = p.t_tiles = p.clustered = 0;
    p.pair_tokens = 256;
    p.starve = paired ? 0 : g_tc_starve;
    if (!paired) g_tc_starve = 0;
    p.trace = nullptr;
#ifdef BC_TC_TRACE
    if (!paired && g_tc_trace && g_tc_trace_next < g_tc_trace_launches) p.trace = g_tc_trace + (size_t)(g_tc_trace_next++) * 1024 * 16;
#endif
    if (paired) {
        switch (epilogue) {
            case EPI_STORE: return launch_pair<EPI_STORE>(mw, mx, p, s);
            case EPI_STORE_F32: return launch_pair<EPI_STORE_F32>(mw, mx, p, s);
            case EPI_ADD_F32: return launch_pair<EPI_ADD_F32>(mw, mx, p, s);
            case EPI_SWIGLU: return launch_pair<EPI_SWIGLU>(mw, mx, p, s);
        }
    }
    switch (epilogue) {
        case EPI_STORE: return launch_bn<EPI_STORE>(bn, stack, mw, mx, p, splits, s);
        case EPI_STORE_F32: return launch_bn<EPI_STORE_F32>(bn, stack, mw, mx, p, splits, s);
        case EPI_ADD_F32: return launch_bn<EPI_ADD_F32>(bn, stack, mw, mx, p, splits, s);
        case EPI_SWIGLU: return launch_bn<EPI_SWIGLU>(bn, false, mw, mx, p, splits, s);
    }
    return BC_ERR_ARG;
}

// This unit's status word (0, or where a bounded wait gave up), its wait limit and its word
// of host memory: bc_gemm_tc_status / _set_wait_cycles / _bind_host_word.
TC_STATUS_EXPORTS(gemm_tc)
