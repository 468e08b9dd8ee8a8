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
//
// Every wait is bounded: after about a second without progress a thread records where it
// gave up in a status word, stops waiting, and the block frees its TMEM and returns.
#include <mutex>
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
};

// Blocks that run at the same time should share operands: the block index walks up to
// TC_RASTER token tiles first, then the weight tiles, then the next band of token tiles.
// A wave of 148 blocks then touches about 16 + 9 operand tiles instead of all the weight
// tiles of one or two token tiles, and each is fetched from HBM once, not once a token tile.
#define TC_RASTER 16

template <int BN, int EPI, bool STACK>
__global__ void __launch_bounds__(TC_THREADS, 1)
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
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // Tiles need 1024-byte alignment for the 128-byte swizzle.
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * 16 + 1];
    __shared__ uint32_t tmem_slot;

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
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                const int k = (k_first + i) * TC_BK;
                load_w(a, full0 + 8 * i, k, n0);
                if (N_ACC == 2) load_w(a + A_BYTES, full0 + 8 * i, k, second_row);
            }
            pdl_wait();
            for (int i = 0; i < ahead; i++) {
                const uint32_t a = smem_u32(smem + (size_t)i * STAGE_BYTES);
                tma_load_2d(a + N_ACC * A_BYTES, &map_x, full0 + 8 * i, (k_first + i) * TC_BK, t0);
            }
            for (int i = ahead; i < k_iters; i++) {
                const int s = i % stages;
                if (!mbar_wait(empty0 + 8 * s, ((i / stages) & 1) ^ 1, 1)) break;
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
            mma_commit(acc_bar);
        }
    } else {
        // Epilogue: this warp reads TMEM lanes 32 q .. 32 q + 31, i.e. weight rows n0 + 32 q + lane.
        const int q = warp & 3;
        const int n_first = n0 + 32 * q + lane;
        const bool split = gridDim.z > 1;
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
        if (lane == 0) ok = mbar_wait(acc_bar, 0, 3);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        tc_fence_after();
        const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16);
        bool finish = !split;   // this warp writes the output
        if (split && p.clustered) {
            // The partial tile goes to this block's shared memory (the ring is drained: every
            // load was consumed before the accumulator barrier fired), [column][row].
            if (ok) {
                float* mine = reinterpret_cast<float*>(smem) + 32 * q + lane;
#pragma unroll 1
                for (int c0 = 0; c0 < N_ACC * BN; c0 += 16) {
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
                for (int c0 = 0; c0 < N_ACC * BN; c0 += 16) {   // the second accumulator follows the first in TMEM and in scratch
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
            finish = arrived == (int)gridDim.z - 1;
            if (finish) {
                __threadfence();
                if (lane == 0) *counter = 0;   // ready for the next launch
            }
        }
        if (finish && ok) {
            const float* all = split ? p.partial + (size_t)tile * gridDim.z * part_tile + 32 * q + lane : nullptr;
            // 16 token columns of one accumulator: apply the epilogue and write.
            auto emit = [&](const uint32_t* v, const uint32_t* u, int cc) {
                const int acc_i = cc / BN, c0 = cc - acc_i * BN;     // which accumulator (stacked weight tile), which token column
                const int n = n_first + TC_BM * acc_i;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int t = t0 + c0 + j;
                    const float val = __uint_as_float(v[j]);
                    if (t < p.T && n < p.N) {
                        const size_t o = (size_t)t * p.N + n;
                        if (EPI == EPI_STORE) ((bf16*)p.out)[o] = __float2bfloat16_rn(val);
                        if (EPI == EPI_STORE_F32) ((float*)p.out)[o] = val;
                        // One thread owns each element, so a fire-and-forget reduction gives the same
                        // sum as a load, add and store, without waiting for the load.
                        if (EPI == EPI_ADD_F32) atomicAdd(&((float*)p.out)[o], val);
                        if (EPI == EPI_SWIGLU) ((bf16*)p.out)[o] = __float2bfloat16_rn(silu_mul(val, __uint_as_float(u[j])));
                    }
                }
            };
            constexpr int TOTAL = OUT_TILES * BN;
            if (!split) {
                // The accumulator comes out of TMEM 16 columns at a time, the next piece on its way
                // while this one is written, so the round trip to TMEM is paid once, not per piece.
                uint32_t va[16], vb[16], ua[16], ub[16];
                tmem_load16(taddr, va);
                if (EPI == EPI_SWIGLU) tmem_load16(taddr + BN, ua);
#pragma unroll 1
                for (int cc = 0; cc < TOTAL; cc += 32) {
                    tmem_load_wait();
                    if (cc + 16 < TOTAL) {
                        tmem_load16(taddr + cc + 16, vb);
                        if (EPI == EPI_SWIGLU) tmem_load16(taddr + BN + cc + 16, ub);
                    }
                    emit(va, ua, cc);
                    if (cc + 16 < TOTAL) {
                        tmem_load_wait();
                        if (cc + 32 < TOTAL) {
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
    if (p.clustered) {
        // Split-K inside a cluster: block z of the cluster finishes the token columns z, z + S,
        // ..: it adds the S partial tiles in the order 0, 1, 2 .. straight out of the blocks'
        // shared memory.  The same sums as through scratch memory, without the round trip.
        cg::cluster_group cl = cg::this_cluster();
        cl.sync();
        if (warp >= 2) {
            const int q = warp & 3, row = 32 * q + lane, n = n0 + row;
            const int S = (int)gridDim.z, rank = (int)blockIdx.z;
            const float* base = reinterpret_cast<const float*>(smem) + row;
            for (int c = rank; c < BN && t0 + c < p.T; c += S) {
                float v = 0.0f, u = 0.0f;
                for (int z = 0; z < S; z++) {
                    const float* theirs = cl.map_shared_rank(base, z);
                    v += theirs[(size_t)c * TC_BM];
                    if (EPI == EPI_SWIGLU) u += theirs[(size_t)(BN + c) * TC_BM];
                }
                if (n < p.N) {
                    const size_t o = (size_t)(t0 + c) * p.N + n;
                    if (EPI == EPI_STORE) ((bf16*)p.out)[o] = __float2bfloat16_rn(v);
                    if (EPI == EPI_STORE_F32) ((float*)p.out)[o] = v;
                    if (EPI == EPI_ADD_F32) atomicAdd(&((float*)p.out)[o], v);
                    if (EPI == EPI_SWIGLU) ((bf16*)p.out)[o] = __float2bfloat16_rn(silu_mul(v, u));
                }
            }
        }
        cl.sync();   // no block may leave while a peer still reads its shared memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
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
    cudaError_t e = p.clustered ? bc_launch_clustered(gemm_tc_kernel<BN, EPI, STACK>, grid, dim3(TC_THREADS), (size_t)smem, s, dim3(1, 1, splits), mw, mx, p)
                                : bc_launch(gemm_tc_kernel<BN, EPI, STACK>, grid, dim3(TC_THREADS), (size_t)smem, s, mw, mx, p);
    if (e != cudaSuccess) {
        bc_set_error("gemm_tc: launch failed: %s", cudaGetErrorString(e));
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
static double wave_fill(long long blocks) { return (double)blocks / (double)(((blocks + 147) / 148) * 148); }
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
    CUtensorMap mw, mx;
    int st = weight_map(&mw, W, w_rows, K);
    if (st != BC_OK) return st;
    st = make_map(&mx, X, T, K, bn);
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
    switch (epilogue) {
        case EPI_STORE: return launch_bn<EPI_STORE>(bn, stack, mw, mx, p, splits, s);
        case EPI_STORE_F32: return launch_bn<EPI_STORE_F32>(bn, stack, mw, mx, p, splits, s);
        case EPI_ADD_F32: return launch_bn<EPI_ADD_F32>(bn, stack, mw, mx, p, splits, s);
        case EPI_SWIGLU: return launch_bn<EPI_SWIGLU>(bn, false, mw, mx, p, splits, s);
    }
    return BC_ERR_ARG;
}

// The status word of the tensor-core kernels: 0, or where a bounded wait gave up.  Reading
// it waits for the device; `reset` clears it.
extern "C" int bc_gemm_tc_status(int reset) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
    if (reset && v != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    }
    return v;
}
