// The tcgen05 / TMA / mbarrier pieces shared by the tensor-core product kernels: tile
// sizes, bounded barrier waits, TMA loads, TMEM allocation and reads, MMA issue, and the
// shared-memory and instruction descriptors.
#pragma once

#include <cuda.h>

#include "common.cuh"

enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3 };

#define TC_BM 128          // weight rows a tile (MMA M)
#define TC_BK 64           // k a stage: 64 bf16 = one 128-byte swizzle row
#define TC_THREADS 192     // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue (the one-block product adds four more from 64 tokens a tile on)
#define TC_SMEM_LIMIT 230400   // dynamic bytes asked for at most; static barriers take a little more
#define TC_WAIT_CYCLES 2000000000ll   // clocks a wait may take before it gives up: about a second

// Status word: 0 while all is well, else (code << 16 | detail) of the first wait that gave up.
// One copy a translation unit (the library builds without relocatable device code): every
// unit that includes this header exports, with TC_STATUS_EXPORTS below, a reader of its own
// word, a setter of its wait limit, and a binder of a word of host memory that the device
// can write: the first wait that gives up leaves its code there too, so the host can look
// after any synchronisation of its own without a copy from the device.
static __device__ int g_tc_status = 0;
static __device__ long long g_tc_wait_cycles = TC_WAIT_CYCLES;
static __device__ int* g_tc_host_word = nullptr;

__device__ __forceinline__ void tc_give_up(int code) {
    const int v = (code << 16) | (int)(blockIdx.x & 0xffff);
    if (atomicCAS(&g_tc_status, 0, v) == 0) {
        int* host = g_tc_host_word;
        if (host) {
            *reinterpret_cast<volatile int*>(host) = v;
            __threadfence_system();
        }
    }
}

#define TC_STATUS_EXPORTS(NAME)                                                                                  \
    extern "C" int bc_##NAME##_status(int reset) {                                                               \
        int v = 0;                                                                                               \
        cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));                                                      \
        if (reset && v != 0) {                                                                                   \
            int zero = 0;                                                                                        \
            cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));                                                 \
        }                                                                                                        \
        return v;                                                                                                \
    }                                                                                                            \
    extern "C" int bc_##NAME##_set_wait_cycles(long long cycles) {                                               \
        if (cycles <= 0) cycles = TC_WAIT_CYCLES;                                                                \
        return (int)cudaMemcpyToSymbol(g_tc_wait_cycles, &cycles, sizeof(cycles));                               \
    }                                                                                                            \
    extern "C" int bc_##NAME##_bind_host_word(int* device_pointer_to_host_word) {                                \
        return (int)cudaMemcpyToSymbol(g_tc_host_word, &device_pointer_to_host_word, sizeof(int*));              \
    }

// ------------------------------------------------------------------------------ PTX pieces
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for a phase of a barrier, at most the wait limit (about a second unless set
// otherwise).  False (and a recorded status) if it gave up; the caller then stops doing work
// but still reaches the teardown.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64(), limit = g_tc_wait_cycles;
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > limit) {
            tc_give_up(code);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Makes this thread's ordinary shared-memory writes visible to the asynchronous proxy (the
// tensor core reads operands through it).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// The same with an L2 policy: weights are read once a step and should leave the L2 first,
// so that activations, partial sums and the cache pages of the step stay.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the A operand in tensor memory: row m of A in lane m, two bf16 a 32-bit column
// (k and k + 1 of a k-step in its low and high half), 8 columns a k-step of 16.
__device__ __forceinline__ void mma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- the same for a pair of blocks on the two SMs of a TPC (cta_group::2): one thread of
// the even block issues MMAs over both blocks' shared memory (each holds its own 128 rows
// of A and its half of B at the same offsets) into both blocks' TMEM.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of the same location in block `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// A TMA load into this block's shared memory whose bytes are counted on a barrier that may
// lie in the pair's other block (a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
                 : "memory");
}
// An arrival on a barrier that may lie in another block of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives, once the pair's MMAs issued so far are done, on the barrier at this offset in
// every block of the mask (both blocks of the pair: 3).  The arrival is multicast, no load is.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(cta_mask)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
        "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: k-major tile of 128-byte rows, 128-byte swizzle, as TMA
// writes it.  Bits 0-13 address/16; 16-29 leading offset/16 (unused for swizzled k-major,
// 1); 32-45 stride between 8-row groups/16 (1024 bytes); 46-47 version 1; 61-63 layout 2
// (SWIZZLE_128B).  Stepping 16 k (32 bytes) inside the swizzle row adds 2 to the address.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// The same tile read the other way round: an operand whose M or N index is the contiguous
// one (a [k, n] matrix with n contiguous, such as values [position, head size] as the B of
// P V), in blocks of [k rows][64 elements] with the 128-byte swizzle, as TMA writes them.
// Eight k rows are 1024 bytes apart (stride offset); the next 64 elements of M or N are
// `next_block` bytes on (leading offset).  Stepping 16 k adds 16 rows (2048 bytes).
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t next_block) {
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)((next_block >> 4) & 0x3fff) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16 for M = 128, float accumulate, bf16 operands, A k-major,
// B k-major or (b_mn) n-major.
__host__ __device__ constexpr uint32_t instr_desc_b(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// Instruction descriptor of kind::f16 for a pair of blocks: M = 256 (128 rows a block).
__host__ __device__ constexpr uint32_t instr_desc_pair(int n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24); }
// Instruction descriptor of kind::f16: float accumulate (bit 4), A and B bf16 (bits 7, 10),
// both k-major (bits 15, 16 clear), N / 8 at bit 17, M / 16 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(int n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24); }

// The gate of the bf16 path: hardware exponential and division (errors of a few float ulp,
// far below the bf16 rounding that follows).
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

