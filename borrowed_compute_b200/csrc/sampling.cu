// Picking the next token from a row of float scores, on the device.
//
// The definition is the reference's (crates/bc-infer/src/sample.rs:24-71):
//   temperature <= 0: the first largest score (argmax, strict >, ascending index);
//   else w_i = e^((s_i - max)/T); order the tokens by w descending, ties by ascending id;
//   keep the shortest prefix whose share of sum(w) reaches top_p (at least one token);
//   draw u = uniform(seed ^ step * 0x9e3779b97f4a7c15) (splitmix64's finaliser, top 24
//   bits), r = u * (kept weight), and walk the kept list until the running weight reaches
//   r; if rounding lets the walk run out, the first token of the list stands.
//
// The reference sorts the whole row on the host.  Here nothing is sorted: a weight's float
// bits order like the weight, so the place where a running sum over the descending order
// crosses a target is found by descending four key bits a pass, 16 bucket sums a pass kept
// in registers and added across the block in a fixed order (no atomics: the same bits every
// run).  Two such walks give the nucleus cut and the draw; tokens of equal weight are told
// apart by id with an ordered count.  A cluster of eight blocks shares a row (each owns a
// span of ids and they exchange sums through distributed shared memory); any vocabulary size.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define SMP_THREADS 512
#define SMP_WARPS (SMP_THREADS / 32)
#define SMP_CLUSTER 8      // blocks that share a row (the portable cluster size)
#define SMP_KEEP 36        // weights a thread keeps in registers: rows of up to 8 x 512 x 36 = 147,456 scores are read once

// splitmix64's finaliser; the top 24 bits over 2^24 (sample.rs:64-71).
__device__ __forceinline__ float uniform_from(uint64_t seed) {
    uint64_t z = seed + 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return (float)(z >> 40) / 16777216.0f;
}

__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
    unsigned u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);     // larger float -> larger unsigned
    if (v != v) u = 0u;                                  // a NaN never wins (sample.rs:27 compares with >)
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
}
__device__ __forceinline__ float argmax_key_value(unsigned long long k) {
    unsigned u = (unsigned)(k >> 32);
    u = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(u);
}

// What one block of a row's cluster leaves for its peers to read through distributed
// shared memory.  Each slot is written once, or alternates between two copies, so that one
// cluster barrier a step is enough.
struct SampleShared {
    unsigned long long best;     // this block's best (score, index) word
    float sum;                   // this block's sum of weights
    float tot[2][16];            // this block's bucket sums of the current descent level (two copies in turn)
    int count[2];                // this block's number of tokens with the cut key / the hit key
    float all[16];               // bucket sums over the whole row (local copy)
    int warp_counts[SMP_WARPS];
};

struct Walk {
    unsigned key;   // float bits of the weight at which the running sum reaches the target
    float above;    // sum of all weights with larger bits
};

// A row is spread over the blocks of a cluster: block c owns ids [c * chunk, (c + 1) * chunk).
struct RowView {
    const float* row;
    int lo, hi;          // this block's ids
    float max_score, inv_t;
    __device__ __forceinline__ float weight(int i) const { return expf((row[i] - max_score) * inv_t); }
};

// Where, going down the weights of the whole row in descending order, the running sum first
// reaches `target` (if rounding keeps it below to the end, the smallest weight stands).
// Four key bits a level: every thread sums the weights of its elements into 16 buckets of
// its own in shared memory, a warp a bucket adds the threads' sums in a fixed order, and
// the blocks' sums are added in rank order, so every block takes the same decision and
// the result is the same bits on every run.
// `kept` holds this thread's weights (elements lo + thread + 512 k, k < n_kept) when the row is
// short enough for that (`cached`): the sixteen passes of the two walks then read registers
// instead of fetching the scores and taking their exponentials again.
__device__ __forceinline__ Walk walk_down(cg::cluster_group& cl, SampleShared& sh, float* hist, const RowView& rv, float target, int& turn,
                                          const float (&kept)[SMP_KEEP], int n_kept, bool cached) {
    unsigned prefix = 0, mask = 0;
    float above = 0.0f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int shift = 28; shift >= 0; shift -= 4) {
#pragma unroll
        for (int j = 0; j < 16; j++) hist[j * SMP_THREADS + threadIdx.x] = 0.0f;
        if (cached) {
#pragma unroll
            for (int k = 0; k < SMP_KEEP; k++)
                if (k < n_kept) {
                    const float w = kept[k];
                    const unsigned key = __float_as_uint(w);
                    if ((key & mask) == prefix) hist[((key >> shift) & 15u) * SMP_THREADS + threadIdx.x] += w;
                }
        } else {
            for (int i = rv.lo + threadIdx.x; i < rv.hi; i += SMP_THREADS) {
                const float w = rv.weight(i);
                const unsigned key = __float_as_uint(w);
                if ((key & mask) == prefix) hist[((key >> shift) & 15u) * SMP_THREADS + threadIdx.x] += w;
            }
        }
        __syncthreads();
        {   // warp j adds bucket j over the threads
            float s = 0.0f;
            for (int k = 0; k < SMP_THREADS / 32; k++) s += hist[warp * SMP_THREADS + lane + 32 * k];
            s = warp_sum(s);
            if (lane == 0) sh.tot[turn][warp] = s;
        }
        cl.sync();
        if (threadIdx.x < 16) {
            float s = 0.0f;
            for (unsigned r = 0; r < cl.num_blocks(); r++) s += cl.map_shared_rank(&sh, r)->tot[turn][threadIdx.x];
            sh.all[threadIdx.x] = s;
        }
        turn ^= 1;
        __syncthreads();
        float running = above;
        int chosen = -1, lowest = -1;
        float above_lowest = above;
        for (int j = 15; j >= 0; j--) {
            const float t = sh.all[j];
            if (t > 0.0f) {
                if (chosen < 0 && running + t >= target) chosen = j;
                lowest = j;
                above_lowest = running;
            }
            if (chosen < 0) running += t;
        }
        if (chosen < 0) {
            chosen = lowest < 0 ? 0 : lowest;
            running = above_lowest;
        }
        above = running;
        prefix |= (unsigned)chosen << shift;
        mask |= 15u << shift;
        __syncthreads();   // sh.all is rewritten at the next level
    }
    return {prefix, above};
}

// Counts, by ascending id, the tokens whose weight has bits `key`.  Returns the row's total;
// `before` gets how many of them have smaller ids than this thread's own span of ids
// [t_lo, t_hi), `mine` how many lie inside it.
__device__ int count_with_key(cg::cluster_group& cl, SampleShared& sh, const RowView& rv, unsigned key, int which, int& before, int& mine,
                              int& t_lo, int& t_hi) {
    const int span = (rv.hi - rv.lo + SMP_THREADS - 1) / SMP_THREADS;
    t_lo = min(rv.hi, rv.lo + (int)threadIdx.x * span);
    t_hi = min(rv.hi, t_lo + span);
    mine = 0;
    for (int i = t_lo; i < t_hi; i++) mine += __float_as_uint(rv.weight(i)) == key;
    // exclusive prefix over the block's threads (ascending ids)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) sh.warp_counts[warp] = incl;
    __syncthreads();
    int warp_before = 0, block_total = 0;
    for (int w = 0; w < SMP_WARPS; w++) {
        if (w < warp) warp_before += sh.warp_counts[w];
        block_total += sh.warp_counts[w];
    }
    if (threadIdx.x == 0) sh.count[which] = block_total;
    cl.sync();
    int blocks_before = 0, total = 0;
    for (unsigned r = 0; r < cl.num_blocks(); r++) {
        const int c = cl.map_shared_rank(&sh, r)->count[which];
        if (r < cl.block_rank()) blocks_before += c;
        total += c;
    }
    before = blocks_before + warp_before + incl - mine;
    return total;
}

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const float* __restrict__ scores, int V, const float* __restrict__ temperature,
                                                             const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                                                             const int* __restrict__ step, int* __restrict__ out) {
    extern __shared__ float hist[];          // [16][SMP_THREADS]: every thread's own bucket sums
    __shared__ SampleShared sh;
    __shared__ unsigned long long warp_best[SMP_WARPS];
    __shared__ float red[32];
    cg::cluster_group cl = cg::this_cluster();
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y;
    const int chunk = (V + (int)cl.num_blocks() - 1) / (int)cl.num_blocks();
    RowView rv;
    rv.row = scores + (size_t)r * V;
    rv.lo = min(V, (int)cl.block_rank() * chunk);
    rv.hi = min(V, rv.lo + chunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // The largest score and its first index, over the cluster.
    unsigned long long best = 0ull;
    for (int i = rv.lo + threadIdx.x; i < rv.hi; i += SMP_THREADS) {
        const unsigned long long k = argmax_key(rv.row[i], i);
        best = k > best ? k : best;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if (lane == 0) warp_best[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SMP_WARPS; w++) best = warp_best[w] > best ? warp_best[w] : best;
        sh.best = best;
    }
    cl.sync();
    best = 0ull;
    for (unsigned b = 0; b < cl.num_blocks(); b++) {
        const unsigned long long k = cl.map_shared_rank(&sh, b)->best;
        best = k > best ? k : best;
    }
    const int top = best == 0ull ? 0 : (int)(0xffffffffu - (unsigned)(best & 0xffffffffull));
    const float temp = temperature[r];
    if (cl.block_rank() == 0 && threadIdx.x == 0) out[r] = top;   // stands unless a draw below replaces it
    if (!(temp > 0.0f)) {                                          // greedy: every block of the cluster leaves here,
        cl.sync();                                                 // but none while a peer still reads its shared memory
        return;
    }
    rv.max_score = argmax_key_value(best);
    rv.inv_t = 1.0f / temp;

    // This thread's weights, kept for the walks below if there are few enough of them.
    float held[SMP_KEEP];
    const bool cached = chunk <= SMP_KEEP * SMP_THREADS;
    const int n_kept = cached ? max(0, (rv.hi - rv.lo - (int)threadIdx.x + SMP_THREADS - 1) / SMP_THREADS) : 0;
    float mine = 0.0f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < SMP_KEEP; k++) {
            held[k] = k < n_kept ? rv.weight(rv.lo + (int)threadIdx.x + k * SMP_THREADS) : 0.0f;
            if (k < n_kept) mine += held[k];
        }
    } else {
        for (int i = rv.lo + threadIdx.x; i < rv.hi; i += SMP_THREADS) mine += rv.weight(i);
    }
    mine = block_sum(mine, red);
    if (threadIdx.x == 0) sh.sum = mine;
    cl.sync();
    float total = 0.0f;
    for (unsigned b = 0; b < cl.num_blocks(); b++) total += cl.map_shared_rank(&sh, b)->sum;

    // The nucleus: everything heavier than the weight at the cut, and of the tokens of
    // exactly that weight the first `n_cut` by id.
    int turn = 0;
    const float want = top_p[r] * total;
    // With top_p of one or more every token is kept: no cut to look for (eight passes less).
    const bool all_kept = top_p[r] >= 1.0f;
    int before, inside, t_lo, t_hi;
    Walk cut = {0u, total};
    int n_cut = 0x7fffffff;
    float kept = total;
    if (!all_kept) {
        cut = walk_down(cl, sh, hist, rv, want, turn, held, n_kept, cached);
        const float w_cut = __uint_as_float(cut.key);
        const int ties_cut = count_with_key(cl, sh, rv, cut.key, 0, before, inside, t_lo, t_hi);
        n_cut = w_cut > 0.0f ? (int)ceilf((want - cut.above) / w_cut) : ties_cut;
        n_cut = max(1, min(n_cut, ties_cut));
        kept = cut.above + (float)n_cut * w_cut;
    }

    const uint64_t st = (uint64_t)(long long)step[r];
    const float rr = uniform_from(seed[r] ^ (st * 0x9e3779b97f4a7c15ull)) * kept;
    const Walk hit = walk_down(cl, sh, hist, rv, rr, turn, held, n_kept, cached);
    const float w_hit = __uint_as_float(hit.key);
    int n_hit = w_hit > 0.0f ? (int)ceilf((rr - hit.above) / w_hit) : 1;
    n_hit = max(1, n_hit);
    // If the walk ran past the kept tokens the first of the list stands (sample.rs:61): `top`, already written.
    const bool past = hit.key < cut.key || (hit.key == cut.key && n_hit > n_cut);
    const int ties_hit = count_with_key(cl, sh, rv, hit.key, 1, before, inside, t_lo, t_hi);
    if (!past) {
        const int wanted = max(1, min(n_hit, ties_hit));            // the wanted-th token of that weight, by ascending id
        if (before < wanted && wanted <= before + inside) {         // it lies in this thread's span: exactly one thread of the cluster
            int seen = before;
            for (int i = t_lo; i < t_hi; i++)
                if (__float_as_uint(rv.weight(i)) == hit.key && ++seen == wanted) {
                    out[r] = i;
                    break;
                }
        }
    }
    cl.sync();   // no block may leave while a peer still reads its shared memory
}

// Greedy picks for a batch in two short launches: blocks scan chunks of a row and fold
// their best into one 64-bit word a row (score bits made sortable in the high half, the
// inverted index in the low half, so the largest word is the largest score and, among
// equals, the smallest index); a second launch unpacks the words and clears them.
#define ARGMAX_CHUNK 4096

__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ scores, int V, unsigned long long* __restrict__ best) {
    __shared__ unsigned long long part[8];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, c0 = blockIdx.x * ARGMAX_CHUNK;
    const float* row = scores + (size_t)r * V;
    unsigned long long mine = 0ull;
    for (int i = c0 + threadIdx.x; i < min(V, c0 + ARGMAX_CHUNK); i += blockDim.x) {
        const unsigned long long k = argmax_key(row[i], i);
        mine = k > mine ? k : mine;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
        mine = other > mine ? other : mine;
    }
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) mine = part[w] > mine ? part[w] : mine;
        atomicMax(&best[r], mine);
    }
}

__global__ void argmax_finish_kernel(unsigned long long* __restrict__ best, int* __restrict__ out, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const unsigned long long k = best[r];
    out[r] = k == 0ull ? 0 : (int)(0xffffffffu - (unsigned)(k & 0xffffffffull));
    best[r] = 0ull;
}

#define ARGMAX_MAX_ROWS 4096
__device__ unsigned long long g_argmax_best[ARGMAX_MAX_ROWS];   // zero between launches

// Blocks that share a row: 0 lets the launcher choose, 1, 2, 4 or 8 force it (measurements and
// tests; every choice gives the same picks).
static int g_smp_share = 0;
extern "C" void bc_sample_set_blocks_per_row(int n) { g_smp_share = (n == 1 || n == 2 || n == 4 || n == 8) ? n : 0; }

// scores [rows, V] float; temperature, top_p, seed (64-bit), step (the position of the row
// sampled) one a row; out [rows] token ids.
extern "C" int bc_sample(const float* scores, int rows, int V, const float* temperature, const float* top_p,
                         const unsigned long long* seed, const int* step, int* out, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && V > 0, "sample: bad sizes rows=%d V=%d", rows, V);
    if (rows == 0) return BC_OK;
    BC_CHECK_ARG(rows <= 65535, "sample: %d rows are more than 65535", rows);
    const size_t smem = 16 * SMP_THREADS * sizeof(float);
    // Blocks a row: eight (a cluster) while all rows' blocks still run at once, one to an SM;
    // with more rows fewer blocks share a row, so that the rows still run side by side instead
    // of in turns (64 rows: 344 us with eight blocks a row, in four turns).
    int share = g_smp_share > 0 ? g_smp_share : SMP_CLUSTER;
    if (g_smp_share == 0) {
        const int sms = bc_sm_count();
        while (share > 1 && rows * share > sms) share /= 2;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(share, rows);
    cfg.blockDim = dim3(SMP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = share;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_bc_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, scores, V, temperature, top_p, seed, step, out);
    if (e != cudaSuccess) {
        bc_set_error("sample: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    BC_LAUNCH_STATUS();
}

extern "C" int bc_argmax(const float* scores, int rows, int V, int* out, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && V > 0, "argmax: bad sizes rows=%d V=%d", rows, V);
    BC_CHECK_ARG(rows <= ARGMAX_MAX_ROWS, "argmax: %d rows are more than %d", rows, ARGMAX_MAX_ROWS);
    if (rows == 0) return BC_OK;
    static unsigned long long* best = nullptr;
    if (!best) {
        cudaError_t e = cudaGetSymbolAddress((void**)&best, g_argmax_best);
        if (e != cudaSuccess) {
            bc_set_error("argmax: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    dim3 grid((V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK, rows);
    bc_launch(argmax_partial_kernel, grid, dim3(256), 0, s, scores, V, best);
    bc_launch(argmax_finish_kernel, dim3((rows + 127) / 128), dim3(128), 0, s, best, out, rows);
    BC_LAUNCH_STATUS();
}
