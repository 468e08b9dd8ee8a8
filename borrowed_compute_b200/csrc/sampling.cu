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
// apart by id with an ordered count.  One block a row; any vocabulary size.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)

struct ArgBest {
    float v;
    int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    // The earlier index wins a tie; a NaN never beats a number (sample.rs:27 compares with >).
    if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
    return a;
}

__device__ int block_argmax(const float* __restrict__ row, int V, ArgBest* scratch, float* max_out) {
    ArgBest best = {-INFINITY, -1};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (best.i < 0 || v > best.v) best = {v, i};
    }
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = best;
    __syncthreads();
    ArgBest b = scratch[0];
    const int warps = (blockDim.x + 31) >> 5;
    for (int w = 1; w < warps; w++) b = better(b, scratch[w]);
    if (max_out) *max_out = b.v;
    return b.i < 0 ? 0 : b.i;
}

// splitmix64's finaliser; the top 24 bits over 2^24 (sample.rs:64-71).
__device__ __forceinline__ float uniform_from(uint64_t seed) {
    uint64_t z = seed + 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return (float)(z >> 40) / 16777216.0f;
}

struct Walk {
    unsigned key;   // float bits of the weight at which the running sum reaches the target
    float above;    // sum of all weights with larger bits
};

// Where, going down the weights in descending order, the running sum first reaches
// `target`.  If rounding keeps the sum below the target to the end, the smallest weight
// that occurs stands.
__device__ Walk walk_down(const float* __restrict__ row, int V, float max_score, float inv_t, float target, float (*part)[16], float* tot) {
    unsigned prefix = 0, mask = 0;
    float above = 0.0f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int shift = 28; shift >= 0; shift -= 4) {
        float b[16];
#pragma unroll
        for (int j = 0; j < 16; j++) b[j] = 0.0f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float w = expf((row[i] - max_score) * inv_t);
            const unsigned key = __float_as_uint(w);
            if ((key & mask) == prefix) {
                const unsigned d = (key >> shift) & 15u;
#pragma unroll
                for (int j = 0; j < 16; j++) b[j] += d == (unsigned)j ? w : 0.0f;
            }
        }
#pragma unroll
        for (int j = 0; j < 16; j++) b[j] = warp_sum(b[j]);
        __syncthreads();
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < 16; j++) part[warp][j] = b[j];
        }
        __syncthreads();
        if (threadIdx.x < 16) {
            float s = 0.0f;
            for (int w = 0; w < SAMPLE_WARPS; w++) s += part[w][threadIdx.x];
            tot[threadIdx.x] = s;
        }
        __syncthreads();
        float running = above;
        int chosen = -1, lowest = -1;
        float above_lowest = above;
        for (int j = 15; j >= 0; j--) {
            const float t = tot[j];
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
    }
    return {prefix, above};
}

// The id of the n-th (1-based, clamped to what exists) token whose weight has bits `key`,
// counting by ascending id, and how many such tokens there are.
__device__ int nth_with_key(const float* __restrict__ row, int V, float max_score, float inv_t, unsigned key, int n, int* counts, int* total_out) {
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
    int mine = 0;
    for (int i = lo; i < hi; i++) mine += __float_as_uint(expf((row[i] - max_score) * inv_t)) == key;
    __syncthreads();
    counts[threadIdx.x] = mine;
    __syncthreads();
    // Threads own ascending id ranges, so a serial prefix over their counts is the order.
    __shared__ int found, total;
    if (threadIdx.x == 0) {
        int sum = 0;
        for (int t = 0; t < (int)blockDim.x; t++) sum += counts[t];
        total = sum;
        int want = max(1, min(n, sum)), before = 0, owner = 0;
        for (int t = 0; t < (int)blockDim.x; t++) {
            if (before + counts[t] >= want) { owner = t; break; }
            before += counts[t];
        }
        counts[0] = owner;
        counts[1] = want - before;
        found = -1;
    }
    __syncthreads();
    const int owner = counts[0], rank = counts[1];
    if ((int)threadIdx.x == owner) {
        int seen = 0;
        for (int i = lo; i < hi; i++) {
            if (__float_as_uint(expf((row[i] - max_score) * inv_t)) == key && ++seen == rank) { found = i; break; }
        }
    }
    __syncthreads();
    if (total_out) *total_out = total;
    return found;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ scores, int V, const float* __restrict__ temperature,
                                                                const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                                                                const int* __restrict__ step, int* __restrict__ out) {
    __shared__ ArgBest best_scratch[SAMPLE_WARPS];
    __shared__ float part[SAMPLE_WARPS][16];
    __shared__ float tot[16];
    __shared__ float red[32];
    __shared__ int counts[SAMPLE_THREADS];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = scores + (size_t)r * V;
    float max_score;
    const int top = block_argmax(row, V, best_scratch, &max_score);
    const float temp = temperature[r];
    if (!(temp > 0.0f)) {
        if (threadIdx.x == 0) out[r] = top;
        return;
    }
    const float inv_t = 1.0f / temp;
    float mine = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mine += expf((row[i] - max_score) * inv_t);
    const float total = block_sum(mine, red);

    // The nucleus: everything heavier than the weight at the cut, and of the tokens of
    // exactly that weight the first `n_cut` by id.
    const float want = top_p[r] * total;
    const Walk cut = walk_down(row, V, max_score, inv_t, want, part, tot);
    const float w_cut = __uint_as_float(cut.key);
    int ties_cut;
    nth_with_key(row, V, max_score, inv_t, cut.key, 1, counts, &ties_cut);
    int n_cut = w_cut > 0.0f ? (int)ceilf((want - cut.above) / w_cut) : ties_cut;
    n_cut = max(1, min(n_cut, ties_cut));
    const float kept = cut.above + (float)n_cut * w_cut;

    const uint64_t st = (uint64_t)(long long)step[r];
    const float rr = uniform_from(seed[r] ^ (st * 0x9e3779b97f4a7c15ull)) * kept;
    const Walk hit = walk_down(row, V, max_score, inv_t, rr, part, tot);
    const float w_hit = __uint_as_float(hit.key);
    int n_hit = w_hit > 0.0f ? (int)ceilf((rr - hit.above) / w_hit) : 1;
    n_hit = max(1, n_hit);
    int pick;
    if (hit.key < cut.key) {
        pick = top;   // the walk ran past the kept tokens: sample.rs:61 falls back to the first
    } else {
        if (hit.key == cut.key && n_hit > n_cut) {
            pick = top;
        } else {
            pick = nth_with_key(row, V, max_score, inv_t, hit.key, n_hit, counts, nullptr);
            if (pick < 0) pick = top;
        }
    }
    if (threadIdx.x == 0) out[r] = pick;
}

// Greedy picks for a batch in two short launches: blocks scan chunks of a row and fold
// their best into one 64-bit word a row (score bits made sortable in the high half, the
// inverted index in the low half, so the largest word is the largest score and, among
// equals, the smallest index); a second launch unpacks the words and clears them.
#define ARGMAX_CHUNK 4096

__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
    unsigned u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);     // larger float -> larger unsigned
    if (v != v) u = 0u;                                  // a NaN never wins
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
}

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

// scores [rows, V] float; temperature, top_p, seed (64-bit), step (the position of the row
// sampled) one a row; out [rows] token ids.
extern "C" int bc_sample(const float* scores, int rows, int V, const float* temperature, const float* top_p,
                         const unsigned long long* seed, const int* step, int* out, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && V > 0, "sample: bad sizes rows=%d V=%d", rows, V);
    if (rows == 0) return BC_OK;
    bc_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, s, scores, V, temperature, top_p, seed, step, out);
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
