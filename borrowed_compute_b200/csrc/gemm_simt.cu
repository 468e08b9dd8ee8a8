// Matrix product on the CUDA cores: Y[m, n] = sum_k X[m, k] * W[n, k], float accumulation
// in ascending k, one fused multiply-add a term.  This is the product of the true 32-bit
// path (tensor cores would round operands to tf32) and the checked twin of the tensor-core
// kernel for bf16 operands.  Reference: the same contraction is k_matmul,
// crates/bc-infer/src/gpu/kernels.h:204-223, one warp a weight row; here a 64x64 output
// tile a block, 4x4 outputs a thread.  An output's sum never depends on how many other rows
// share the launch, because each thread walks k in order on its own.
//
// Epilogues: store in the operand type; store as float (scores); add into a float buffer
// (the residual stream); SwiGLU over a weight that stacks gate rows on up rows.
#include "common.cuh"

enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3 };

#define BM 64
#define BN 64
#define BK 16

template <class T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float* o) {
        float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float* o) {
        uint2 v = *reinterpret_cast<const uint2*>(p);
        o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
        o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
    }
};

// Loads a 64 x 16 tile of a K-major matrix (rows row0.., columns k0..) into smem[k][row].
template <class T, bool VEC>
__device__ __forceinline__ void load_tile(const T* __restrict__ src, int rows, int K, int row0, int k0, float (*smem)[BM + 4]) {
    const int r = threadIdx.x >> 2, kq = (threadIdx.x & 3) * 4;
    const int row = row0 + r, k = k0 + kq;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (row < rows) {
        const T* p = src + (size_t)row * K + k;
        if (VEC && k + 3 < K) {
            Vec4<T>::load(p, v);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (k + j < K) v[j] = to_f32(p[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) smem[kq + j][r] = v[j];
}

template <class T, int EPI, bool VEC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, T* __restrict__ out_act,
                                                        float* __restrict__ out_f32, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    __shared__ float Cs[EPI == EPI_SWIGLU ? BK : 1][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    float acc2[EPI == EPI_SWIGLU ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        load_tile<T, VEC>(X, M, K, m0, k0, As);
        load_tile<T, VEC>(W, N, K, n0, k0, Bs);
        if (EPI == EPI_SWIGLU) load_tile<T, VEC>(W + (size_t)N * K, N, K, n0, k0, Cs);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            if (EPI == EPI_SWIGLU) {
                float c[4];
#pragma unroll
                for (int j = 0; j < 4; j++) c[j] = Cs[k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc2[i][j] = fmaf(a[i], c[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = (size_t)m * N + n;
            if (EPI == EPI_STORE) out_act[o] = from_f32<T>(acc[i][j]);
            if (EPI == EPI_STORE_F32) out_f32[o] = acc[i][j];
            if (EPI == EPI_ADD_F32) out_f32[o] += acc[i][j];
            if (EPI == EPI_SWIGLU) {
                const float g = acc[i][j];
                out_act[o] = from_f32<T>(g / (1.0f + expf(-g)) * acc2[EPI == EPI_SWIGLU ? i : 0][j]);
            }
        }
    }
}

template <class T, int EPI>
static int launch(const void* X, const void* W, void* out, int M, int N, int K, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const bool vec = K % 4 == 0 && ((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0);
    T* oa = (EPI == EPI_STORE || EPI == EPI_SWIGLU) ? (T*)out : nullptr;
    float* of = (EPI == EPI_STORE_F32 || EPI == EPI_ADD_F32) ? (float*)out : nullptr;
    if (vec)
        bc_launch(gemm_simt_kernel<T, EPI, true>, grid, dim3(256), 0, s, (const T*)X, (const T*)W, oa, of, M, N, K);
    else
        bc_launch(gemm_simt_kernel<T, EPI, false>, grid, dim3(256), 0, s, (const T*)X, (const T*)W, oa, of, M, N, K);
    BC_LAUNCH_STATUS();
}

// X [M, K] and W [N, K] (for SwiGLU: W [2N, K], gate rows then up rows) in the operand
// type; `out` is [M, N] in the operand type (store, SwiGLU) or float (store_f32, add_f32).
template <class T>
static int dispatch(const void* X, const void* W, void* out, int M, int N, int K, int epilogue, cudaStream_t s) {
    BC_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    BC_CHECK_ARG((M + BM - 1) / BM <= 65535, "gemm_simt: %d rows are more than 65535 tiles of %d", M, BM);
    if (M == 0) return BC_OK;
    switch (epilogue) {
        case EPI_STORE: return launch<T, EPI_STORE>(X, W, out, M, N, K, s);
        case EPI_STORE_F32: return launch<T, EPI_STORE_F32>(X, W, out, M, N, K, s);
        case EPI_ADD_F32: return launch<T, EPI_ADD_F32>(X, W, out, M, N, K, s);
        case EPI_SWIGLU: return launch<T, EPI_SWIGLU>(X, W, out, M, N, K, s);
    }
    bc_set_error("gemm_simt: unknown epilogue %d", epilogue);
    return BC_ERR_ARG;
}

extern "C" int bc_gemm_simt_f32(const void* X, const void* W, void* out, int M, int N, int K, int epilogue, cudaStream_t s) {
    return dispatch<float>(X, W, out, M, N, K, epilogue, s);
}
extern "C" int bc_gemm_simt_bf16(const void* X, const void* W, void* out, int M, int N, int K, int epilogue, cudaStream_t s) {
    return dispatch<bf16>(X, W, out, M, N, K, epilogue, s);
}
