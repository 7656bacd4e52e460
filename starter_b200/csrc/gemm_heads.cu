// One product per head: C[m, h, :] = A[m, h, :] * W[h]^T for W [heads, N, K], on the CUDA cores, any sizes.
//
// A and C are views with a row stride and a head stride (their last axis is contiguous), so a head's columns can
// be read out of, and written into, wider rows without a copy.  Each output is one running 32-bit sum over
// k = 0..K-1 in order: a row's result does not depend on the rows around it.  It is the product of the 32-bit
// path and of small shapes; many rows in bfloat16 go to the library's batched product.
#include "common.cuh"

#define GH_BM 64
#define GH_BN 64
#define GH_BK 16

template <class T>
__global__ void __launch_bounds__(256) gemm_heads_kernel(const T* __restrict__ A, long long a_row, long long a_head,
                                                         const T* __restrict__ W, T* __restrict__ C, long long c_row,
                                                         long long c_head, int M, int N, int K) {
    __shared__ float As[GH_BK][GH_BM + 4];
    __shared__ float Ws[GH_BK][GH_BN + 4];
    pdl_wait();
    const int tid = threadIdx.x, head = blockIdx.z;
    const T* Ah = A + head * a_head;
    const T* Wh = W + (long long)head * N * K;
    T* Ch = C + head * c_head;
    const int m0 = blockIdx.y * GH_BM, n0 = blockIdx.x * GH_BN;
    const int tx = tid % 16, ty = tid / 16;
    const int lr = tid / 4, lk = (tid % 4) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GH_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + e][lr] = (am < M && k < K) ? to_f<T>(Ah[am * a_row + k]) : 0.f;
            Ws[lk + e][lr] = (wn < N && k < K) ? to_f<T>(Wh[(long long)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GH_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) Ch[m * c_row + n] = from_f<T>(acc[i][j]);
        }
    }
}

// A handful of rows (a decode step): a warp per output column of a head, the lanes striding over K, every row's sum
// reduced across the warp.  The tiled kernel above spends a step of 8 rows on 64-row tiles and a barrier every 16
// columns of K (33 us for 16 heads of 128 x 512 on a B200); this one is bound by the few hundred KB it reads.
#define GH_SMALL_M 16

template <class T>
__global__ void __launch_bounds__(256) gemm_heads_rows_kernel(const T* __restrict__ A, long long a_row, long long a_head,
                                                              const T* __restrict__ W, T* __restrict__ C, long long c_row,
                                                              long long c_head, int M, int N, int K) {
    pdl_wait();
    const int head = blockIdx.y, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const T* w = W + ((long long)head * N + n) * K;
    const T* a = A + head * a_head;
    float acc[GH_SMALL_M];
#pragma unroll
    for (int m = 0; m < GH_SMALL_M; ++m) acc[m] = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float wv = to_f<T>(w[k]);
#pragma unroll
        for (int m = 0; m < GH_SMALL_M; ++m)
            if (m < M) acc[m] = fmaf(to_f<T>(a[m * a_row + k]), wv, acc[m]);
    }
#pragma unroll
    for (int m = 0; m < GH_SMALL_M; ++m) {
        if (m < M) {
            const float v = warp_sum(acc[m]);
            if (lane == 0) C[head * c_head + m * c_row + n] = from_f<T>(v);
        }
    }
}

// Strides in elements.
extern "C" int sb_gemm_heads(int dtype, const void* A, long long a_row, long long a_head, const void* W, void* C, long long c_row,
                             long long c_head, int M, int N, int K, int heads, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return 0;
    if (M <= GH_SMALL_M && heads <= 65535) {
        dim3 small((N + 7) / 8, heads);
        if (dtype == SB_F32)
            sb_launch(gemm_heads_rows_kernel<float>, small, 256, 0, stream, (const float*)A, a_row, a_head, (const float*)W, (float*)C,
                      c_row, c_head, M, N, K);
        else
            sb_launch(gemm_heads_rows_kernel<__nv_bfloat16>, small, 256, 0, stream, (const __nv_bfloat16*)A, a_row, a_head,
                      (const __nv_bfloat16*)W, (__nv_bfloat16*)C, c_row, c_head, M, N, K);
        SB_LAUNCH_CHECK();
    }
    dim3 grid((N + GH_BN - 1) / GH_BN, (M + GH_BM - 1) / GH_BM, heads);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == SB_F32)
        sb_launch(gemm_heads_kernel<float>, grid, 256, 0, stream, (const float*)A, a_row, a_head, (const float*)W, (float*)C, c_row,
                  c_head, M, N, K);
    else
        sb_launch(gemm_heads_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)A, a_row, a_head,
                  (const __nv_bfloat16*)W, (__nv_bfloat16*)C, c_row, c_head, M, N, K);
    SB_LAUNCH_CHECK();
}
