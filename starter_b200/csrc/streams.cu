// A residual kept in several 32-bit copies side by side, x [rows, S * width]: the embedding rows that start it, and
// the one row kernel a branch costs.
//
//   return of the branch before (when one waits):   X'_t = sum_s mix[s][t] X_s + out[t] * y      (all t from the old X)
//   read of the next branch:                        n = RMSNorm(sum_s read[s] X'_s) * weight
//
// Everything is 32-bit; n is rounded once, when it is stored in the run's type.  A row's result depends on that row
// only.  Without `read` the kernel only takes the return.
#include "common.cuh"

#define STREAMS_MAX 8

template <class T>
__global__ void embed_streams_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ out, int hidden,
                                     int vocab, float scale, int copies, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_BAD_TOKEN);
        tok = 0;
    }
    const T* src = table + (long long)tok * hidden;
    float* dst = out + (long long)row * hidden * copies;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = to_f<T>(src[c]) * scale;
        for (int s = 0; s < copies; ++s) dst[(long long)s * hidden + c] = v;
    }
}

struct StreamWeights {
    float mix[STREAMS_MAX * STREAMS_MAX];   // [from][to]
    float out[STREAMS_MAX];
    float read[STREAMS_MAX];
};

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned int*>(&a);
    raw.y = *reinterpret_cast<const unsigned int*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// One block per row, VW columns per thread and turn (4 when the width is a multiple of 4: 16-byte reads of the 32-bit
// streams).  First pass: the return (in place) and the sum of squares of the blend; second pass: the blend scaled and
// stored.  The blend of a thread's first turn stays in registers (one turn covers rows of up to 4 * threads columns);
// later turns read their columns again (still in L1).
template <class T, class W, int S, int VW>
__global__ void __launch_bounds__(512)
stream_norm_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ mix,
                                   const float* __restrict__ out_w, const float* __restrict__ read_w, const W* __restrict__ weight,
                                   T* __restrict__ n, int width, float eps) {
    __shared__ float red[33];
    __shared__ StreamWeights sw;
    if (threadIdx.x < S * S) sw.mix[threadIdx.x] = y != nullptr ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        sw.out[threadIdx.x] = y != nullptr ? out_w[threadIdx.x] : 0.f;
        sw.read[threadIdx.x] = read_w != nullptr ? read_w[threadIdx.x] : 0.f;
    }
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    float* xr = x + (long long)blockIdx.x * width * S;
    const T* yr = y != nullptr ? y + (long long)blockIdx.x * width : nullptr;
    float ss = 0.f;
    float keep[VW];
#pragma unroll
    for (int i = 0; i < VW; ++i) keep[i] = 0.f;
    for (int c = threadIdx.x * VW; c < width; c += blockDim.x * VW) {
        float v[S][VW];
#pragma unroll
        for (int s = 0; s < S; ++s) {
            if (VW == 4) {
                const float4 t = ld4(xr + (long long)s * width + c);
                v[s][0] = t.x; v[s][1] = t.y; v[s][2] = t.z; v[s][VW - 1] = t.w;
            } else {
                v[s][0] = xr[(long long)s * width + c];
            }
        }
        if (yr != nullptr) {
            float yv[VW];
            if (VW == 4) {
                const float4 t = ld4(yr + c);
                yv[0] = t.x; yv[1] = t.y; yv[2] = t.z; yv[VW - 1] = t.w;
            } else {
                yv[0] = to_f<T>(yr[c]);
            }
            float nv[S][VW];
#pragma unroll
            for (int t = 0; t < S; ++t)
#pragma unroll
                for (int i = 0; i < VW; ++i) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < S; ++s) a = fmaf(sw.mix[s * S + t], v[s][i], a);
                    nv[t][i] = fmaf(sw.out[t], yv[i], a);
                }
#pragma unroll
            for (int t = 0; t < S; ++t) {
#pragma unroll
                for (int i = 0; i < VW; ++i) v[t][i] = nv[t][i];
                if (VW == 4) st4(xr + (long long)t * width + c, make_float4(nv[t][0], nv[t][1], nv[t][2], nv[t][VW - 1]));
                else xr[(long long)t * width + c] = nv[t][0];
            }
        }
#pragma unroll
        for (int i = 0; i < VW; ++i) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < S; ++s) u = fmaf(sw.read[s], v[s][i], u);
            ss = fmaf(u, u, ss);
            if (c < blockDim.x * VW) keep[i] = u;
        }
    }
    if (read_w == nullptr) return;
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
    T* nr = n + (long long)blockIdx.x * width;
    for (int c = threadIdx.x * VW; c < width; c += blockDim.x * VW) {
        float u[VW];
        if (c < blockDim.x * VW) {
#pragma unroll
            for (int i = 0; i < VW; ++i) u[i] = keep[i];
        } else {
#pragma unroll
            for (int i = 0; i < VW; ++i) {
                u[i] = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) u[i] = fmaf(sw.read[s], xr[(long long)s * width + c + i], u[i]);
            }
        }
        if (VW == 4) {
            const float4 w4 = ld4(weight + c);
            st4(nr + c, make_float4(__fmul_rn(__fmul_rn(u[0], rstd), w4.x), __fmul_rn(__fmul_rn(u[1], rstd), w4.y),
                                    __fmul_rn(__fmul_rn(u[2], rstd), w4.z), __fmul_rn(__fmul_rn(u[VW - 1], rstd), w4.w)));
        } else {
            nr[c] = from_f<T>(__fmul_rn(__fmul_rn(u[0], rstd), to_f<W>(weight[c])));
        }
    }
}

extern "C" {

int sb_embed_streams(int dtype, const int* tokens, const void* table, float* out, int rows, int hidden, int vocab, float scale,
                     int copies, int* status, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (copies < 1) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == SB_F32)
        sb_launch(embed_streams_kernel<float>, rows, threads, 0, stream, tokens, (const float*)table, out, hidden, vocab, scale, copies,
                  status);
    else
        sb_launch(embed_streams_kernel<__nv_bfloat16>, rows, threads, 0, stream, tokens, (const __nv_bfloat16*)table, out, hidden,
                  vocab, scale, copies, status);
    SB_LAUNCH_CHECK();
}

// dtype: the run's type (y and n); w_dtype: the norm weight's.  y, mix, out_w null: no return waits.  read_w null: only
// the return is taken.
int sb_stream_norm(int dtype, int w_dtype, float* x, const void* y, const float* mix, const float* out_w, const float* read_w,
                   const void* weight, void* n, int rows, int width, int streams, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (streams < 1 || streams > STREAMS_MAX) return (int)cudaErrorInvalidValue;
    if (y == nullptr && read_w == nullptr) return 0;
    const bool vec = width % 4 == 0;
    const int cols = vec ? width / 4 : width;
    const int threads = cols >= 512 && streams <= 4 ? 512 : (cols >= 256 ? 256 : 128);   // many streams: many registers per thread
    typedef __nv_bfloat16 bf;
#define SB_SN(T, W, S)                                                                                                              \
    do {                                                                                                                            \
        if (vec)                                                                                                                    \
            sb_launch(stream_norm_kernel<T, W, S, 4>, rows, threads, 0, stream, x, (const T*)y, mix, out_w, read_w, (const W*)weight, \
                      (T*)n, width, eps);                                                                                           \
        else                                                                                                                        \
            sb_launch(stream_norm_kernel<T, W, S, 1>, rows, threads, 0, stream, x, (const T*)y, mix, out_w, read_w, (const W*)weight, \
                      (T*)n, width, eps);                                                                                           \
    } while (0)
#define SB_SN_S(T, W)                          \
    switch (streams) {                         \
        case 1: SB_SN(T, W, 1); break;         \
        case 2: SB_SN(T, W, 2); break;         \
        case 3: SB_SN(T, W, 3); break;         \
        case 4: SB_SN(T, W, 4); break;         \
        case 5: SB_SN(T, W, 5); break;         \
        case 6: SB_SN(T, W, 6); break;         \
        case 7: SB_SN(T, W, 7); break;         \
        default: SB_SN(T, W, 8); break;        \
    }
    if (dtype == SB_F32 && w_dtype == SB_F32) { SB_SN_S(float, float) }
    else if (dtype == SB_BF16 && w_dtype == SB_BF16) { SB_SN_S(bf, bf) }
    else if (dtype == SB_BF16 && w_dtype == SB_F32) { SB_SN_S(bf, float) }
    else return (int)cudaErrorInvalidValue;
#undef SB_SN_S
#undef SB_SN
    SB_LAUNCH_CHECK();
}

}  // extern "C"
