// Row-wise kernels of models that keep a 32-bit residual stream: embedding rows widened to 32-bit, RMSNorm in
// groups with the residual sum in front, the clamped gated activation, tanh.
//
// TX is the residual's type, T the run's activation type (what branches read and write), W the weight's.  Sums of
// squares, the scaling and the residual sum are 32-bit; a result is rounded once, when it is stored.
#include "common.cuh"

__global__ void embed_wide_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table, float* __restrict__ out,
                                  int hidden, int vocab, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_BAD_TOKEN);
        tok = 0;
    }
    const __nv_bfloat16* src = table + (long long)tok * hidden;
    float* dst = out + (long long)row * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = __bfloat162float(src[c]);
}

// Four consecutive values of a row as floats, whatever the type they are stored in.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned int*>(&a);
    raw.y = *reinterpret_cast<const unsigned int*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// One block per row.  x <- x + (d1 + d2) first when deltas are given (either may be null); then every group of
// width / groups consecutive columns is divided by its own root mean square and multiplied by the weight.
// VEC: the group's width is a multiple of 4, so a thread takes four columns at a time (16-byte reads of a 32-bit row).
template <class TX, class T, class W, bool VEC>
__global__ void grouped_rmsnorm_kernel(TX* __restrict__ x, const T* __restrict__ d1, const T* __restrict__ d2,
                                       const W* __restrict__ weight, T* __restrict__ out, int width, int groups, float eps) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const long long base = (long long)blockIdx.x * width;
    TX* xr = x + base;
    const int gw = width / groups;
    for (int g = 0; g < groups; ++g) {
        const int c0 = g * gw, c1 = c0 + gw;
        float ss = 0.f;
        if (VEC) {
            for (int c = c0 + 4 * threadIdx.x; c < c1; c += 4 * blockDim.x) {
                float4 v = load4(xr + c);
                if (d1 != nullptr) {
                    float4 d = load4(d1 + base + c);
                    if (d2 != nullptr) {
                        const float4 e = load4(d2 + base + c);
                        d = make_float4(__fadd_rn(d.x, e.x), __fadd_rn(d.y, e.y), __fadd_rn(d.z, e.z), __fadd_rn(d.w, e.w));
                    }
                    v = make_float4(rnd<TX>(__fadd_rn(v.x, d.x)), rnd<TX>(__fadd_rn(v.y, d.y)), rnd<TX>(__fadd_rn(v.z, d.z)),
                                    rnd<TX>(__fadd_rn(v.w, d.w)));
                    store4(xr + c, v);
                }
                ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            }
        } else {
            for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
                float v = to_f<TX>(xr[c]);
                if (d1 != nullptr) {
                    float d = to_f<T>(d1[base + c]);
                    if (d2 != nullptr) d = __fadd_rn(d, to_f<T>(d2[base + c]));
                    v = rnd<TX>(__fadd_rn(v, d));
                    xr[c] = from_f<TX>(v);
                }
                ss = fmaf(v, v, ss);
            }
        }
        ss = block_sum(ss, red);
        const float rstd = 1.0f / sqrtf(ss / (float)gw + eps);
        if (VEC) {
            for (int c = c0 + 4 * threadIdx.x; c < c1; c += 4 * blockDim.x) {   // the thread's own four values again: still in L1
                const float4 v = load4(xr + c), w4 = load4(weight + c);
                store4(out + base + c, make_float4(__fmul_rn(__fmul_rn(v.x, rstd), w4.x), __fmul_rn(__fmul_rn(v.y, rstd), w4.y),
                                                   __fmul_rn(__fmul_rn(v.z, rstd), w4.z), __fmul_rn(__fmul_rn(v.w, rstd), w4.w)));
            }
        } else {
            for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x)
                out[base + c] = from_f<T>(__fmul_rn(__fmul_rn(to_f<TX>(xr[c]), rstd), to_f<W>(weight[c])));
        }
    }
}

// g' = min(g, limit), u' = clamp(u, -limit, limit); out = g' * sigmoid(alpha * g') * (u' + 1).  gu holds [g | u].
template <class T>
__global__ void gated_clamp_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, float alpha, float limit) {
    pdl_wait();
    const long long row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const float g = fminf(to_f<T>(gu[row * 2 * inter + c]), limit);
    const float u = fminf(fmaxf(to_f<T>(gu[row * 2 * inter + inter + c]), -limit), limit);
    out[row * inter + c] = from_f<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

// bfloat16 rows whose half-width is a multiple of 8: eight values per thread, 16-byte accesses.
__global__ void gated_clamp_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter, long long total8,
                                       float alpha, float limit) {
    pdl_wait();
    const int per_row = inter / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / per_row;
        const int c = (int)(i % per_row) * 8;
        const uint4 graw = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + c);
        const uint4 uraw = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter + c);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 res;
        __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 gf = __bfloat1622float2(gh[e]), uf = __bfloat1622float2(uh[e]);
            const float g0 = fminf(gf.x, limit), g1 = fminf(gf.y, limit);
            const float u0 = fminf(fmaxf(uf.x, -limit), limit), u1 = fminf(fmaxf(uf.y, -limit), limit);
            rh[e] = __floats2bfloat162_rn(g0 / (1.0f + expf(-alpha * g0)) * (u0 + 1.0f), g1 / (1.0f + expf(-alpha * g1)) * (u1 + 1.0f));
        }
        *reinterpret_cast<uint4*>(out + row * inter + c) = res;
    }
}

template <class T>
__global__ void tanh_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f<T>(tanhf(to_f<T>(x[i])));
}

extern "C" {

int sb_embed_wide(const int* tokens, const void* table, void* out, int rows, int hidden, int vocab, int* status,
                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    sb_launch(embed_wide_kernel, rows, hidden >= 1024 ? 256 : 128, 0, stream, tokens, (const __nv_bfloat16*)table, (float*)out,
              hidden, vocab, status);
    SB_LAUNCH_CHECK();
}

// x_dtype: type of x (the residual); dtype: type of the deltas and of out; w_dtype: type of the weight.
int sb_grouped_rmsnorm(int x_dtype, int dtype, int w_dtype, void* x, const void* d1, const void* d2, const void* weight, void* out,
                       int rows, int width, int groups, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (groups < 1 || width % groups) return (int)cudaErrorInvalidValue;
    const int gw = width / groups;
    const bool vec = gw % 4 == 0;
    int threads = vec ? (gw / 4 + 31) / 32 * 32 : (gw >= 1024 ? 256 : 128);
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
    typedef __nv_bfloat16 bf;
#define SB_GN(TX, T, W)                                                                                                        \
    do {                                                                                                                       \
        if (vec)                                                                                                               \
            sb_launch(grouped_rmsnorm_kernel<TX, T, W, true>, rows, threads, 0, stream, (TX*)x, (const T*)d1, (const T*)d2,    \
                      (const W*)weight, (T*)out, width, groups, eps);                                                          \
        else                                                                                                                   \
            sb_launch(grouped_rmsnorm_kernel<TX, T, W, false>, rows, threads, 0, stream, (TX*)x, (const T*)d1, (const T*)d2,   \
                      (const W*)weight, (T*)out, width, groups, eps);                                                          \
    } while (0)
    if (x_dtype == SB_F32 && dtype == SB_F32 && w_dtype == SB_F32) SB_GN(float, float, float);
    else if (x_dtype == SB_F32 && dtype == SB_BF16 && w_dtype == SB_BF16) SB_GN(float, bf, bf);
    else if (x_dtype == SB_F32 && dtype == SB_BF16 && w_dtype == SB_F32) SB_GN(float, bf, float);
    else if (x_dtype == SB_BF16 && dtype == SB_BF16 && w_dtype == SB_BF16) SB_GN(bf, bf, bf);
    else if (x_dtype == SB_BF16 && dtype == SB_BF16 && w_dtype == SB_F32) SB_GN(bf, bf, float);
    else return (int)cudaErrorInvalidValue;
#undef SB_GN
    SB_LAUNCH_CHECK();
}

int sb_gated_clamp(int dtype, const void* gu, void* out, int rows, int inter, float alpha, float limit, cudaStream_t stream) {
    if (rows <= 0 || inter <= 0) return 0;
    if (dtype == SB_BF16 && inter % 8 == 0) {
        const long long total8 = (long long)rows * (inter / 8);
        const int blocks = (int)((total8 + 255) / 256 < 8192 ? (total8 + 255) / 256 : 8192);
        sb_launch(gated_clamp_vec_kernel, blocks, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total8, alpha, limit);
        SB_LAUNCH_CHECK();
    }
    dim3 grid(rows, (inter + 255) / 256);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == SB_F32)
        sb_launch(gated_clamp_kernel<float>, grid, 256, 0, stream, (const float*)gu, (float*)out, inter, alpha, limit);
    else
        sb_launch(gated_clamp_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter,
                  alpha, limit);
    SB_LAUNCH_CHECK();
}

int sb_tanh(int dtype, const void* x, void* out, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (dtype == SB_F32)
        sb_launch(tanh_kernel<float>, blocks, 256, 0, stream, (const float*)x, (float*)out, n);
    else
        sb_launch(tanh_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
