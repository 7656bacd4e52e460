// Attention with options on the score and the mask, over a paged cache whose keys and values may have different
// widths, and the kernels that fill such a cache.
//
//   score(i, j) = (q_i . k_j) * scale * head_scale[h]  -  slope[h] * (i - j)
//   visible:      j <= i,  i - j < window (if any),  i / chunk == j / chunk (if any)
//   weights:      softmax over the visible keys; with a sink s_h the denominator holds exp(s_h) once more
//
// Scores, the running maximum, the exponentials, the weights and the sums over values are 32-bit in every run:
// a weight is not rounded before it meets its value.  Values are read from their own pages, or out of the key rows
// (their first v_dim columns) for a cache that keeps one row per token for both.
//
// This file holds the general kernel (a warp per row and query head, keys 32 at a time in order of position: a
// row's result depends on its position and its keys only); attention_flex_mma.cu holds the tensor-core kernels.
#include "attention_flex.cuh"

template <class T> __device__ __forceinline__ float dot_cols(const float* qs, const T* kr, int D);
template <> __device__ __forceinline__ float dot_cols<float>(const float* qs, const float* kr, int D) {
    float dot = 0.f;
    if ((D & 3) == 0) {
        for (int d = 0; d < D; d += 4) {
            const float4 v = *reinterpret_cast<const float4*>(kr + d);
            dot = fmaf(qs[d], v.x, dot);
            dot = fmaf(qs[d + 1], v.y, dot);
            dot = fmaf(qs[d + 2], v.z, dot);
            dot = fmaf(qs[d + 3], v.w, dot);
        }
    } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], kr[d], dot);
    }
    return dot;
}
template <> __device__ __forceinline__ float dot_cols<__nv_bfloat16>(const float* qs, const __nv_bfloat16* kr, int D) {
    float dot = 0.f;
    if ((D & 7) == 0) {
        for (int d = 0; d < D; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                dot = fmaf(qs[d + 2 * e], f.x, dot);
                dot = fmaf(qs[d + 2 * e + 1], f.y, dot);
            }
        }
    } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], __bfloat162float(kr[d]), dot);
    }
    return dot;
}

template <class T>
__global__ void flex_attention_general_kernel(SbFlex p, SbBatch batch, T* __restrict__ out) {
    extern __shared__ float qs[];
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int kvh = head / (p.n_heads / p.n_kv_heads);
    int slot, pos;
    row_place(batch, row, slot, pos);
    const int lo = flex_first_key(p, pos);
    const T* qr = (const T*)p.q + (long long)row * p.q_row + (long long)head * p.q_head;
    for (int d = lane; d < p.k_dim; d += 32) qs[d] = to_f<T>(qr[d]);
    __syncwarp();
    const float hs = p.head_scale != nullptr ? p.scale * p.head_scale[head] : p.scale;
    const float slope = p.slopes != nullptr ? p.slopes[head] : 0.f;

    float m = -INFINITY, l = 0.f;
    float acc[FLEX_MAX_V / 32];
#pragma unroll
    for (int j = 0; j < FLEX_MAX_V / 32; ++j) acc[j] = 0.f;
    const T* kbase = (const T*)p.k;
    const T* vbase = (const T*)p.v;
    for (int n0 = (lo / 32) * 32; n0 <= pos; n0 += 32) {
        const int n = n0 + lane;
        const long long tok = (n >= lo && n <= pos) ? flex_token(p, slot, n, kvh) : -1;
        float s = -INFINITY;
        if (tok >= 0) s = dot_cols<T>(qs, kbase + tok * p.k_dim, p.k_dim) * hs - slope * (float)(pos - n);
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;
        const float w = tok >= 0 ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(w);
        m = m_new;
#pragma unroll
        for (int j = 0; j < FLEX_MAX_V / 32; ++j) acc[j] *= alpha;
        const long long vtok = flex_value_token(p, tok, kvh);
        for (int t = 0; t < 32; ++t) {
            const long long vt = __shfl_sync(0xffffffffu, vtok, t);
            const float wt = __shfl_sync(0xffffffffu, w, t);
            if (vt < 0) continue;
            const T* vr = vbase + vt * p.v_row;
#pragma unroll
            for (int j = 0; j < FLEX_MAX_V / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < p.v_dim) acc[j] = fmaf(wt, to_f<T>(vr[d]), acc[j]);
            }
        }
    }
    if (p.sink != nullptr) {   // one more term in the denominator, no value behind it
        const float sk = p.sink[head];
        const float m_new = fmaxf(m, sk);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int j = 0; j < FLEX_MAX_V / 32; ++j) acc[j] *= alpha;
    }
    T* orow = out + ((long long)row * p.n_heads + head) * p.v_dim;
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < FLEX_MAX_V / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < p.v_dim) orow[d] = from_f<T>(acc[j] * inv);
    }
}

// One block per row, one warp per key/value head at a time: the key is copied, the value is divided by its root
// mean square over v_dim (when norm is set) and both go to the row's place in the cache.
template <class T>
__global__ void kv_store_kernel(const T* __restrict__ k, long long k_row, const T* __restrict__ v, long long v_row, SbBatch batch,
                                SbFlex p, int norm, float eps, int* status) {
    pdl_wait();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    int slot, pos;
    row_place(batch, row, slot, pos);
    for (int g = warp; g < p.n_kv_heads; g += n_warps) {
        const long long tok = flex_token(p, slot, pos, g);
        if (tok < 0) {
            if (lane == 0) atomicOr(status, SB_STATUS_NO_PAGE);
            continue;
        }
        const T* ks = k + row * k_row + (long long)g * p.k_dim;
        T* kd = (T*)p.k + tok * p.k_dim;
        for (int d = lane; d < p.k_dim; d += 32) kd[d] = ks[d];
        const T* vs = v + row * v_row + (long long)g * p.v_dim;
        T* vd = (T*)p.v + tok * p.v_row;
        float rstd = 1.f;
        if (norm) {
            float ss = 0.f;
            for (int d = lane; d < p.v_dim; d += 32) {
                const float x = to_f<T>(vs[d]);
                ss = fmaf(x, x, ss);
            }
            ss = warp_sum(ss);
            rstd = 1.0f / sqrtf(ss / (float)p.v_dim + eps);
        }
        for (int d = lane; d < p.v_dim; d += 32) vd[d] = norm ? from_f<T>(to_f<T>(vs[d]) * rstd) : vs[d];
    }
}

// Columns [0, rot) of every head turn in neighbouring pairs by position * freqs[pair]; later columns are copied.
// angle, sine and cosine are 32-bit.
template <class T>
__global__ void rotate_pairs_kernel(const T* __restrict__ src, long long s_row, long long s_head, T* __restrict__ dst, long long d_row,
                                    long long d_head, SbBatch batch, const float* __restrict__ freqs, int n_heads, int cols, int rot) {
    pdl_wait();
    const int row = blockIdx.x;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const int half = rot / 2, per_head = half + (cols - rot);
    for (int e = threadIdx.x; e < n_heads * per_head; e += blockDim.x) {
        const int h = e / per_head, c = e % per_head;
        const T* s = src + row * s_row + h * s_head;
        T* d = dst + row * d_row + h * d_head;
        if (c < half) {
            float sn, cs;
            sincosf((float)pos * freqs[c], &sn, &cs);
            const float a = to_f<T>(s[2 * c]), b = to_f<T>(s[2 * c + 1]);
            d[2 * c] = from_f<T>(a * cs - b * sn);
            d[2 * c + 1] = from_f<T>(b * cs + a * sn);
        } else {
            d[rot + c - half] = s[rot + c - half];
        }
    }
}

// One block per row of down = [query latent (q_rank) | key/value latent (kv_rank) | shared rotated part (rot_dim)]:
// the query latent normed into cq, the key/value latent normed and the shared part rotated into the row's one
// cache row [kv_rank + rot_dim]; the same row also into row_out [rows, kv_rank + rot_dim] when that is given.
template <class T, class W>
__global__ void latent_prepare_kernel(const T* __restrict__ down, T* __restrict__ cq, SbBatch batch, SbFlex p, int q_rank, int kv_rank,
                                      int rot_dim, const W* __restrict__ q_norm, const W* __restrict__ kv_norm, float eps,
                                      const float* __restrict__ freqs, int rot, int* status, T* __restrict__ row_out) {
    __shared__ float red[33];
    pdl_wait();
    const int row = blockIdx.x;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const T* dr = down + (long long)row * (q_rank + kv_rank + rot_dim);
    T* ro = row_out != nullptr ? row_out + (long long)row * (kv_rank + rot_dim) : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
        const float x = to_f<T>(dr[c]);
        ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, red);
    float rstd = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
        cq[(long long)row * q_rank + c] = from_f<T>(__fmul_rn(__fmul_rn(to_f<T>(dr[c]), rstd), to_f<W>(q_norm[c])));
    const long long tok = flex_token(p, slot, pos, 0);
    ss = 0.f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const float x = to_f<T>(dr[q_rank + c]);
        ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, red);
    if (tok < 0) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_NO_PAGE);
        return;
    }
    rstd = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    T* kd = (T*)p.k + tok * p.k_dim;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const T val = from_f<T>(__fmul_rn(__fmul_rn(to_f<T>(dr[q_rank + c]), rstd), to_f<W>(kv_norm[c])));
        kd[c] = val;
        if (ro != nullptr) ro[c] = val;
    }
    const T* sr = dr + q_rank + kv_rank;
    const int half = rot / 2;
    for (int c = threadIdx.x; c < half + (rot_dim - rot); c += blockDim.x) {
        if (c < half) {
            float sn, cs;
            sincosf((float)pos * freqs[c], &sn, &cs);
            const float a = to_f<T>(sr[2 * c]), b = to_f<T>(sr[2 * c + 1]);
            const T x = from_f<T>(a * cs - b * sn), y = from_f<T>(b * cs + a * sn);
            kd[kv_rank + 2 * c] = x;
            kd[kv_rank + 2 * c + 1] = y;
            if (ro != nullptr) {
                ro[kv_rank + 2 * c] = x;
                ro[kv_rank + 2 * c + 1] = y;
            }
        } else {
            kd[kv_rank + rot + c - half] = sr[rot + c - half];
            if (ro != nullptr) ro[kv_rank + rot + c - half] = sr[rot + c - half];
        }
    }
}

extern "C" {

int sb_flex_attention_general(int dtype, SbFlex p, SbBatch batch, void* out, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (p.v_dim > FLEX_MAX_V || p.n_heads % p.n_kv_heads || p.k_dim > 8192) return (int)cudaErrorInvalidValue;
    dim3 grid(batch.n_rows, p.n_heads);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)p.k_dim * sizeof(float);
    if (dtype == SB_F32)
        sb_launch(flex_attention_general_kernel<float>, grid, 32, smem, stream, p, batch, (float*)out);
    else
        sb_launch(flex_attention_general_kernel<__nv_bfloat16>, grid, 32, smem, stream, p, batch, (__nv_bfloat16*)out);
    SB_LAUNCH_CHECK();
}

int sb_kv_store(int dtype, const void* k, long long k_row, const void* v, long long v_row, SbBatch batch, SbFlex p, int norm, float eps,
                int* status, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    const int threads = 32 * (p.n_kv_heads < 8 ? p.n_kv_heads : 8);
    if (dtype == SB_F32)
        sb_launch(kv_store_kernel<float>, batch.n_rows, threads, 0, stream, (const float*)k, k_row, (const float*)v, v_row, batch, p,
                  norm, eps, status);
    else
        sb_launch(kv_store_kernel<__nv_bfloat16>, batch.n_rows, threads, 0, stream, (const __nv_bfloat16*)k, k_row,
                  (const __nv_bfloat16*)v, v_row, batch, p, norm, eps, status);
    SB_LAUNCH_CHECK();
}

int sb_rotate_pairs(int dtype, const void* src, long long s_row, long long s_head, void* dst, long long d_row, long long d_head,
                    SbBatch batch, const float* freqs, int n_heads, int cols, int rot, cudaStream_t stream) {
    if (batch.n_rows <= 0 || cols <= 0) return 0;
    if (rot < 0 || rot > cols || rot % 2) return (int)cudaErrorInvalidValue;
    if (dtype == SB_F32)
        sb_launch(rotate_pairs_kernel<float>, batch.n_rows, 128, 0, stream, (const float*)src, s_row, s_head, (float*)dst, d_row, d_head,
                  batch, freqs, n_heads, cols, rot);
    else
        sb_launch(rotate_pairs_kernel<__nv_bfloat16>, batch.n_rows, 128, 0, stream, (const __nv_bfloat16*)src, s_row, s_head,
                  (__nv_bfloat16*)dst, d_row, d_head, batch, freqs, n_heads, cols, rot);
    SB_LAUNCH_CHECK();
}

int sb_latent_prepare(int dtype, int w_dtype, const void* down, void* cq, SbBatch batch, SbFlex p, int q_rank, int kv_rank, int rot_dim,
                      const void* q_norm, const void* kv_norm, float eps, const float* freqs, int rot, int* status, void* row_out,
                      cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (rot < 0 || rot > rot_dim || rot % 2 || p.k_dim != kv_rank + rot_dim) return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf;
#define SB_LP(T, W)                                                                                                          \
    sb_launch(latent_prepare_kernel<T, W>, batch.n_rows, 128, 0, stream, (const T*)down, (T*)cq, batch, p, q_rank, kv_rank, rot_dim, \
              (const W*)q_norm, (const W*)kv_norm, eps, freqs, rot, status, (T*)row_out)
    if (dtype == SB_F32 && w_dtype == SB_F32) SB_LP(float, float);
    else if (dtype == SB_BF16 && w_dtype == SB_BF16) SB_LP(bf, bf);
    else if (dtype == SB_BF16 && w_dtype == SB_F32) SB_LP(bf, float);
    else return (int)cudaErrorInvalidValue;
#undef SB_LP
    SB_LAUNCH_CHECK();
}

}  // extern "C"
