// Gated linear attention: the recurrence over a sequence's rows, with the head's norm and the gate in its epilogue.
//
//   a_t = sigmoid(z_t + bias) ** (1 / tau)                      (a decay per key channel)
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,    o_t = S_t^T (q_t * q_scale)
//   y_t = o_t / sqrt(mean(o_t^2) + eps) * norm * silu(g_t)      (per head, over the value channels)
//
// A sequence's record in the state group is [heads][key channel][value channel] floats.  The kernel walks a
// sequence's rows in order from the record and writes it back, so a step of many tokens leaves what the same tokens
// would leave one by one.  State, the logarithm of the sigmoid, the division by tau, the exponential, the unit norm and
// the gate are 32-bit; q, k, v, g come in the run's type as views of wider rows, z in 32-bit.
#include "common.cuh"

#define GLA_TB 32   // tokens whose q, k, v, decay and gate are staged in shared memory at a time
#define GLA_IG 8    // threads that share a value channel: each holds ceil(D / 8) key channels of that column of the state

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
    // log(sigmoid(z)) = -softplus(-z), taken on the side that does not overflow
    const float ls = z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
    return expf(ls * inv_tau);
}

// One block per (sequence, head).  Thread (jg, ig) owns, in registers, the state's entries S[i][j] for the E = ceil(D / 8)
// key channels i = ig * E .. and the CJ value channels j = jg, jg + JG, ...  (JG = threads / 8).  The eight threads of a
// column are neighbouring lanes and add their shares of o_t[j] with three shuffles.  Every entry of the state is a
// recurrence of its own, so the walk over a sequence's tokens costs a few dependent operations per token.
template <class T, int EMAX, int CJ>
__global__ void __launch_bounds__(CJ == 1 ? 1024 : 512)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g, long long ld,
                const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ norm_w, float eps,
                float inv_tau, float q_scale, float* __restrict__ state, long long state_stride, SbBatch batch, int H, int D, int V,
                T* __restrict__ y) {
    extern __shared__ float sm[];
    float* qs = sm;                  // [GLA_TB][D]
    float* ks = qs + GLA_TB * D;
    float* as = ks + GLA_TB * D;
    float* vs = as + GLA_TB * D;     // [GLA_TB][V]
    float* os = vs + GLA_TB * V;
    float* gs = os + GLA_TB * V;     // silu(g)
    float* bs = gs + GLA_TB * V;     // [D]
    __shared__ float rstd_s[GLA_TB];
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, n_threads = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, n_warps = n_threads >> 5;
    const int JG = n_threads / GLA_IG, jg = tid / GLA_IG, ig = tid % GLA_IG;
    const int E = (D + GLA_IG - 1) / GLA_IG, i0 = ig * E;
    for (int i = tid; i < D; i += n_threads) bs[i] = bias[head * D + i];   // weights: they do not depend on the kernel before
    pdl_wait();
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    float* Sg = state + (long long)slot * state_stride + (long long)head * D * V;
    float S[EMAX][CJ];
#pragma unroll
    for (int e = 0; e < EMAX; ++e)
#pragma unroll
        for (int c = 0; c < CJ; ++c) {
            const int j = jg + c * JG;
            S[e][c] = (j < V && e < E && i0 + e < D) ? Sg[(long long)(i0 + e) * V + j] : 0.f;
        }
    for (int t0 = row0; t0 < row1; t0 += GLA_TB) {
        const int nt = min(GLA_TB, row1 - t0);
        __syncthreads();
#pragma unroll 2
        for (int e = tid; e < nt * D; e += n_threads) {
            const int tt = e / D, i = e - tt * D;
            const long long at = (long long)(t0 + tt) * ld + head * D + i;
            qs[e] = to_f<T>(q[at]) * q_scale;
            ks[e] = to_f<T>(k[at]);
            as[e] = z[(long long)(t0 + tt) * H * D + head * D + i];
        }
#pragma unroll 1
        for (int e = tid; e < nt * D; e += n_threads) as[e] = decay_of(as[e] + bs[e % D], inv_tau);   // the thread's own entries
#pragma unroll 2
        for (int e = tid; e < nt * V; e += n_threads) {
            const int tt = e / V, j = e - tt * V;
            const long long at = (long long)(t0 + tt) * ld + head * V + j;
            const float gv = to_f<T>(g[at]);
            vs[e] = to_f<T>(v[at]);
            gs[e] = gv / (1.0f + expf(-gv));
        }
        __syncthreads();
#pragma unroll 1
        for (int tt = 0; tt < nt; ++tt) {
            float vj[CJ], o[CJ];
#pragma unroll
            for (int c = 0; c < CJ; ++c) {
                const int j = jg + c * JG;
                vj[c] = j < V ? vs[tt * V + j] : 0.f;
                o[c] = 0.f;
            }
            const float* qt = qs + tt * D + i0;
            const float* kt = ks + tt * D + i0;
            const float* at = as + tt * D + i0;
#pragma unroll
            for (int e = 0; e < EMAX; ++e) {
                if (e < E && i0 + e < D) {
                    const float qe = qt[e], ke = kt[e], ae = at[e];
#pragma unroll
                    for (int c = 0; c < CJ; ++c) {
                        S[e][c] = fmaf(ae, S[e][c], ke * vj[c]);
                        o[c] = fmaf(qe, S[e][c], o[c]);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < CJ; ++c) {
                o[c] += __shfl_xor_sync(0xffffffffu, o[c], 1);
                o[c] += __shfl_xor_sync(0xffffffffu, o[c], 2);
                o[c] += __shfl_xor_sync(0xffffffffu, o[c], 4);
                const int j = jg + c * JG;
                if (ig == 0 && j < V) os[tt * V + j] = o[c];
            }
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += n_warps) {   // the head's root mean square, a warp per token
            float ss = 0.f;
            for (int c = lane; c < V; c += 32) ss = fmaf(os[tt * V + c], os[tt * V + c], ss);
            ss = warp_sum(ss);
            if (lane == 0) rstd_s[tt] = 1.0f / sqrtf(ss / (float)V + eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * V; e += n_threads) {
            const int tt = e / V, c = e - tt * V;
            y[((long long)(t0 + tt) * H + head) * V + c] = from_f<T>(os[e] * rstd_s[tt] * norm_w[c] * gs[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < EMAX; ++e)
#pragma unroll
        for (int c = 0; c < CJ; ++c) {
            const int j = jg + c * JG;
            if (j < V && e < E && i0 + e < D) Sg[(long long)(i0 + e) * V + j] = S[e][c];
        }
}

// Heads beyond what the kernel above holds in registers: the state stays in global memory (it is the sequence's record
// anyway), thread j owns value channel j and walks the key channels of its column token by token.  Slow and plain.
template <class T>
__global__ void gla_scan_wide_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                                     long long ld, const float* __restrict__ z, const float* __restrict__ bias,
                                     const float* __restrict__ norm_w, float eps, float inv_tau, float q_scale,
                                     float* __restrict__ state, long long state_stride, SbBatch batch, int H, int D, int V,
                                     T* __restrict__ y) {
    extern __shared__ float sm[];
    float* qs = sm;          // the token's q, k and decay, [D] each
    float* ks = qs + D;
    float* as = ks + D;
    float* os = as + D;      // the token's raw outputs [V]
    __shared__ float red[33];
    pdl_wait();
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    float* Sg = state + (long long)slot * state_stride + (long long)head * D * V;
    for (int t = row0; t < row1; ++t) {
        __syncthreads();
        for (int i = tid; i < D; i += blockDim.x) {
            const long long at = (long long)t * ld + head * D + i;
            qs[i] = to_f<T>(q[at]) * q_scale;
            ks[i] = to_f<T>(k[at]);
            as[i] = decay_of(z[(long long)t * H * D + head * D + i] + bias[head * D + i], inv_tau);
        }
        __syncthreads();
        float ss = 0.f;
        for (int j = tid; j < V; j += blockDim.x) {   // the same thread owns column j at every token
            const float vj = to_f<T>(v[(long long)t * ld + head * V + j]);
            float o = 0.f;
            for (int i = 0; i < D; ++i) {
                const float nv = fmaf(as[i], Sg[(long long)i * V + j], ks[i] * vj);
                Sg[(long long)i * V + j] = nv;
                o = fmaf(qs[i], nv, o);
            }
            os[j] = o;
            ss = fmaf(o, o, ss);
        }
        ss = block_sum(ss, red);
        const float rstd = 1.0f / sqrtf(ss / (float)V + eps);
        for (int j = tid; j < V; j += blockDim.x) {
            const float gv = to_f<T>(g[(long long)t * ld + head * V + j]);
            y[((long long)t * H + head) * V + j] = from_f<T>(os[j] * rstd * norm_w[j] * (gv / (1.0f + expf(-gv))));
        }
    }
}

extern "C" {

// q, k [rows, H * D], v, g [rows, H * V]: views whose rows are `ld` elements apart; z [rows, H * D] 32-bit, contiguous;
// state [slots][H * D * V] with `state_stride` floats between slots; y [rows, H * V] contiguous.
int sb_gla_scan(int dtype, const void* q, const void* k, const void* v, const void* g, long long ld, const float* z, const float* bias,
                const float* norm_w, float eps, float tau, float q_scale, float* state, long long state_stride, SbBatch batch, int H,
                int D, int V, void* y, cudaStream_t stream) {
    if (batch.n_seqs <= 0 || batch.n_rows <= 0) return 0;
    if (D < 1 || V < 1 || D > 4096 || V > 4096 || H > 65535 || !(tau > 0.f)) return (int)cudaErrorInvalidValue;
    const float inv_tau = 1.0f / tau;
    dim3 grid(batch.n_seqs, H);
    typedef __nv_bfloat16 bf;
    const size_t smem = (size_t)(GLA_TB * (3 * D + 3 * V) + D) * sizeof(float);
    if (D > 128 || V > 256 || smem > 200 * 1024) {
        const int wt = V < 1024 ? (V + 31) / 32 * 32 : 1024;
        const size_t wsmem = (size_t)(3 * D + V) * sizeof(float);
        if (dtype == SB_F32)
            sb_launch(gla_scan_wide_kernel<float>, grid, wt, wsmem, stream, (const float*)q, (const float*)k, (const float*)v,
                      (const float*)g, ld, z, bias, norm_w, eps, inv_tau, q_scale, state, state_stride, batch, H, D, V, (float*)y);
        else
            sb_launch(gla_scan_wide_kernel<bf>, grid, wt, wsmem, stream, (const bf*)q, (const bf*)k, (const bf*)v, (const bf*)g, ld, z,
                      bias, norm_w, eps, inv_tau, q_scale, state, state_stride, batch, H, D, V, (bf*)y);
        SB_LAUNCH_CHECK();
    }
    const int cj = V <= 128 ? 1 : 4;   // a column per thread up to 1024 threads, four beyond (512 threads)
    const int threads = ((V + cj - 1) / cj * GLA_IG + 31) / 32 * 32;
#define SB_GLA(T, EMAX, CJ)                                                                                                       \
    do {                                                                                                                          \
        if (smem > 48 * 1024) {                                                                                                   \
            const cudaError_t err = cudaFuncSetAttribute(gla_scan_kernel<T, EMAX, CJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                         (int)smem);                                                              \
            if (err != cudaSuccess) return (int)err;                                                                              \
        }                                                                                                                         \
        sb_launch(gla_scan_kernel<T, EMAX, CJ>, grid, threads, smem, stream, (const T*)q, (const T*)k, (const T*)v, (const T*)g, ld, z, \
                  bias, norm_w, eps, inv_tau, q_scale, state, state_stride, batch, H, D, V, (T*)y);                               \
    } while (0)
#define SB_GLA_E(T, CJ)                          \
    do {                                         \
        if (D <= 32) SB_GLA(T, 4, CJ);           \
        else if (D <= 64) SB_GLA(T, 8, CJ);      \
        else SB_GLA(T, 16, CJ);                  \
    } while (0)
#define SB_GLA_SIZES(T)                          \
    do {                                         \
        if (cj == 1) SB_GLA_E(T, 1);             \
        else SB_GLA_E(T, 4);                     \
    } while (0)
    if (dtype == SB_F32) SB_GLA_SIZES(float);
    else SB_GLA_SIZES(bf);
#undef SB_GLA_SIZES
#undef SB_GLA_E
#undef SB_GLA
    SB_LAUNCH_CHECK();
}

}  // extern "C"
