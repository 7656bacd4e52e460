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

#define GLA_VB 64   // value channels (columns of the state) per block

// One block per (sequence, head, group of GLA_VB value channels), 8 threads per value channel.  Thread (jl, ig) owns, in
// registers, the state's entries S[i][j] of its column j for E = ceil(D / 8) key channels.  The eight threads of a column
// are neighbouring lanes and add their shares of o_t[j] with three shuffles.  Every entry of the state is a recurrence
// of its own, so the walk over a sequence's tokens costs a few dependent operations per token; four tokens are unrolled
// so that one token's shuffles overlap the next tokens' products.  EXACT: D = 8 * EMAX, so no entry needs a bounds test
// and q, k and the decay are read 16 bytes at a time; a thread's key channels are then dealt out four at a time,
// ((e / 4) * 8 + ig) * 4 + e % 4, so that the eight lanes of a column read 128 consecutive bytes.  Columns are
// independent of one another, so a head's columns may be shared out over several blocks; the head's norm then runs in
// gla_finish_kernel from the raw outputs in o_raw (null: one block holds all columns and norms them itself).
template <class T, int EMAX, bool EXACT>
__global__ void __launch_bounds__(GLA_VB * GLA_IG)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g, long long ld,
                const float* __restrict__ z, const float* __restrict__ bias, const float* __restrict__ norm_w, float eps,
                float inv_tau, float q_scale, float* __restrict__ state, long long state_stride, SbBatch batch, int H, int D, int V,
                T* __restrict__ y, float* __restrict__ o_raw) {
    extern __shared__ float sm[];
    float* qs = sm;                  // [GLA_TB][D]
    float* ks = qs + GLA_TB * D;
    float* as = ks + GLA_TB * D;
    float* vs = as + GLA_TB * D;     // [GLA_TB][GLA_VB]
    float* os = vs + GLA_TB * GLA_VB;
    float* gs = os + GLA_TB * GLA_VB;   // silu(g)
    float* bs = gs + GLA_TB * GLA_VB;   // [D]
    __shared__ float rstd_s[GLA_TB];
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, n_threads = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, n_warps = n_threads >> 5;
    const int j0 = blockIdx.z * GLA_VB, nv = min(GLA_VB, V - j0);
    const int jl = tid / GLA_IG, ig = tid % GLA_IG, j = j0 + jl;
    const bool col = jl < nv;
    const int E = (D + GLA_IG - 1) / GLA_IG, i0 = ig * E;
    auto chan = [&](int e) { return EXACT ? ((e >> 2) * GLA_IG + ig) * 4 + (e & 3) : i0 + e; };   // key channel of entry e
    for (int i = tid; i < D; i += n_threads) bs[i] = bias[head * D + i];   // weights: they do not depend on the kernel before
    pdl_wait();
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    float* Sg = state + (long long)slot * state_stride + (long long)head * D * V;
    float S[EMAX];
#pragma unroll
    for (int e = 0; e < EMAX; ++e) S[e] = (col && e < E && chan(e) < D) ? Sg[(long long)chan(e) * V + j] : 0.f;
    for (int t0 = row0; t0 < row1; t0 += GLA_TB) {
        const int nt = min(GLA_TB, row1 - t0);
        __syncthreads();
#pragma unroll 4
        for (int e = tid; e < nt * D; e += n_threads) {   // unrolled: the loads of four turns are in flight together
            const int tt = EXACT ? e / (8 * EMAX) : e / D, i = e - tt * D;   // an exact head size divides by a constant
            const long long at = (long long)(t0 + tt) * ld + head * D + i;
            qs[e] = to_f<T>(q[at]) * q_scale;
            ks[e] = to_f<T>(k[at]);
            as[e] = z[(long long)(t0 + tt) * H * D + head * D + i];
        }
#pragma unroll 4
        for (int e = tid; e < nt * nv; e += n_threads) {
            const int tt = e / nv, c = e - tt * nv;
            const long long at = (long long)(t0 + tt) * ld + head * V + j0 + c;
            vs[tt * GLA_VB + c] = to_f<T>(v[at]);
            if (o_raw == nullptr) {
                const float gv = to_f<T>(g[at]);
                gs[tt * GLA_VB + c] = gv / (1.0f + expf(-gv));
            }
        }
#pragma unroll 1
        for (int e = tid; e < nt * D; e += n_threads) as[e] = decay_of(as[e] + bs[EXACT ? e % (8 * EMAX) : e % D], inv_tau);   // the thread's own entries
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = col ? vs[tt * GLA_VB + jl] : 0.f;
            float o = 0.f;
            if (EXACT) {   // two entries of the state per instruction (fma.rn.f32x2): the time here is the instruction count
                constexpr int DC = 8 * EMAX;
                const float2 v2 = make_float2(vj, vj), zero = make_float2(0.f, 0.f);
                float2 o2 = zero;
#pragma unroll
                for (int e = 0; e < EMAX; e += 4) {
                    const int at = tt * DC + ((e >> 2) * GLA_IG + ig) * 4;
                    const float4 q4 = *reinterpret_cast<const float4*>(qs + at);
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + at);
                    const float4 a4 = *reinterpret_cast<const float4*>(as + at);
                    float2 s01 = make_float2(S[e], S[e + 1]), s23 = make_float2(S[e + 2], S[e + 3]);
                    s01 = fma_pair(make_float2(a4.x, a4.y), s01, fma_pair(make_float2(k4.x, k4.y), v2, zero));
                    s23 = fma_pair(make_float2(a4.z, a4.w), s23, fma_pair(make_float2(k4.z, k4.w), v2, zero));
                    o2 = fma_pair(make_float2(q4.x, q4.y), s01, o2);
                    o2 = fma_pair(make_float2(q4.z, q4.w), s23, o2);
                    S[e] = s01.x;
                    S[e + 1] = s01.y;
                    S[e + 2] = s23.x;
                    S[e + 3] = s23.y;
                }
                o = o2.x + o2.y;
            } else {
                const float* qt = qs + tt * D + i0;
                const float* kt = ks + tt * D + i0;
                const float* at = as + tt * D + i0;
#pragma unroll
                for (int e = 0; e < EMAX; ++e) {
                    if (e < E && i0 + e < D) {
                        S[e] = fmaf(at[e], S[e], kt[e] * vj);
                        o = fmaf(qt[e], S[e], o);
                    }
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            o += __shfl_xor_sync(0xffffffffu, o, 4);
            if (ig == 0 && col) os[tt * GLA_VB + jl] = o;
        }
        __syncthreads();
        if (o_raw != nullptr) {
            for (int e = tid; e < nt * nv; e += n_threads) {
                const int tt = e / nv, c = e - tt * nv;
                o_raw[((long long)(t0 + tt) * H + head) * V + j0 + c] = os[tt * GLA_VB + c];
            }
            continue;
        }
        for (int tt = warp; tt < nt; tt += n_warps) {   // the head's root mean square, a warp per token
            float ss = 0.f;
            for (int c = lane; c < nv; c += 32) ss = fmaf(os[tt * GLA_VB + c], os[tt * GLA_VB + c], ss);
            ss = warp_sum(ss);
            if (lane == 0) rstd_s[tt] = 1.0f / sqrtf(ss / (float)V + eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * nv; e += n_threads) {
            const int tt = e / nv, c = e - tt * nv;
            y[((long long)(t0 + tt) * H + head) * V + c] =
                from_f<T>(os[tt * GLA_VB + c] * rstd_s[tt] * norm_w[c] * gs[tt * GLA_VB + c]);
        }
    }
#pragma unroll
    for (int e = 0; e < EMAX; ++e)
        if (col && e < E && chan(e) < D) Sg[(long long)chan(e) * V + j] = S[e];
}

// One warp per (row, head): the head's unit norm over its V raw outputs, the norm weight and the gate.
template <class T>
__global__ void gla_finish_kernel(const float* __restrict__ o_raw, const T* __restrict__ g, long long ld, const float* __restrict__ norm_w,
                                  float eps, int rows, int H, int V, T* __restrict__ y) {
    pdl_wait();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)rows * H) return;
    const long long row = wid / H;
    const int head = (int)(wid % H);
    const float* o = o_raw + (row * H + head) * V;
    float ss = 0.f;
    for (int c = lane; c < V; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)V + eps);
    for (int c = lane; c < V; c += 32) {
        const float gv = to_f<T>(g[row * ld + head * V + c]);
        y[(row * H + head) * V + c] = from_f<T>(o[c] * rstd * norm_w[c] * (gv / (1.0f + expf(-gv))));
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
// state [slots][H * D * V] with `state_stride` floats between slots; y [rows, H * V] contiguous; o_raw: [rows, H * V]
// floats of scratch for heads of more than GLA_VB value channels (their columns are shared out over blocks).
int sb_gla_scan(int dtype, const void* q, const void* k, const void* v, const void* g, long long ld, const float* z, const float* bias,
                const float* norm_w, float eps, float tau, float q_scale, float* state, long long state_stride, SbBatch batch, int H,
                int D, int V, void* y, float* o_raw, cudaStream_t stream) {
    if (batch.n_seqs <= 0 || batch.n_rows <= 0) return 0;
    if (D < 1 || V < 1 || D > 4096 || V > 4096 || H > 65535 || !(tau > 0.f)) return (int)cudaErrorInvalidValue;
    const float inv_tau = 1.0f / tau;
    typedef __nv_bfloat16 bf;
    const size_t smem = (size_t)(GLA_TB * (3 * D + 3 * GLA_VB) + D) * sizeof(float);
    const int chunks = (V + GLA_VB - 1) / GLA_VB;
    if (D > 128 || chunks > 64 || (chunks > 1 && o_raw == nullptr)) {
        dim3 grid(batch.n_seqs, H);
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
    dim3 grid(batch.n_seqs, H, chunks);
    const int threads = (min(V, GLA_VB) * GLA_IG + 31) / 32 * 32;
    float* raw = chunks > 1 ? o_raw : nullptr;
#define SB_GLA(T, EMAX, EXACT)                                                                                                    \
    do {                                                                                                                          \
        if (smem > 48 * 1024) {                                                                                                   \
            const cudaError_t err = cudaFuncSetAttribute(gla_scan_kernel<T, EMAX, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                         (int)smem);                                                              \
            if (err != cudaSuccess) return (int)err;                                                                              \
        }                                                                                                                         \
        sb_launch(gla_scan_kernel<T, EMAX, EXACT>, grid, threads, smem, stream, (const T*)q, (const T*)k, (const T*)v, (const T*)g, ld, \
                  z, bias, norm_w, eps, inv_tau, q_scale, state, state_stride, batch, H, D, V, (T*)y, raw);                       \
    } while (0)
#define SB_GLA_SIZES(T)                              \
    do {                                             \
        if (D == 32) SB_GLA(T, 4, true);             \
        else if (D == 64) SB_GLA(T, 8, true);        \
        else if (D == 128) SB_GLA(T, 16, true);      \
        else if (D <= 32) SB_GLA(T, 4, false);       \
        else if (D <= 64) SB_GLA(T, 8, false);       \
        else SB_GLA(T, 16, false);                   \
    } while (0)
    if (dtype == SB_F32) SB_GLA_SIZES(float);
    else SB_GLA_SIZES(bf);
#undef SB_GLA_SIZES
#undef SB_GLA
    if (raw != nullptr) {
        const long long warps = (long long)batch.n_rows * H;
        const unsigned int blocks = (unsigned int)((warps * 32 + 255) / 256);
        if (dtype == SB_F32)
            sb_launch(gla_finish_kernel<float>, blocks, 256, 0, stream, (const float*)raw, (const float*)g, ld, norm_w, eps, batch.n_rows,
                      H, V, (float*)y);
        else
            sb_launch(gla_finish_kernel<bf>, blocks, 256, 0, stream, (const float*)raw, (const bf*)g, ld, norm_w, eps, batch.n_rows, H, V,
                      (bf*)y);
    }
    SB_LAUNCH_CHECK();
}

}  // extern "C"
