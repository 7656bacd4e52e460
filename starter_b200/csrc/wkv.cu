// The linear recurrence with a matrix state per head (the "wkv" mixer): the blends of a token's input with the
// previous token's, and the recurrence itself.
//
//   blend_m = n + (n' - n) * mu_m                                   n' = previous token's input, zeros at a sequence's start
//   out_t = (S + (u * k_t) v_t^T)^T r_t       S <- decay_t[:, None] * S + k_t v_t^T       decay_t = exp(-exp(pre_t + w0))
//   y_t = out_t / rms(out_t per head) * norm * silu(g_t)
//
// A sequence's record in the state group is [heads][key channel][value channel] floats, then the last token's
// input (32-bit).  The recurrence kernel walks a sequence's rows in order from the record and writes it back, so a
// step of many tokens leaves what the same tokens would leave one by one.  State, decay, the two exponentials, the
// unit norm and the gate are 32-bit; r, k, v, g come in the run's type.
#include "common.cuh"

// One block per row: out[m][row][c] = n + (prev - n) * mu[m][c], prev from the row before or, for a sequence's
// first row of the step, from the sequence's record.
template <class T, class W>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ state, long long state_stride, int prev_offset,
                                   const W* __restrict__ mu, int n_mix, SbBatch batch, int width, T* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int s = batch.row_seq[row];
    const bool first = row == batch.cu_q[s];
    const float* rec = state + (long long)batch.seq_slot[s] * state_stride + prev_offset;
    const T* cur = h + (long long)row * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float x = to_f<T>(cur[c]);
        const float before = first ? rec[c] : to_f<T>(cur[c - width]);
        const float d = before - x;
        for (int m = 0; m < n_mix; ++m)
            out[((long long)m * batch.n_rows + row) * width + c] = from_f<T>(fmaf(d, to_f<W>(mu[(long long)m * width + c]), x));
    }
}

// bfloat16 rows and blend vectors whose width is a multiple of 8: eight columns per thread, 16-byte accesses.
__global__ void token_shift_vec_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ state, long long state_stride,
                                       int prev_offset, const __nv_bfloat16* __restrict__ mu, int n_mix, SbBatch batch, int width,
                                       __nv_bfloat16* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int s = batch.row_seq[row];
    const bool first = row == batch.cu_q[s];
    const float* rec = state + (long long)batch.seq_slot[s] * state_stride + prev_offset;
    const __nv_bfloat16* cur = h + (long long)row * width;
    for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
        float x[8], d[8];
        const uint4 raw = *reinterpret_cast<const uint4*>(cur + c);
        const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(xh[e]);
            x[2 * e] = f.x;
            x[2 * e + 1] = f.y;
        }
        if (first) {
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] = rec[c + e] - x[e];
        } else {
            const uint4 praw = *reinterpret_cast<const uint4*>(cur + c - width);
            const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&praw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(ph[e]);
                d[2 * e] = f.x - x[2 * e];
                d[2 * e + 1] = f.y - x[2 * e + 1];
            }
        }
        for (int m = 0; m < n_mix; ++m) {
            const uint4 mraw = *reinterpret_cast<const uint4*>(mu + (long long)m * width + c);
            const __nv_bfloat162* mh = reinterpret_cast<const __nv_bfloat162*>(&mraw);
            uint4 res;
            __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(mh[e]);
                rh[e] = __floats2bfloat162_rn(fmaf(d[2 * e], f.x, x[2 * e]), fmaf(d[2 * e + 1], f.y, x[2 * e + 1]));
            }
            *reinterpret_cast<uint4*>(out + ((long long)m * batch.n_rows + row) * width + c) = res;
        }
    }
}

#define WKV_TB 32   // tokens whose r, k, v and decay are staged in shared memory at a time
#define WKV_IG 8    // threads that share a group of value channels: each holds D / 8 key channels of those columns of the state
#define WKV_CJ 1    // value channels (columns of the state) per thread

// One block per (sequence, head), ceil(D / WKV_CJ) * 8 threads.  Thread (jg, ig) owns the state's entries S[i][j] for the
// E = ceil(D / 8) key channels i = ig * E .. ig * E + E - 1 and the WKV_CJ value channels from j = WKV_CJ * jg on, in
// registers.  The eight threads of a column group are neighbouring lanes and add their shares of out_t[j] with three
// shuffles.  EXACT: D = 8 * EMAX, so no entry needs a bounds test and r, k and the decay are read 16 bytes at a time;
// a thread's key channels are then dealt out four at a time ((e / 4) * 8 + ig) * 4 + e % 4, so that the eight lanes
// of a group read 128 consecutive bytes (no bank conflict), and what a thread reads serves its four columns: measured
// on a B200 the shared-memory pipe, not arithmetic, bounds this kernel (a warp per column group re-reads r, k, decay).  Every entry of the state is a recurrence
// of its own, so the walk over a sequence's tokens costs a few dependent operations per token, whatever the head's size.
template <class T, int EMAX, bool EXACT>
__global__ void __launch_bounds__(EMAX * WKV_IG * WKV_IG / WKV_CJ)
wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                const float* __restrict__ decay_pre, const float* __restrict__ w0, const float* __restrict__ u,
                const float* __restrict__ norm_w, float eps, const T* __restrict__ h, int width, float* __restrict__ state,
                long long state_stride, int prev_offset, SbBatch batch, int H, int D, T* __restrict__ y) {
    extern __shared__ float sm[];
    float* rs = sm;                  // [WKV_TB][D]
    float* ks = rs + WKV_TB * D;
    float* ws = ks + WKV_TB * D;
    float* vs = ws + WKV_TB * D;
    float* os = vs + WKV_TB * D;
    float* gs = os + WKV_TB * D;     // silu(g)
    float* us = gs + WKV_TB * D;     // [D]
    float* w0s = us + D;             // [D]
    __shared__ float rstd_s[WKV_TB];
    __shared__ float bonus_s[WKV_TB];   // sum_i r_i u_i k_i of each staged token: the current token's own share, per unit of v_j
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, n_threads = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, n_warps = n_threads >> 5;
    const int j = (tid / WKV_IG) * WKV_CJ, ig = tid % WKV_IG;   // j: the first of this thread's four columns
    const int E = (D + WKV_IG - 1) / WKV_IG, i0 = ig * E;
    auto chan = [&](int e) { return EXACT ? ((e >> 2) * WKV_IG + ig) * 4 + (e & 3) : i0 + e; };   // key channel of entry e
    for (int i = tid; i < D; i += n_threads) {   // weights: they do not depend on the kernel before this one
        us[i] = u[head * D + i];
        w0s[i] = w0[head * D + i];
    }
    pdl_wait();
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    const int HD = H * D;
    float* Sg = state + (long long)slot * state_stride + (long long)head * D * D;
    float S[EMAX][WKV_CJ];
#pragma unroll
    for (int e = 0; e < EMAX; ++e)
#pragma unroll
        for (int c = 0; c < WKV_CJ; ++c) S[e][c] = (j + c < D && e < E && chan(e) < D) ? Sg[chan(e) * D + j + c] : 0.f;
    for (int t0 = row0; t0 < row1; t0 += WKV_TB) {
        const int nt = min(WKV_TB, row1 - t0);
        __syncthreads();
#pragma unroll 4
        for (int e = tid; e < nt * D; e += n_threads) {   // unrolled: the loads of four turns are in flight together
            const long long at = (long long)(t0 + e / D) * HD + head * D + e % D;
            const float gv = to_f<T>(g[at]);
            rs[e] = to_f<T>(r[at]);
            ks[e] = to_f<T>(k[at]);
            vs[e] = to_f<T>(v[at]);
            ws[e] = expf(-expf(decay_pre[at] + w0s[e % D]));
            gs[e] = gv / (1.0f + expf(-gv));
        }
        __syncthreads();
        // out_t[j] = sum_i r_i S[i][j] + v_j * sum_i r_i u_i k_i: the second sum is the same for every column
        for (int tt = warp; tt < nt; tt += n_warps) {
            float c = 0.f;
            for (int i = lane; i < D; i += 32) c = fmaf(rs[tt * D + i] * us[i], ks[tt * D + i], c);
            c = warp_sum(c);
            if (lane == 0) bonus_s[tt] = c;
        }
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {   // unrolled: a token's shuffles overlap the next tokens' products
            float vj[WKV_CJ], o[WKV_CJ];
#pragma unroll
            for (int c = 0; c < WKV_CJ; ++c) {
                vj[c] = (EXACT || j + c < D) ? vs[tt * D + j + c] : 0.f;
                o[c] = 0.f;
            }
            const float* rt = rs + tt * D + i0;
            const float* kt = ks + tt * D + i0;
            const float* wt = ws + tt * D + i0;
            if (EXACT) {   // 16-byte reads, the same address for the lanes of one key group
#pragma unroll
                for (int e = 0; e < EMAX; e += 4) {
                    {
                        const int at = tt * D + ((e >> 2) * WKV_IG + ig) * 4;
                        const float4 r4 = *reinterpret_cast<const float4*>(rs + at);
                        const float4 k4 = *reinterpret_cast<const float4*>(ks + at);
                        const float4 w4 = *reinterpret_cast<const float4*>(ws + at);
                        const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q)
#pragma unroll
                            for (int c = 0; c < WKV_CJ; ++c) {
                                o[c] = fmaf(rr[q], S[e + q][c], o[c]);
                                S[e + q][c] = fmaf(ww[q], S[e + q][c], kk[q] * vj[c]);
                            }
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < EMAX; ++e) {
                    if (e < E && i0 + e < D) {
                        const float re = rt[e], ke = kt[e], we = wt[e];
#pragma unroll
                        for (int c = 0; c < WKV_CJ; ++c) {
                            o[c] = fmaf(re, S[e][c], o[c]);
                            S[e][c] = fmaf(we, S[e][c], ke * vj[c]);
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < WKV_CJ; ++c) {
                o[c] += __shfl_xor_sync(0xffffffffu, o[c], 1);
                o[c] += __shfl_xor_sync(0xffffffffu, o[c], 2);
                o[c] += __shfl_xor_sync(0xffffffffu, o[c], 4);
                if (ig == 0 && (EXACT || j + c < D)) os[tt * D + j + c] = fmaf(vj[c], bonus_s[tt], o[c]);
            }
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += n_warps) {   // the head's root mean square, a warp per token
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(os[tt * D + c], os[tt * D + c], ss);
            ss = warp_sum(ss);
            if (lane == 0) rstd_s[tt] = 1.0f / sqrtf(ss / (float)D + eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * D; e += n_threads) {
            const int tt = e / D, c = e % D;
            y[(long long)(t0 + tt) * HD + head * D + c] = from_f<T>(os[e] * rstd_s[tt] * norm_w[head * D + c] * gs[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < EMAX; ++e)
#pragma unroll
        for (int c = 0; c < WKV_CJ; ++c)
            if (j + c < D && e < E && chan(e) < D) Sg[chan(e) * D + j + c] = S[e][c];
    if (head == 0 && row1 > row0) {   // the last token's input: what the next step's first row blends with
        float* rec = state + (long long)slot * state_stride + prev_offset;
        const T* last = h + (long long)(row1 - 1) * width;
        for (int c = tid; c < width; c += n_threads) rec[c] = to_f<T>(last[c]);
    }
}

// Heads of more than 128 channels: the state stays in global memory (it is the sequence's record anyway), thread j owns
// value channel j and walks the key channels of its column token by token.  Slow and plain; the sizes models have go
// through the kernel above.
template <class T>
__global__ void wkv_scan_wide_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                                     const float* __restrict__ decay_pre, const float* __restrict__ w0, const float* __restrict__ u,
                                     const float* __restrict__ norm_w, float eps, const T* __restrict__ h, int width,
                                     float* __restrict__ state, long long state_stride, int prev_offset, SbBatch batch, int H, int D,
                                     T* __restrict__ y) {
    extern __shared__ float sm[];
    float* rs = sm;          // the token's r, k and decay, [D] each
    float* ks = rs + D;
    float* ws = ks + D;
    float* os = ws + D;      // the token's raw outputs
    __shared__ float red[33];
    pdl_wait();
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    const int HD = H * D;
    float* Sg = state + (long long)slot * state_stride + (long long)head * D * D;
    for (int t = row0; t < row1; ++t) {
        const long long at = (long long)t * HD + head * D;
        __syncthreads();
        for (int i = tid; i < D; i += blockDim.x) {
            rs[i] = to_f<T>(r[at + i]);
            ks[i] = to_f<T>(k[at + i]);
            ws[i] = expf(-expf(decay_pre[at + i] + w0[head * D + i]));
        }
        __syncthreads();
        float ss = 0.f;
        for (int j = tid; j < D; j += blockDim.x) {   // the same thread owns column j at every token: nobody else touches it
            const float vj = to_f<T>(v[at + j]);
            float o = 0.f;
            for (int i = 0; i < D; ++i) {
                const float old = Sg[(long long)i * D + j], kv = ks[i] * vj;
                o = fmaf(rs[i], fmaf(u[head * D + i], kv, old), o);
                Sg[(long long)i * D + j] = fmaf(ws[i], old, kv);
            }
            os[j] = o;
            ss = fmaf(o, o, ss);
        }
        ss = block_sum(ss, red);
        const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
        for (int j = tid; j < D; j += blockDim.x) {
            const float gv = to_f<T>(g[at + j]);
            y[at + j] = from_f<T>(os[j] * rstd * norm_w[head * D + j] * (gv / (1.0f + expf(-gv))));
        }
    }
    if (head == 0 && row1 > row0) {
        float* rec = state + (long long)slot * state_stride + prev_offset;
        const T* last = h + (long long)(row1 - 1) * width;
        for (int c = tid; c < width; c += blockDim.x) rec[c] = to_f<T>(last[c]);
    }
}

extern "C" {

int sb_token_shift(int dtype, int w_dtype, const void* h, const float* state, long long state_stride, int prev_offset, const void* mu,
                   int n_mix, SbBatch batch, int width, void* out, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    typedef __nv_bfloat16 bf;
    if (dtype == SB_BF16 && w_dtype == SB_BF16 && width % 8 == 0) {
        sb_launch(token_shift_vec_kernel, batch.n_rows, threads, 0, stream, (const bf*)h, state, state_stride, prev_offset,
                  (const bf*)mu, n_mix, batch, width, (bf*)out);
        SB_LAUNCH_CHECK();
    }
#define SB_TS(T, W)                                                                                                        \
    sb_launch(token_shift_kernel<T, W>, batch.n_rows, threads, 0, stream, (const T*)h, state, state_stride, prev_offset, (const W*)mu, \
              n_mix, batch, width, (T*)out)
    if (dtype == SB_F32 && w_dtype == SB_F32) SB_TS(float, float);
    else if (dtype == SB_BF16 && w_dtype == SB_BF16) SB_TS(bf, bf);
    else if (dtype == SB_BF16 && w_dtype == SB_F32) SB_TS(bf, float);
    else return (int)cudaErrorInvalidValue;
#undef SB_TS
    SB_LAUNCH_CHECK();
}

int sb_wkv_scan(int dtype, const void* r, const void* k, const void* v, const void* g, const float* decay_pre, const float* w0,
                const float* u, const float* norm_w, float eps, const void* h, int width, float* state, long long state_stride,
                int prev_offset, SbBatch batch, int H, int D, void* y, cudaStream_t stream) {
    if (batch.n_seqs <= 0 || batch.n_rows <= 0) return 0;
    if (D < 1 || D > 4096 || H > 65535) return (int)cudaErrorInvalidValue;
    if (D > 128) {
        dim3 wide(batch.n_seqs, H);
        const int wt = D < 1024 ? (D + 31) / 32 * 32 : 1024;
        if (dtype == SB_F32)
            sb_launch(wkv_scan_wide_kernel<float>, wide, wt, (size_t)4 * D * sizeof(float), stream, (const float*)r, (const float*)k,
                      (const float*)v, (const float*)g, decay_pre, w0, u, norm_w, eps, (const float*)h, width, state, state_stride,
                      prev_offset, batch, H, D, (float*)y);
        else
            sb_launch(wkv_scan_wide_kernel<__nv_bfloat16>, wide, wt, (size_t)4 * D * sizeof(float), stream, (const __nv_bfloat16*)r,
                      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)g, decay_pre, w0, u, norm_w, eps,
                      (const __nv_bfloat16*)h, width, state, state_stride, prev_offset, batch, H, D, (__nv_bfloat16*)y);
        SB_LAUNCH_CHECK();
    }
    dim3 grid(batch.n_seqs, H);
    const size_t smem = (size_t)(6 * WKV_TB + 2) * D * sizeof(float);
    const int threads = ((D + WKV_CJ - 1) / WKV_CJ * WKV_IG + 31) / 32 * 32;
    typedef __nv_bfloat16 bf;
#define SB_WKV(T, EMAX, EXACT)                                                                                                \
    do {                                                                                                                      \
        if (smem > 48 * 1024) {                                                                                               \
            const cudaError_t err = cudaFuncSetAttribute(wkv_scan_kernel<T, EMAX, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                         (int)smem);                                                          \
            if (err != cudaSuccess) return (int)err;                                                                          \
        }                                                                                                                     \
        sb_launch(wkv_scan_kernel<T, EMAX, EXACT>, grid, threads, smem, stream, (const T*)r, (const T*)k, (const T*)v, (const T*)g, \
                  decay_pre, w0, u, norm_w, eps, (const T*)h, width, state, state_stride, prev_offset, batch, H, D, (T*)y);    \
    } while (0)
#define SB_WKV_SIZES(T)                              \
    do {                                             \
        if (D == 32) SB_WKV(T, 4, true);             \
        else if (D == 64) SB_WKV(T, 8, true);        \
        else if (D == 128) SB_WKV(T, 16, true);      \
        else if (D <= 32) SB_WKV(T, 4, false);       \
        else if (D <= 64) SB_WKV(T, 8, false);       \
        else SB_WKV(T, 16, false);                   \
    } while (0)
    if (dtype == SB_F32) SB_WKV_SIZES(float);
    else SB_WKV_SIZES(bf);
#undef SB_WKV_SIZES
#undef SB_WKV
    SB_LAUNCH_CHECK();
}

}  // extern "C"
