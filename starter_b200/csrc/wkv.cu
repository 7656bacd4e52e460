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

#define WKV_TB 16   // tokens whose r, k and decay are staged in shared memory at a time

// One block per (sequence, head); thread j owns value channel j: column j of the state, D floats in registers.
template <class T, int DMAX>
__global__ void __launch_bounds__(DMAX) wkv_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                                        const T* __restrict__ g, const float* __restrict__ decay_pre,
                                                        const float* __restrict__ w0, const float* __restrict__ u,
                                                        const float* __restrict__ norm_w, float eps, const T* __restrict__ h, int width,
                                                        float* __restrict__ state, long long state_stride, int prev_offset,
                                                        SbBatch batch, int H, int D, T* __restrict__ y) {
    extern __shared__ float sm[];
    float* rs = sm;                  // [WKV_TB][D]
    float* ks = rs + WKV_TB * D;
    float* ws = ks + WKV_TB * D;
    float* os = ws + WKV_TB * D;
    float* us = os + WKV_TB * D;     // [D]
    float* w0s = us + D;             // [D]
    __shared__ float rstd_s[WKV_TB];
    const int s = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const int lane = j & 31, warp = j >> 5, n_warps = DMAX / 32;
    for (int i = j; i < D; i += DMAX) {   // weights: they do not depend on the kernel before this one
        us[i] = u[head * D + i];
        w0s[i] = w0[head * D + i];
    }
    pdl_wait();
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    const int HD = H * D, col = head * D + j;
    const bool own = j < D;
    float* Sg = state + (long long)slot * state_stride + (long long)head * D * D;
    float S[DMAX];
#pragma unroll
    for (int i = 0; i < DMAX; ++i) S[i] = (own && i < D) ? Sg[i * D + j] : 0.f;
    const float nw = own ? norm_w[col] : 0.f;
    for (int t0 = row0; t0 < row1; t0 += WKV_TB) {
        const int nt = min(WKV_TB, row1 - t0);
        __syncthreads();
        for (int e = j; e < nt * D; e += DMAX) {
            const long long at = (long long)(t0 + e / D) * HD + head * D + e % D;
            rs[e] = to_f<T>(r[at]);
            ks[e] = to_f<T>(k[at]);
            ws[e] = expf(-expf(decay_pre[at] + w0s[e % D]));
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = own ? to_f<T>(v[(long long)(t0 + tt) * HD + col]) : 0.f;
            const float* rt = rs + tt * D;
            const float* kt = ks + tt * D;
            const float* wt = ws + tt * D;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < DMAX; ++i) {
                if (i < D) {
                    const float kv = kt[i] * vj;
                    o = fmaf(rt[i], fmaf(us[i], kv, S[i]), o);
                    S[i] = fmaf(wt[i], S[i], kv);
                }
            }
            if (own) os[tt * D + j] = o;
        }
        __syncthreads();
        for (int tt = warp; tt < nt; tt += n_warps) {   // the head's root mean square, a warp per token
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(os[tt * D + c], os[tt * D + c], ss);
            ss = warp_sum(ss);
            if (lane == 0) rstd_s[tt] = 1.0f / sqrtf(ss / (float)D + eps);
        }
        __syncthreads();
        if (own) {
            for (int tt = 0; tt < nt; ++tt) {
                const long long at = (long long)(t0 + tt) * HD + col;
                const float gv = to_f<T>(g[at]);
                y[at] = from_f<T>(os[tt * D + j] * rstd_s[tt] * nw * (gv / (1.0f + expf(-gv))));
            }
        }
    }
    if (own) {
#pragma unroll
        for (int i = 0; i < DMAX; ++i)
            if (i < D) Sg[i * D + j] = S[i];
    }
    if (head == 0 && row1 > row0) {   // the last token's input: what the next step's first row blends with
        float* rec = state + (long long)slot * state_stride + prev_offset;
        const T* last = h + (long long)(row1 - 1) * width;
        for (int c = j; c < width; c += DMAX) rec[c] = to_f<T>(last[c]);
    }
}

extern "C" {

int sb_token_shift(int dtype, int w_dtype, const void* h, const float* state, long long state_stride, int prev_offset, const void* mu,
                   int n_mix, SbBatch batch, int width, void* out, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    typedef __nv_bfloat16 bf;
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
    if (D < 1 || D > 128 || H > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(batch.n_seqs, H);
    const size_t smem = (size_t)(4 * WKV_TB + 2) * D * sizeof(float);
    typedef __nv_bfloat16 bf;
#define SB_WKV(T, DMAX)                                                                                                      \
    sb_launch(wkv_scan_kernel<T, DMAX>, grid, DMAX, smem, stream, (const T*)r, (const T*)k, (const T*)v, (const T*)g, decay_pre, w0, u, \
              norm_w, eps, (const T*)h, width, state, state_stride, prev_offset, batch, H, D, (T*)y)
    if (dtype == SB_F32) {
        if (D <= 32) SB_WKV(float, 32);
        else if (D <= 64) SB_WKV(float, 64);
        else SB_WKV(float, 128);
    } else {
        if (D <= 32) SB_WKV(bf, 32);
        else if (D <= 64) SB_WKV(bf, 64);
        else SB_WKV(bf, 128);
    }
#undef SB_WKV
    SB_LAUNCH_CHECK();
}

}  // extern "C"
