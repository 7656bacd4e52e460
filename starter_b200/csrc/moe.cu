// Mixture of experts: the router, the order of the chosen (token, expert) pairs by expert, the experts' products for a
// handful of pairs, and the weighted sum that brings a token's experts together.
//
//   s = softmax(W_r h) over experts + identity outputs                      (32-bit)
//   chosen = the `top` largest of s + correction;  weight = s / (sum of the chosen s + 1e-20) * scale
//   y = base + sum over chosen e of weight_e * (e is an identity output ? h : down_e(act(gate_e h, up_e h)))
//
// A pair is (row, k): the k-th choice of a row.  Pairs of identity outputs read no matrix.  For many rows the pairs are
// put in the order of their experts (a slot per pair), so that one grouped product per matrix serves the step; for a
// few pairs each pair streams its expert's matrices through the kernels below (a warp per output column).
#include "common.cuh"

#define MOE_MAX_OUTPUTS 1024   // experts + identity outputs that the router kernel takes
#define MOE_MAX_TOP 32

// One block of 128 threads per row: logits by warps, softmax and the choice by the first warp.
template <class T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ correction,
                                 int* __restrict__ chosen, float* __restrict__ weight, int width, int n_out, int top, float scale) {
    __shared__ float s_s[MOE_MAX_OUTPUTS];      // logits, then scores
    __shared__ float c_s[MOE_MAX_OUTPUTS];      // choice scores; -inf once taken
    pdl_wait();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const T* hr = h + (long long)row * width;
    for (int e = warp; e < n_out; e += n_warps) {
        const float* wr = router + (long long)e * width;
        float dot = 0.f;
        for (int c = lane; c < width; c += 32) dot = fmaf(to_f<T>(hr[c]), wr[c], dot);
        dot = warp_sum(dot);
        if (lane == 0) s_s[e] = dot;
    }
    __syncthreads();
    if (warp != 0) return;
    float mx = -INFINITY;
    for (int e = lane; e < n_out; e += 32) mx = fmaxf(mx, s_s[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_out; e += 32) {
        const float w = expf(s_s[e] - mx);
        s_s[e] = w;
        sum += w;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < n_out; e += 32) {
        s_s[e] *= inv;
        c_s[e] = s_s[e] + correction[e];
    }
    __syncwarp();
    float total = 0.f;
    int mine = -1;   // lane k keeps the k-th choice
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_out; e += 32)
            if (c_s[e] > best) {
                best = c_s[e];
                at = e;
            }
        for (int o = 16; o > 0; o >>= 1) {   // the largest; of equals the lowest index
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) {
                best = ob;
                at = oa;
            }
        }
        if (at == 0x7fffffff) at = 0;
        if (lane == k) mine = at;
        total += s_s[at];
        __syncwarp();
        if (lane == 0) c_s[at] = -INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        chosen[(long long)row * top + lane] = mine;
        weight[(long long)row * top + lane] = s_s[mine] / (total + 1e-20f) * scale;
    }
}

// One block: counts per expert, their running sums (ends[e] = pairs of experts 0..e), and a slot for every pair of a
// real expert, expert by expert (-1 for pairs of identity outputs).  Within an expert the pairs keep their order.
__global__ void moe_sort_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ ends,
                                int* __restrict__ slot_of_pair, int* __restrict__ pair_of_slot) {
    extern __shared__ int cnt[];   // [n_experts] counts, then starts
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < n_experts) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int c = cnt[e];
            cnt[e] = run;
            run += c;
            ends[e] = run;
        }
    }
    __syncthreads();
    // in order: a warp takes an expert and walks the pairs with ballots, so that a pair's slot does not depend on timing
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < n_experts; e += n_warps) {
        int at = cnt[e];
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            const bool hit = p < n_pairs && chosen[p] == e;
            const unsigned int mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int slot = at + __popc(mask & ((1u << lane) - 1u));
                slot_of_pair[p] = slot;
                pair_of_slot[slot] = p;
            }
            at += __popc(mask);
        }
    }
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= n_experts) slot_of_pair[p] = -1;
    }
}

// xs[slot] = h[row of the slot's pair], 16 bytes per thread where the rows allow.
template <class T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ pair_of_slot, const int* __restrict__ ends,
                                  int n_experts, int top, int width, T* __restrict__ xs) {
    pdl_wait();
    const int slot = blockIdx.x;
    if (slot >= ends[n_experts - 1]) return;
    const T* src = h + (long long)(pair_of_slot[slot] / top) * width;
    T* dst = xs + (long long)slot * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
}

// A pair's gate and up products with the activation: act[pair][c] for the block's columns, a warp per column.
template <class T>
__global__ void moe_pair_gate_up_kernel(const T* __restrict__ h, const int* __restrict__ chosen, const T* __restrict__ w_gate_up,
                                        T* __restrict__ act, int top, int n_experts, int width, int ff, float alpha, float limit) {
    pdl_wait();
    const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int e = chosen[pair];
    if (e < 0 || e >= n_experts) return;
    const T* hr = h + (long long)(pair / top) * width;
    const T* wg = w_gate_up + (long long)e * 2 * ff * width;
    for (int c = blockIdx.y * n_warps + warp; c < ff; c += gridDim.y * n_warps) {
        const T* g_row = wg + (long long)c * width;
        const T* u_row = wg + (long long)(ff + c) * width;
        float g = 0.f, u = 0.f;
        for (int i = lane; i < width; i += 32) {
            const float x = to_f<T>(hr[i]);
            g = fmaf(x, to_f<T>(g_row[i]), g);
            u = fmaf(x, to_f<T>(u_row[i]), u);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) {
            g = fminf(rnd<T>(g), limit);
            u = fminf(fmaxf(rnd<T>(u), -limit), limit);
            act[(long long)pair * ff + c] = from_f<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
        }
    }
}

// A pair's down product: down[pair][c], a warp per column.
template <class T>
__global__ void moe_pair_down_kernel(const T* __restrict__ act, const int* __restrict__ chosen, const T* __restrict__ w_down,
                                     T* __restrict__ down, int n_experts, int width, int ff) {
    pdl_wait();
    const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int e = chosen[pair];
    if (e < 0 || e >= n_experts) return;
    const T* ar = act + (long long)pair * ff;
    const T* wd = w_down + (long long)e * width * ff;
    for (int c = blockIdx.y * n_warps + warp; c < width; c += gridDim.y * n_warps) {
        const T* row = wd + (long long)c * ff;
        float d = 0.f;
        for (int i = lane; i < ff; i += 32) d = fmaf(to_f<T>(ar[i]), to_f<T>(row[i]), d);
        d = warp_sum(d);
        if (lane == 0) down[(long long)pair * width + c] = from_f<T>(d);
    }
}

// y[row] = base[row] + sum_k weight[row][k] * (identity ? h[row] : down[place of pair (row, k)]), summed in 32-bit in
// the order of k.  slot_of_pair null: a pair's result lies at the pair's own index.
template <class T>
__global__ void moe_combine_kernel(const T* __restrict__ h, const T* __restrict__ down, const T* __restrict__ base,
                                   const int* __restrict__ chosen, const float* __restrict__ weight, const int* __restrict__ slot_of_pair,
                                   T* __restrict__ y, int top, int n_experts, int width) {
    __shared__ int place_s[MOE_MAX_TOP];
    __shared__ float w_s[MOE_MAX_TOP];
    pdl_wait();
    const long long row = blockIdx.x;
    if (threadIdx.x < top) {
        const long long pair = row * top + threadIdx.x;
        const int e = chosen[pair];
        w_s[threadIdx.x] = weight[pair];
        place_s[threadIdx.x] = (e < 0 || e >= n_experts) ? -1 : (slot_of_pair != nullptr ? slot_of_pair[pair] : (int)pair);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = base != nullptr ? to_f<T>(base[row * width + c]) : 0.f;
        const float hv = to_f<T>(h[row * width + c]);
        for (int k = 0; k < top; ++k) {
            const int at = place_s[k];
            acc = fmaf(w_s[k], at < 0 ? hv : to_f<T>(down[(long long)at * width + c]), acc);
        }
        y[row * width + c] = from_f<T>(acc);
    }
}

extern "C" {

int sb_moe_route(int dtype, const void* h, const float* router, const float* correction, int* chosen, float* weight, int rows,
                 int width, int n_out, int top, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n_out < 1 || n_out > MOE_MAX_OUTPUTS || top < 1 || top > MOE_MAX_TOP || top > n_out) return (int)cudaErrorInvalidValue;
    if (dtype == SB_F32)
        sb_launch(moe_route_kernel<float>, rows, 128, 0, stream, (const float*)h, router, correction, chosen, weight, width, n_out, top,
                  scale);
    else
        sb_launch(moe_route_kernel<__nv_bfloat16>, rows, 128, 0, stream, (const __nv_bfloat16*)h, router, correction, chosen, weight,
                  width, n_out, top, scale);
    SB_LAUNCH_CHECK();
}

int sb_moe_sort(const int* chosen, int n_pairs, int n_experts, int* ends, int* slot_of_pair, int* pair_of_slot, cudaStream_t stream) {
    if (n_pairs <= 0 || n_experts <= 0) return 0;
    if (n_experts > 8192) return (int)cudaErrorInvalidValue;
    sb_launch(moe_sort_kernel, 1, 1024, (size_t)n_experts * sizeof(int), stream, chosen, n_pairs, n_experts, ends, slot_of_pair,
              pair_of_slot);
    SB_LAUNCH_CHECK();
}

int sb_moe_gather(int dtype, const void* h, const int* pair_of_slot, const int* ends, int n_experts, int n_pairs, int top, int width,
                  void* xs, cudaStream_t stream) {
    if (n_pairs <= 0 || n_experts <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == SB_F32)
        sb_launch(moe_gather_kernel<float>, n_pairs, threads, 0, stream, (const float*)h, pair_of_slot, ends, n_experts, top, width,
                  (float*)xs);
    else
        sb_launch(moe_gather_kernel<__nv_bfloat16>, n_pairs, threads, 0, stream, (const __nv_bfloat16*)h, pair_of_slot, ends, n_experts,
                  top, width, (__nv_bfloat16*)xs);
    SB_LAUNCH_CHECK();
}

int sb_moe_pairs(int dtype, const void* h, const int* chosen, const void* w_gate_up, const void* w_down, void* act, void* down,
                 int n_pairs, int top, int n_experts, int width, int ff, float alpha, float limit, cudaStream_t stream) {
    if (n_pairs <= 0 || n_experts <= 0) return 0;
    const int threads = 256, warps = threads / 32;
    // enough blocks along the columns for a few per SM when the pairs are few
    const int want = n_pairs >= 592 ? 1 : (592 + n_pairs - 1) / n_pairs;
    dim3 g1(n_pairs, (unsigned int)max(1, min(want, (ff + warps - 1) / warps)));
    dim3 g2(n_pairs, (unsigned int)max(1, min(want, (width + warps - 1) / warps)));
    typedef __nv_bfloat16 bf;
    if (dtype == SB_F32) {
        sb_launch(moe_pair_gate_up_kernel<float>, g1, threads, 0, stream, (const float*)h, chosen, (const float*)w_gate_up, (float*)act,
                  top, n_experts, width, ff, alpha, limit);
        sb_launch(moe_pair_down_kernel<float>, g2, threads, 0, stream, (const float*)act, chosen, (const float*)w_down, (float*)down,
                  n_experts, width, ff);
    } else {
        sb_launch(moe_pair_gate_up_kernel<bf>, g1, threads, 0, stream, (const bf*)h, chosen, (const bf*)w_gate_up, (bf*)act, top,
                  n_experts, width, ff, alpha, limit);
        sb_launch(moe_pair_down_kernel<bf>, g2, threads, 0, stream, (const bf*)act, chosen, (const bf*)w_down, (bf*)down, n_experts,
                  width, ff);
    }
    SB_LAUNCH_CHECK();
}

int sb_moe_combine(int dtype, const void* h, const void* down, const void* base, const int* chosen, const float* weight,
                   const int* slot_of_pair, void* y, int rows, int top, int n_experts, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP) return (int)cudaErrorInvalidValue;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == SB_F32)
        sb_launch(moe_combine_kernel<float>, rows, threads, 0, stream, (const float*)h, (const float*)down, (const float*)base, chosen,
                  weight, slot_of_pair, (float*)y, top, n_experts, width);
    else
        sb_launch(moe_combine_kernel<__nv_bfloat16>, rows, threads, 0, stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)down,
                  (const __nv_bfloat16*)base, chosen, weight, slot_of_pair, (__nv_bfloat16*)y, top, n_experts, width);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
