// The attention of attention_flex.cu on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit sums), for
// prompts and for decoding alike.
//
// A block of four warps owns 16 rows of scores: the query heads that share one key/value head (up to 16 of them) at
// 16 / heads consecutive positions of one sequence.  So a page of keys is fetched once for all heads that read it:
// for a cache with a single shared row per token (values inside the key rows) the 16 rows are 16 heads of one token,
// which is what decoding through a latent needs.  Keys come a page (64 tokens) at a time through a two-stage cp.async
// pipeline; rows of a page that lie outside the block's range of visible keys are filled with zeros instead of being
// read, so that whatever an earlier sequence left in a page never meets a weight.
//
// Per page: each warp multiplies the 16 query rows with 16 of the 64 keys; the scores meet in shared memory, where
// scale, per-head temperature, distance penalty and the mask (causal, window, chunk) are applied and the running
// maximum, the exponentials and the row sums are taken, all 32-bit.  A weight w is handed to the tensor cores as two
// bfloat16 numbers hi + lo (hi = bf16(w), lo = bf16(w - hi)), so that it keeps 16 bits instead of 8 when it meets its
// value; each warp then owns a quarter of the value columns and adds hi * V and lo * V to its 32-bit sums.
//
// With several blocks per (sequence, key/value head) along the keys (decoding: few rows, many keys) every block
// leaves its unnormalised sums, maximum and row sum in scratch and a second kernel merges them; the sink joins the
// denominator in whichever kernel divides.
#include "attention_flex.cuh"
#include "mma_utils.cuh"

#define FM_KEYS 64
#define FM_ROWS 16
#define FM_THREADS 128
#define FM_SLD 68   // floats per row of the score tile
#define FM_PLD 72   // bfloat16 per row of a weight tile

__device__ __forceinline__ void cp_async_16_or_zero(void* smem_dst, const void* gmem_src, bool real) {
    const unsigned int s = (unsigned int)__cvta_generic_to_shared(smem_dst);
    const int n = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem_src), "r"(n));
}

template <int VD>
__global__ void __launch_bounds__(FM_THREADS)
flex_attention_mma_kernel(SbFlex p, SbBatch batch, __nv_bfloat16* __restrict__ out, int tiles_per_seq, int n_splits,
                          float* __restrict__ partial, int values_in_keys) {
    typedef __nv_bfloat16 bf;
    constexpr int VW = VD / 4, NT = VW / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KD = p.k_dim, kld = KD + 8, vld = values_in_keys ? kld : VD + 8;
    bf* Qs = reinterpret_cast<bf*>(smem_raw);
    bf* Ks = Qs + FM_ROWS * kld;
    bf* Vs = values_in_keys ? Ks : Ks + 2 * FM_KEYS * kld;
    const size_t v_stage = values_in_keys ? (size_t)FM_KEYS * kld : (size_t)FM_KEYS * vld;
    bf* after = values_in_keys ? Ks + 2 * FM_KEYS * kld : Vs + 2 * FM_KEYS * vld;
    float* Ss = reinterpret_cast<float*>(after);
    bf* Ph = reinterpret_cast<bf*>(Ss + FM_ROWS * FM_SLD);
    bf* Pl = Ph + FM_ROWS * FM_PLD;
    float* alpha_s = reinterpret_cast<float*>(Pl + FM_ROWS * FM_PLD);
    float* l_s = alpha_s + FM_ROWS;
    float* m_s = l_s + FM_ROWS;

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t = lane & 3;
    const int HG = p.n_heads / p.n_kv_heads;
    const int HGB = HG < FM_ROWS ? HG : FM_ROWS;          // heads of the group that this block owns
    const int HSUB = HG / HGB;
    const int QR = FM_ROWS / HGB;                          // positions that this block owns
    const int s = blockIdx.x / tiles_per_seq, tile = blockIdx.x % tiles_per_seq;
    const int kvh = blockIdx.y / HSUB, head0 = kvh * HG + (blockIdx.y % HSUB) * HGB;
    const int split = blockIdx.z;
    pdl_wait();
    const int slot = batch.seq_slot[s], q0 = batch.cu_q[s], nq = batch.cu_q[s + 1] - q0;
    const int first = tile * QR;
    if (first >= nq) return;
    const int n_here = min(QR, nq - first);
    const int pos_first = batch.lengths[slot] + first, pos_last = pos_first + n_here - 1;
    const int key_lo = flex_first_key(p, pos_first), key_hi = pos_last;
    int page_lo = key_lo / SB_PAGE, page_hi = key_hi / SB_PAGE;
    if (n_splits > 1) {
        const int per = (page_hi - page_lo + n_splits) / n_splits;
        page_lo += split * per;
        page_hi = min(page_hi, page_lo + per - 1);
    }

    // the queries of the block's 16 rows: row r = position (r / HGB), head (r % HGB); rows past the sequence's are zeros
    {
        const int cpr = KD / 8;
        for (int c = tid; c < FM_ROWS * cpr; c += FM_THREADS) {
            const int r = c / cpr, cc = c % cpr, qi = r / HGB, hh = r % HGB;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (qi < n_here)
                val = *reinterpret_cast<const uint4*>((const bf*)p.q + (long long)(q0 + first + qi) * p.q_row +
                                                      (long long)(head0 + hh) * p.q_head + cc * 8);
            *reinterpret_cast<uint4*>(Qs + r * kld + cc * 8) = val;
        }
    }
    auto load_page = [&](int page_idx, int buf) {
        int lp = page_idx;
        if (p.ring_pages) lp %= p.ring_pages;
        const int page = lp < p.table_width ? p.table[(long long)slot * p.table_width + lp] : -1;
        const long long tok0 = ((long long)(page < 0 ? 0 : page) * p.n_kv_heads + kvh) * SB_PAGE;
        const bf* ksrc = (const bf*)p.k + tok0 * KD;
        const int cpr = KD / 8;
        for (int c = tid; c < FM_KEYS * cpr; c += FM_THREADS) {
            const int r = c / cpr, cc = c % cpr, key = page_idx * SB_PAGE + r;
            cp_async_16_or_zero(Ks + (size_t)buf * FM_KEYS * kld + r * kld + cc * 8, ksrc + (long long)r * KD + cc * 8,
                                page >= 0 && key >= key_lo && key <= key_hi);
        }
        if (!values_in_keys) {
            const bf* vsrc = (const bf*)p.v + flex_value_page(p, page < 0 ? 0 : page, kvh) * p.v_row;
            constexpr int vcpr = VD / 8;
            for (int c = tid; c < FM_KEYS * vcpr; c += FM_THREADS) {
                const int r = c / vcpr, cc = c % vcpr, key = page_idx * SB_PAGE + r;
                cp_async_16_or_zero(Vs + (size_t)buf * v_stage + r * vld + cc * 8, vsrc + (long long)r * p.v_row + cc * 8,
                                    page >= 0 && key >= key_lo && key <= key_hi);
            }
        }
        cp_async_commit();
    };

    // what the softmax lanes keep: lane -> row w * 4 + lane / 8, keys (lane % 8) * 8 .. + 7 of the page
    const int srow = w * 4 + (lane >> 3), sub = lane & 7;
    const int s_qi = srow / HGB, s_head = head0 + srow % HGB;
    const bool s_valid = s_qi < n_here;
    const int s_pos = pos_first + s_qi, s_lo = flex_first_key(p, s_pos);
    const float hs = p.head_scale != nullptr ? p.scale * p.head_scale[s_head] : p.scale;
    const float slope = p.slopes != nullptr ? p.slopes[s_head] : 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

    if (page_lo <= page_hi) load_page(page_lo, 0);
    for (int pg = page_lo; pg <= page_hi; ++pg) {
        const int buf = (pg - page_lo) & 1;
        if (pg + 1 <= page_hi) {
            load_page(pg + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf* Kb = Ks + (size_t)buf * FM_KEYS * kld;
        const bf* Vb = Vs + (size_t)buf * v_stage;
        {   // scores of the 16 rows against keys 16 w .. 16 w + 15 of the page
            float sacc[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
            const bf* qa = Qs + (lane & 15) * kld + (lane >> 4) * 8;
            const bf* kb = Kb + (16 * w + (lane & 7) + (lane >> 4) * 8) * kld + ((lane >> 3) & 1) * 8;
            for (int k0 = 0; k0 < KD; k0 += 16) {
                unsigned int a[4], b[4];
                ldmatrix_x4(a, qa + k0);
                ldmatrix_x4(b, kb + k0);
                mma_bf16(sacc[0], a, b[0], b[1]);
                mma_bf16(sacc[1], a, b[2], b[3]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int col = 16 * w + 8 * i + 2 * t;
                *reinterpret_cast<float2*>(Ss + g * FM_SLD + col) = make_float2(sacc[i][0], sacc[i][1]);
                *reinterpret_cast<float2*>(Ss + (g + 8) * FM_SLD + col) = make_float2(sacc[i][2], sacc[i][3]);
            }
        }
        __syncthreads();
        {   // mask, running maximum, weights
            float sv[8];
            float mx = -INFINITY;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int n = pg * SB_PAGE + sub * 8 + e;
                const bool seen = s_valid && n >= s_lo && n <= s_pos;
                sv[e] = seen ? Ss[srow * FM_SLD + sub * 8 + e] * hs - slope * (float)(s_pos - n) : -INFINITY;
                mx = fmaxf(mx, sv[e]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_new = fmaxf(m_run, mx);
            float alpha = 1.f, sum = 0.f;
            unsigned int hi[4], lo[4];
            if (m_new == -INFINITY) {
#pragma unroll
                for (int e = 0; e < 4; ++e) hi[e] = lo[e] = 0u;
            } else {
                alpha = expf(m_run - m_new);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float w0 = expf(sv[2 * e] - m_new), w1 = expf(sv[2 * e + 1] - m_new);
                    sum += w0 + w1;
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(w0, w1);
                    const float2 back = __bfloat1622float2(h2);
                    hi[e] = *reinterpret_cast<const unsigned int*>(&h2);
                    lo[e] = pack_bf16(w0 - back.x, w1 - back.y);
                }
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            l_run = l_run * alpha + sum;
            m_run = m_new;
            *reinterpret_cast<uint4*>(Ph + srow * FM_PLD + sub * 8) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(Pl + srow * FM_PLD + sub * 8) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            if (sub == 0) alpha_s[srow] = alpha;
        }
        __syncthreads();
        {   // this warp's quarter of the value columns
            const float a0 = alpha_s[g], a1 = alpha_s[g + 8];
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[i][0] *= a0;
                acc[i][1] *= a0;
                acc[i][2] *= a1;
                acc[i][3] *= a1;
            }
            const bf* pa = Ph + (lane & 15) * FM_PLD + (lane >> 4) * 8;
            const bf* pl = Pl + (lane & 15) * FM_PLD + (lane >> 4) * 8;
            const bf* vb = Vb + ((lane & 7) + ((lane >> 3) & 1) * 8) * vld + w * VW + (lane >> 4) * 8;
#pragma unroll
            for (int k0 = 0; k0 < FM_KEYS; k0 += 16) {
                unsigned int ah[4], al[4];
                ldmatrix_x4(ah, pa + k0);
                ldmatrix_x4(al, pl + k0);
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    unsigned int b[4];
                    ldmatrix_x4_trans(b, vb + k0 * vld + i * 8);
                    mma_bf16(acc[i], ah, b[0], b[1]);
                    mma_bf16(acc[i], al, b[0], b[1]);
                    mma_bf16(acc[i + 1], ah, b[2], b[3]);
                    mma_bf16(acc[i + 1], al, b[2], b[3]);
                }
            }
        }
        __syncthreads();   // the next turn overwrites this page's buffer, the scores and the weights
    }
    if (sub == 0) {
        l_s[srow] = l_run;
        m_s[srow] = m_run;
    }
    __syncthreads();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half, qi = r / HGB, head = head0 + r % HGB;
        if (qi >= n_here) continue;
        const long long grow = q0 + first + qi;
        float m = m_s[r], l = l_s[r];
        if (n_splits == 1) {
            float a = 1.f;
            if (p.sink != nullptr) {
                const float sk = p.sink[head], mf = fmaxf(m, sk);
                a = expf(m - mf);
                l = l * a + expf(sk - mf);
            }
            const float mul = a / l;
            bf* o = out + (grow * p.n_heads + head) * VD + w * VW;
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + 2 * t) =
                    __floats2bfloat162_rn(acc[i][2 * half] * mul, acc[i][2 * half + 1] * mul);
        } else {
            float* o = partial + ((grow * p.n_heads + head) * n_splits + split) * (VD + 2);
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<float2*>(o + w * VW + i * 8 + 2 * t) = make_float2(acc[i][2 * half], acc[i][2 * half + 1]);
            if (w == 0 && t == 0) {
                o[VD] = m;
                o[VD + 1] = l;
            }
        }
    }
}

// One block per (row, head): the splits' sums, scaled to their common maximum (the sink's too), added and divided.
__global__ void flex_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, const float* __restrict__ sink,
                                  int n_heads, int n_splits, int VD) {
    pdl_wait();
    const long long rh = (long long)blockIdx.x * n_heads + blockIdx.y;
    const float* base = partial + rh * n_splits * (VD + 2);
    float m = sink != nullptr ? sink[blockIdx.y] : -INFINITY;
    for (int sidx = 0; sidx < n_splits; ++sidx) m = fmaxf(m, base[(long long)sidx * (VD + 2) + VD]);
    float l = sink != nullptr ? expf(sink[blockIdx.y] - m) : 0.f;
    for (int sidx = 0; sidx < n_splits; ++sidx) {
        const float ms = base[(long long)sidx * (VD + 2) + VD];
        if (ms != -INFINITY) l += base[(long long)sidx * (VD + 2) + VD + 1] * expf(ms - m);
    }
    for (int c = threadIdx.x; c < VD; c += blockDim.x) {
        float o = 0.f;
        for (int sidx = 0; sidx < n_splits; ++sidx) {
            const float ms = base[(long long)sidx * (VD + 2) + VD];
            if (ms != -INFINITY) o = fmaf(base[(long long)sidx * (VD + 2) + c], expf(ms - m), o);
        }
        out[rh * VD + c] = __float2bfloat16_rn(o / l);
    }
}

// The kernel for prompts: 64 rows per block, a warp per 16 rows.  Each warp multiplies its rows with all 64 keys of a
// page, keeps the scores in registers, takes mask, maximum, exponentials and row sums there (the four lanes of a row
// meet by two shuffles), hands the weights to the tensor cores straight from those registers (hi + lo again) and owns
// all value columns of its rows: inside a page the warps do not meet at all.  For values of up to 128 columns (the sums
// of a warp's 16 rows over all columns live in its registers).  Rows are (position, head of the group) pairs, 64 / heads
// positions per block, so a page is still fetched once for all heads that read it.
#define FR_ROWS 64

template <int VD>
__global__ void __launch_bounds__(FM_THREADS)
flex_attention_rows64_kernel(SbFlex p, SbBatch batch, __nv_bfloat16* __restrict__ out, int tiles_per_seq, int values_in_keys) {
    typedef __nv_bfloat16 bf;
    constexpr int NT = VD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KD = p.k_dim, kld = KD + 8, vld = values_in_keys ? kld : VD + 8;
    bf* Qs = reinterpret_cast<bf*>(smem_raw);
    bf* Ks = Qs + FR_ROWS * kld;
    bf* Vs = values_in_keys ? Ks : Ks + 2 * FM_KEYS * kld;
    const size_t v_stage = values_in_keys ? (size_t)FM_KEYS * kld : (size_t)FM_KEYS * vld;

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, t = lane & 3;
    const int HG = p.n_heads / p.n_kv_heads;           // divides 64
    const int QR = FR_ROWS / HG;                        // positions that this block owns
    const int s = blockIdx.x / tiles_per_seq, tile = tiles_per_seq - 1 - blockIdx.x % tiles_per_seq;   // latest rows (most keys) first
    const int kvh = blockIdx.y, head0 = kvh * HG;
    pdl_wait();
    const int slot = batch.seq_slot[s], q0 = batch.cu_q[s], nq = batch.cu_q[s + 1] - q0;
    const int first = tile * QR;
    if (first >= nq) return;
    const int n_here = min(QR, nq - first);
    const int pos_first = batch.lengths[slot] + first, pos_last = pos_first + n_here - 1;
    const int key_lo = flex_first_key(p, pos_first), key_hi = pos_last;
    const int page_lo = key_lo / SB_PAGE, page_hi = key_hi / SB_PAGE;
    {
        const int cpr = KD / 8;
        for (int c = tid; c < FR_ROWS * cpr; c += FM_THREADS) {
            const int r = c / cpr, cc = c % cpr, qi = r / HG, hh = r % HG;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (qi < n_here)
                val = *reinterpret_cast<const uint4*>((const bf*)p.q + (long long)(q0 + first + qi) * p.q_row +
                                                      (long long)(head0 + hh) * p.q_head + cc * 8);
            *reinterpret_cast<uint4*>(Qs + r * kld + cc * 8) = val;
        }
    }
    auto load_page = [&](int page_idx, int buf) {
        int lp = page_idx;
        if (p.ring_pages) lp %= p.ring_pages;
        const int page = lp < p.table_width ? p.table[(long long)slot * p.table_width + lp] : -1;
        const long long tok0 = ((long long)(page < 0 ? 0 : page) * p.n_kv_heads + kvh) * SB_PAGE;
        const bf* ksrc = (const bf*)p.k + tok0 * KD;
        const int cpr = KD / 8;
        for (int c = tid; c < FM_KEYS * cpr; c += FM_THREADS) {
            const int r = c / cpr, cc = c % cpr, key = page_idx * SB_PAGE + r;
            cp_async_16_or_zero(Ks + (size_t)buf * FM_KEYS * kld + r * kld + cc * 8, ksrc + (long long)r * KD + cc * 8,
                                page >= 0 && key >= key_lo && key <= key_hi);
        }
        if (!values_in_keys) {
            const bf* vsrc = (const bf*)p.v + flex_value_page(p, page < 0 ? 0 : page, kvh) * p.v_row;
            constexpr int vcpr = VD / 8;
            for (int c = tid; c < FM_KEYS * vcpr; c += FM_THREADS) {
                const int r = c / vcpr, cc = c % vcpr, key = page_idx * SB_PAGE + r;
                cp_async_16_or_zero(Vs + (size_t)buf * v_stage + r * vld + cc * 8, vsrc + (long long)r * p.v_row + cc * 8,
                                    page >= 0 && key >= key_lo && key <= key_hi);
            }
        }
        cp_async_commit();
    };

    // this thread's two rows: w * 16 + g and + 8
    int r_pos[2], r_lo[2], r_head[2];
    bool r_valid[2];
    float r_hs[2], r_slope[2], m_run[2], l_run[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = w * 16 + g + 8 * half, qi = r / HG;
        r_head[half] = head0 + r % HG;
        r_valid[half] = qi < n_here;
        r_pos[half] = pos_first + qi;
        r_lo[half] = flex_first_key(p, r_pos[half]);
        r_hs[half] = p.head_scale != nullptr ? p.scale * p.head_scale[r_head[half]] : p.scale;
        r_slope[half] = p.slopes != nullptr ? p.slopes[r_head[half]] : 0.f;
        m_run[half] = -INFINITY;
        l_run[half] = 0.f;
    }
    const int w_last = pos_first + min(n_here - 1, (w * 16 + 15) / HG);   // the last position among this warp's rows
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

    load_page(page_lo, 0);
    for (int pg = page_lo; pg <= page_hi; ++pg) {
        const int buf = (pg - page_lo) & 1;
        if (pg + 1 <= page_hi) {
            load_page(pg + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (pg * SB_PAGE <= w_last && w * 16 / HG < n_here) {   // a page past this warp's rows holds nothing they see
            const bf* Kb = Ks + (size_t)buf * FM_KEYS * kld;
            const bf* Vb = Vs + (size_t)buf * v_stage;
            float sacc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
            const bf* qa = Qs + (w * 16 + (lane & 15)) * kld + (lane >> 4) * 8;
            const bf* kb = Kb + ((lane & 7) + (lane >> 4) * 8) * kld + ((lane >> 3) & 1) * 8;
            for (int k0 = 0; k0 < KD; k0 += 16) {
                unsigned int a[4];
                ldmatrix_x4(a, qa + k0);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    unsigned int b[4];
                    ldmatrix_x4(b, kb + i * 8 * kld + k0);
                    mma_bf16(sacc[i], a, b[0], b[1]);
                    mma_bf16(sacc[i + 1], a, b[2], b[3]);
                }
            }
            // mask and scale in place; sacc[i][2 * half + e] is row half, key pg * 64 + 8 i + 2 t + e
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int n = pg * SB_PAGE + 8 * i + 2 * t + e;
                        const bool seen = r_valid[half] && n >= r_lo[half] && n <= r_pos[half];
                        const float sc = seen ? sacc[i][2 * half + e] * r_hs[half] - r_slope[half] * (float)(r_pos[half] - n) : -INFINITY;
                        sacc[i][2 * half + e] = sc;
                        mx[half] = fmaxf(mx[half], sc);
                    }
            float alpha[2], m_new[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
                mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
                m_new[half] = fmaxf(m_run[half], mx[half]);
                alpha[half] = m_new[half] == -INFINITY ? 1.f : expf(m_run[half] - m_new[half]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float wv = m_new[half] == -INFINITY ? 0.f : expf(sacc[i][2 * half + e] - m_new[half]);
                        sacc[i][2 * half + e] = wv;
                        sum[half] += wv;
                    }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                sum[half] += __shfl_xor_sync(0xffffffffu, sum[half], 1);
                sum[half] += __shfl_xor_sync(0xffffffffu, sum[half], 2);
                l_run[half] = l_run[half] * alpha[half] + sum[half];
                m_run[half] = m_new[half];
            }
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[i][0] *= alpha[0];
                acc[i][1] *= alpha[0];
                acc[i][2] *= alpha[1];
                acc[i][3] *= alpha[1];
            }
            const bf* vb = Vb + ((lane & 7) + ((lane >> 3) & 1) * 8) * vld + (lane >> 4) * 8;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {   // 16 keys at a time: the weights of score tiles 2 kk and 2 kk + 1 as one operand
                unsigned int ah[4], al[4];
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    const float w0 = sacc[2 * kk + (part >> 1)][2 * (part & 1)], w1 = sacc[2 * kk + (part >> 1)][2 * (part & 1) + 1];
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(w0, w1);
                    const float2 back = __bfloat1622float2(h2);
                    ah[part] = *reinterpret_cast<const unsigned int*>(&h2);
                    al[part] = pack_bf16(w0 - back.x, w1 - back.y);
                }
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    unsigned int b[4];
                    ldmatrix_x4_trans(b, vb + kk * 16 * vld + i * 8);
                    mma_bf16(acc[i], ah, b[0], b[1]);
                    mma_bf16(acc[i], al, b[0], b[1]);
                    mma_bf16(acc[i + 1], ah, b[2], b[3]);
                    mma_bf16(acc[i + 1], al, b[2], b[3]);
                }
            }
        }
        __syncthreads();   // the next turn overwrites this page's buffer
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        if (!r_valid[half]) continue;
        const int r = w * 16 + g + 8 * half;
        const long long grow = q0 + first + r / HG;
        float a = 1.f, l = l_run[half];
        if (p.sink != nullptr) {
            const float sk = p.sink[r_head[half]], mf = fmaxf(m_run[half], sk);
            a = expf(m_run[half] - mf);
            l = l * a + expf(sk - mf);
        }
        const float mul = a / l;
        bf* o = out + (grow * p.n_heads + r_head[half]) * VD;
#pragma unroll
        for (int i = 0; i < NT; ++i)
            *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + 2 * t) = __floats2bfloat162_rn(acc[i][2 * half] * mul, acc[i][2 * half + 1] * mul);
    }
}

static size_t flex_rows64_smem(int KD, int VD, int values_in_keys) {
    size_t b = (size_t)(FR_ROWS + 2 * FM_KEYS) * (KD + 8) * 2;
    if (!values_in_keys) b += (size_t)2 * FM_KEYS * (VD + 8) * 2;
    return b;
}

template <int VD>
static int launch_flex_rows64(SbFlex p, SbBatch batch, void* out, int max_q_len, int values_in_keys, cudaStream_t stream) {
    const size_t smem = flex_rows64_smem(p.k_dim, VD, values_in_keys);
    static size_t allowed = 0;
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(flex_attention_rows64_kernel<VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    const int HG = p.n_heads / p.n_kv_heads, QR = FR_ROWS / HG;
    const int tiles = (max_q_len + QR - 1) / QR;
    dim3 grid((unsigned int)(batch.n_seqs * tiles), (unsigned int)p.n_kv_heads, 1);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    sb_launch(flex_attention_rows64_kernel<VD>, grid, FM_THREADS, smem, stream, p, batch, (__nv_bfloat16*)out, tiles, values_in_keys);
    SB_LAUNCH_CHECK();
}

static size_t flex_mma_smem(int KD, int VD, int values_in_keys) {
    size_t b = (size_t)(FM_ROWS + 2 * FM_KEYS) * (KD + 8) * 2;
    if (!values_in_keys) b += (size_t)2 * FM_KEYS * (VD + 8) * 2;
    return b + FM_ROWS * FM_SLD * 4 + 2 * FM_ROWS * FM_PLD * 2 + 3 * FM_ROWS * 4;
}

template <int VD>
static int launch_flex_mma(SbFlex p, SbBatch batch, void* out, int max_q_len, int n_splits, float* partial, int values_in_keys,
                           cudaStream_t stream) {
    const size_t smem = flex_mma_smem(p.k_dim, VD, values_in_keys);
    static size_t allowed = 0;
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(flex_attention_mma_kernel<VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    const int HG = p.n_heads / p.n_kv_heads, HGB = HG < FM_ROWS ? HG : FM_ROWS, QR = FM_ROWS / HGB;
    const int tiles = (max_q_len + QR - 1) / QR;
    dim3 grid((unsigned int)(batch.n_seqs * tiles), (unsigned int)(p.n_kv_heads * (HG / HGB)), (unsigned int)n_splits);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
    sb_launch(flex_attention_mma_kernel<VD>, grid, FM_THREADS, smem, stream, p, batch, (__nv_bfloat16*)out, tiles, n_splits, partial,
              values_in_keys);
    if (n_splits > 1)
        sb_launch(flex_merge_kernel, dim3(batch.n_rows, p.n_heads), 128, 0, stream, (const float*)partial, (__nv_bfloat16*)out, p.sink,
                  p.n_heads, n_splits, VD);
    SB_LAUNCH_CHECK();
}

extern "C" {

// Bytes of shared memory a block would ask for, or -1 for sizes the kernel does not take: key width a multiple of
// 16, value width 64, 128, 256 or 512, and 1, 2, 4, 8 or a multiple of 16 query heads per key/value head.
long long sb_flex_attention_mma_smem(int k_dim, int v_dim, int heads_per_kv, int values_in_keys) {
    if (k_dim % 16 || k_dim < 16) return -1;
    if (v_dim != 64 && v_dim != 128 && v_dim != 256 && v_dim != 512) return -1;
    if (!(heads_per_kv == 1 || heads_per_kv == 2 || heads_per_kv == 4 || heads_per_kv == 8 || (heads_per_kv > 0 && heads_per_kv % 16 == 0)))
        return -1;
    if (values_in_keys && v_dim > k_dim) return -1;
    return (long long)flex_mma_smem(k_dim, v_dim, values_in_keys);
}

// Bytes of shared memory a block of the kernel for prompts would ask for, or -1 for sizes it does not take: key width
// a multiple of 16, values of 64 or 128 columns, a number of query heads per key/value head that divides 64.
long long sb_flex_attention_rows64_smem(int k_dim, int v_dim, int heads_per_kv, int values_in_keys) {
    if (k_dim % 16 || k_dim < 16 || (v_dim != 64 && v_dim != 128)) return -1;
    if (heads_per_kv < 1 || heads_per_kv > 64 || 64 % heads_per_kv) return -1;
    if (values_in_keys && v_dim > k_dim) return -1;
    return (long long)flex_rows64_smem(k_dim, v_dim, values_in_keys);
}

int sb_flex_attention_rows64(SbFlex p, SbBatch batch, void* out, int max_q_len, int values_in_keys, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (sb_flex_attention_rows64_smem(p.k_dim, p.v_dim, p.n_heads / p.n_kv_heads, values_in_keys) < 0 || max_q_len < 1)
        return (int)cudaErrorInvalidValue;
    if (p.v_dim == 64) return launch_flex_rows64<64>(p, batch, out, max_q_len, values_in_keys, stream);
    return launch_flex_rows64<128>(p, batch, out, max_q_len, values_in_keys, stream);
}

// bfloat16 only.  partial: (rows * heads * n_splits * (v_dim + 2)) floats when n_splits > 1.
int sb_flex_attention_mma(SbFlex p, SbBatch batch, void* out, int max_q_len, int n_splits, float* partial, int values_in_keys,
                          cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (sb_flex_attention_mma_smem(p.k_dim, p.v_dim, p.n_heads / p.n_kv_heads, values_in_keys) < 0 || max_q_len < 1 || n_splits < 1)
        return (int)cudaErrorInvalidValue;
    switch (p.v_dim) {
        case 64: return launch_flex_mma<64>(p, batch, out, max_q_len, n_splits, partial, values_in_keys, stream);
        case 128: return launch_flex_mma<128>(p, batch, out, max_q_len, n_splits, partial, values_in_keys, stream);
        case 256: return launch_flex_mma<256>(p, batch, out, max_q_len, n_splits, partial, values_in_keys, stream);
        default: return launch_flex_mma<512>(p, batch, out, max_q_len, n_splits, partial, values_in_keys, stream);
    }
}

}  // extern "C"
