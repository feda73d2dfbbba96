// Attention through a cached latent on the tensor cores (bfloat16 operands, 32-bit accumulation and softmax).
// The cache row [latent | rotated key part] is key AND value: one shared-memory tile per 64 cached positions
// serves S = Q K^T over its whole width and O = P V over its first columns, so a position's row is fetched once
// for all heads of all the tokens of a tile. Queries arrive already in the latent space (latent_attention.cu).
//
//  * prompt portions: a CTA owns 64 rows, a row being one (token, head) of one request; key tiles of 64 through
//    the block table by cp.async, two in flight; online softmax; causal and window masks by absolute position;
//  * decoded tokens: a CTA owns up to 16 heads of one token; its four warps take 16 keys of every tile each and
//    merge through shared memory; long windows are split over CTAs and a second kernel merges the parts in a
//    fixed order.
//
// mma.sync m16n8k16 with ldmatrix from padded tiles; DKP = row width rounded up to 16 (the padding columns are
// zero in the tile and in the queries), DVP = the output columns computed (latent width rounded up).
#include "attention_common.cuh"

namespace {

constexpr int LM_BLOCK_N = 64;
constexpr int LM_WARPS = 4;

__device__ __forceinline__ void lm_cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int DKP> struct LTile {
    static constexpr int ROW_BYTES = DKP * 2 + 16;       // 4 mod 8 words: the rows of an 8x8 block fall into distinct banks
    static constexpr int BYTES = LM_BLOCK_N * ROW_BYTES;
    static constexpr int CPR = DKP / 8;
};

// Rows key0..key0+63 of the request into a tile; rows outside [lo, hi] or without a page, and columns beyond
// `width`, are zero.
template <int DKP>
__device__ __forceinline__ void lm_load_tile(unsigned char* tile, const __nv_bfloat16* __restrict__ pages, const int* __restrict__ bt,
                                             int page_size, int shift, int num_pages, int width, int key0, int lo, int hi, int tid) {
    constexpr int CPR = LTile<DKP>::CPR, TOTAL = LM_BLOCK_N * CPR;
#pragma unroll 2
    for (int i = tid; i < TOTAL; i += LM_WARPS * 32) {
        const int r = i / CPR, c = i - r * CPR;
        const int j = key0 + r;
        bool valid = (j >= lo) && (j <= hi) && (c * 8 < width);
        size_t off = 0;
        if (valid) {
            const int lp = shift >= 0 ? (j >> shift) : (j / page_size);
            const int slot = shift >= 0 ? (j & (page_size - 1)) : (j - lp * page_size);
            const int page = bt[lp];
            valid = page >= 0 && page < num_pages;
            if (valid) off = ((size_t)page * page_size + slot) * width + c * 8;
        }
        lm_cp_async_16(tile + r * LTile<DKP>::ROW_BYTES + c * 16, pages + off, valid);
    }
}

template <int DKP, int NT>
__device__ __forceinline__ void lm_qk(float (&s)[NT][4], const unsigned (&q)[DKP / 16][4], const unsigned char* tile, int row0, int lane) {
    const int mat = lane >> 3, rr = lane & 7;
    const int key_off = (mat >> 1) * 8 + rr, dim_off = (mat & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < DKP / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            unsigned b[4];
            ldmatrix_x4(b, tile + (row0 + np * 16 + key_off) * LTile<DKP>::ROW_BYTES + (kk * 16 + dim_off) * 2);
            mma_bf16(s[2 * np], q[kk], b[0], b[1]);
            mma_bf16(s[2 * np + 1], q[kk], b[2], b[3]);
        }
    }
}

template <int DKP, int DVP, int KB>
__device__ __forceinline__ void lm_pv(float (&o)[DVP / 8][4], const unsigned (&p)[KB][4], const unsigned char* tile, int row0, int lane) {
    const int mat = lane >> 3, rr = lane & 7;
    const int key_off = (mat & 1) * 8 + rr, dim_off = (mat >> 1) * 8;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
        for (int dp = 0; dp < DVP / 16; ++dp) {
            unsigned b[4];
            ldmatrix_x4_trans(b, tile + (row0 + kb * 16 + key_off) * LTile<DKP>::ROW_BYTES + (dp * 16 + dim_off) * 2);
            mma_bf16(o[2 * dp], p[kb], b[0], b[1]);
            mma_bf16(o[2 * dp + 1], p[kb], b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------ prompt portions
// grid: (row tiles of 64, requests). qa: [tokens, heads, DKP] bfloat16; out: [tokens, heads, rank] floats.
template <int DKP, int DVP>
__global__ void __launch_bounds__(LM_WARPS * 32, DKP <= 160 ? 3 : 2)
latent_prefill_mma_kernel(const __nv_bfloat16* __restrict__ qa, float* __restrict__ out, const int* __restrict__ q_start,
                          const int* __restrict__ ctx_lens, const int* __restrict__ block_table, int bt_stride, int page_size,
                          const __nv_bfloat16* __restrict__ pages, int num_pages, int heads, int rank, int width, float scale, int window,
                          const float* __restrict__ sink) {
        pdl_wait();      // everything this kernel reads may come from the kernel before
    extern __shared__ __align__(16) unsigned char smem[];
    const int req = blockIdx.y;
    const int row_begin = q_start[req], q_len = q_start[req + 1] - row_begin;
    const int rows_total = q_len * heads;
    // the tiles at a prompt's end see the most keys: they go first, the light ones fill the last wave
    const int row0 = (gridDim.x - 1 - blockIdx.x) * (LM_WARPS * 16);
    if (row0 >= rows_total) return;
    const int pos0 = ctx_lens[req] - q_len;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2;
    const int* bt = block_table + (size_t)req * bt_stride;
    const int shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    int vis_lo[2], vis_hi[2];
    const __nv_bfloat16* q_ptr[2];
    long long out_off[2];
    float sink2[2] = {0.f, 0.f};        // the head's sink in the units of the running maximum (log2)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + warp * 16 + g + 8 * r;
        if (row < rows_total) {
            const int ti = row / heads, head = row - ti * heads;
            if (sink != nullptr) sink2[r] = sink[head] * LOG2E;
            const int p = pos0 + ti;
            vis_hi[r] = p;
            vis_lo[r] = window > 0 ? max(0, p - window + 1) : 0;
            q_ptr[r] = qa + ((size_t)(row_begin + ti) * heads + head) * DKP;
            out_off[r] = ((long long)(row_begin + ti) * heads + head) * rank;
        } else {
            vis_hi[r] = -1; vis_lo[r] = 0; q_ptr[r] = nullptr; out_off[r] = -1;
        }
    }
    const int last_row = min(rows_total, row0 + LM_WARPS * 16) - 1;
    const int hi_cta = pos0 + last_row / heads;
    const int lo_cta = window > 0 ? max(0, pos0 + row0 / heads - window + 1) : 0;
    const int t_begin = lo_cta / LM_BLOCK_N, t_end = hi_cta / LM_BLOCK_N;

    unsigned q[DKP / 16][4];
    load_q<DKP>(q, q_ptr, lane);
    float o[DVP / 8][4];
#pragma unroll
    for (int d = 0; d < DVP / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale2 = scale * LOG2E;
    unsigned char* buf[2] = {smem, smem + LTile<DKP>::BYTES};

    lm_load_tile<DKP>(buf[0], pages, bt, page_size, shift, num_pages, width, t_begin * LM_BLOCK_N, lo_cta, hi_cta, tid);
    lm_commit();
    for (int tile = t_begin; tile <= t_end; ++tile) {
        const int cur = (tile - t_begin) & 1;
        if (tile < t_end)
            lm_load_tile<DKP>(buf[cur ^ 1], pages, bt, page_size, shift, num_pages, width, (tile + 1) * LM_BLOCK_N, lo_cta, hi_cta, tid);
        lm_commit();
        lm_wait<1>();
        __syncthreads();
        float s[LM_BLOCK_N / 8][4];
#pragma unroll
        for (int n = 0; n < LM_BLOCK_N / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        lm_qk<DKP, LM_BLOCK_N / 8>(s, q, buf[cur], 0, lane);
        unsigned p[LM_BLOCK_N / 16][4];
        softmax_block<DVP, LM_BLOCK_N / 8>(s, p, o, m_run, l_run, scale2, tile * LM_BLOCK_N, vis_lo, vis_hi, lane);
        lm_pv<DKP, DVP, LM_BLOCK_N / 16>(o, p, buf[cur], 0, lane);
        __syncthreads();
    }
    lm_wait<0>();
    pdl_launch_dependents();        // only now: the next kernel's blocks would take room from tiles still at work
    const int t = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (out_off[r] < 0) continue;
        float l = l_run[r], f = 1.0f;
        if (sink != nullptr) {      // one more term in the denominator, at the larger of the two maxima
            const float m_fin = fmaxf(m_run[r], sink2[r]);
            f = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_fin);
            l = l * f + exp2f(sink2[r] - m_fin);
        }
        const float inv = l > 0.f ? f / l : 0.f;
        float* orow = out + out_off[r];
#pragma unroll
        for (int d = 0; d < DVP / 8; ++d)
            if (d * 8 + 2 * t < rank)
                *reinterpret_cast<float2*>(orow + d * 8 + 2 * t) = make_float2(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------------ decoded tokens
// grid: (splits, tokens, groups of 16 heads). Every token has q_len 1; its position is ctx_len - 1.
// part_o: [tokens, heads, splits, DVP] floats, part_ml: [tokens, heads, splits, 2] (max in log2 units, sum).
template <int DKP, int DVP>
__global__ void __launch_bounds__(LM_WARPS * 32)
latent_decode_mma_kernel(const __nv_bfloat16* __restrict__ qa, float* __restrict__ out, const int* __restrict__ ctx_lens,
                         const int* __restrict__ block_table, int bt_stride, int page_size, const __nv_bfloat16* __restrict__ pages,
                         int num_pages, int heads, int rank, int width, float scale, int window, int splits,
                         float* __restrict__ part_o, float* __restrict__ part_ml, const float* __restrict__ sink) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    extern __shared__ __align__(16) unsigned char smem[];
    const int split = blockIdx.x, token = blockIdx.y, h0 = blockIdx.z * 16;
    const int n_rows = min(16, heads - h0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int p = ctx_lens[token] - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int* bt = block_table + (size_t)token * bt_stride;
    const int shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    const int t_first = lo / LM_BLOCK_N, t_last = p / LM_BLOCK_N;
    const int n_tiles = t_last - t_first + 1;
    const int per = (n_tiles + splits - 1) / splits;
    const int t_begin = t_first + split * per;
    const int t_end = min(t_last, t_begin + per - 1);

    int vis_lo[2] = {lo, lo}, vis_hi[2] = {g < n_rows ? p : -1, g + 8 < n_rows ? p : -1};
    const __nv_bfloat16* q_ptr[2] = {nullptr, nullptr};
    if (g < n_rows) q_ptr[0] = qa + ((size_t)token * heads + h0 + g) * DKP;
    if (g + 8 < n_rows) q_ptr[1] = qa + ((size_t)token * heads + h0 + g + 8) * DKP;
    unsigned q[DKP / 16][4];
    load_q<DKP>(q, q_ptr, lane);
    float o[DVP / 8][4];
#pragma unroll
    for (int d = 0; d < DVP / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale2 = scale * LOG2E;
    unsigned char* buf[2] = {smem, smem + LTile<DKP>::BYTES};
    if (t_begin <= t_end) lm_load_tile<DKP>(buf[0], pages, bt, page_size, shift, num_pages, width, t_begin * LM_BLOCK_N, lo, p, tid);
    lm_commit();
    if (t_begin + 1 <= t_end) lm_load_tile<DKP>(buf[1], pages, bt, page_size, shift, num_pages, width, (t_begin + 1) * LM_BLOCK_N, lo, p, tid);
    lm_commit();
    for (int tile = t_begin; tile <= t_end; ++tile) {
        const int cur = (tile - t_begin) & 1;
        lm_wait<1>();
        __syncthreads();
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
        lm_qk<DKP, 2>(s, q, buf[cur], warp * 16, lane);
        unsigned pf[1][4];
        softmax_block<DVP, 2>(s, pf, o, m_run, l_run, scale2, tile * LM_BLOCK_N + warp * 16, vis_lo, vis_hi, lane);
        lm_pv<DKP, DVP, 1>(o, pf, buf[cur], warp * 16, lane);
        __syncthreads();
        if (tile + 2 <= t_end) lm_load_tile<DKP>(buf[cur], pages, bt, page_size, shift, num_pages, width, (tile + 2) * LM_BLOCK_N, lo, p, tid);
        lm_commit();
    }
    lm_wait<0>();
    __syncthreads();
    // merge the four warps through shared memory (the tiles are no longer needed), warps in ascending order
    constexpr int MS = DVP + 4;
    float* sm_o = reinterpret_cast<float*>(smem);                 // [WARPS][16][MS]
    float* sm_ml = sm_o + LM_WARPS * 16 * MS;                     // [WARPS][16][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
#pragma unroll
        for (int d = 0; d < DVP / 8; ++d)
            *reinterpret_cast<float2*>(&sm_o[(warp * 16 + row) * MS + d * 8 + 2 * t]) = make_float2(o[d][2 * r], o[d][2 * r + 1]);
        if (t == 0) {
            sm_ml[(warp * 16 + row) * 2] = m_run[r];
            sm_ml[(warp * 16 + row) * 2 + 1] = l_run[r];
        }
    }
    __syncthreads();
    for (int i = tid; i < n_rows * DVP; i += LM_WARPS * 32) {
        const int row = i / DVP, d = i - row * DVP;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < LM_WARPS; ++w) m = fmaxf(m, sm_ml[(w * 16 + row) * 2]);
        float l = 0.f, acc = 0.f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < LM_WARPS; ++w) {
                const float mw = sm_ml[(w * 16 + row) * 2];
                const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
                l += sm_ml[(w * 16 + row) * 2 + 1] * f;
                acc += sm_o[(w * 16 + row) * MS + d] * f;
            }
        }
        const int head = h0 + row;
        if (splits == 1) {
            if (sink != nullptr) {
                const float s2 = sink[head] * LOG2E, m_fin = fmaxf(m, s2);
                const float f = (m == -INFINITY) ? 0.f : exp2f(m - m_fin);
                l = l * f + exp2f(s2 - m_fin);
                acc *= f;
            }
            if (d < rank) out[((size_t)token * heads + head) * rank + d] = l > 0.f ? acc / l : 0.f;
        } else {
            const size_t slot = ((size_t)token * heads + head) * splits + split;
            part_o[slot * DVP + d] = acc;
            if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
        }
    }
}

// Merges the splits of every (token, head) in split order. One block per (token, head): every warp finds the maximum
// and the denominator for itself (lanes over the splits) and keeps the splits' factors in shared memory; then a thread
// owns an output column and adds the splits' parts in ascending order, eight loads in flight.
constexpr int LM_FACTORS = 64;      // splits whose factors are kept; beyond, a factor is computed where it is used

__global__ void __launch_bounds__(128)
latent_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, float* __restrict__ out,
                             int rows, int splits, int dvp, int rank, const float* __restrict__ sink, int heads) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float fac[4][LM_FACTORS];
    const int w = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (w >= rows) return;
    const float* ml = part_ml + (size_t)w * splits * 2;
    float m = -INFINITY;
    for (int s = lane; s < splits; s += 32) m = fmaxf(m, ml[2 * s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float sink2 = sink != nullptr ? sink[w % heads] * LOG2E : -INFINITY;
    m = fmaxf(m, sink2);        // the sink is one more part: a sum of exp(sink) at its own maximum, no output
    float l = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 32) {       // lane sums in split order within its stride; the warp sum is a fixed tree
        const int s = s0 + lane;
        float f = 0.f;
        if (s < splits) {
            const float ms = ml[2 * s];
            if (ms != -INFINITY) f = exp2f(ms - m);
            l += ml[2 * s + 1] * f;
            if (s < LM_FACTORS) fac[warp][s] = f;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (sink != nullptr) l += exp2f(sink2 - m);
    __syncwarp();
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    const float* po = part_o + (size_t)w * splits * dvp;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            float f;
            if (s < LM_FACTORS) f = fac[warp][s];
            else { const float ms = ml[2 * s]; f = ms != -INFINITY ? exp2f(ms - m) : 0.f; }
            acc = fmaf(po[(size_t)s * dvp + d], f, acc);
        }
        out[(size_t)w * rank + d] = acc * inv;
    }
}

template <int DKP, int DVP>
int lm_launch(bool decode, const __nv_bfloat16* qa, float* out, const int* q_start, const int* ctx_lens, const int* bt, int bt_stride,
              int page_size, const __nv_bfloat16* pages, int num_pages, int requests, int max_q_len, int heads, int rank, int width,
              float scale, int window, int splits, float* part_o, float* part_ml, const float* sink, cudaStream_t stream) {
    if (!decode) {
        const size_t smem = 2 * (size_t)LTile<DKP>::BYTES;
        NIB_CUDA(cudaFuncSetAttribute(latent_prefill_mma_kernel<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const dim3 grid(ceil_div((long long)max_q_len * heads, LM_WARPS * 16), requests);
        NIB_CUDA(launch_pdl(latent_prefill_mma_kernel<DKP, DVP>, dim3(grid), dim3(LM_WARPS * 32), (size_t)(smem), stream, qa, out, q_start, ctx_lens, bt, bt_stride, page_size,
                                                                                   pages, num_pages, heads, rank, width, scale, window, sink));
        NIB_LAUNCH_CHECK();
        return 0;
    }
    size_t smem = 2 * (size_t)LTile<DKP>::BYTES;
    const size_t merge = (size_t)LM_WARPS * 16 * (DVP + 4 + 2) * sizeof(float);
    if (merge > smem) smem = merge;
    NIB_CUDA(cudaFuncSetAttribute(latent_decode_mma_kernel<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid(splits, requests, ceil_div(heads, 16));
    NIB_CUDA(launch_pdl(latent_decode_mma_kernel<DKP, DVP>, dim3(grid), dim3(LM_WARPS * 32), (size_t)(smem), stream, qa, out, ctx_lens, bt, bt_stride, page_size, pages, num_pages,
                                                                              heads, rank, width, scale, window, splits, part_o, part_ml, sink));
    NIB_LAUNCH_CHECK();
    if (splits > 1) {
        const int rows = requests * heads;
        NIB_CUDA(launch_pdl(latent_decode_combine_kernel, dim3(rows), dim3(128), (size_t)(0), stream, part_o, part_ml, out, rows, splits, DVP, rank, sink, heads));
        NIB_LAUNCH_CHECK();
    }
    return 0;
}

// the output columns computed for a latent of `rank` columns in a tile of dkp columns
int lm_dvp(int rank, int dkp) {
    for (int v : {32, 64, 128})
        if (rank <= v && v <= dkp) return v;
    return dkp;
}

// ------------------------------------------------------------------------------------------ per-head products
// The two maps between a head's own space and the latent space, for many tokens at once: one small matrix per head,
// 16 tokens per warp, the head's matrix staged in shared memory 64 output columns at a time. A comes from 32-bit
// activations, rounded to bfloat16 as it is put into fragments.
__device__ __forceinline__ void lm_a_from_f32(unsigned (&a)[4], const float* const (&row)[2], int k0, int k, int lane) {
    const int t = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (row[r]) {
            const int c = k0 + 2 * t;
            if (c < k) v[0] = row[r][c];
            if (c + 1 < k) v[1] = row[r][c + 1];
            if (c + 8 < k) v[2] = row[r][c + 8];
            if (c + 9 < k) v[3] = row[r][c + 9];
        }
        a[r] = pack_bf16(v[0], v[1]);
        a[2 + r] = pack_bf16(v[2], v[3]);
    }
}

// out[t, h, n] = sum_k a[t, h, k] * w[h, n, k] (w: [heads, n, k] bfloat16, its rows are the output features).
// grid: (token tiles of 64, heads). a: floats, `lda` elements per token, the head's k values at h * k.
// TO: bfloat16, or float with an optional bias [heads, n]. The head's n outputs of token t start at
// out + t * ldo + h * out_head_stride.
template <int KP, typename TO>
__global__ void __launch_bounds__(LM_WARPS * 32)
head_product_nk_kernel(const float* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w, const float* __restrict__ bias,
                       TO* __restrict__ out, int ldo, long long out_head_stride, int tokens, int n, int k,
                       const float* __restrict__ gate, int ldg) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const float* row[2];
    int tok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tok[r] = blockIdx.x * (LM_WARPS * 16) + warp * 16 + g + 8 * r;
        row[r] = tok[r] < tokens ? a + (size_t)tok[r] * lda + (size_t)h * k : nullptr;
    }
    unsigned af[KP / 16][4];
#pragma unroll
    for (int kk = 0; kk < KP / 16; ++kk) lm_a_from_f32(af[kk], row, kk * 16, k, lane);
    const __nv_bfloat16* wh = w + (size_t)h * n * k;
    for (int n0 = 0; n0 < n; n0 += LM_BLOCK_N) {
        __syncthreads();
        constexpr int CPR = LTile<KP>::CPR;
        for (int i = tid; i < LM_BLOCK_N * CPR; i += LM_WARPS * 32) {
            const int r = i / CPR, c = i - r * CPR;
            const bool valid = n0 + r < n && c * 8 < k;
            lm_cp_async_16(smem + r * LTile<KP>::ROW_BYTES + c * 16, wh + (valid ? (size_t)(n0 + r) * k + c * 8 : 0), valid);
        }
        lm_commit();
        lm_wait<0>();
        __syncthreads();
        float s[LM_BLOCK_N / 8][4];
#pragma unroll
        for (int j = 0; j < LM_BLOCK_N / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
        lm_qk<KP, LM_BLOCK_N / 8>(s, af, smem, 0, lane);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (tok[r] >= tokens) continue;
            TO* o = out + (size_t)tok[r] * ldo + (size_t)h * out_head_stride + n0;
#pragma unroll
            for (int j = 0; j < LM_BLOCK_N / 8; ++j) {
                const int f = n0 + j * 8 + 2 * t4;
                if (f >= n) continue;
                if constexpr (sizeof(TO) == 2) {
                    float v0 = s[j][2 * r], v1 = s[j][2 * r + 1];
                    if (gate != nullptr) {      // times sigmoid(gate) at the output's own place (heads side by side, n wide)
                        const float* gr = gate + (size_t)tok[r] * ldg + (size_t)h * n + f;
                        v0 *= 1.0f / (1.0f + expf(-gr[0]));
                        v1 *= 1.0f / (1.0f + expf(-gr[1]));
                    }
                    *reinterpret_cast<unsigned*>(o + j * 8 + 2 * t4) = pack_bf16(v0, v1);
                } else {
                    const float b0 = bias ? bias[(size_t)h * n + f] : 0.f, b1 = bias ? bias[(size_t)h * n + f + 1] : 0.f;
                    *reinterpret_cast<float2*>(o + j * 8 + 2 * t4) = make_float2(s[j][2 * r] + b0, s[j][2 * r + 1] + b1);
                }
            }
        }
    }
}

// qa[t, h, c] = sum_d q[t, h, d] * w[h, d, c] for c < n (w: [heads, k, n] bfloat16, its rows are the inputs), then the
// rotated part: qa[t, h, n + 2i], [.. + 1] = the pair q[t, h, k + 2i], [.. + 1] turned by position * freq[i] (with
// half_layout the pair is i, i + rot/2), and zeros up to ldq. grid: (token tiles of 64, heads). q: floats, `ldq_in` elements per token, a head's k + rot values together.
template <int KP>
__global__ void __launch_bounds__(LM_WARPS * 32)
head_product_kn_kernel(const float* __restrict__ q, int ldq_in, const __nv_bfloat16* __restrict__ w, const float* __restrict__ freq,
                       float mag, const int* __restrict__ positions, __nv_bfloat16* __restrict__ qa, int ldq, int tokens, int heads,
                       int n, int k, int rot, int half_layout) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const float* row[2];
    int tok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tok[r] = blockIdx.x * (LM_WARPS * 16) + warp * 16 + g + 8 * r;
        row[r] = tok[r] < tokens ? q + (size_t)tok[r] * ldq_in + (size_t)h * (k + rot) : nullptr;
    }
    unsigned af[KP / 16][4];
#pragma unroll
    for (int kk = 0; kk < KP / 16; ++kk) lm_a_from_f32(af[kk], row, kk * 16, k, lane);
    const __nv_bfloat16* wh = w + (size_t)h * k * n;
    for (int n0 = 0; n0 < n; n0 += LM_BLOCK_N) {
        __syncthreads();
        constexpr int CPR = LM_BLOCK_N / 8;         // a tile row holds 64 output columns of one input d
        for (int i = tid; i < KP * CPR; i += LM_WARPS * 32) {
            const int d = i / CPR, c = i - d * CPR;
            const bool valid = d < k && n0 + c * 8 < n;
            lm_cp_async_16(smem + d * LTile<LM_BLOCK_N>::ROW_BYTES + c * 16, wh + (valid ? (size_t)d * n + n0 + c * 8 : 0), valid);
        }
        lm_commit();
        lm_wait<0>();
        __syncthreads();
        float o[LM_BLOCK_N / 8][4];
#pragma unroll
        for (int j = 0; j < LM_BLOCK_N / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
        lm_pv<LM_BLOCK_N, LM_BLOCK_N, KP / 16>(o, af, smem, 0, lane);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (tok[r] >= tokens) continue;
            __nv_bfloat16* dst = qa + ((size_t)tok[r] * heads + h) * ldq + n0;
#pragma unroll
            for (int j = 0; j < LM_BLOCK_N / 8; ++j)
                if (n0 + j * 8 + 2 * t4 < n)
                    *reinterpret_cast<unsigned*>(dst + j * 8 + 2 * t4) = pack_bf16(o[j][2 * r], o[j][2 * r + 1]);
        }
    }
    // the rotated part and the padding of the warp's 16 rows
    for (int rr = 0; rr < 16; ++rr) {
        const int token = blockIdx.x * (LM_WARPS * 16) + warp * 16 + rr;
        if (token >= tokens) break;
        const float* qr = q + (size_t)token * ldq_in + (size_t)h * (k + rot) + k;
        __nv_bfloat16* dst = qa + ((size_t)token * heads + h) * ldq + n;
        const float pos = (float)positions[token];
        for (int i = lane; i < rot / 2; i += 32) {
            const float ang = pos * freq[i];
            const float cs = cosf(ang) * mag, sn = sinf(ang) * mag;
            const int ia = half_layout ? i : 2 * i, ib = half_layout ? i + rot / 2 : 2 * i + 1;
            const float x = qr[ia], y = qr[ib];
            dst[ia] = __float2bfloat16_rn(x * cs - y * sn);
            dst[ib] = __float2bfloat16_rn(y * cs + x * sn);
        }
        for (int c = n + rot + lane; c < ldq; c += 32) qa[((size_t)token * heads + h) * ldq + c] = __float2bfloat16_rn(0.f);
    }
}

}  // namespace

// 1 if the tensor-core kernels take this shape: rows of up to 192 elements whose byte size is a multiple of 16.
NIB_API int nib_latent_attention_mma_supported(int rank, int rot) {
    const int width = rank + rot;
    return (width % 8 == 0 && rank % 8 == 0 && width >= 16 && width <= 192) ? 1 : 0;
}

// The padded query row width the kernels read (zeros beyond rank + rot).
NIB_API int nib_latent_attention_mma_qwidth(int rank, int rot) { return (rank + rot + 15) / 16 * 16; }

// decode != 0: every request brings one token (q_start is not read); part_o / part_ml: scratch for splits > 1;
// sink: nullptr, or one number per head whose exponential joins every row's softmax denominator
// ([requests, heads, splits, dvp] and [requests, heads, splits, 2] floats, dvp <= 192).
NIB_API int nib_latent_attention_mma(int decode, const void* qa, void* out, const int* q_start, const int* ctx_lens,
                                     const int* block_table, int bt_stride, int page_size, const void* pages, int num_pages,
                                     int requests, int max_q_len, int heads, int rank, int rot, float scale, int window,
                                     int splits, float* part_o, float* part_ml, const float* sink, cudaStream_t stream) {
    NIB_REQUIRE(nib_latent_attention_mma_supported(rank, rot) == 1, "latent attention (tensor cores): latent %d + %d is not supported", rank, rot);
    NIB_REQUIRE(requests >= 0 && heads > 0 && page_size > 0 && num_pages > 0 && window >= 0 && splits >= 1, "latent attention (tensor cores): bad sizes");
    NIB_REQUIRE(!decode || splits == 1 || (part_o != nullptr && part_ml != nullptr), "latent attention (tensor cores): splits need scratch");
    if (requests == 0 || max_q_len == 0) return 0;
    const int width = rank + rot, dkp = nib_latent_attention_mma_qwidth(rank, rot), dvp = lm_dvp(rank, dkp);
#define NIB_LM(DKP, DVP)                                                                                                          \
    if (dkp == DKP && dvp == DVP)                                                                                                 \
        return lm_launch<DKP, DVP>(decode != 0, (const __nv_bfloat16*)qa, (float*)out, q_start, ctx_lens, block_table,   \
                                   bt_stride, page_size, (const __nv_bfloat16*)pages, num_pages, requests, max_q_len, heads, rank, \
                                   width, scale, window, splits, part_o, part_ml, sink, stream);
    NIB_LM(16, 16) NIB_LM(32, 32) NIB_LM(48, 32) NIB_LM(48, 48) NIB_LM(64, 32) NIB_LM(64, 64) NIB_LM(80, 32) NIB_LM(80, 64) NIB_LM(80, 80)
    NIB_LM(96, 32) NIB_LM(96, 64) NIB_LM(96, 96) NIB_LM(112, 32) NIB_LM(112, 64) NIB_LM(112, 112) NIB_LM(128, 32) NIB_LM(128, 64) NIB_LM(128, 128)
    NIB_LM(144, 64) NIB_LM(144, 128) NIB_LM(160, 64) NIB_LM(160, 128) NIB_LM(176, 64) NIB_LM(176, 128) NIB_LM(192, 64) NIB_LM(192, 128)
    NIB_LM(144, 32) NIB_LM(160, 32) NIB_LM(176, 32) NIB_LM(192, 32) NIB_LM(144, 144) NIB_LM(160, 160) NIB_LM(176, 176) NIB_LM(192, 192)
#undef NIB_LM
    NIB_REQUIRE(false, "latent attention (tensor cores): no kernel for a row of %d and a latent of %d", dkp, dvp);
    return 0;
}

// 1 if the per-head products on the tensor cores take these sizes (k: the contraction, n: the output columns).
NIB_API int nib_head_product_supported(int kn_layout, int k, int n) {
    if (kn_layout) return (k >= 1 && k <= 128 && n % 8 == 0 && n >= 8) ? 1 : 0;
    return (k % 8 == 0 && k >= 8 && k <= 192 && n % 2 == 0 && n >= 2) ? 1 : 0;
}

// out[t, h, :n] = a[t, h, :k] . w[h]^T (+ bias[h]), w: [heads, n, k]: values out of the latent space (k = latent,
// n = value width, bfloat16 out), or the gates of a block-diagonal map (float out with bias, out_f32 != 0). The head's
// outputs of token t start at out + t * ldo + h * out_head_stride (elements).
NIB_API int nib_head_product_nk(const float* a, int lda, const void* w, const float* bias, void* out, int ldo,
                                long long out_head_stride, int out_f32, int tokens, int heads, int n, int k, const float* gate, int ldg,
                                cudaStream_t stream) {
    NIB_REQUIRE(nib_head_product_supported(0, k, n) == 1 && tokens >= 0 && heads > 0, "per-head product: sizes k=%d n=%d are not supported", k, n);
    NIB_REQUIRE(gate == nullptr || !out_f32, "per-head product: the gate goes with outputs in the storage type");
    if (tokens == 0) return 0;
    const dim3 grid(ceil_div(tokens, LM_WARPS * 16), heads);
    const int kp = (k + 15) / 16 * 16;
#define NIB_HP(KP)                                                                                                                  \
    if (kp == KP) {                                                                                                                 \
        if (out_f32)                                                                                                                \
            NIB_CUDA(launch_pdl(head_product_nk_kernel<KP, float>, grid, dim3(LM_WARPS * 32), (size_t)LTile<KP>::BYTES, stream, a, lda, \
                                (const __nv_bfloat16*)w, bias, (float*)out, ldo, out_head_stride, tokens, n, k, gate, ldg));       \
        else                                                                                                                        \
            NIB_CUDA(launch_pdl(head_product_nk_kernel<KP, __nv_bfloat16>, grid, dim3(LM_WARPS * 32), (size_t)LTile<KP>::BYTES, stream, a, lda, \
                                (const __nv_bfloat16*)w, bias, (__nv_bfloat16*)out, ldo, out_head_stride, tokens, n, k, gate, ldg)); \
        return 0;                                                                                                                   \
    }
    NIB_HP(16) NIB_HP(32) NIB_HP(48) NIB_HP(64) NIB_HP(80) NIB_HP(96) NIB_HP(112) NIB_HP(128) NIB_HP(144) NIB_HP(160) NIB_HP(176) NIB_HP(192)
#undef NIB_HP
    NIB_REQUIRE(false, "per-head product: k=%d", k);
    return 0;
}

// qa[t, h] = [q[t, h, :k] . w[h] | q[t, h, k:] rotated | zeros], w: [heads, k, n] (queries into the latent space:
// k = the head's plain width, n = latent); qa: bfloat16 rows of ldq elements per (token, head).
NIB_API int nib_head_product_kn(const float* q, int ldq_in, const void* w, const float* freq, float mag, const int* positions,
                                void* qa, int ldq, int tokens, int heads, int n, int k, int rot, int half_layout, cudaStream_t stream) {
    NIB_REQUIRE(nib_head_product_supported(1, k, n) == 1 && tokens >= 0 && heads > 0 && rot % 2 == 0 && ldq >= n + rot,
                "per-head product: sizes k=%d n=%d are not supported", k, n);
    if (tokens == 0) return 0;
    const dim3 grid(ceil_div(tokens, LM_WARPS * 16), heads);
    const int kp = (k + 15) / 16 * 16;
#define NIB_HP(KP)                                                                                                                   \
    if (kp == KP) {                                                                                                                  \
        NIB_CUDA(launch_pdl(head_product_kn_kernel<KP>, grid, dim3(LM_WARPS * 32), (size_t)(KP * LTile<LM_BLOCK_N>::ROW_BYTES), stream, \
                            q, ldq_in, (const __nv_bfloat16*)w, freq, mag, positions, (__nv_bfloat16*)qa, ldq, tokens, heads, n, k, rot, half_layout)); \
        return 0;                                                                                                                    \
    }
    NIB_HP(16) NIB_HP(32) NIB_HP(48) NIB_HP(64) NIB_HP(80) NIB_HP(96) NIB_HP(112) NIB_HP(128)
#undef NIB_HP
    NIB_REQUIRE(false, "per-head product: k=%d", k);
    return 0;
}
