// Softmax attention with options on the tensor cores (bfloat16, mma.sync m16n8k16): the same mathematics as
// attention_flex.cu for keys of up to 128 and values of up to 128 elements (multiples of 8, the two may differ), any
// mix of prompt portions and decoded tokens.
//
// grid: (row tiles of 64, requests, kv heads); the rows of a request and kv head are r = token * n_rep + g, so keys and
// values are read once per kv head. Key tiles of 64 come through the block table by cp.async into padded shared-memory
// tiles, two in flight; a head narrower than the tile's 64 or 128 columns is filled up with zeros on the way (the
// products then add zeros). Scores leave the tensor cores as floats: scale, soft cap, distance bias and the masks
// (causal, window, chunk; all by absolute position) are applied in 32-bit, then the online softmax of
// attention_common.cuh. Key tiles start at absolute multiples of 64, so a position's result does not depend on what else
// is in the batch; it depends on the cut only through which rows share a tile, i.e. by rounding. With `sinks` the
// denominator of a row of head h holds exp(sinks[h]) once more (no key, no value): it enters where a row is normalized,
// here or, with split keys, in the merge.
#include "attention_common.cuh"

namespace {

constexpr int FB_N = 64;     // keys per tile
constexpr int FWARPS = 4;

__device__ __forceinline__ void fx_cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void fx_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void fx_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// FB_N rows of D bfloat16, each padded by 16 bytes (the eight rows of an ldmatrix block then fall into distinct banks).
template <int D> struct FxTile {
    static constexpr int ROW_BYTES = D * 2 + 16;
    static constexpr int BYTES = FB_N * ROW_BYTES;
    static constexpr int CPR = D / 8;            // 16-byte chunks per row
};

// Rows key0..key0+63 of one kv head of a paged tensor whose rows hold `width` <= D elements; rows outside [lo, hi] or
// without a page, and the columns from `width` on, are zero.
template <int D>
__device__ __forceinline__ void fx_load_tile(unsigned char* tile, const __nv_bfloat16* __restrict__ pages, int width,
                                             const int* __restrict__ bt, int page_size, int num_pages, int kv_heads, int kvh,
                                             int key0, int lo, int hi, int tid) {
    constexpr int CPR = FxTile<D>::CPR;
    for (int i = tid; i < FB_N * CPR; i += FWARPS * 32) {
        const int r = i / CPR, c = i - r * CPR;
        const int j = key0 + r;
        bool valid = (j >= lo) && (j <= hi) && (c * 8 < width);
        size_t off = 0;
        if (valid) {
            const int lp = j / page_size;
            const int page = bt[lp];
            valid = page >= 0 && page < num_pages;
            if (valid) off = (((size_t)page * kv_heads + kvh) * page_size + (j - lp * page_size)) * width + c * 8;
        }
        fx_cp_async_16(tile + r * FxTile<D>::ROW_BYTES + c * 16, pages + off, valid);
    }
}

// S[16 x 64] += Q[16 x D] . K^T
template <int D>
__device__ __forceinline__ void fx_qk(float (&s)[FB_N / 8][4], const unsigned (&q)[D / 16][4], const unsigned char* k_tile, int lane) {
    const int mat = lane >> 3, rr = lane & 7;
    const int key_off = (mat >> 1) * 8 + rr, dim_off = (mat & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < FB_N / 16; ++np) {
            unsigned b[4];
            ldmatrix_x4(b, k_tile + (np * 16 + key_off) * FxTile<D>::ROW_BYTES + (kk * 16 + dim_off) * 2);
            mma_bf16(s[2 * np], q[kk], b[0], b[1]);
            mma_bf16(s[2 * np + 1], q[kk], b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x 64] . V
template <int D>
__device__ __forceinline__ void fx_pv(float (&o)[D / 8][4], const unsigned (&p)[FB_N / 16][4], const unsigned char* v_tile, int lane) {
    const int mat = lane >> 3, rr = lane & 7;
    const int key_off = (mat & 1) * 8 + rr, dim_off = (mat >> 1) * 8;
#pragma unroll
    for (int kb = 0; kb < FB_N / 16; ++kb) {
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            unsigned b[4];
            ldmatrix_x4_trans(b, v_tile + (kb * 16 + key_off) * FxTile<D>::ROW_BYTES + (dp * 16 + dim_off) * 2);
            mma_bf16(o[2 * dp], p[kb], b[0], b[1]);
            mma_bf16(o[2 * dp + 1], p[kb], b[2], b[3]);
        }
    }
}

template <typename TO> __device__ __forceinline__ void fx_store2(TO* p, float a, float b);
template <> __device__ __forceinline__ void fx_store2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <> __device__ __forceinline__ void fx_store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<unsigned*>(p) = pack_bf16(a, b);
}

template <int DKP, int DVP, typename TO>
__global__ void __launch_bounds__(FWARPS * 32)
attention_flex_mma_kernel(const __nv_bfloat16* __restrict__ q_in, int q_stride, TO* __restrict__ out,
                          const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
                          const int* __restrict__ block_table, int bt_stride, int page_size,
                          const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages, int num_pages,
                          int heads, int kv_heads, int dk, int dv, float scale, float softcap, const float* __restrict__ slopes,
                          int window, int chunk, float out_scale, int splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                          const float* __restrict__ sinks) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int req = blockIdx.y, kvh = blockIdx.z;
    const int n_rep = heads / kv_heads;
    const int row_begin = q_start[req], q_len = q_start[req + 1] - row_begin;
    const int rows_total = q_len * n_rep;
    // splits > 1 (steps of a few tokens per request: all rows fit one tile): blockIdx.x is a share of the key tiles
    const int split = splits > 1 ? blockIdx.x : 0;
    // the last row tiles of a prompt see the most keys: they start first, so that the kernel does not end on its longest CTA
    const int row0 = splits > 1 ? 0 : (gridDim.x - 1 - blockIdx.x) * (FWARPS * 16);
    if (row0 >= rows_total) return;
    const int ctx = ctx_lens[req];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2;
    if (ctx <= 0) {                                   // a padding row of a replayed step: shares that hold nothing
        if (splits > 1)
            for (int row = tid; row < rows_total; row += FWARPS * 32) {
                const int ti = row / n_rep, head = kvh * n_rep + (row - ti * n_rep);
                const size_t slot = ((size_t)(row_begin + ti) * heads + head) * splits + split;
                part_ml[slot * 2] = -INFINITY;
                part_ml[slot * 2 + 1] = 0.f;
            }
        return;
    }
    const int pos0 = ctx - q_len;                     // position of the request's first token in this step
    const int* bt = block_table + (size_t)req * bt_stride;

    auto first_visible = [&](int p) {
        int lo = window > 0 ? max(0, p - window + 1) : 0;
        if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
        return lo;
    };
    int vis_lo[2], vis_hi[2];
    float slope2[2], sink2[2];
    const __nv_bfloat16* q_ptr[2];
    long long out_off[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + warp * 16 + g + 8 * r;
        if (row < rows_total) {
            const int ti = row / n_rep, head = kvh * n_rep + (row - ti * n_rep);
            const int p = pos0 + ti;
            vis_hi[r] = p;
            vis_lo[r] = first_visible(p);
            slope2[r] = slopes != nullptr ? slopes[head] * LOG2E : 0.f;
            sink2[r] = sinks != nullptr ? sinks[head] * LOG2E : -INFINITY;
            q_ptr[r] = q_in + (size_t)(row_begin + ti) * q_stride + (size_t)head * dk;
            out_off[r] = ((long long)(row_begin + ti) * heads + head) * dv;
        } else {
            vis_hi[r] = -1; vis_lo[r] = 0; slope2[r] = 0.f; sink2[r] = -INFINITY; q_ptr[r] = nullptr; out_off[r] = -1;
        }
    }
    // key range of the whole CTA: the first visible key does not decrease with the position
    const int last_row = min(rows_total, row0 + FWARPS * 16) - 1;
    const int hi_cta = pos0 + last_row / n_rep;
    const int lo_cta = first_visible(pos0 + row0 / n_rep);
    int t_begin = lo_cta / FB_N, t_end = hi_cta / FB_N;
    if (splits > 1) {       // this CTA's share of the tiles; it may be empty
        const int per = (t_end - t_begin + splits) / splits;
        t_begin += split * per;
        t_end = min(t_end, t_begin + per - 1);
    }

    pdl_wait();     // queries, and the keys and values of this step's tokens, come from the kernels before
    unsigned q[DKP / 16][4];
    {
        const int t = lane & 3;
#pragma unroll
        for (int kk = 0; kk < DKP / 16; ++kk) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                unsigned lo = 0u, hi = 0u;
                if (q_ptr[r]) {
                    if (kk * 16 < dk) lo = *reinterpret_cast<const unsigned*>(q_ptr[r] + kk * 16 + 2 * t);
                    if (kk * 16 + 8 < dk) hi = *reinterpret_cast<const unsigned*>(q_ptr[r] + kk * 16 + 8 + 2 * t);
                }
                q[kk][r] = lo;
                q[kk][2 + r] = hi;
            }
        }
    }
    float o[DVP / 8][4];
#pragma unroll
    for (int d = 0; d < DVP / 8; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;

    unsigned char* k_buf[2] = {smem, smem + FxTile<DKP>::BYTES};
    unsigned char* v_buf[2] = {smem + 2 * FxTile<DKP>::BYTES, smem + 2 * FxTile<DKP>::BYTES + FxTile<DVP>::BYTES};

    if (t_begin <= t_end) {
        fx_load_tile<DKP>(k_buf[0], k_pages, dk, bt, page_size, num_pages, kv_heads, kvh, t_begin * FB_N, lo_cta, hi_cta, tid);
        fx_load_tile<DVP>(v_buf[0], v_pages, dv, bt, page_size, num_pages, kv_heads, kvh, t_begin * FB_N, lo_cta, hi_cta, tid);
    }
    fx_commit();

    for (int tile = t_begin; tile <= t_end; ++tile) {
        const int cur = (tile - t_begin) & 1;
        if (tile < t_end) {
            fx_load_tile<DKP>(k_buf[cur ^ 1], k_pages, dk, bt, page_size, num_pages, kv_heads, kvh, (tile + 1) * FB_N, lo_cta, hi_cta, tid);
            fx_load_tile<DVP>(v_buf[cur ^ 1], v_pages, dv, bt, page_size, num_pages, kv_heads, kvh, (tile + 1) * FB_N, lo_cta, hi_cta, tid);
        }
        fx_commit();
        fx_wait<1>();
        __syncthreads();

        float s[FB_N / 8][4];
#pragma unroll
        for (int n = 0; n < FB_N / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        fx_qk<DKP>(s, q, k_buf[cur], lane);
        // scale, cap and distance bias in 32-bit, into base-2 units; the masks follow in softmax_block
        {
            const int t = lane & 3;
#pragma unroll
            for (int n = 0; n < FB_N / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const int key = tile * FB_N + n * 8 + 2 * t + (e & 1);
                    float x = s[n][e] * scale;
                    // tanh(y) = 1 - 2 / (1 + e^(2y)) with the fast exponential and division: off by a few 1e-7 in absolute
                    // terms, far below the rounding of the probabilities to bfloat16 that follows
                    if (softcap > 0.f) x = softcap * (1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x * inv_cap)));
                    s[n][e] = fmaf(x, LOG2E, -slope2[r] * (float)(vis_hi[r] - key));
                }
            }
        }
        unsigned p[FB_N / 16][4];
        softmax_block<DVP, FB_N / 8>(s, p, o, m_run, l_run, 1.0f, tile * FB_N, vis_lo, vis_hi, lane);
        fx_pv<DVP>(o, p, v_buf[cur], lane);
        __syncthreads();    // the tile may be overwritten by the load issued in the next iteration
    }
    fx_wait<0>();
    pdl_launch_dependents();

    const int t = lane & 3;
    if (splits > 1) {       // sums, maxima (base-2 units) and unnormalized outputs of this share; a second kernel merges them
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (out_off[r] < 0) continue;
            const size_t slot = (size_t)(out_off[r] / dv) * splits + split;        // (token * heads + head) * splits + split
            if (t == 0) { part_ml[slot * 2] = m_run[r]; part_ml[slot * 2 + 1] = l_run[r]; }
#pragma unroll
            for (int d = 0; d < DVP / 8; ++d)
                if (d * 8 < dv) *reinterpret_cast<float2*>(part_o + slot * dv + d * 8 + 2 * t) = make_float2(o[d][2 * r], o[d][2 * r + 1]);
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (out_off[r] < 0) continue;
        float corr = 1.0f;
        if (sink2[r] != -INFINITY) {        // the sink: one more term of the denominator (base-2 units like the maxima)
            const float m_new = fmaxf(m_run[r], sink2[r]);
            corr = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
            l_run[r] = l_run[r] * corr + exp2f(sink2[r] - m_new);
        }
        const float inv = l_run[r] > 0.f ? out_scale * corr / l_run[r] : 0.f;
        TO* orow = out + out_off[r];
#pragma unroll
        for (int d = 0; d < DVP / 8; ++d)
            if (d * 8 < dv) fx_store2<TO>(orow + d * 8 + 2 * t, o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
    }
}

// Merges the shares of one (token, head), in share order: a block of 128 threads per row of part_o.
template <typename TO>
__global__ void __launch_bounds__(128)
attention_flex_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, TO* __restrict__ out, int splits, int dv,
                            float out_scale, const float* __restrict__ sinks, int heads) {
    pdl_wait();
    const size_t row = blockIdx.x;      // token * heads + head
    const float sink2 = sinks != nullptr ? sinks[row % heads] * LOG2E : -INFINITY;
    float m = sink2;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(row * splits + s) * 2]);
    float l = sink2 != -INFINITY ? exp2f(sink2 - m) : 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = part_ml[(row * splits + s) * 2];
        if (ms != -INFINITY) l += part_ml[(row * splits + s) * 2 + 1] * exp2f(ms - m);
    }
    const float inv = l > 0.f ? out_scale / l : 0.f;
    for (int d = threadIdx.x; d < dv; d += 128) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(row * splits + s) * 2];
            if (ms != -INFINITY) acc += part_o[(row * splits + s) * dv + d] * exp2f(ms - m);
        }
        Elem<TO>::store(out + row * dv + d, acc * inv);
    }
}

template <int DKP, int DVP, typename TO>
int fx_launch(const void* q, int q_stride, void* out, const int* q_start, const int* ctx_lens, const int* block_table, int bt_stride,
              int page_size, const void* k_pages, const void* v_pages, int num_pages, int n_req, int max_q_len, int heads, int kv_heads,
              int dk, int dv, float scale, float softcap, const float* slopes, int window, int chunk, float out_scale, int splits,
              float* part_o, float* part_ml, int m_tokens, const float* sinks, cudaStream_t stream) {
    static bool configured = false;
    const int smem = 2 * FxTile<DKP>::BYTES + 2 * FxTile<DVP>::BYTES;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(attention_flex_mma_kernel<DKP, DVP, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    const int n_rep = heads / kv_heads;
    dim3 grid(splits > 1 ? splits : ceil_div((long long)max_q_len * n_rep, FWARPS * 16), n_req, kv_heads);
    NIB_CUDA(launch_pdl(attention_flex_mma_kernel<DKP, DVP, TO>, grid, dim3(FWARPS * 32), (size_t)smem, stream, (const __nv_bfloat16*)q, q_stride,
                        (TO*)out, q_start, ctx_lens, block_table, bt_stride, page_size, (const __nv_bfloat16*)k_pages,
                        (const __nv_bfloat16*)v_pages, num_pages, heads, kv_heads, dk, dv, scale, softcap, slopes, window, chunk, out_scale,
                        splits, part_o, part_ml, sinks));
    if (splits > 1)
        NIB_CUDA(launch_pdl(attention_flex_merge_kernel<TO>, dim3(m_tokens * heads), dim3(128), (size_t)0, stream, (const float*)part_o,
                            (const float*)part_ml, (TO*)out, splits, dv, out_scale, sinks, heads));
    return 0;
}

}  // namespace

NIB_API int nib_attention_flex_mma_supported(int heads, int kv_heads, int dk, int dv, int q_stride) {
    return (heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0 && dk % 8 == 0 && dv % 8 == 0 && dk <= 128 &&
            dv <= 128 && q_stride % 2 == 0) ? 1 : 0;
}

// q: rows of q_stride bfloat16 whose first heads*dk are the prepared queries; out: [tokens, heads*dv] floats (out_f32)
// or bfloat16; q_start [n_req + 1], ctx_lens [n_req]; max_q_len: the most tokens a request brings. splits > 1: the key
// tiles of every request are shared out to that many CTAs (part_o: [m_tokens * heads * splits * dv] floats, part_ml:
// [m_tokens * heads * splits * 2]) and a second kernel merges the shares.
NIB_API int nib_attention_flex_mma(const void* q, int q_stride, void* out, int out_f32, const int* q_start, const int* ctx_lens,
                                   const int* block_table, int bt_stride, int page_size, const void* k_pages, const void* v_pages,
                                   int num_pages, int n_req, int max_q_len, int heads, int kv_heads, int dk, int dv, float scale,
                                   float softcap, const float* slopes, int window, int chunk, float out_scale, int splits, float* part_o,
                                   float* part_ml, int m_tokens, const float* sinks, cudaStream_t stream) {
    NIB_REQUIRE(nib_attention_flex_mma_supported(heads, kv_heads, dk, dv, q_stride) == 1, "attention (tensor cores): head sizes %d / %d or head counts %d / %d are not taken", dk, dv, heads, kv_heads);
    NIB_REQUIRE(n_req >= 0 && max_q_len > 0 && page_size > 0 && num_pages > 0 && window >= 0 && chunk >= 0 && softcap >= 0.f, "attention (tensor cores): bad sizes");
    NIB_REQUIRE(splits <= 1 || (max_q_len * (heads / kv_heads) <= 64 && part_o != nullptr && part_ml != nullptr),
                "attention (tensor cores): keys are split over CTAs only when a request's rows fit one tile, and with scratch");
    if (n_req == 0) return 0;
#define NIB_FXM(DKP, DVP)                                                                                                                   \
    do {                                                                                                                                    \
        const int rc = out_f32 ? fx_launch<DKP, DVP, float>(q, q_stride, out, q_start, ctx_lens, block_table, bt_stride, page_size, k_pages, \
                                                            v_pages, num_pages, n_req, max_q_len, heads, kv_heads, dk, dv, scale, softcap,   \
                                                            slopes, window, chunk, out_scale, splits, part_o, part_ml, m_tokens, sinks, stream) \
                                   : fx_launch<DKP, DVP, __nv_bfloat16>(q, q_stride, out, q_start, ctx_lens, block_table, bt_stride,         \
                                                                        page_size, k_pages, v_pages, num_pages, n_req, max_q_len, heads,     \
                                                                        kv_heads, dk, dv, scale, softcap, slopes, window, chunk, out_scale,  \
                                                                        splits, part_o, part_ml, m_tokens, sinks, stream);                   \
        if (rc != 0) return rc;                                                                                                             \
    } while (0)
    if (dk <= 64 && dv <= 64) NIB_FXM(64, 64);
    else if (dk <= 64) NIB_FXM(64, 128);
    else if (dv <= 64) NIB_FXM(128, 64);
    else NIB_FXM(128, 128);
#undef NIB_FXM
    NIB_LAUNCH_CHECK();
    return 0;
}
