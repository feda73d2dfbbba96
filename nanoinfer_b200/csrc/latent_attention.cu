// Attention through a low-rank latent, over the paged cache. What is cached per position is ONE row for all heads:
// the normed latent c [rank] followed by a rotated key part [rot] that the heads share. A head's key is
// [W_uk,h c | rotated part] and its value W_uv,h c; instead of expanding them for every cached position, the
// query is carried into the latent space (q_lat = W_uk,h^T q_plain), the scores are taken against the cached rows
// as they are, the softmax-weighted sum of the cached latents is formed, and W_uv,h is applied once to that sum:
//   score_j = (q_lat . c_j + q_rot . kr_j) * scale,   out_h = W_uv,h (sum_j p_j c_j).
// So a step reads each cached row once per (token, head) and the per-head matrices once per token.
//
// Rotation: interleaved pairs (2i, 2i+1) or, with `half_layout`, pairs (i, i + rot/2); angle = position * freq[i] formed
// in 32-bit from a frequency vector that the position encoding supplies (any scaling rule changes the vector only),
// cos and sin times a magnitude. With `sink` (one number per head) the softmax's denominator also holds exp(sink[head]):
// a key without a value that every query sees once, not scaled.
// Keys are taken in blocks of 32 that start at absolute multiples of 32 (online softmax), so a position's result
// does not depend on how the request was cut into steps. All arithmetic is 32-bit; T is the storage type of the
// cache and of the weights.
#include "common.cuh"

constexpr int LAT_WARPS = 4;
constexpr int LAT_MAX_RANK = 512;      // latent width
constexpr int LAT_MAX_ROW = 640;       // latent + rotated part

// ---------------------------------------------------------------------------------- cache write
// z: [tokens, rank + rot] floats (the down projection's output). Row -> page: rms norm of the first rank values
// times gain, the last rot values rotated. One warp per token.
template <typename T>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_store_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ gain, float eps,
                    const float* __restrict__ freq, float mag, const int* __restrict__ positions,
                    const int* __restrict__ req_index, const int* __restrict__ block_table, int bt_stride, int page_size,
                    T* __restrict__ pages, int num_pages, int tokens, int rank, int rot, int half_layout) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int t = blockIdx.x * LAT_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)req_index[t] * bt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) return;      // a padding row owns no page
    const float* zr = z + (size_t)t * ldz;
    T* row = pages + ((size_t)page * page_size + (pos % page_size)) * (rank + rot);
    float ss = 0.f;
    for (int c = lane; c < rank; c += 32) ss = fmaf(zr[c], zr[c], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int c = lane; c < rank; c += 32) Elem<T>::store(row + c, zr[c] * scale * gain[c]);
    for (int i = lane; i < rot / 2; i += 32) {
        const float ang = (float)pos * freq[i];
        const float cs = cosf(ang) * mag, sn = sinf(ang) * mag;
        const int ia = half_layout ? i : 2 * i, ib = half_layout ? i + rot / 2 : 2 * i + 1;
        const float a = zr[rank + ia], b = zr[rank + ib];
        Elem<T>::store(row + rank + ia, a * cs - b * sn);
        Elem<T>::store(row + rank + ib, b * cs + a * sn);
    }
}

NIB_API int nib_latent_store(const float* z, int ldz, const float* gain, float eps, const float* freq, float mag,
                             const int* positions, const int* req_index, const int* block_table, int bt_stride,
                             int page_size, void* pages, int num_pages, int tokens, int rank, int rot, int dtype,
                             int half_layout, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && page_size > 0, "latent_store: bad sizes");
    if (tokens == 0) return 0;
    const int grid = ceil_div(tokens, LAT_WARPS);
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(latent_store_kernel<float>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, z, ldz, gain, eps, freq, mag, positions, req_index,
            block_table, bt_stride, page_size, (float*)pages, num_pages, tokens, rank, rot, half_layout));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(latent_store_kernel<__nv_bfloat16>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, z, ldz, gain, eps, freq, mag, positions, req_index,
            block_table, bt_stride, page_size, (__nv_bfloat16*)pages, num_pages, tokens, rank, rot, half_layout));
    else
        NIB_REQUIRE(false, "latent_store: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- queries into the latent space
// q: [tokens, heads, dn + rot] floats. qa: [tokens, heads, ldq] of TQ (float for the general kernel, bfloat16 rows
// padded with zeros for the tensor-core kernels):
//   qa[:rank] = sum_d q[d] * w_uk[h*dn + d, :]   (w_uk: [heads*dn, rank], as stored),   qa[rank:rank+rot] = rotated q[dn:].
// One warp per (token, head); lanes over the latent's columns, so the rows of w_uk are read coalesced.
template <typename T, typename TQ>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_query_kernel(const float* __restrict__ q, int ldq_in, const T* __restrict__ w_uk, const float* __restrict__ freq, float mag,
                    const int* __restrict__ positions, TQ* __restrict__ qa, int ldq, int tokens, int heads, int dn, int rank, int rot,
                    int half_layout) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long w = (long long)blockIdx.x * LAT_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)tokens * heads) return;
    const int t = (int)(w / heads), h = (int)(w % heads);
    const float* qr = q + (size_t)t * ldq_in + (size_t)h * (dn + rot);
    TQ* o = qa + (size_t)w * ldq;
    const T* wh = w_uk + (size_t)h * dn * rank;
    for (int c0 = 0; c0 < rank; c0 += 32 * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int d = 0; d < dn; ++d) {
            const float qd = qr[d];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = c0 + lane + 32 * i;
                if (c < rank) acc[i] = fmaf(qd, Elem<T>::load(wh + (size_t)d * rank + c), acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + lane + 32 * i;
            if (c < rank) Elem<TQ>::store(o + c, acc[i]);
        }
    }
    const int pos = positions[t];
    for (int i = lane; i < rot / 2; i += 32) {
        const float ang = (float)pos * freq[i];
        const float cs = cosf(ang) * mag, sn = sinf(ang) * mag;
        const int ia = half_layout ? i : 2 * i, ib = half_layout ? i + rot / 2 : 2 * i + 1;
        const float a = qr[dn + ia], b = qr[dn + ib];
        Elem<TQ>::store(o + rank + ia, a * cs - b * sn);
        Elem<TQ>::store(o + rank + ib, b * cs + a * sn);
    }
    for (int c = rank + rot + lane; c < ldq; c += 32) Elem<TQ>::store(o + c, 0.f);
}

// dtype: the weights' type; q_dtype: the type of qa's elements; ldq: qa's row width per (token, head), >= rank + rot.
NIB_API int nib_latent_query(const float* q, int ldq_in, const void* w_uk, const float* freq, float mag, const int* positions,
                             void* qa, int ldq, int q_dtype, int tokens, int heads, int dn, int rank, int rot, int dtype,
                             int half_layout, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && heads > 0 && dn > 0 && rank > 0 && rot >= 0 && rot % 2 == 0 && ldq >= rank + rot, "latent_query: bad sizes");
    if (tokens == 0) return 0;
    const int grid = ceil_div((long long)tokens * heads, LAT_WARPS);
    if (dtype == NIB_F32 && q_dtype == NIB_F32)
        NIB_CUDA(launch_pdl(latent_query_kernel<float, float>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, q, ldq_in, (const float*)w_uk, freq, mag, positions, (float*)qa, ldq, tokens, heads, dn, rank, rot, half_layout));
    else if (dtype == NIB_BF16 && q_dtype == NIB_F32)
        NIB_CUDA(launch_pdl(latent_query_kernel<__nv_bfloat16, float>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, q, ldq_in, (const __nv_bfloat16*)w_uk, freq, mag, positions, (float*)qa, ldq, tokens, heads, dn, rank, rot, half_layout));
    else if (dtype == NIB_BF16 && q_dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(latent_query_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, q, ldq_in, (const __nv_bfloat16*)w_uk, freq, mag, positions, (__nv_bfloat16*)qa, ldq, tokens, heads, dn, rank, rot, half_layout));
    else
        NIB_REQUIRE(false, "latent_query: unsupported types %d / %d", dtype, q_dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- attention over cached rows
// qa: [tokens, heads, rank + rot] floats; pages: [num_pages, page_size, rank + rot] of T; out: [tokens, heads, rank]
// floats, the softmax-weighted sum of the visible rows' latents. One warp per (token, head): a lane scores one key
// of a block of 32, then the lanes share the block's rows column-wise for the weighted sum.
template <typename T>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_attention_kernel(const float* __restrict__ qa, float* __restrict__ out, const int* __restrict__ positions,
                        const int* __restrict__ req_index, const int* __restrict__ block_table, int bt_stride, int page_size,
                        const T* __restrict__ pages, int num_pages, int tokens, int heads, int rank, int rot, float scale, int window,
                        const float* __restrict__ sink) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float q_s[LAT_WARPS][LAT_MAX_ROW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * LAT_WARPS + warp;
    if (w >= (long long)tokens * heads) return;
    const int token = (int)(w / heads);
    const int width = rank + rot;
    const int pos = positions[token];
    const int* bt = block_table + (size_t)req_index[token] * bt_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const float* q = qa + (size_t)w * width;
    for (int d = lane; d < width; d += 32) q_s[warp][d] = q[d];
    __syncwarp();

    float m_run = -INFINITY, l_run = 0.f;
    float acc[LAT_MAX_RANK / 32];
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] = 0.f;
    for (int kb = (lo / 32) * 32; kb <= pos; kb += 32) {
        const int j = kb + lane;
        float s = -INFINITY;
        long long row = -1;
        if (j >= lo && j <= pos) {
            const int page = bt[j / page_size];
            if (page >= 0 && page < num_pages) {
                row = ((long long)page * page_size + (j % page_size)) * width;
                const T* kr = pages + row;
                float dot = 0.f;
                for (int d = 0; d < width; ++d) dot = fmaf(q_s[warp][d], Elem<T>::load(kr + d), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m_run, warp_max(s));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, row, jj);
            if (pj == 0.f || rj < 0) continue;      // uniform over the warp
            const T* vr = pages + rj;
#pragma unroll
            for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < rank) acc[i] = fmaf(pj, Elem<T>::load(vr + d), acc[i]);
            }
        }
        m_run = m_new;
    }
    float* o = out + (size_t)w * rank;
    if (sink != nullptr) {      // one more term in the denominator; the sums are brought to the larger of the two maxima
        const float sk = sink[(int)(w % heads)];
        const float m_fin = fmaxf(m_run, sk);
        const float f = (m_run == -INFINITY) ? 0.f : expf(m_run - m_fin);
        l_run = l_run * f + expf(sk - m_fin);
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] *= f;
    }
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) o[d] = acc[i] * inv;
    }
}

NIB_API int nib_latent_attention(const float* qa, float* out, const int* positions, const int* req_index,
                                 const int* block_table, int bt_stride, int page_size, const void* pages, int num_pages,
                                 int tokens, int heads, int rank, int rot, float scale, int window, int dtype,
                                 const float* sink, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && heads > 0 && rank > 0 && rank <= LAT_MAX_RANK && rank + rot <= LAT_MAX_ROW,
                "latent attention: latent %d (+%d rotated) is outside 1..%d (row up to %d)", rank, rot, LAT_MAX_RANK, LAT_MAX_ROW);
    NIB_REQUIRE(page_size > 0 && num_pages > 0 && window >= 0, "latent attention: bad page_size/num_pages/window");
    if (tokens == 0) return 0;
    const int grid = ceil_div((long long)tokens * heads, LAT_WARPS);
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(latent_attention_kernel<float>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, qa, out, positions, req_index, block_table, bt_stride,
            page_size, (const float*)pages, num_pages, tokens, heads, rank, rot, scale, window, sink));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(latent_attention_kernel<__nv_bfloat16>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, qa, out, positions, req_index, block_table, bt_stride,
            page_size, (const __nv_bfloat16*)pages, num_pages, tokens, heads, rank, rot, scale, window, sink));
    else
        NIB_REQUIRE(false, "latent attention: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- values out of the latent space
// lat: [tokens, heads, rank] floats; w_uv: [heads*dv, rank] as stored; out: [tokens, heads*dv] of T:
//   out[t, h*dv + j] = sum_c w_uv[h*dv + j, c] * lat[t, h, c], times sigmoid(gate[t, h*dv + j]) with a gate.
// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_value_kernel(const float* __restrict__ lat, const T* __restrict__ w_uv, T* __restrict__ out, int ldo, int tokens,
                    int heads, int dv, int rank, const float* __restrict__ gate, int ldg) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float l_s[LAT_WARPS][LAT_MAX_RANK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * LAT_WARPS + warp;
    if (w >= (long long)tokens * heads) return;
    const int t = (int)(w / heads), h = (int)(w % heads);
    for (int c = lane; c < rank; c += 32) l_s[warp][c] = lat[(size_t)w * rank + c];
    __syncwarp();
    for (int j = 0; j < dv; ++j) {
        const T* wr = w_uv + ((size_t)h * dv + j) * rank;
        float acc = 0.f;
        for (int c = lane; c < rank; c += 32) acc = fmaf(Elem<T>::load(wr + c), l_s[warp][c], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            if (gate != nullptr) acc *= 1.0f / (1.0f + expf(-gate[(size_t)t * ldg + (size_t)h * dv + j]));
            Elem<T>::store(out + (size_t)t * ldo + (size_t)h * dv + j, acc);
        }
    }
}

NIB_API int nib_latent_value(const float* lat, const void* w_uv, void* out, int ldo, int tokens, int heads, int dv, int rank,
                             int dtype, const float* gate, int ldg, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && heads > 0 && dv > 0 && rank > 0 && rank <= LAT_MAX_RANK, "latent_value: bad sizes");
    if (tokens == 0) return 0;
    const int grid = ceil_div((long long)tokens * heads, LAT_WARPS);
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(latent_value_kernel<float>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, lat, (const float*)w_uv, (float*)out, ldo, tokens, heads, dv, rank, gate, ldg));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(latent_value_kernel<__nv_bfloat16>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(0), stream, lat, (const __nv_bfloat16*)w_uv, (__nv_bfloat16*)out, ldo, tokens, heads, dv, rank, gate, ldg));
    else
        NIB_REQUIRE(false, "latent_value: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}
