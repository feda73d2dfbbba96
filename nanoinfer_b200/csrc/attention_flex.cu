// Softmax attention over the paged cache with the options that decoder designs combine, and the kernel that prepares
// its operands. All arithmetic is 32-bit whatever the storage type T (float or bfloat16).
//
//  * attention_prepare: from the 32-bit rows [q | k | v] of a step (after projection, bias and any convolution): every q
//    and k head optionally divided by its root mean square and multiplied by a gain of the head's size (shared by the
//    heads), the first `rot` elements of every q and k head turned by angle = position * freq[i] (element i paired with
//    i + rot/2, or 2i with 2i + 1 in the interleaved layout; the angle is formed in 32-bit), then optionally every q and
//    k head divided by its root mean square once more, without a gain (a norm AFTER the rotation), queries written in the
//    storage type, keys and values written into their pages. Keys are `dk` wide, values `dv`; the values may be the keys
//    as projected (before norm and rotation), the rows then hold [q | k] only. One warp per (token, head of q, k or v).
//    With FXP_NORM_WHOLE the root mean square is taken over ALL heads of a token's q (and of its k) at once and the gain
//    has the size of the whole projection. With `v_first` a value becomes (1 - lambda) v + lambda v_first, where v_first
//    holds the same token's values of another layer (32-bit rows) and lambda = vmix[0]; the blend is what is cached.
//  * attention_flex: one warp per (token, query head). A query at position p of its request sees the keys j <= p,
//    with a window only j > p - window, with a chunk only floor(j / chunk) == floor(p / chunk) (counted from the
//    request's position 0). score = (q . k) * scale; with a cap c: c tanh(score / c); with slopes: minus
//    slope[head] * (p - j). Keys are taken in blocks of 32 that start at absolute multiples of 32 with a running
//    maximum and sum, so a position's result does not depend on how the request was cut into steps, nor on what else
//    is in the batch. With `sinks` the softmax's denominator holds exp(sinks[head]) once more: a term without key and
//    value, neither scaled nor capped. The output (dv wide per head) is multiplied by out_scale and written as float or T.
#include "common.cuh"

constexpr int FX_MAX_D = 256;
constexpr int FX_WARPS = 4;

// flags of attention_prepare
enum { FXP_INTERLEAVED = 1, FXP_UNIT_NORM_AFTER = 2, FXP_VALUES_ARE_KEYS = 4, FXP_NORM_WHOLE = 8 };

// One (token, head of q, k or v) by one warp. whole_q / whole_k: with FXP_NORM_WHOLE the factors 1 / rms of the token's
// whole q and k projections (computed once per token by the caller), else unused.
template <typename T>
__device__ __forceinline__ void prepare_unit(const float* __restrict__ qkv, int ld, T* __restrict__ q_out, const float* __restrict__ q_gain,
                                             const float* __restrict__ k_gain, float eps, const float* __restrict__ freq, int rot,
                                             const int* __restrict__ positions, const int* __restrict__ req_index,
                                             const int* __restrict__ block_table, int bt_stride, int page_size, T* __restrict__ k_pages,
                                             T* __restrict__ v_pages, int num_pages, int heads, int kv_heads, int dk, int dv, int writes, int flags,
                                             const float* __restrict__ v_first, int ld_first, const float* __restrict__ vmix, int t, int s,
                                             float whole_q, float whole_k, float* x_s, int lane) {
    const int pos = positions[t];
    const bool is_q = s < heads, is_k = !is_q && s < heads + kv_heads;
    const int head = is_q ? s : (is_k ? s - heads : s - heads - kv_heads);
    const int d = (is_q || is_k) ? dk : dv;
    // a value head that is the key head as projected reads the key's columns (the rows then hold no values)
    const bool v_is_k = (flags & FXP_VALUES_ARE_KEYS) != 0;
    const float* src = qkv + (size_t)t * ld + (is_q ? (size_t)head * dk : ((is_k || v_is_k) ? (size_t)heads * dk + (size_t)head * dk
                                                                                   : (size_t)(heads + kv_heads) * dk + (size_t)head * dv));
    T* dst = nullptr;
    if (is_q) {
        dst = q_out + (size_t)t * heads * dk + (size_t)head * dk;
    } else if (writes) {
        const int page = block_table[(size_t)req_index[t] * bt_stride + pos / page_size];
        if (page >= 0 && page < num_pages)      // a padding row of a replayed step holds no pages
            dst = (is_k ? k_pages : v_pages) + (((size_t)page * kv_heads + head) * page_size + (pos % page_size)) * d;
    }
    if (dst == nullptr) return;
    if (!is_q && !is_k) {
        if (v_first != nullptr) {       // the blend with another layer's values of this token
            const float lam = vmix[0];
            const float* fr = v_first + (size_t)t * ld_first + (size_t)head * dv;
            for (int c = lane; c < d; c += 32) Elem<T>::store(dst + c, (1.0f - lam) * src[c] + lam * fr[c]);
            return;
        }
        for (int c = lane; c < d; c += 32) Elem<T>::store(dst + c, src[c]);
        return;
    }
    const float* gain = is_q ? q_gain : k_gain;
    float norm = 1.0f;
    if (gain != nullptr && (flags & FXP_NORM_WHOLE)) {
        norm = is_q ? whole_q : whole_k;
        if (norm < 0.f) {       // not summed by the caller: this warp sums the whole projection itself (steps of few tokens)
            const int n_all = (is_q ? heads : kv_heads) * dk;
            const float* all = qkv + (size_t)t * ld + (is_q ? 0 : (size_t)heads * dk);
            float ss = 0.f;
            for (int c = lane; c < n_all; c += 32) ss = fmaf(all[c], all[c], ss);
            norm = 1.0f / sqrtf(warp_sum(ss) / (float)n_all + eps);
        }
        gain += (size_t)head * dk;
    } else if (gain != nullptr) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) ss = fmaf(src[c], src[c], ss);
        norm = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
    }
    for (int c = lane; c < d; c += 32) x_s[c] = gain != nullptr ? src[c] * norm * gain[c] : src[c];
    __syncwarp();
    const int half = rot >> 1;
    const bool interleaved = (flags & FXP_INTERLEAVED) != 0;
    float y[FX_MAX_D / 32];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < FX_MAX_D / 32; ++j) {
        const int c = lane + 32 * j;
        if (c >= d) break;
        float v = x_s[c];
        if (c < rot) {
            // the pair's first element is turned with minus, its second with plus; pairs are (i, i + rot/2) or (2i, 2i + 1)
            const bool first = interleaved ? (c & 1) == 0 : c < half;
            const int i = interleaved ? (c >> 1) : (c < half ? c : c - half);
            const int mate = interleaved ? (c ^ 1) : (c < half ? c + half : c - half);
            const float a = (float)pos * freq[i];
            const float cs = cosf(a), sn = sinf(a);
            v = first ? v * cs - x_s[mate] * sn : v * cs + x_s[mate] * sn;
        }
        y[j] = v;
        ss = fmaf(v, v, ss);
    }
    float after = 1.0f;
    if (flags & FXP_UNIT_NORM_AFTER) after = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
#pragma unroll
    for (int j = 0; j < FX_MAX_D / 32; ++j) {
        const int c = lane + 32 * j;
        if (c >= d) break;
        Elem<T>::store(dst + c, y[j] * after);
    }
    __syncwarp();       // x_s is the warp's own and may be filled again for its next unit
}

// A warp per (token, head of q, k or v), four of them a block; with FXP_NORM_WHOLE such a warp sums the squares of the
// token's whole projection itself. With `by_token` (FXP_NORM_WHOLE and many tokens): a block per token, which first sums
// the squares of the token's whole q and whole k once, then its warps take the token's heads in turn. Either way the
// additions of a token's sum have one fixed order within a launch; the two orders differ by rounding.
template <typename T>
__global__ void __launch_bounds__(FX_WARPS * 32)
attention_prepare_kernel(const float* __restrict__ qkv, int ld, T* __restrict__ q_out, const float* __restrict__ q_gain,
                         const float* __restrict__ k_gain, float eps, const float* __restrict__ freq, int rot,
                         const int* __restrict__ positions, const int* __restrict__ req_index, const int* __restrict__ block_table,
                         int bt_stride, int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages, int num_pages,
                         int tokens, int heads, int kv_heads, int dk, int dv, int writes, int flags,
                         const float* __restrict__ v_first, int ld_first, const float* __restrict__ vmix, int by_token) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float x_s[FX_WARPS][FX_MAX_D];
    __shared__ float red[2][FX_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (by_token) {
        const int t = blockIdx.x;
        const float* row = qkv + (size_t)t * ld;
        const int nq = heads * dk, nk = kv_heads * dk;
        float sq = 0.f, sk = 0.f;
        for (int c = threadIdx.x; c < nq; c += FX_WARPS * 32) sq = fmaf(row[c], row[c], sq);
        for (int c = threadIdx.x; c < nk; c += FX_WARPS * 32) sk = fmaf(row[nq + c], row[nq + c], sk);
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
        __syncthreads();
        sq = sk = 0.f;
#pragma unroll
        for (int w = 0; w < FX_WARPS; ++w) { sq += red[0][w]; sk += red[1][w]; }
        const float whole_q = 1.0f / sqrtf(sq / (float)nq + eps), whole_k = 1.0f / sqrtf(sk / (float)nk + eps);
        for (int s = warp; s < heads + 2 * kv_heads; s += FX_WARPS)
            prepare_unit<T>(qkv, ld, q_out, q_gain, k_gain, eps, freq, rot, positions, req_index, block_table, bt_stride, page_size, k_pages, v_pages,
                            num_pages, heads, kv_heads, dk, dv, writes, flags, v_first, ld_first, vmix, t, s, whole_q, whole_k, x_s[warp], lane);
        return;
    }
    const int units = heads + 2 * kv_heads;
    const long long wid = (long long)blockIdx.x * FX_WARPS + warp;
    if (wid >= (long long)tokens * units) return;
    prepare_unit<T>(qkv, ld, q_out, q_gain, k_gain, eps, freq, rot, positions, req_index, block_table, bt_stride, page_size, k_pages, v_pages,
                    num_pages, heads, kv_heads, dk, dv, writes, flags, v_first, ld_first, vmix, (int)(wid / units), (int)(wid % units), -1.0f, -1.0f,
                    x_s[warp], lane);
}


// ---- the same for bfloat16 storage, eight elements a thread --------------------------------------------------------------
// A block per token; a work item is eight consecutive elements of a head (two 16-byte loads of floats, one 16-byte store of
// bfloat16), or, inside the rotated part of a q or k head, the eight elements at c and their mates at c + rot/2 together,
// so that an angle's sine and cosine are formed once a pair. Takes: no norm or the norm over the whole projection, pairs
// (i, i + rot/2) with rot a multiple of 16, head sizes in multiples of 8, values of their own (blended or not). The token's
// page and slot are looked up once. Same arithmetic per element as the kernel above.
__device__ __forceinline__ void load8(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
    uint4 u;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(x[0], x[1]); u.x = *reinterpret_cast<unsigned*>(&t);
    t = __floats2bfloat162_rn(x[2], x[3]); u.y = *reinterpret_cast<unsigned*>(&t);
    t = __floats2bfloat162_rn(x[4], x[5]); u.z = *reinterpret_cast<unsigned*>(&t);
    t = __floats2bfloat162_rn(x[6], x[7]); u.w = *reinterpret_cast<unsigned*>(&t);
    *reinterpret_cast<uint4*>(p) = u;
}

__global__ void __launch_bounds__(128)
attention_prepare_vec_kernel(const float* __restrict__ qkv, int ld, __nv_bfloat16* __restrict__ q_out, const float* __restrict__ q_gain,
                             const float* __restrict__ k_gain, float eps, const float* __restrict__ freq, int rot,
                             const int* __restrict__ positions, const int* __restrict__ req_index, const int* __restrict__ block_table,
                             int bt_stride, int page_size, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, int num_pages,
                             int heads, int kv_heads, int dk, int dv, int writes, const float* __restrict__ v_first, int ld_first,
                             const float* __restrict__ vmix) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float red[2][4];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* row = qkv + (size_t)t * ld;
    const int nq = heads * dk, nk = kv_heads * dk;
    float whole_q = 1.0f, whole_k = 1.0f;
    if (q_gain != nullptr) {        // the norm over the whole projection: one sum of squares for q, one for k
        float sq = 0.f, sk = 0.f;
        for (int c = tid * 4; c < nq; c += 128 * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + c);
            sq = fmaf(v.x, v.x, sq); sq = fmaf(v.y, v.y, sq); sq = fmaf(v.z, v.z, sq); sq = fmaf(v.w, v.w, sq);
        }
        for (int c = tid * 4; c < nk; c += 128 * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + nq + c);
            sk = fmaf(v.x, v.x, sk); sk = fmaf(v.y, v.y, sk); sk = fmaf(v.z, v.z, sk); sk = fmaf(v.w, v.w, sk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
        __syncthreads();
        sq = (red[0][0] + red[0][1]) + (red[0][2] + red[0][3]);
        sk = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]);
        whole_q = 1.0f / sqrtf(sq / (float)nq + eps);
        whole_k = 1.0f / sqrtf(sk / (float)nk + eps);
    }
    const int pos = positions[t];
    long long slot = -1;        // (page * kv_heads) * page_size + offset in the page; a kv head adds head * page_size
    if (writes) {
        const int page = block_table[(size_t)req_index[t] * bt_stride + pos / page_size];
        if (page >= 0 && page < num_pages) slot = (long long)page * kv_heads * page_size + (pos % page_size);   // else: a padding row of a replayed step
    }
    const int half = rot >> 1;
    const int per_head = half / 8 + (dk - rot) / 8;             // work items of a q or k head
    const int items_qk = (heads + kv_heads) * per_head, items_v = kv_heads * (dv / 8);
    const float lam = v_first != nullptr ? vmix[0] : 0.f;
    for (int it = tid; it < items_qk + items_v; it += 128) {
        if (it >= items_qk) {                                   // eight elements of a value head
            if (slot < 0) continue;
            const int c = (it - items_qk) * 8, head = c / dv, off = c - head * dv;
            float x[8];
            load8(row + nq + nk + c, x);
            if (v_first != nullptr) {
                float f[8];
                load8(v_first + (size_t)t * ld_first + c, f);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = (1.0f - lam) * x[e] + lam * f[e];
            }
            store8(v_pages + ((size_t)slot + (size_t)head * page_size) * dv + off, x);
            continue;
        }
        const int hq = it / per_head, w = it - hq * per_head;  // head among q's then k's; item within it
        const bool is_q = hq < heads;
        const int head = is_q ? hq : hq - heads;
        if (!is_q && slot < 0) continue;
        const float* src = row + (size_t)hq * dk;                // q heads and k heads lie one behind the other
        const float* gain = is_q ? q_gain : k_gain;
        const float norm = is_q ? whole_q : whole_k;
        __nv_bfloat16* dst = is_q ? q_out + (size_t)t * nq + (size_t)head * dk
                                  : k_pages + ((size_t)slot + (size_t)head * page_size) * dk;
        if (w < half / 8) {                                     // eight rotated pairs: elements c.. and c + rot/2..
            const int c = w * 8;
            float a[8], b[8];
            load8(src + c, a);
            load8(src + c + half, b);
            if (gain != nullptr) {
                float ga[8], gb[8];
                load8(gain + (size_t)head * dk + c, ga);
                load8(gain + (size_t)head * dk + c + half, gb);
#pragma unroll
                for (int e = 0; e < 8; ++e) { a[e] = a[e] * norm * ga[e]; b[e] = b[e] * norm * gb[e]; }
            }
            float fr[8];
            load8(freq + c, fr);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float sn, cs;
                sincosf((float)pos * fr[e], &sn, &cs);
                const float u = a[e], v = b[e];
                a[e] = u * cs - v * sn;
                b[e] = v * cs + u * sn;
            }
            store8(dst + c, a);
            store8(dst + c + half, b);
        } else {                                                // eight elements that are not rotated
            const int c = rot + (w - half / 8) * 8;
            float a[8];
            load8(src + c, a);
            if (gain != nullptr) {
                float ga[8];
                load8(gain + (size_t)head * dk + c, ga);
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = a[e] * norm * ga[e];
            }
            store8(dst + c, a);
        }
    }
}

NIB_API int nib_attention_prepare(const float* qkv, int ld, void* q_out, const float* q_gain, const float* k_gain, float eps,
                                  const float* freq, int rot, const int* positions, const int* req_index, const int* block_table,
                                  int bt_stride, int page_size, void* k_pages, void* v_pages, int num_pages, int tokens, int heads,
                                  int kv_heads, int dk, int dv, int writes, int dtype, int flags, const float* v_first, int ld_first,
                                  const float* vmix, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0, "attention_prepare: bad head counts");
    NIB_REQUIRE(dk > 0 && dk <= FX_MAX_D && dv > 0 && dv <= FX_MAX_D, "attention_prepare: head sizes %d / %d are outside 1..%d", dk, dv, FX_MAX_D);
    NIB_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dk && (rot == 0 || freq != nullptr), "attention_prepare: bad rotated width %d", rot);
    NIB_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "attention_prepare: q and k are normed together or not at all");
    NIB_REQUIRE(!(flags & FXP_NORM_WHOLE) || q_gain != nullptr, "attention_prepare: a norm over the whole projection needs its gains");
    NIB_REQUIRE(!(flags & FXP_VALUES_ARE_KEYS) || dk == dv, "attention_prepare: values that are the keys have the keys' width");
    NIB_REQUIRE(!writes || (page_size > 0 && num_pages > 0 && block_table != nullptr), "attention_prepare: bad pages");
    NIB_REQUIRE(v_first == nullptr || (vmix != nullptr && ld_first >= kv_heads * dv && !(flags & FXP_VALUES_ARE_KEYS)),
                "attention_prepare: a blend of values needs its factor and rows of at least kv_heads * dv floats");
    if (tokens == 0) return 0;
    // bfloat16 storage in the common forms, with enough tokens to fill the GPU with a block each: eight elements a thread
    const bool aligned16 = ((uintptr_t)qkv % 16 == 0) && ld % 4 == 0 && (uintptr_t)q_out % 16 == 0 && (!writes || ((uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0))
        && (q_gain == nullptr || ((uintptr_t)q_gain % 16 == 0 && (uintptr_t)k_gain % 16 == 0)) && (rot == 0 || (uintptr_t)freq % 16 == 0)
        && (v_first == nullptr || ((uintptr_t)v_first % 16 == 0 && ld_first % 4 == 0));
    if (dtype == NIB_BF16 && tokens >= 256 && aligned16 && dk % 8 == 0 && dv % 8 == 0 && rot % 16 == 0 && (flags & ~FXP_NORM_WHOLE) == 0
        && ((q_gain != nullptr) == ((flags & FXP_NORM_WHOLE) != 0))) {
        NIB_CUDA(launch_pdl(attention_prepare_vec_kernel, dim3(tokens), dim3(128), (size_t)0, stream, qkv, ld, (__nv_bfloat16*)q_out, q_gain, k_gain, eps, freq,
                            rot, positions, req_index, block_table, bt_stride, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages, heads,
                            kv_heads, dk, dv, writes, v_first, ld_first, vmix));
        NIB_LAUNCH_CHECK();
        return 0;
    }
    // a block per token pays when the tokens alone fill the GPU; a step of few tokens wants a warp per head
    const int by_token = ((flags & FXP_NORM_WHOLE) && tokens >= 512) ? 1 : 0;
    const dim3 grid(by_token ? tokens : ceil_div((long long)tokens * (heads + 2 * kv_heads), FX_WARPS)), block(FX_WARPS * 32);
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(attention_prepare_kernel<float>, grid, block, (size_t)0, stream, qkv, ld, (float*)q_out, q_gain, k_gain, eps, freq, rot,
                            positions, req_index, block_table, bt_stride, page_size, (float*)k_pages, (float*)v_pages, num_pages, tokens, heads,
                            kv_heads, dk, dv, writes, flags, v_first, ld_first, vmix, by_token));
    else if (dtype == NIB_BF16)
        NIB_CUDA(launch_pdl(attention_prepare_kernel<__nv_bfloat16>, grid, block, (size_t)0, stream, qkv, ld, (__nv_bfloat16*)q_out, q_gain, k_gain,
                            eps, freq, rot, positions, req_index, block_table, bt_stride, page_size, (__nv_bfloat16*)k_pages,
                            (__nv_bfloat16*)v_pages, num_pages, tokens, heads, kv_heads, dk, dv, writes, flags, v_first, ld_first, vmix, by_token));
    else
        NIB_REQUIRE(false, "attention_prepare: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q_s, const T* __restrict__ kr, int dk) {
    float dot = 0.f;
    for (int d = 0; d < dk; ++d) dot = fmaf(q_s[d], Elem<T>::load(kr + d), dot);
    return dot;
}

// bfloat16 rows of a multiple of 8 elements are read 16 bytes at a time (rows then start on 16-byte boundaries)
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q_s, const __nv_bfloat16* __restrict__ kr, int dk) {
    float dot = 0.f;
    if ((dk & 7) == 0) {
        const uint4* k4 = reinterpret_cast<const uint4*>(kr);
        for (int d8 = 0; d8 < dk / 8; ++d8) {
            const uint4 raw = k4[d8];
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                dot = fmaf(q_s[d8 * 8 + 2 * i], f.x, dot);
                dot = fmaf(q_s[d8 * 8 + 2 * i + 1], f.y, dot);
            }
        }
        return dot;
    }
    for (int d = 0; d < dk; ++d) dot = fmaf(q_s[d], __bfloat162float(kr[d]), dot);
    return dot;
}

template <typename T, typename TO>
__global__ void __launch_bounds__(FX_WARPS * 32)
attention_flex_kernel(const T* __restrict__ q, int q_stride, TO* __restrict__ out, const int* __restrict__ positions,
                      const int* __restrict__ req_index, const int* __restrict__ block_table, int bt_stride, int page_size,
                      const T* __restrict__ k_pages, const T* __restrict__ v_pages, int num_pages, int m_tokens, int heads,
                      int kv_heads, int dk, int dv, float scale, float softcap, const float* __restrict__ slopes, int window,
                      int chunk, float out_scale, const float* __restrict__ sinks) {
    __shared__ __align__(16) float q_s[FX_WARPS][FX_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * FX_WARPS + warp;
    if (w >= (long long)m_tokens * heads) return;
    const int token = (int)(w / heads), head = (int)(w % heads);
    const int kvh = head / (heads / kv_heads);
    const int pos = positions[token];
    const int* bt = block_table + (size_t)req_index[token] * bt_stride;
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const float slope = slopes != nullptr ? slopes[head] : 0.f;
    const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;

    const T* qr = q + (size_t)token * q_stride + (size_t)head * dk;
    for (int d = lane; d < dk; d += 32) q_s[warp][d] = Elem<T>::load(qr + d);
    __syncwarp();

    float m_run = -INFINITY, l_run = 0.f;
    float acc[FX_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < FX_MAX_D / 32; ++i) acc[i] = 0.f;

    for (int kb = (lo / 32) * 32; kb <= pos; kb += 32) {
        const int j = kb + lane;
        const bool valid = (j >= lo) && (j <= pos);
        float s = -INFINITY;
        long long slot = -1;  // row of this lane's key in the pages: (page * kv_heads + kvh) * page_size + offset
        if (valid) {
            const int page = bt[j / page_size];
            if (page >= 0 && page < num_pages) {
                slot = ((long long)page * kv_heads + kvh) * page_size + (j % page_size);
                s = dot_row<T>(q_s[warp], k_pages + slot * dk, dk) * scale;
                if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
                s -= slope * (float)(pos - j);
            }
        }
        const float m_new = fmaxf(m_run, warp_max(s));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < FX_MAX_D / 32; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long rj = __shfl_sync(0xffffffffu, slot, jj);
            if (pj == 0.f || rj < 0) continue;  // uniform over the warp
            const T* vr = v_pages + rj * dv;
#pragma unroll
            for (int i = 0; i < FX_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, Elem<T>::load(vr + d), acc[i]);
            }
        }
        m_run = m_new;
    }
    TO* o = out + (size_t)token * heads * dv + (size_t)head * dv;
    float corr_sink = 1.0f;
    if (sinks != nullptr) {     // one more term of the denominator, with no value
        const float sk = sinks[head];
        const float m_new = fmaxf(m_run, sk);
        corr_sink = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr_sink + expf(sk - m_new);
    }
    const float inv = l_run > 0.f ? out_scale * corr_sink / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < FX_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) Elem<TO>::store(o + d, acc[i] * inv);
    }
}

// q: rows of q_stride elements whose first heads*dk are the prepared queries. out: [m_tokens, heads*dv], float when
// out_f32, else T. Pages: k [num_pages, kv_heads, page_size, dk], v [num_pages, kv_heads, page_size, dv].
NIB_API int nib_attention_flex(const void* q, int q_stride, void* out, int out_f32, const int* positions, const int* req_index,
                               const int* block_table, int bt_stride, int page_size, const void* k_pages, const void* v_pages,
                               int num_pages, int m_tokens, int heads, int kv_heads, int dk, int dv, float scale, float softcap,
                               const float* slopes, int window, int chunk, float out_scale, const float* sinks, int dtype,
                               cudaStream_t stream) {
    NIB_REQUIRE(m_tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "attention: bad head counts %d / %d", heads, kv_heads);
    NIB_REQUIRE(dk > 0 && dk <= FX_MAX_D && dv > 0 && dv <= FX_MAX_D, "attention: head sizes %d / %d are outside 1..%d", dk, dv, FX_MAX_D);
    NIB_REQUIRE(page_size > 0 && num_pages > 0 && window >= 0 && chunk >= 0 && softcap >= 0.f, "attention: bad page_size/num_pages/window/chunk/cap");
    if (m_tokens == 0) return 0;
    const int blocks = ceil_div((long long)m_tokens * heads, FX_WARPS);
#define NIB_FX_LAUNCH(T, TO)                                                                                                       \
    attention_flex_kernel<T, TO><<<blocks, FX_WARPS * 32, 0, stream>>>((const T*)q, q_stride, (TO*)out, positions, req_index, block_table, \
        bt_stride, page_size, (const T*)k_pages, (const T*)v_pages, num_pages, m_tokens, heads, kv_heads, dk, dv, scale, softcap, slopes,  \
        window, chunk, out_scale, sinks)
    if (dtype == NIB_F32) NIB_FX_LAUNCH(float, float);
    else if (dtype == NIB_BF16 && out_f32) NIB_FX_LAUNCH(__nv_bfloat16, float);
    else if (dtype == NIB_BF16) NIB_FX_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else NIB_REQUIRE(false, "attention: unknown dtype %d", dtype);
#undef NIB_FX_LAUNCH
    NIB_LAUNCH_CHECK();
    return 0;
}
