// Row-wise and element-wise kernels that several designs share: the PolyNorm activation (a mix of the
// rms-normed first three powers of a row), the weighted sum of a step's earlier residual streams, a
// unary function with a change of storage type, and the norm-and-gate of a recurrent mixer's heads.
// All arithmetic is 32-bit; T is the storage type of the activations that leave (float or bfloat16).
#include "common.cuh"

__device__ __forceinline__ float block_sum_256(float v, float* part) {
    // fixed order: warp butterflies, then the eight warps' sums added ascending by every thread
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w];
    __syncthreads();
    return t;
}

// ---------------------------------------------------------------------------------- PolyNorm
// out[t, :] = c0 z / rms(z) + c1 z^2 / rms(z^2) + c2 z^3 / rms(z^3) + c3, rms(y) = sqrt(mean(y^2) + eps).
// One block of 256 threads per row; the row is read twice (sums of z^2, z^4, z^6; then the result).
template <typename T>
__global__ void __launch_bounds__(256)
poly_norm_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ coef, T* __restrict__ out, int ldo,
                 int width, float eps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float part[8];
    const float* zr = z + (size_t)blockIdx.x * ldz;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int c = threadIdx.x; c < width; c += 256) {
        const float v = zr[c], v2 = v * v, v3 = v2 * v;
        s2 = fmaf(v, v, s2);
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    s2 = block_sum_256(s2, part);
    s4 = block_sum_256(s4, part);
    s6 = block_sum_256(s6, part);
    const float inv = 1.0f / (float)width;
    const float n1 = coef[0] / sqrtf(s2 * inv + eps), n2 = coef[1] / sqrtf(s4 * inv + eps), n3 = coef[2] / sqrtf(s6 * inv + eps);
    const float c3 = coef[3];
    T* o = out + (size_t)blockIdx.x * ldo;
    for (int c = threadIdx.x; c < width; c += 256) {
        const float v = zr[c], v2 = v * v;
        Elem<T>::store(o + c, fmaf(n1, v, fmaf(n2, v2, fmaf(n3, v2 * v, c3))));
    }
}

NIB_API int nib_poly_norm(const float* z, int ldz, const float* coef, void* out, int ldo, int rows, int width, float eps,
                          int dtype, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && width > 0 && ldz >= width && ldo >= width, "poly_norm: bad sizes rows=%d width=%d", rows, width);
    if (rows == 0) return 0;
    if (dtype == NIB_F32) NIB_CUDA(launch_pdl(poly_norm_kernel<float>, dim3(rows), dim3(256), (size_t)(0), stream, z, ldz, coef, (float*)out, ldo, width, eps));
    else if (dtype == NIB_BF16) NIB_CUDA(launch_pdl(poly_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), (size_t)(0), stream, z, ldz, coef, (__nv_bfloat16*)out, ldo, width, eps));
    else NIB_REQUIRE(false, "poly_norm: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- weighted sum of streams
// hist holds `cap` streams of `n_elem` floats each. The newest stream is x (it becomes hist[n - 1]); x then
// becomes sum_{j < n} coef[j] * hist[j], added in ascending j.
__global__ void depth_mix_kernel(float* __restrict__ hist, float* __restrict__ x, const float* __restrict__ coef, int n,
                                 long long n_elem) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elem) return;
    const float newest = x[i];
    hist[(size_t)(n - 1) * n_elem + i] = newest;
    float acc = 0.f;
    for (int j = 0; j < n - 1; ++j) acc = fmaf(coef[j], hist[(size_t)j * n_elem + i], acc);
    x[i] = fmaf(coef[n - 1], newest, acc);
}

// the same with four elements a thread (n_elem a multiple of 4, 16-byte aligned streams)
__global__ void depth_mix4_kernel(float4* __restrict__ hist, float4* __restrict__ x, const float* __restrict__ coef, int n,
                                  long long n_vec) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const float4 newest = x[i];
    hist[(size_t)(n - 1) * n_vec + i] = newest;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < n - 1; ++j) {
        const float c = coef[j];
        const float4 h = hist[(size_t)j * n_vec + i];
        acc.x = fmaf(c, h.x, acc.x); acc.y = fmaf(c, h.y, acc.y); acc.z = fmaf(c, h.z, acc.z); acc.w = fmaf(c, h.w, acc.w);
    }
    const float c = coef[n - 1];
    x[i] = make_float4(fmaf(c, newest.x, acc.x), fmaf(c, newest.y, acc.y), fmaf(c, newest.z, acc.z), fmaf(c, newest.w, acc.w));
}

NIB_API int nib_depth_mix(float* hist, float* x, const float* coef, int n, long long n_elem, cudaStream_t stream) {
    NIB_REQUIRE(n >= 1 && n_elem >= 0, "depth_mix: bad sizes n=%d", n);
    if (n_elem == 0) return 0;
    if (n_elem % 4 == 0 && (((uintptr_t)hist | (uintptr_t)x) & 15) == 0)
        NIB_CUDA(launch_pdl(depth_mix4_kernel, dim3(ceil_div(n_elem / 4, 256)), dim3(256), (size_t)(0), stream, (float4*)hist, (float4*)x, coef, n, n_elem / 4));
    else
        NIB_CUDA(launch_pdl(depth_mix_kernel, dim3(ceil_div(n_elem, 256)), dim3(256), (size_t)(0), stream, hist, x, coef, n, n_elem));
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- unary function + cast
// out[t, c] = f(in[t, c]) for c < width; kind 0: tanh, 1: identity, 2: sigmoid.
template <typename T>
__global__ void unary_kernel(const float* __restrict__ in, int ld_in, T* __restrict__ out, int ld_out, int rows, int width, int kind) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    float v = in[(size_t)t * ld_in + c];
    if (kind == 0) v = tanhf(v);
    else if (kind == 2) v = 1.0f / (1.0f + expf(-v));
    Elem<T>::store(out + (size_t)t * ld_out + c, v);
}

NIB_API int nib_unary(const float* in, int ld_in, void* out, int ld_out, int rows, int width, int kind, int dtype,
                      cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && width > 0 && kind >= 0 && kind <= 2, "unary: bad arguments");
    if (rows == 0) return 0;
    const int blocks = ceil_div((long long)rows * width, 256);
    if (dtype == NIB_F32) NIB_CUDA(launch_pdl(unary_kernel<float>, dim3(blocks), dim3(256), (size_t)(0), stream, in, ld_in, (float*)out, ld_out, rows, width, kind));
    else if (dtype == NIB_BF16) NIB_CUDA(launch_pdl(unary_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), (size_t)(0), stream, in, ld_in, (__nv_bfloat16*)out, ld_out, rows, width, kind));
    else NIB_REQUIRE(false, "unary: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- per-head norm and gate
// out[t, h*d + j] = o[t, h, j] / sqrt(mean_j o[t, h, :]^2 + eps) * gain[h*d + j] * sigmoid(gate[t, h*d + j]).
// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg,
                      const float* __restrict__ gain, T* __restrict__ out, int ld_out, int tokens, int heads, int d, float eps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)tokens * heads) return;
    const int t = (int)(w / heads), h = (int)(w % heads);
    const float* orow = o + (size_t)t * ldo + (size_t)h * d;
    float ss = 0.f;
    for (int j = lane; j < d; j += 32) ss = fmaf(orow[j], orow[j], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int j = lane; j < d; j += 32) {
        const float g = gate[(size_t)t * ldg + (size_t)h * d + j];
        const float v = orow[j] * scale * gain[h * d + j] * (1.0f / (1.0f + expf(-g)));
        Elem<T>::store(out + (size_t)t * ld_out + (size_t)h * d + j, v);
    }
}

NIB_API int nib_head_norm_gate(const float* o, int ldo, const float* gate, int ldg, const float* gain, void* out, int ld_out,
                               int tokens, int heads, int d, float eps, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && heads > 0 && d > 0, "head_norm_gate: bad sizes");
    if (tokens == 0) return 0;
    const int blocks = ceil_div((long long)tokens * heads, 4);
    if (dtype == NIB_F32) NIB_CUDA(launch_pdl(head_norm_gate_kernel<float>, dim3(blocks), dim3(128), (size_t)(0), stream, o, ldo, gate, ldg, gain, (float*)out, ld_out, tokens, heads, d, eps));
    else if (dtype == NIB_BF16) NIB_CUDA(launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), (size_t)(0), stream, o, ldo, gate, ldg, gain, (__nv_bfloat16*)out, ld_out, tokens, heads, d, eps));
    else NIB_REQUIRE(false, "head_norm_gate: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- two RMS norms of one row
// out_a = x / rms(x) * gain_a and out_b = x / rms(x) * gain_b: the two branches of a parallel block read the same
// stream, so the row is read and its statistic computed once. One warp per row, the row in registers (NV float4 a
// lane); widths that are multiples of 4 up to 128 * NV.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
rmsnorm_pair_kernel(const float* __restrict__ x, const float* __restrict__ gain_a, const float* __restrict__ gain_b,
                    T* __restrict__ out_a, T* __restrict__ out_b, int n_rows, int hidden, float eps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int n4 = hidden >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)r * hidden);
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c >= n4) continue;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gain_a) + c), gb = __ldg(reinterpret_cast<const float4*>(gain_b) + c);
        const float sx = v[i].x * scale, sy = v[i].y * scale, sz = v[i].z * scale, sw = v[i].w * scale;
        T* oa = out_a + (size_t)r * hidden + 4 * c;
        T* ob = out_b + (size_t)r * hidden + 4 * c;
        Elem<T>::store(oa, sx * ga.x); Elem<T>::store(oa + 1, sy * ga.y); Elem<T>::store(oa + 2, sz * ga.z); Elem<T>::store(oa + 3, sw * ga.w);
        Elem<T>::store(ob, sx * gb.x); Elem<T>::store(ob + 1, sy * gb.y); Elem<T>::store(ob + 2, sz * gb.z); Elem<T>::store(ob + 3, sw * gb.w);
    }
}

// 1 if nib_rmsnorm_pair takes rows of this width.
NIB_API int nib_rmsnorm_pair_supported(int hidden) { return (hidden % 4 == 0 && hidden > 0 && hidden <= 4096) ? 1 : 0; }

NIB_API int nib_rmsnorm_pair(const float* x, const float* gain_a, const float* gain_b, void* out_a, void* out_b, int n_rows,
                             int hidden, float eps, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(n_rows >= 0 && nib_rmsnorm_pair_supported(hidden) == 1, "rmsnorm_pair: bad sizes rows=%d hidden=%d", n_rows, hidden);
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "rmsnorm_pair: unknown dtype %d", dtype);
    NIB_REQUIRE((((uintptr_t)x | (uintptr_t)gain_a | (uintptr_t)gain_b) & 15) == 0, "rmsnorm_pair: rows and gains must start on 16-byte boundaries");
    if (n_rows == 0) return 0;
    const int warps = n_rows >= 8 ? 8 : n_rows;
    const dim3 grid(ceil_div(n_rows, warps)), block(32 * warps);
#define NIB_RP(T, NV) NIB_CUDA(launch_pdl(rmsnorm_pair_kernel<T, NV>, dim3(grid), dim3(block), (size_t)(0), stream, x, gain_a, gain_b, (T*)out_a, (T*)out_b, n_rows, hidden, eps))
    if (dtype == NIB_F32) {
        if (hidden <= 1024) NIB_RP(float, 8); else if (hidden <= 2048) NIB_RP(float, 16); else NIB_RP(float, 32);
    } else {
        if (hidden <= 1024) NIB_RP(__nv_bfloat16, 8); else if (hidden <= 2048) NIB_RP(__nv_bfloat16, 16); else NIB_RP(__nv_bfloat16, 32);
    }
#undef NIB_RP
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- weighted sum of streams + two norms
// nib_depth_mix followed by nib_rmsnorm_pair of the result, with the row in registers in between: x joins the
// streams as hist[n - 1], becomes their weighted sum (ascending j), and the sum's two RMS norms leave as out_a, out_b.
// One warp per row; widths that are multiples of 4 up to 128 * NV.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
depth_mix_norm_pair_kernel(float* __restrict__ hist, float* __restrict__ x, const float* __restrict__ coef, int n,
                           const float* __restrict__ gain_a, const float* __restrict__ gain_b, T* __restrict__ out_a,
                           T* __restrict__ out_b, int n_rows, int hidden, float eps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int n4 = hidden >> 2;
    const size_t stream4 = (size_t)n_rows * n4;
    float4* xr = reinterpret_cast<float4*>(x) + (size_t)r * n4;
    float4* hr = reinterpret_cast<float4*>(hist) + (size_t)r * n4;
    // One stream at a time, all of the lane's chunks of it in flight together: a lane waits for memory once per stream.
    float4 v[NV], newest[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        newest[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int j = 0; j < n - 1; ++j) {
        const float cj = coef[j];
        float4 h[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            h[i] = c < n4 ? hr[(size_t)j * stream4 + c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            v[i].x = fmaf(cj, h[i].x, v[i].x); v[i].y = fmaf(cj, h[i].y, v[i].y);
            v[i].z = fmaf(cj, h[i].z, v[i].z); v[i].w = fmaf(cj, h[i].w, v[i].w);
        }
    }
    const float c_new = coef[n - 1];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        v[i].x = fmaf(c_new, newest[i].x, v[i].x); v[i].y = fmaf(c_new, newest[i].y, v[i].y);
        v[i].z = fmaf(c_new, newest[i].z, v[i].z); v[i].w = fmaf(c_new, newest[i].w, v[i].w);
        if (c < n4) {
            hr[(size_t)(n - 1) * stream4 + c] = newest[i];
            xr[c] = v[i];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c >= n4) continue;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gain_a) + c), gb = __ldg(reinterpret_cast<const float4*>(gain_b) + c);
        const float sx = v[i].x * scale, sy = v[i].y * scale, sz = v[i].z * scale, sw = v[i].w * scale;
        T* oa = out_a + (size_t)r * hidden + 4 * c;
        T* ob = out_b + (size_t)r * hidden + 4 * c;
        Elem<T>::store(oa, sx * ga.x); Elem<T>::store(oa + 1, sy * ga.y); Elem<T>::store(oa + 2, sz * ga.z); Elem<T>::store(oa + 3, sw * ga.w);
        Elem<T>::store(ob, sx * gb.x); Elem<T>::store(ob + 1, sy * gb.y); Elem<T>::store(ob + 2, sz * gb.z); Elem<T>::store(ob + 3, sw * gb.w);
    }
}

// The same for a handful of rows (a decode step): a block of 256 threads per row, so that a row's streams are fetched
// by 256 threads at once instead of by one warp; four streams in flight per thread.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
depth_mix_norm_pair_row_kernel(float* __restrict__ hist, float* __restrict__ x, const float* __restrict__ coef, int n,
                               const float* __restrict__ gain_a, const float* __restrict__ gain_b, T* __restrict__ out_a,
                               T* __restrict__ out_b, int n_rows, int hidden, float eps) {
    __shared__ float part[8];
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int r = blockIdx.x, tid = threadIdx.x;
    const int n4 = hidden >> 2;
    const size_t stream4 = (size_t)n_rows * n4;
    float4* xr = reinterpret_cast<float4*>(x) + (size_t)r * n4;
    float4* hr = reinterpret_cast<float4*>(hist) + (size_t)r * n4;
    float4 v[NV], newest[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = tid + 256 * i;
        newest[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll 4
    for (int j = 0; j < n - 1; ++j) {           // ascending j, as everywhere
        const float cj = coef[j];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = tid + 256 * i;
            const float4 h = c < n4 ? hr[(size_t)j * stream4 + c] : make_float4(0.f, 0.f, 0.f, 0.f);
            v[i].x = fmaf(cj, h.x, v[i].x); v[i].y = fmaf(cj, h.y, v[i].y);
            v[i].z = fmaf(cj, h.z, v[i].z); v[i].w = fmaf(cj, h.w, v[i].w);
        }
    }
    const float c_new = coef[n - 1];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = tid + 256 * i;
        v[i].x = fmaf(c_new, newest[i].x, v[i].x); v[i].y = fmaf(c_new, newest[i].y, v[i].y);
        v[i].z = fmaf(c_new, newest[i].z, v[i].z); v[i].w = fmaf(c_new, newest[i].w, v[i].w);
        if (c < n4) {
            hr[(size_t)(n - 1) * stream4 + c] = newest[i];
            xr[c] = v[i];
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = block_sum_256(ss, part);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = tid + 256 * i;
        if (c >= n4) continue;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(gain_a) + c), gb = __ldg(reinterpret_cast<const float4*>(gain_b) + c);
        const float sx = v[i].x * scale, sy = v[i].y * scale, sz = v[i].z * scale, sw = v[i].w * scale;
        T* oa = out_a + (size_t)r * hidden + 4 * c;
        T* ob = out_b + (size_t)r * hidden + 4 * c;
        Elem<T>::store(oa, sx * ga.x); Elem<T>::store(oa + 1, sy * ga.y); Elem<T>::store(oa + 2, sz * ga.z); Elem<T>::store(oa + 3, sw * ga.w);
        Elem<T>::store(ob, sx * gb.x); Elem<T>::store(ob + 1, sy * gb.y); Elem<T>::store(ob + 2, sz * gb.z); Elem<T>::store(ob + 3, sw * gb.w);
    }
}

// Takes the widths nib_rmsnorm_pair takes (nib_rmsnorm_pair_supported).
NIB_API int nib_depth_mix_norm_pair(float* hist, float* x, const float* coef, int n, const float* gain_a, const float* gain_b,
                                    void* out_a, void* out_b, int n_rows, int hidden, float eps, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(n >= 1 && n_rows >= 0 && nib_rmsnorm_pair_supported(hidden) == 1, "depth_mix_norm_pair: bad sizes rows=%d hidden=%d", n_rows, hidden);
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "depth_mix_norm_pair: unknown dtype %d", dtype);
    NIB_REQUIRE((((uintptr_t)hist | (uintptr_t)x | (uintptr_t)gain_a | (uintptr_t)gain_b) & 15) == 0, "depth_mix_norm_pair: 16-byte boundaries");
    if (n_rows == 0) return 0;
    if (n_rows <= 32) {         // which kernel runs depends on the step's size alone
#define NIB_DR(T, NV) NIB_CUDA(launch_pdl(depth_mix_norm_pair_row_kernel<T, NV>, dim3(n_rows), dim3(256), (size_t)0, stream, hist, x, coef, n, gain_a, gain_b, (T*)out_a, (T*)out_b, n_rows, hidden, eps))
        if (dtype == NIB_F32) {
            if (hidden <= 1024) NIB_DR(float, 1); else if (hidden <= 2048) NIB_DR(float, 2); else NIB_DR(float, 4);
        } else {
            if (hidden <= 1024) NIB_DR(__nv_bfloat16, 1); else if (hidden <= 2048) NIB_DR(__nv_bfloat16, 2); else NIB_DR(__nv_bfloat16, 4);
        }
#undef NIB_DR
        return 0;
    }
    const int warps = n_rows >= 8 ? 8 : n_rows;
    const dim3 grid(ceil_div(n_rows, warps)), block(32 * warps);
#define NIB_DP(T, NV) NIB_CUDA(launch_pdl(depth_mix_norm_pair_kernel<T, NV>, grid, block, (size_t)0, stream, hist, x, coef, n, gain_a, gain_b, (T*)out_a, (T*)out_b, n_rows, hidden, eps))
    if (dtype == NIB_F32) {
        if (hidden <= 1024) NIB_DP(float, 8); else if (hidden <= 2048) NIB_DP(float, 16); else NIB_DP(float, 32);
    } else {
        if (hidden <= 1024) NIB_DP(__nv_bfloat16, 8); else if (hidden <= 2048) NIB_DP(__nv_bfloat16, 16); else NIB_DP(__nv_bfloat16, 32);
    }
#undef NIB_DP
    return 0;
}

// ---------------------------------------------------------------------------------- gate, norm in groups, skip
// For a row o of n floats cut into `groups` equal parts (a warp per (token, part)):
//     y = o (+ coef[c / (n / n_coef)] * skip)          a skip connection with one coefficient per head
//     y = y * act(gate)                                 if gate_first
//     y = y / sqrt(mean_part(y^2) + eps)                if norm
//     y = y * gain[c % gain_len]                        gain_len = n (a gain per channel) or a part's size (shared)
//     y = y * act(gate)                                 if not gate_first
//     out = y * out_scale
// act: 1 sigmoid, 2 silu, 0 none. With norm the part is read twice (sum of squares, then the result).
__device__ __forceinline__ float gate_act(float g, int kind) {
    const float s = 1.0f / (1.0f + expf(-g));
    return kind == 1 ? s : g * s;
}

template <typename T>
__global__ void __launch_bounds__(128)
gated_norm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg, int gate_kind, int gate_first,
                  const float* __restrict__ gain, int gain_len, const float* __restrict__ skip, int lds,
                  const float* __restrict__ coef, int coef_span, int norm, float eps, float out_scale,
                  T* __restrict__ out, int ld_out, int tokens, int groups, int width) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)tokens * groups) return;
    const int t = (int)(w / groups), c0 = (int)(w % groups) * width;
    const float* orow = o + (size_t)t * ldo;
    const float* grow = gate != nullptr ? gate + (size_t)t * ldg : nullptr;
    const float* srow = skip != nullptr ? skip + (size_t)t * lds : nullptr;
    const bool early = grow != nullptr && gate_kind != 0 && gate_first != 0;
    const bool late = grow != nullptr && gate_kind != 0 && gate_first == 0;
    float scale = 1.0f;
    if (norm) {
        float ss = 0.f;
        for (int j = lane; j < width; j += 32) {
            const int c = c0 + j;
            float y = orow[c];
            if (srow != nullptr) y = fmaf(coef[c / coef_span], srow[c], y);
            if (early) y *= gate_act(grow[c], gate_kind);
            ss = fmaf(y, y, ss);
        }
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)width + eps);
    }
    for (int j = lane; j < width; j += 32) {
        const int c = c0 + j;
        float y = orow[c];
        if (srow != nullptr) y = fmaf(coef[c / coef_span], srow[c], y);
        if (early) y *= gate_act(grow[c], gate_kind);
        y *= scale;
        if (gain != nullptr) y *= gain[c % gain_len];
        if (late) y *= gate_act(grow[c], gate_kind);
        Elem<T>::store(out + (size_t)t * ld_out + c, y * out_scale);
    }
}

// The same for wide parts (a state-space mixer's norm over thousands of channels): a block of 256 threads per
// (token, part), so that the few rows of a decode step are not walked by one warp each.
template <typename T>
__global__ void __launch_bounds__(256)
gated_norm_block_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ gate, int ldg, int gate_kind, int gate_first,
                        const float* __restrict__ gain, int gain_len, const float* __restrict__ skip, int lds,
                        const float* __restrict__ coef, int coef_span, int norm, float eps, float out_scale,
                        T* __restrict__ out, int ld_out, int tokens, int groups, int width) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float part[8];
    const int t = blockIdx.x / groups, c0 = (blockIdx.x % groups) * width;
    const float* orow = o + (size_t)t * ldo;
    const float* grow = gate != nullptr ? gate + (size_t)t * ldg : nullptr;
    const float* srow = skip != nullptr ? skip + (size_t)t * lds : nullptr;
    const bool early = grow != nullptr && gate_kind != 0 && gate_first != 0;
    const bool late = grow != nullptr && gate_kind != 0 && gate_first == 0;
    float scale = 1.0f;
    if (norm) {
        float ss = 0.f;
        for (int j = threadIdx.x; j < width; j += 256) {
            const int c = c0 + j;
            float y = orow[c];
            if (srow != nullptr) y = fmaf(coef[c / coef_span], srow[c], y);
            if (early) y *= gate_act(grow[c], gate_kind);
            ss = fmaf(y, y, ss);
        }
        scale = 1.0f / sqrtf(block_sum_256(ss, part) / (float)width + eps);
    }
    for (int j = threadIdx.x; j < width; j += 256) {
        const int c = c0 + j;
        float y = orow[c];
        if (srow != nullptr) y = fmaf(coef[c / coef_span], srow[c], y);
        if (early) y *= gate_act(grow[c], gate_kind);
        y *= scale;
        if (gain != nullptr) y *= gain[c % gain_len];
        if (late) y *= gate_act(grow[c], gate_kind);
        Elem<T>::store(out + (size_t)t * ld_out + c, y * out_scale);
    }
}

NIB_API int nib_gated_norm(const float* o, int ldo, const float* gate, int ldg, int gate_kind, int gate_first, const float* gain,
                           int gain_len, const float* skip, int lds, const float* coef, int n_coef, int groups, int norm, float eps,
                           float out_scale, void* out, int ld_out, int tokens, int n, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && n > 0 && groups > 0 && n % groups == 0, "gated_norm: %d channels do not split into %d parts", n, groups);
    NIB_REQUIRE(gain == nullptr || (gain_len > 0 && n % gain_len == 0), "gated_norm: a gain of %d does not tile %d channels", gain_len, n);
    NIB_REQUIRE(skip == nullptr || (coef != nullptr && n_coef > 0 && n % n_coef == 0), "gated_norm: bad skip coefficients");
    NIB_REQUIRE(gate_kind >= 0 && gate_kind <= 2, "gated_norm: unknown gate kind %d", gate_kind);
    if (tokens == 0) return 0;
    const int width = n / groups, span = skip != nullptr ? n / n_coef : 1;
    if (width > 256) {
        const dim3 grid(tokens * groups);
        if (dtype == NIB_F32) NIB_CUDA(launch_pdl(gated_norm_block_kernel<float>, grid, dim3(256), (size_t)(0), stream, o, ldo, gate, ldg, gate_kind, gate_first, gain, gain_len, skip, lds, coef, span, norm, eps, out_scale, (float*)out, ld_out, tokens, groups, width));
        else if (dtype == NIB_BF16) NIB_CUDA(launch_pdl(gated_norm_block_kernel<__nv_bfloat16>, grid, dim3(256), (size_t)(0), stream, o, ldo, gate, ldg, gate_kind, gate_first, gain, gain_len, skip, lds, coef, span, norm, eps, out_scale, (__nv_bfloat16*)out, ld_out, tokens, groups, width));
        else NIB_REQUIRE(false, "gated_norm: unknown dtype %d", dtype);
        NIB_LAUNCH_CHECK();
        return 0;
    }
    const int blocks = ceil_div((long long)tokens * groups, 4);
    if (dtype == NIB_F32) NIB_CUDA(launch_pdl(gated_norm_kernel<float>, dim3(blocks), dim3(128), (size_t)(0), stream, o, ldo, gate, ldg, gate_kind, gate_first, gain, gain_len, skip, lds, coef, span, norm, eps, out_scale, (float*)out, ld_out, tokens, groups, width));
    else if (dtype == NIB_BF16) NIB_CUDA(launch_pdl(gated_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), (size_t)(0), stream, o, ldo, gate, ldg, gate_kind, gate_first, gain, gain_len, skip, lds, coef, span, norm, eps, out_scale, (__nv_bfloat16*)out, ld_out, tokens, groups, width));
    else NIB_REQUIRE(false, "gated_norm: unknown dtype %d", dtype);
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- norm of a branch's output, added
// x[t] += mult * y[t] / sqrt(mean(y[t]^2) + eps) * gain: the residual sum of a block whose norm stands on the
// sublayer's OUTPUT. With `h_out` the new x is also written in the storage type (what the next sublayer reads);
// with `clear` y is left zeroed, ready for the next sublayer's products to add into. A block per row when rows are
// few (a decode step), else a warp per row. All arithmetic is 32-bit. With `next_gain` what goes to `h_out` is not the
// new x but the NEXT sublayer's norm of it, x / sqrt(mean(x^2) + next_eps) * next_gain: a block with a norm before and
// after each sublayer then makes one pass over the rows per sublayer.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_add_kernel(float* __restrict__ y, const float* __restrict__ gain, float* __restrict__ x, T* __restrict__ h_out,
                   int rows, int width, float eps, float mult, int clear, int vec, const float* __restrict__ next_gain, float next_eps) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ float part[THREADS / 32];
    constexpr bool BLOCK_ROW = THREADS > 32 * 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = BLOCK_ROW ? blockIdx.x : blockIdx.x * (THREADS / 32) + warp;
    if (row >= rows) return;        // a whole block (block per row) or a whole warp (warp per row) leaves together
    const int first = BLOCK_ROW ? threadIdx.x : lane, step = BLOCK_ROW ? THREADS : 32;
    float* yr = y + (size_t)row * width;
    float* xr = x + (size_t)row * width;
    float ss = 0.f;
    if (vec) {      // rows of whole 16-byte groups: four elements a load
        for (int c = first * 4; c < width; c += step * 4) {
            const float4 v = *reinterpret_cast<const float4*>(yr + c);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int c = first; c < width; c += step) ss = fmaf(yr[c], yr[c], ss);
    }
    ss = warp_sum(ss);
    if (BLOCK_ROW) {
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < THREADS / 32; ++w) ss += part[w];      // the same order in every thread
    }
    const float scale = mult / sqrtf(ss / (float)width + eps);
    if (next_gain != nullptr) {
        // the sum, the sum of squares of the new row, and then the next norm of it (the row comes back from L1/L2)
        float s2 = 0.f;
        if (vec) {
            for (int c = first * 4; c < width; c += step * 4) {
                const float4 yv = *reinterpret_cast<const float4*>(yr + c), g = __ldg(reinterpret_cast<const float4*>(gain + c));
                float4 v = *reinterpret_cast<const float4*>(xr + c);
                v.x += yv.x * scale * g.x; v.y += yv.y * scale * g.y; v.z += yv.z * scale * g.z; v.w += yv.w * scale * g.w;
                *reinterpret_cast<float4*>(xr + c) = v;
                s2 = fmaf(v.x, v.x, s2); s2 = fmaf(v.y, v.y, s2); s2 = fmaf(v.z, v.z, s2); s2 = fmaf(v.w, v.w, s2);
                if (clear) *reinterpret_cast<float4*>(yr + c) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        } else {
            for (int c = first; c < width; c += step) {
                const float v = xr[c] + yr[c] * scale * gain[c];
                xr[c] = v;
                s2 = fmaf(v, v, s2);
                if (clear) yr[c] = 0.f;
            }
        }
        s2 = warp_sum(s2);
        if (BLOCK_ROW) {
            __syncthreads();        // every thread has read the first sum's parts
            if (lane == 0) part[warp] = s2;
            __syncthreads();
            s2 = 0.f;
            for (int w = 0; w < THREADS / 32; ++w) s2 += part[w];
        }
        const float scale2 = 1.0f / sqrtf(s2 / (float)width + next_eps);
        if (h_out == nullptr) return;
        if (vec) {      // (every thread reads back what it wrote itself)
            for (int c = first * 4; c < width; c += step * 4) {
                const float4 g = __ldg(reinterpret_cast<const float4*>(next_gain + c));
                float4 v = *reinterpret_cast<const float4*>(xr + c);
                v.x *= scale2 * g.x; v.y *= scale2 * g.y; v.z *= scale2 * g.z; v.w *= scale2 * g.w;
                T* ho = h_out + (size_t)row * width + c;
                if constexpr (sizeof(T) == 4) {
                    *reinterpret_cast<float4*>(ho) = v;
                } else {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const unsigned*>(&lo);
                    pk.y = *reinterpret_cast<const unsigned*>(&hi);
                    *reinterpret_cast<uint2*>(ho) = pk;
                }
            }
        } else {
            for (int c = first; c < width; c += step) Elem<T>::store(h_out + (size_t)row * width + c, xr[c] * scale2 * next_gain[c]);
        }
        return;
    }
    if (vec) {
        for (int c = first * 4; c < width; c += step * 4) {
            const float4 yv = *reinterpret_cast<const float4*>(yr + c), g = __ldg(reinterpret_cast<const float4*>(gain + c));
            float4 v = *reinterpret_cast<const float4*>(xr + c);
            v.x += yv.x * scale * g.x; v.y += yv.y * scale * g.y; v.z += yv.z * scale * g.z; v.w += yv.w * scale * g.w;
            *reinterpret_cast<float4*>(xr + c) = v;
            if (h_out != nullptr) {
                T* ho = h_out + (size_t)row * width + c;
                if constexpr (sizeof(T) == 4) {
                    *reinterpret_cast<float4*>(ho) = v;
                } else {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const unsigned*>(&lo);
                    pk.y = *reinterpret_cast<const unsigned*>(&hi);
                    *reinterpret_cast<uint2*>(ho) = pk;
                }
            }
            if (clear) *reinterpret_cast<float4*>(yr + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    for (int c = first; c < width; c += step) {
        const float v = xr[c] + yr[c] * scale * gain[c];
        xr[c] = v;
        if (h_out != nullptr) Elem<T>::store(h_out + (size_t)row * width + c, v);
        if (clear) yr[c] = 0.f;
    }
}

NIB_API int nib_rmsnorm_add(float* y, const float* gain, float* x, void* h_out, int rows, int width, float eps, float mult,
                            int clear, int dtype, const float* next_gain, float next_eps, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && width > 0, "rmsnorm_add: bad sizes");
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "rmsnorm_add: unknown dtype %d", dtype);
    if (rows == 0) return 0;
    const bool block_row = rows <= 64 && width >= 512;
    const int vec = (width % 4 == 0 && (((uintptr_t)y | (uintptr_t)gain | (uintptr_t)x | (uintptr_t)h_out | (uintptr_t)next_gain) & 15) == 0) ? 1 : 0;
#define NIB_RA(T, THREADS, GRID) \
    NIB_CUDA(launch_pdl(rmsnorm_add_kernel<T, THREADS>, dim3(GRID), dim3(THREADS), (size_t)0, stream, y, gain, x, (T*)h_out, rows, width, eps, mult, clear, vec, next_gain, next_eps))
    if (block_row) {
        if (dtype == NIB_F32) NIB_RA(float, 256, rows); else NIB_RA(__nv_bfloat16, 256, rows);
    } else {
        if (dtype == NIB_F32) NIB_RA(float, 128, ceil_div(rows, 4)); else NIB_RA(__nv_bfloat16, 128, ceil_div(rows, 4));
    }
#undef NIB_RA
    NIB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------- identity outputs of a router
// The router outputs from `n_real` on have no weights: such a choice stands for the token's input itself, so
// out[t] += (sum of the weights of the token's choices e >= n_real) * h[t]. A block per token.
template <typename T>
__global__ void __launch_bounds__(256)
moe_identity_kernel(const T* __restrict__ h, int ldh, const int* __restrict__ sel_e, const float* __restrict__ sel_w, int top, int n_real,
                    float* __restrict__ out, int ldo, int hidden) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int t = blockIdx.x;
    float wsum = 0.f;
    bool any = false;
    for (int k = 0; k < top; ++k)       // ascending order of choice, the same in every thread
        if (sel_e[(size_t)t * top + k] >= n_real) { wsum += sel_w[(size_t)t * top + k]; any = true; }
    if (!any) return;
    for (int c = threadIdx.x; c < hidden; c += 256) out[(size_t)t * ldo + c] += wsum * Elem<T>::load(h + (size_t)t * ldh + c);
}

NIB_API int nib_moe_identity(const void* h, int ldh, const int* sel_e, const float* sel_w, int top, int n_real, float* out, int ldo, int hidden,
                             int tokens, int dtype, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && sel_e != nullptr && sel_w != nullptr && out != nullptr && h != nullptr && top > 0 && hidden > 0 && n_real >= 0,
                "moe_identity: bad arguments");
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "moe_identity: unknown dtype %d", dtype);
    if (tokens == 0) return 0;
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(moe_identity_kernel<float>, dim3(tokens), dim3(256), (size_t)0, stream, (const float*)h, ldh, sel_e, sel_w, top, n_real, out, ldo, hidden));
    else
        NIB_CUDA(launch_pdl(moe_identity_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), (size_t)0, stream, (const __nv_bfloat16*)h, ldh, sel_e, sel_w, top,
                            n_real, out, ldo, hidden));
    NIB_LAUNCH_CHECK();
    return 0;
}
