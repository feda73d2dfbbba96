// Routed experts: every token goes through `top` of `experts` small gated feed-forwards, chosen by a router.
//
//  * moe_route: from the 32-bit router logits z [tokens, experts]: the `top` largest (the first of equal ones), and
//    for each its weight sigmoid(z) (not renormalized). One warp per token.
//  * moe_group: the (token, choice) entries ordered by expert: row_of[entry] = its row in that order, src_of[row] = the
//    entry, and a table of row tiles (expert, first row, rows), none of which spans two experts. One block; the table's
//    length depends on the routing, so the products below are launched with the largest grid the sizes allow and a
//    block without a tile leaves at once: the launches never depend on the batch's content.
//  * moe_gemm (CUDA cores; any sizes, float or bfloat16): per tile, rows gathered through src_of:
//      gate/up:  act[row] = silu(w g) * (w u),  g = W_gate,e h, u = W_up,e h,  w = the entry's weight
//                (the weight stands on the expert's INPUT; W (w h) = w (W h), so it is applied in 32-bit to the products),
//      down:     y[row] = W_down,e act[row] as floats; with one choice per token straight into the token's output row.
//    Every output element is accumulated by one thread over ascending k: a row's result depends on the row alone.
//  * moe_combine: out[t] += sum over the token's choices, in ascending order of choice, of y[row_of[t, choice]].
//
// Options that other designs of a mixture combine (all off = the form above):
//  * scores: softmax over all router outputs instead of sigmoid (MOE_SOFTMAX); a correction per output that is added to
//    the scores for the CHOICE only (`corr`); the chosen scores divided by their sum + 1e-20 (MOE_RENORM);
//  * the weight on the expert's OUTPUT instead of its input (`w_out`);
//  * experts without a gate: W_down relu(W_up x)^2 (mode 2 of the products);
//  * router outputs from `n_real` on that stand for no expert (the caller adds what they mean, see moe_identity in
//    pointwise.cu): they are chosen and weighted like the others, but get no row tiles;
//  * `always` experts that every token uses (a shared expert, cut into pieces of the experts' width): they are the first
//    `always` of the stacked experts, so a chosen router output o becomes expert o + always; every token gets `always` more
//    entries behind its `top` chosen ones, each weighted by sigmoid of one more logit that stands behind the router's in
//    the token's row (zr[experts]). The entries of a token are then `top + always` wide.
#include "common.cuh"
#include <climits>

constexpr int MOE_MAX_EXPERTS = 1024;

enum { MOE_SOFTMAX = 1, MOE_RENORM = 2 };

// One warp chooses for one token: the `top` largest of zr[0..experts) (the first of equal ones) and their sigmoids.
// With options the logits are first turned into scores IN PLACE (softmax over all of them, or sigmoid), the choice goes
// by score + corr, and the weights are the chosen scores, divided by their sum + 1e-20 with MOE_RENORM.
__device__ __forceinline__ void route_token(float* zr, int experts, int top, int lane, int* sel_e, float* sel_w, int mode, const float* corr,
                                            int always) {
    unsigned taken = 0;     // bit j: this lane's expert lane + 32 j is chosen already
    if (always > 0 && lane == 0) {
        const float g = 1.0f / (1.0f + expf(-zr[experts]));
        for (int j = 0; j < always; ++j) { sel_e[top + j] = j; sel_w[top + j] = g; }
    }
    if (mode != 0 || corr != nullptr) {
        if (mode & MOE_SOFTMAX) {
            float mx = -INFINITY;
            for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, zr[e]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int e = lane; e < experts; e += 32) sum += expf(zr[e] - mx);
            sum = warp_sum(sum);
            for (int e = lane; e < experts; e += 32) zr[e] = expf(zr[e] - mx) / sum;
        } else {
            for (int e = lane; e < experts; e += 32) zr[e] = 1.0f / (1.0f + expf(-zr[e]));
        }
        __syncwarp();
        float total = 0.f;      // lane 0: the chosen scores' sum, in the order of choice
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int bi = INT_MAX;
            for (int j = 0; lane + 32 * j < experts; ++j) {
                if ((taken >> j) & 1u) continue;
                const int e = lane + 32 * j;
                const float v = zr[e] + (corr != nullptr ? corr[e] : 0.f);
                if (bi == INT_MAX || v > best) { best = v; bi = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != INT_MAX && (bi == INT_MAX || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
            }
            if (bi == INT_MAX) bi = 0;
            if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
            if (lane == 0) {
                sel_e[k] = bi + always;
                sel_w[k] = zr[bi];
                total += zr[bi];
            }
        }
        if (lane == 0 && (mode & MOE_RENORM)) {
            const float inv = 1.0f / (total + 1e-20f);
            for (int k = 0; k < top; ++k) sel_w[k] *= inv;
        }
        return;
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = INT_MAX;
        for (int j = 0; lane + 32 * j < experts; ++j) {
            if ((taken >> j) & 1u) continue;
            const int e = lane + 32 * j;
            const float v = zr[e];
            if (bi == INT_MAX || v > best) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != INT_MAX && (bi == INT_MAX || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
        }
        if (bi == INT_MAX) bi = 0;
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (lane == 0) {
            sel_e[k] = bi + always;
            sel_w[k] = 1.0f / (1.0f + expf(-best));
        }
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(float* __restrict__ z, int ldz, int* __restrict__ sel_e, float* __restrict__ sel_w, int tokens, int experts, int top, int mode,
                 const float* __restrict__ corr, int always) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    route_token(z + (size_t)t * ldz, experts, top, lane, sel_e + (size_t)t * (top + always), sel_w + (size_t)t * (top + always), mode, corr, always);
}

// The (token, choice) entries ordered by expert, by one block of any size. tiles: [max_tiles, 3] = (expert, first row,
// rows); n_tiles[0] = how many are in use. cnt, off, toff, cur: shared arrays of MOE_MAX_EXPERTS ints.
// Router outputs from n_real on are no experts: their entries get rows (behind all experts' rows) but no tiles.
__device__ __forceinline__ void group_entries(const int* sel_e, int n, int experts, int tile_rows, int* row_of, int* src_of, int* tiles,
                                              int* n_tiles, int max_tiles, int* cnt, int* off, int* toff, int* cur, int n_real) {
    const int tid = threadIdx.x, lane = tid & 31;
    for (int e = tid; e < experts; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) atomicAdd(&cnt[sel_e[i]], 1);
    __syncthreads();
    if (tid < 32) {     // exclusive sums of the rows and of the tiles, 32 experts at a time
        int run = 0, trun = 0;
        for (int base = 0; base < experts; base += 32) {
            const int c = base + lane < experts ? cnt[base + lane] : 0;
            const int tl = base + lane < n_real ? (c + tile_rows - 1) / tile_rows : 0;
            int ic = c, it = tl;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int a = __shfl_up_sync(0xffffffffu, ic, o), b = __shfl_up_sync(0xffffffffu, it, o);
                if (lane >= o) { ic += a; it += b; }
            }
            if (base + lane < experts) { off[base + lane] = run + ic - c; toff[base + lane] = trun + it - tl; }
            run += __shfl_sync(0xffffffffu, ic, 31);
            trun += __shfl_sync(0xffffffffu, it, 31);
        }
        if (lane == 0) n_tiles[0] = min(trun, max_tiles);
    }
    __syncthreads();
    for (int e = tid; e < n_real; e += blockDim.x) {
        const int c = cnt[e];
        for (int j = 0; j * tile_rows < c; ++j) {
            const int ti = toff[e] + j;
            if (ti < max_tiles) {
                tiles[3 * ti] = e;
                tiles[3 * ti + 1] = off[e] + j * tile_rows;
                tiles[3 * ti + 2] = min(tile_rows, c - j * tile_rows);
            }
        }
    }
    // a token's entries keep their order within an expert's rows only by chance: nothing reads that order
    for (int i = tid; i < n; i += blockDim.x) {
        const int e = sel_e[i];
        const int pos = off[e] + atomicAdd(&cur[e], 1);
        row_of[i] = pos;
        src_of[pos] = i;
    }
}

__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ sel_e, int n, int experts, int tile_rows, int* __restrict__ row_of, int* __restrict__ src_of,
                 int* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles, int n_real) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ int cnt[MOE_MAX_EXPERTS], off[MOE_MAX_EXPERTS], toff[MOE_MAX_EXPERTS], cur[MOE_MAX_EXPERTS];
    group_entries(sel_e, n, experts, tile_rows, row_of, src_of, tiles, n_tiles, max_tiles, cnt, off, toff, cur, n_real);
}

// A step of few tokens in ONE launch of one block: router logits z = W_router h (32-bit sums over the stored h), the
// choice, the grouping, and with `rows` the tokens' rows copied into the grouped order (what the tensor-core products read).
// w_router may hold `extra` more rows behind the router's: their logits (a gate per token) leave in z_extra [tokens, extra].
constexpr int MOE_STEP_MAX_Z = 2048;     // tokens * experts

// Sixteen bytes of a row as floats: 8 bfloat16 or 4 floats.
__device__ __forceinline__ void unpack16(const uint4& u, const __nv_bfloat16*, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(p[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
__device__ __forceinline__ void unpack16(const uint4& u, const float*, float (&f)[8]) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    f[4] = f[5] = f[6] = f[7] = 0.f;
}

// `vec`: rows and bases are 16-byte aligned and the width is a multiple of 16 bytes, so rows move 16 bytes at a time.
template <typename T>
__global__ void __launch_bounds__(1024)
moe_step_kernel(const T* __restrict__ h, int ldh, const T* __restrict__ w_router, int tokens, int hidden, int experts, int top,
                int* __restrict__ sel_e, float* __restrict__ sel_w, int tile_rows, int* __restrict__ row_of, int* __restrict__ src_of,
                int* __restrict__ tiles, int* __restrict__ n_tiles, int max_tiles, T* __restrict__ rows, int vec, int mode,
                const float* __restrict__ corr, int n_real, int extra, float* __restrict__ z_extra, int always) {
    constexpr int V = 16 / (int)sizeof(T);
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    __shared__ int cnt[MOE_MAX_EXPERTS], off[MOE_MAX_EXPERTS], toff[MOE_MAX_EXPERTS], cur[MOE_MAX_EXPERTS];
    __shared__ float z[MOE_STEP_MAX_Z];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    const int outs = experts + extra;
    for (int p = warp; p < tokens * outs; p += warps) {      // a warp per (token, router output)
        const int t = p / outs, e = p - t * outs;
        const T* hr = h + (size_t)t * ldh;
        const T* wr = w_router + (size_t)e * hidden;
        float acc = 0.f;
        if (vec) {
#pragma unroll 4
            for (int k = lane * V; k < hidden; k += 32 * V) {
                float a[8], b[8];
                unpack16(__ldg(reinterpret_cast<const uint4*>(hr + k)), hr, a);
                unpack16(__ldg(reinterpret_cast<const uint4*>(wr + k)), wr, b);
#pragma unroll
                for (int i = 0; i < V; ++i) acc = fmaf(a[i], b[i], acc);
            }
        } else {
            for (int k = lane; k < hidden; k += 32) acc = fmaf(Elem<T>::load(hr + k), Elem<T>::load(wr + k), acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            z[p] = acc;
            if (e >= experts && z_extra != nullptr) z_extra[(size_t)t * extra + (e - experts)] = acc;
        }
    }
    __syncthreads();
    for (int t = warp; t < tokens; t += warps)
        route_token(z + t * outs, experts, top, lane, sel_e + (size_t)t * (top + always), sel_w + (size_t)t * (top + always), mode, corr, always);
    __syncthreads();        // the block's own writes to sel_e are visible to all of its threads
    top += always;          // from here on a token's entries are its chosen and its always-used experts
    experts += always;
    const int n = tokens * top;
    group_entries(sel_e, n, experts, tile_rows, row_of, src_of, tiles, n_tiles, max_tiles, cnt, off, toff, cur, n_real);
    if (rows == nullptr) return;
    __syncthreads();
    if (vec) {
        const int per_row = hidden / V;
#pragma unroll 4
        for (int i = tid; i < n * per_row; i += blockDim.x) {
            const int r = i / per_row, c = (i - r * per_row) * V;
            *reinterpret_cast<uint4*>(rows + (size_t)r * hidden + c) = __ldg(reinterpret_cast<const uint4*>(h + (size_t)(src_of[r] / top) * ldh + c));
        }
    } else {
        for (int i = tid; i < n * hidden; i += blockDim.x) {
            const int r = i / hidden, c = i - r * hidden;
            rows[(size_t)r * hidden + c] = h[(size_t)(src_of[r] / top) * ldh + c];
        }
    }
}

// MODE 0: down; 1: gate and up, silu(g) u; 2: up alone, relu(u)^2. w_out: the weight multiplies the down product's result
// instead of the first product's input.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, void* __restrict__ out, int ldo,
                     const int* __restrict__ tiles, const int* __restrict__ n_tiles, const int* __restrict__ src_of,
                     const float* __restrict__ sel_w, int top, int N, int K, int scatter, int w_out) {
    constexpr bool GATE_UP = MODE == 1, FIRST = MODE != 0;
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    if ((int)blockIdx.y >= n_tiles[0]) return;
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    __shared__ float Us[GATE_UP ? BK : 1][GATE_UP ? BN + 1 : 1];
    __shared__ int a_row[BM];       // the activation row each of the tile's rows reads
    __shared__ int o_row[BM];       // the row it writes
    __shared__ float a_wgt[BM];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * BN;
    const T* We = W + (size_t)expert * (GATE_UP ? 2 : 1) * N * K;
    if (tid < BM) {
        const int p = row0 + tid;
        int ar = -1, orow = -1;
        float wg = 0.f;
        if (tid < rows) {
            const int entry = src_of[p];
            ar = FIRST ? entry / top : p;
            orow = (!FIRST && scatter) ? entry / top : p;
            wg = (FIRST == (w_out != 0)) ? 1.0f : sel_w[entry];     // the weight belongs to the other product
        }
        a_row[tid] = ar; o_row[tid] = orow; a_wgt[tid] = wg;
    }
    __syncthreads();

    float acc[TM][TN], acc2[GATE_UP ? TM : 1][GATE_UP ? TN : 1];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    if (GATE_UP) {
#pragma unroll
        for (int i = 0; i < (GATE_UP ? TM : 1); ++i)
#pragma unroll
            for (int j = 0; j < (GATE_UP ? TN : 1); ++j) acc2[i][j] = 0.f;
    }
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gk = k0 + kk;
            float a = 0.f, w = 0.f, u = 0.f;
            if (gk < K) {
                if (a_row[r] >= 0) a = Elem<T>::load(A + (size_t)a_row[r] * lda + gk);
                if (n0 + r < N) {
                    w = Elem<T>::load(We + (size_t)(n0 + r) * K + gk);
                    if (GATE_UP) u = Elem<T>::load(We + (size_t)(N + n0 + r) * K + gk);
                }
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
            if (GATE_UP) Us[kk][r] = u;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
            if (GATE_UP) {
                float u[TN];
#pragma unroll
                for (int j = 0; j < TN; ++j) u[j] = Us[kk][tx * TN + j];
#pragma unroll
                for (int i = 0; i < (GATE_UP ? TM : 1); ++i)
#pragma unroll
                    for (int j = 0; j < (GATE_UP ? TN : 1); ++j) acc2[i][j] = fmaf(a[i], u[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            const size_t o = (size_t)o_row[r] * ldo + n;
            if (GATE_UP) {
                const float g = acc[i][j] * a_wgt[r], u = acc2[GATE_UP ? i : 0][GATE_UP ? j : 0] * a_wgt[r];
                Elem<T>::store((T*)out + o, g / (1.0f + expf(-g)) * u);
            } else if (FIRST) {
                const float u = fmaxf(acc[i][j] * a_wgt[r], 0.f);
                Elem<T>::store((T*)out + o, u * u);
            } else if (scatter) {
                ((float*)out)[o] += acc[i][j] * a_wgt[r];
            } else {
                ((float*)out)[o] = acc[i][j] * a_wgt[r];
            }
        }
    }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of, float* __restrict__ out, int tokens, int width, int top) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * width) return;
    const int t = (int)(i / width), c = (int)(i % width);
    float acc = out[i];
    for (int k = 0; k < top; ++k) acc += y[(size_t)row_of[(size_t)t * top + k] * width + c];
    out[i] = acc;
}

// mode: MOE_SOFTMAX | MOE_RENORM; corr: [experts] or null. With a mode or a correction z is overwritten by the scores.
// always > 0: sel_e and sel_w are [tokens, top + always], z holds one more logit behind the router's (ldz > experts).
NIB_API int nib_moe_route(float* z, int ldz, int* sel_e, float* sel_w, int tokens, int experts, int top, int mode, const float* corr,
                          int always, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && experts > 0 && experts + always <= MOE_MAX_EXPERTS && top > 0 && top <= experts && always >= 0 && (always == 0 || ldz > experts),
                "moe_route: %d experts (up to %d), %d chosen, %d always", experts, MOE_MAX_EXPERTS, top, always);
    if (tokens == 0) return 0;
    NIB_CUDA(launch_pdl(moe_route_kernel, dim3(ceil_div(tokens, 4)), dim3(128), (size_t)0, stream, z, ldz, sel_e, sel_w, tokens, experts, top, mode, corr, always));
    NIB_LAUNCH_CHECK();
    return 0;
}

// The largest number of tiles that `entries` rows in `experts` groups can make.
NIB_API int nib_moe_max_tiles(int entries, int experts, int tile_rows) {
    const long long by_rows = (entries + tile_rows - 1) / tile_rows + experts;
    return (int)(by_rows < entries ? by_rows : entries);
}

// experts: the router's outputs; the first n_real of them are experts and get row tiles.
NIB_API int nib_moe_group(const int* sel_e, int entries, int experts, int tile_rows, int* row_of, int* src_of, int* tiles, int* n_tiles,
                          int max_tiles, int n_real, cudaStream_t stream) {
    NIB_REQUIRE(entries >= 0 && experts > 0 && experts <= MOE_MAX_EXPERTS && tile_rows > 0 && max_tiles >= nib_moe_max_tiles(entries, experts, tile_rows)
                && n_real >= 0 && n_real <= experts, "moe_group: bad sizes");
    if (entries == 0) return 0;
    NIB_CUDA(launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)0, stream, sel_e, entries, experts, tile_rows, row_of, src_of, tiles, n_tiles, max_tiles, n_real));
    NIB_LAUNCH_CHECK();
    return 0;
}

// 1 if a step of these sizes takes the one-launch form.
NIB_API int nib_moe_step_supported(int tokens, int hidden, int experts, int top) {
    return tokens > 0 && experts > 0 && experts <= MOE_MAX_EXPERTS && top > 0 && top <= experts && (long long)tokens * experts <= MOE_STEP_MAX_Z
        && (long long)tokens * experts * hidden <= (1LL << 21) && (long long)tokens * top * hidden <= (1LL << 20);
}
// (with `extra` rows behind the router's, ask with experts + extra outputs)

// Router, choice, grouping and (rows != null) the gathered rows of a step of few tokens. h [tokens, hidden] and w_router
// [experts, hidden] in the storage type; the other arguments as for moe_route and moe_group.
NIB_API int nib_moe_step(const void* h, int ldh, const void* w_router, int tokens, int hidden, int experts, int top, int* sel_e, float* sel_w,
                         int tile_rows, int* row_of, int* src_of, int* tiles, int* n_tiles, int max_tiles, void* rows, int dtype, int mode,
                         const float* corr, int n_real, int extra, float* z_extra, int always, cudaStream_t stream) {
    // (with `always`: n_real counts the always-used experts too; the tables are made for top + always entries a token)
    NIB_REQUIRE(extra >= 0 && always >= 0 && nib_moe_step_supported(tokens, hidden, experts + extra, top) == 1 && top <= experts && ldh >= hidden
                && (long long)tokens * (top + always) * hidden <= (1LL << 20)
                && tile_rows > 0 && max_tiles >= nib_moe_max_tiles(tokens * (top + always), experts + always, tile_rows) && n_real >= 0
                && n_real <= experts + always && experts + always <= MOE_MAX_EXPERTS && (always == 0 || extra == 1),
                "moe_step: bad sizes");
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "moe_step: unknown dtype %d", dtype);
    const int per16 = dtype == NIB_F32 ? 4 : 8;
    const int vec = (hidden % per16 == 0 && ldh % per16 == 0 && (((uintptr_t)h | (uintptr_t)w_router | (uintptr_t)rows) & 15) == 0) ? 1 : 0;
    if (dtype == NIB_F32)
        NIB_CUDA(launch_pdl(moe_step_kernel<float>, dim3(1), dim3(1024), (size_t)0, stream, (const float*)h, ldh, (const float*)w_router, tokens, hidden,
                            experts, top, sel_e, sel_w, tile_rows, row_of, src_of, tiles, n_tiles, max_tiles, (float*)rows, vec, mode, corr, n_real, extra, z_extra, always));
    else
        NIB_CUDA(launch_pdl(moe_step_kernel<__nv_bfloat16>, dim3(1), dim3(1024), (size_t)0, stream, (const __nv_bfloat16*)h, ldh,
                            (const __nv_bfloat16*)w_router, tokens, hidden, experts, top, sel_e, sel_w, tile_rows, row_of, src_of, tiles, n_tiles,
                            max_tiles, (__nv_bfloat16*)rows, vec, mode, corr, n_real, extra, z_extra, always));
    NIB_LAUNCH_CHECK();
    return 0;
}

// gate_up 1: A = the tokens' activations [tokens, K] (rows gathered through src_of), W [experts, 2N, K] (gate rows, then
// up rows), out [entries, N] in the storage type; 2: the same with W [experts, N, K] (no gate) and relu(.)^2. 0: A = [entries, K] in the grouped order, W [experts, N, K], out floats:
// [entries, N] in the grouped order, or with scatter (one choice per token) added into the token's row of [tokens, N].
// The tiles must have been made for rows of 64.
NIB_API int nib_moe_gemm_simt(int gate_up, const void* A, int lda, const void* W, void* out, int ldo, const int* tiles, const int* n_tiles,
                              int max_tiles, const int* src_of, const float* sel_w, int top, int N, int K, int scatter, int dtype,
                              int w_out, cudaStream_t stream) {
    NIB_REQUIRE(N > 0 && K > 0 && top > 0 && max_tiles >= 0 && (!scatter || top == 1) && gate_up >= 0 && gate_up <= 2, "moe_gemm: bad sizes");
    NIB_REQUIRE(dtype == NIB_F32 || dtype == NIB_BF16, "moe_gemm: unknown dtype %d", dtype);
    if (max_tiles == 0) return 0;
    const dim3 grid(ceil_div(N, 64), max_tiles), block(256);
#define NIB_MG(T, GU) \
    NIB_CUDA(launch_pdl(moe_gemm_simt_kernel<T, GU>, grid, block, (size_t)0, stream, (const T*)A, lda, (const T*)W, out, ldo, tiles, n_tiles, src_of, sel_w, top, N, K, scatter, w_out))
    if (dtype == NIB_F32) { if (gate_up == 1) NIB_MG(float, 1); else if (gate_up == 2) NIB_MG(float, 2); else NIB_MG(float, 0); }
    else { if (gate_up == 1) NIB_MG(__nv_bfloat16, 1); else if (gate_up == 2) NIB_MG(__nv_bfloat16, 2); else NIB_MG(__nv_bfloat16, 0); }
#undef NIB_MG
    NIB_LAUNCH_CHECK();
    return 0;
}

NIB_API int nib_moe_combine(const float* y, const int* row_of, float* out, int tokens, int width, int top, cudaStream_t stream) {
    NIB_REQUIRE(tokens >= 0 && width > 0 && top > 0, "moe_combine: bad sizes");
    if (tokens == 0) return 0;
    NIB_CUDA(launch_pdl(moe_combine_kernel, dim3(ceil_div((long long)tokens * width, 256)), dim3(256), (size_t)0, stream, y, row_of, out, tokens, width, top));
    NIB_LAUNCH_CHECK();
    return 0;
}
