// Routed experts on the 5th-generation tensor cores of sm_100a: the two products of the experts' feed-forwards over the
// (token, choice) rows in the order moe_group leaves them (rows of one expert together), bfloat16 operands, 32-bit
// accumulation in tensor memory.
//
//   gate/up:  act[row] = silu(w g) * (w u),  g = W_gate,e x, u = W_up,e x, w = the row's score (it stands on the expert's
//             input; W (w x) = w (W x), so it is applied in 32-bit to the two accumulators),
//   down:     y[row] = W_down,e act[row] as floats, or added into the token's output row: plainly with one choice per
//             token, else by reductions in memory (the order of a token's choices, and with it the last bit of a sum of
//             three or more, is not fixed; two addends onto zeros give the same sum in either order).
//
// Experts without a gate (mode 2): act[row] = relu(w u)^2 from one accumulator. With `w_out` the score multiplies the
// down product's result (in 32-bit, in its epilogue) instead of the first product's accumulators.
//
// A work item is (row tile of the table that moe_group wrote, tile of 128 output features). The table's length depends on
// the routing and lives on the device: the grid is as large as the sizes allow (one CTA per SM at most) and every CTA reads
// the count when it starts, so the launch never depends on the batch's content. A row tile never spans two experts, and
// its expert picks the rows of the weight map ([experts * rows, K] as one matrix). The activation tile starts at the
// tile's first row and is TOK rows long whatever the tile holds: what it reads beyond the tile's rows (the next expert's
// rows, or zeros past the end) goes through the tensor core and is never stored.
//
// Orientation and pipeline are those of the dense product (gemm_tcgen05.cu): the weight rows are the instruction's M side
// (128 features = the 128 lanes of tensor memory), the rows its N side (TOK = 32 for a decode step's few rows per expert,
// 128 else); warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = epilogue, one output feature per thread; stages of 64
// elements of K with the 128-byte swizzle; two accumulator buffers. Every wait is bounded: one that runs out records a code
// in an error word, the CTA stops issuing, waits (bounded) for its copies in flight, frees its tensor memory and returns.
#include "tcgen05.cuh"
#include <mutex>
#include <unordered_map>

using namespace nibp;
using namespace nibt;

namespace {

constexpr int BLOCK_F = 128;     // output features per CTA (UMMA M)
constexpr int BLOCK_K = 64;      // elements of K per stage: 128 bytes, one swizzle atom
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

__device__ int g_moe_tc_error = 0;   // 0, or (role << 16 | blockIdx.x) of the first wait that ran out

template <int TOK, bool DUAL> struct Cfg {
    static constexpr int W_BYTES = BLOCK_F * BLOCK_K * 2;                 // 16 KB
    static constexpr int A_BYTES = TOK * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * W_BYTES + A_BYTES;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
    static constexpr int ACC_COLS = (DUAL ? 2 : 1) * TOK;                 // columns of one accumulator buffer
    static constexpr int TMEM_COLS = tmem_cols(2 * ACC_COLS);             // two buffers
    static_assert(2 * ACC_COLS <= 512, "two accumulator buffers must fit the 512 TMEM columns");
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

template <int TOK, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
moe_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, void* __restrict__ out, int ldo,
              const int* __restrict__ tiles, const int* __restrict__ n_tiles, int max_tiles, const int* __restrict__ src_of,
              const float* __restrict__ sel_w, int top, int n_out, int k_dim, int w_rows, int scatter, int splits, int kb_per_split, int w_out) {
    constexpr bool GATE_UP = MODE == 1, FIRST = MODE != 0;     // FIRST: the product that reads the tokens' rows and writes activations
    constexpr bool DUAL = GATE_UP;
    const bool use_w = FIRST != (w_out != 0);                  // whether this product is the one the score multiplies
    // Row tiles of 128: the operands change places, so the ROWS are the instruction's M side (the TMEM lanes) and the 128
    // features its columns; a thread of the epilogue then owns a row and writes 16 consecutive features at a time.
    constexpr bool SWAP = (TOK == BLOCK_F);
    using C = Cfg<TOK, DUAL>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + C::STAGES * C::STAGE_BYTES);
    unsigned long long* empty_bar = full_bar + C::STAGES;
    unsigned long long* acc_full_bar = empty_bar + C::STAGES;     // [2]
    unsigned long long* acc_empty_bar = acc_full_bar + 2;         // [2]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty_bar + 2);
    __shared__ volatile int s_failed;
    __shared__ float s_wgt[4][TOK];      // per epilogue warp: the scores of the tile's rows
    __shared__ int s_row[4][TOK];        // ... and the row each writes (-1: none)

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f_tiles = (n_out + BLOCK_F - 1) / BLOCK_F;
    const int k_blocks = (k_dim + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0) {
        s_failed = 0;
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full_bar[b], 1); mbar_init(&acc_empty_bar[b], 4); }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();         // from here on the kernel reads what earlier kernels wrote (the table, the rows)
    int nt = __ldcg(n_tiles);
    if (nt > max_tiles) nt = max_tiles;
    // work item = (row tile, feature tile, split of K), splits fastest, then feature tiles. With K split (the down product
    // of a short step, whose tiles alone leave SMs idle) every item adds its partial sums into the output by reductions.
    const int items = nt * f_tiles * splits;
    const bool reduce = scatter == 2 || splits > 1;

    if (warp == 0 && lane == 0) {
        // ---------------- producer: TMA loads of the expert's weight rows and of the tile's rows, stage after stage
        int it = 0, issued = 0;
        for (int item = blockIdx.x; item < items && !s_failed; item += gridDim.x) {
            const int split = item % splits, rest = item / splits;
            const int tile = rest / f_tiles, f0 = (rest - tile * f_tiles) * BLOCK_F;
            const int expert = __ldg(tiles + 3 * tile), row0 = __ldg(tiles + 3 * tile + 1);
            const int wrow = expert * w_rows + f0;
            const int kb_end = min(k_blocks, (split + 1) * kb_per_split);
            for (int kb = split * kb_per_split; kb < kb_end; ++kb, ++it) {
                const int s = it % C::STAGES;
                if (!mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1)) {
                    atomicCAS(&g_moe_tc_error, 0, (1 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                    break;
                }
                unsigned char* st = smem + s * C::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
                tma_load_2d(st, &map_w, &full_bar[s], kb * BLOCK_K, wrow);
                if (DUAL) tma_load_2d(st + C::W_BYTES, &map_w, &full_bar[s], kb * BLOCK_K, wrow + n_out);
                tma_load_2d(st + (DUAL ? 2 : 1) * C::W_BYTES, &map_a, &full_bar[s], kb * BLOCK_K, row0);
                issued = it + 1;
            }
        }
        if (s_failed) {
            // copies already issued still target this CTA's shared memory: wait for them, bounded
            for (int i = max(0, issued - C::STAGES); i < issued; ++i)
                mbar_wait(&full_bar[i % C::STAGES], (i / C::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr unsigned idesc = SWAP ? instr_desc(TOK, BLOCK_F) : instr_desc(BLOCK_F, TOK);
        int it = 0, local = 0;
        for (int item = blockIdx.x; item < items && !s_failed; item += gridDim.x, ++local) {
            const int buf = local & 1;
            // the epilogue has drained this buffer (two tiles ago)
            if (!mbar_wait(&acc_empty_bar[buf], ((local >> 1) & 1) ^ 1)) {
                atomicCAS(&g_moe_tc_error, 0, (4 << 16) | (int)blockIdx.x);
                s_failed = 1;
                break;
            }
            tc_fence_after();
            const unsigned acc = tmem_base + buf * C::ACC_COLS;
            const int kb_begin = (item % splits) * kb_per_split, kb_end = min(k_blocks, kb_begin + kb_per_split);
            for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                const int s = it % C::STAGES;
                if (!mbar_wait(&full_bar[s], (it / C::STAGES) & 1)) {
                    atomicCAS(&g_moe_tc_error, 0, (2 << 16) | (int)blockIdx.x);
                    s_failed = 1;
                    break;
                }
                tc_fence_after();
                const unsigned st = smem_u32(smem + s * C::STAGE_BYTES);
                const unsigned long long w_desc = desc_kmajor(st);
                const unsigned long long u_desc = desc_kmajor(st + C::W_BYTES);
                const unsigned long long a_desc = desc_kmajor(st + (DUAL ? 2 : 1) * C::W_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const unsigned long long adv = (unsigned long long)((k * UMMA_K * 2) >> 4);   // 32 bytes per step
                    const bool accumulate = (kb > kb_begin) || (k > 0);
                    if (SWAP) {
                        tc_mma(acc, a_desc + adv, w_desc + adv, idesc, accumulate);
                        if (DUAL) tc_mma(acc + BLOCK_F, a_desc + adv, u_desc + adv, idesc, accumulate);
                    } else {
                        tc_mma(acc, w_desc + adv, a_desc + adv, idesc, accumulate);
                        if (DUAL) tc_mma(acc + TOK, u_desc + adv, a_desc + adv, idesc, accumulate);
                    }
                }
                tc_commit(&empty_bar[s]);        // the stage is free when these MMAs have read it
            }
            if (s_failed) break;
            tc_commit(&acc_full_bar[buf]);       // the accumulator is complete when all MMAs are done
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: TMEM -> registers -> global, one output feature per thread
        const int quad = warp & 3;                       // the TMEM lanes this warp may read: 32*quad..
        int local = 0;
        for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
            const int buf = local & 1;
            const int rest = item / splits;
            const int tile = rest / f_tiles, f0 = (rest - tile * f_tiles) * BLOCK_F;
            const int row0 = __ldg(tiles + 3 * tile + 1), rows = min(TOK, __ldg(tiles + 3 * tile + 2));
            const int f = f0 + quad * 32 + lane;
            if constexpr (SWAP) {
                // ---- this thread owns row row0 + t of the tile; its lane holds the tile's 128 features
                const int t = quad * 32 + lane;
                const bool live = t < rows;
                float wg = 0.f;
                size_t orow = 0;
                if (live) {
                    const int entry = __ldg(src_of + row0 + t);
                    wg = use_w ? __ldg(sel_w + entry) : 1.0f;
                    orow = (size_t)((!FIRST && scatter) ? entry / top : row0 + t) * ldo;
                }
                bool ok = !s_failed && mbar_wait(&acc_full_bar[buf], (local >> 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0 && !s_failed) { atomicCAS(&g_moe_tc_error, 0, (3 << 16) | (int)blockIdx.x); s_failed = 1; }
                    break;
                }
                tc_fence_after();
                const unsigned lane_addr = tmem_base + buf * C::ACC_COLS + ((unsigned)(quad * 32) << 16);
#pragma unroll 1
                for (int c = 0; c < BLOCK_F; c += 16) {
                    if (f0 + c >= n_out) break;
                    unsigned rv[16], ru[16];
                    tmem_ld16_async(lane_addr + c, rv);
                    if (DUAL) tmem_ld16_async(lane_addr + BLOCK_F + c, ru);
                    tmem_wait_ld();
                    if (!live) continue;
                    float x[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (GATE_UP) {
                            const float g = __uint_as_float(rv[j]) * wg, up = __uint_as_float(ru[j]) * wg;
                            x[j] = __fdividef(g, 1.0f + __expf(-g)) * up;      // the dense gated product's epilogue has the same forms
                        } else if (FIRST) {
                            const float u = fmaxf(__uint_as_float(rv[j]) * wg, 0.f);
                            x[j] = u * u;
                        } else {
                            x[j] = __uint_as_float(rv[j]) * wg;
                        }
                    }
                    const int f = f0 + c;
                    const bool whole = f + 16 <= n_out;       // 16 features: 32 bytes of bfloat16 or 64 of floats, aligned
                    if (FIRST) {
                        __nv_bfloat16* o = (__nv_bfloat16*)out + orow + f;
                        if (whole) {
                            uint4 p0, p1;
                            p0.x = pack_bf16(x[0], x[1]); p0.y = pack_bf16(x[2], x[3]); p0.z = pack_bf16(x[4], x[5]); p0.w = pack_bf16(x[6], x[7]);
                            p1.x = pack_bf16(x[8], x[9]); p1.y = pack_bf16(x[10], x[11]); p1.z = pack_bf16(x[12], x[13]); p1.w = pack_bf16(x[14], x[15]);
                            reinterpret_cast<uint4*>(o)[0] = p0;
                            reinterpret_cast<uint4*>(o)[1] = p1;
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (f + j < n_out) o[j] = __float2bfloat16(x[j]);
                        }
                    } else {
                        float* o = (float*)out + orow + f;
                        if (whole && reduce) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4) red_add_v4(o + j, x[j], x[j + 1], x[j + 2], x[j + 3]);
                        } else if (whole) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                float4 cur = scatter ? *reinterpret_cast<float4*>(o + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                                cur.x += x[j]; cur.y += x[j + 1]; cur.z += x[j + 2]; cur.w += x[j + 3];
                                *reinterpret_cast<float4*>(o + j) = cur;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                if (f + j >= n_out) break;
                                if (reduce) atomicAdd(o + j, x[j]);
                                else if (scatter) o[j] += x[j];
                                else o[j] = x[j];
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
                continue;
            }
            // what the epilogue reads besides the accumulator is fetched while the tensor core still works on the tile
            __syncwarp();
            for (int c = lane; c < TOK; c += 32) {
                float wg = 0.f;
                int orow = -1;
                if (c < rows) {
                    const int entry = __ldg(src_of + row0 + c);
                    wg = use_w ? __ldg(sel_w + entry) : 1.0f;
                    orow = (!FIRST && scatter) ? entry / top : row0 + c;
                }
                s_wgt[quad][c] = wg;
                s_row[quad][c] = orow;
            }
            __syncwarp();
            bool ok = !s_failed && mbar_wait(&acc_full_bar[buf], (local >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !s_failed) { atomicCAS(&g_moe_tc_error, 0, (3 << 16) | (int)blockIdx.x); s_failed = 1; }
                break;
            }
            tc_fence_after();
            const unsigned lane_addr = tmem_base + buf * C::ACC_COLS + ((unsigned)(quad * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < rows; c += 16) {
                float v[16], u[16];
                tmem_ld16(lane_addr + c, v);
                if (DUAL) tmem_ld16(lane_addr + TOK + c, u);
                if (f < n_out) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c + j >= rows) break;
                        const size_t o = (size_t)s_row[quad][c + j] * ldo + f;
                        const float wg = s_wgt[quad][c + j];
                        if (GATE_UP) {
                            const float g = v[j] * wg, up = u[j] * wg;
                            ((__nv_bfloat16*)out)[o] = __float2bfloat16(__fdividef(g, 1.0f + __expf(-g)) * up);
                        } else if (FIRST) {
                            const float r = fmaxf(v[j] * wg, 0.f);
                            ((__nv_bfloat16*)out)[o] = __float2bfloat16(r * r);
                        } else if (reduce) {
                            atomicAdd((float*)out + o, v[j] * wg);   // a token's choices, or the splits of K, meet in its row in no fixed order
                        } else if (scatter) {
                            ((float*)out)[o] += v[j] * wg;       // one choice per token: nobody else writes this row
                        } else {
                            ((float*)out)[o] = v[j] * wg;
                        }
                    }
                }
            }
            // this warp has read its part of the buffer: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// dst[row] = src[src_of[row] / top]: the tokens' rows in the grouped order, 16 bytes per thread and step.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, int lds, __nv_bfloat16* __restrict__ dst, int ldd, const int* __restrict__ src_of,
                       int rows, int width, int top) {
    pdl_launch_dependents();
    pdl_wait();      // everything this kernel reads may come from the kernel before
    const int per_row = width / 8;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * per_row) return;
    const int r = (int)(i / per_row), c = (int)(i % per_row) * 8;
    const int t = __ldg(src_of + r) / top;
    *reinterpret_cast<uint4*>(dst + (size_t)r * ldd + c) = __ldg(reinterpret_cast<const uint4*>(src + (size_t)t * lds + c));
}

// Map of a row-major bfloat16 matrix [rows, k] with row stride ld elements; box = 64 x box_rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld, int box_rows) {
    NibEncodeTiledFn enc = nib_tensor_map_encoder();
    NIB_REQUIRE(enc != nullptr, "experts (tensor cores): cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NIB_REQUIRE(r == CUDA_SUCCESS, "experts (tensor cores): cuTensorMapEncodeTiled failed with code %d (rows=%lld k=%lld ld=%lld)", (int)r, rows, k, ld);
    return 0;
}

struct MapKey {
    const void* p; long long rows, k;
    bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && k == o.k; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& x) const {
        return std::hash<const void*>()(x.p) ^ (std::hash<long long>()(x.rows) * 31) ^ (std::hash<long long>()(x.k) * 131);
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_expert_maps;   // weights live as long as the model
std::mutex g_expert_map_mutex;

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            sms = 1;
    }
    return sms;
}

template <int TOK, int MODE>
int launch_moe_tc(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int ldo, const int* tiles, const int* n_tiles, int max_tiles,
                  const int* src_of, const float* sel_w, int top, int N, int K, int w_rows, int scatter, int splits, int w_out,
                  cudaStream_t stream) {
    constexpr bool FIRST = MODE != 0;       // the first product, gated or not: its output cannot be split along K
    using C = Cfg<TOK, MODE == 1>;
    static bool configured = false;
    if (!configured) {
        NIB_CUDA(cudaFuncSetAttribute(moe_tc_kernel<TOK, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        configured = true;
    }
    const int k_blocks = ceil_div(K, BLOCK_K);
    if (splits < 1 || FIRST || scatter == 0) splits = 1;      // only sums into the output can be split along K
    if (splits > k_blocks) splits = k_blocks;
    const int kb_per_split = ceil_div(k_blocks, splits);
    splits = ceil_div(k_blocks, kb_per_split);               // no split without work
    const long long most = (long long)max_tiles * ceil_div(N, BLOCK_F) * splits;
    const int sms = sm_count();
    NIB_CUDA(launch_pdl(moe_tc_kernel<TOK, MODE>, dim3((unsigned)(most < sms ? most : sms)), dim3(THREADS), (size_t)C::SMEM, stream, mw, ma, out, ldo,
                        tiles, n_tiles, max_tiles, src_of, sel_w, top, N, K, w_rows, scatter, splits, kb_per_split, w_out));
    return 0;
}

}  // namespace

// 1 if the tensor-core kernels take these operands: widths in multiples of 8 (16-byte rows), 16-byte aligned bases, and a
// weight matrix whose row count fits a tensor map's 32-bit coordinates.
NIB_API int nib_moe_tc_supported(const void* h, int ldh, const void* w_gate_up, const void* w_down, int experts, int hidden, int ff) {
    if (hidden <= 0 || ff <= 0 || hidden % 8 || ff % 8 || ldh % 8) return 0;
    if (((uintptr_t)h & 15) || ((uintptr_t)w_gate_up & 15) || ((uintptr_t)w_down & 15)) return 0;
    if ((long long)experts * 2 * ff >= (1LL << 31) || (long long)experts * hidden >= (1LL << 31)) return 0;
    return nib_tensor_map_encoder() != nullptr;
}

// The error word of the kernels' bounded waits: 0, or (role << 16 | block) of the first wait that ran out (role 1
// producer, 2 MMA issuer, 3 epilogue, 4 MMA issuer waiting for the epilogue). Reading it synchronises with the device; it
// is cleared.
NIB_API int nib_moe_tc_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_moe_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_moe_tc_error, &zero, sizeof(int));
    return v;
}

// dst [rows, width] = the rows of src [tokens, width] in the grouped order (row r reads token src_of[r] / top).
NIB_API int nib_moe_gather_rows(const void* src, int lds, void* dst, int ldd, const int* src_of, int rows, int width, int top, cudaStream_t stream) {
    NIB_REQUIRE(rows >= 0 && width > 0 && width % 8 == 0 && lds % 8 == 0 && ldd % 8 == 0 && top > 0, "moe_gather_rows: bad sizes");
    NIB_REQUIRE((((uintptr_t)src | (uintptr_t)dst) & 15) == 0, "moe_gather_rows: bases must be 16-byte aligned");
    if (rows == 0) return 0;
    NIB_CUDA(launch_pdl(moe_gather_rows_kernel, dim3(ceil_div((long long)rows * (width / 8), 256)), dim3(256), (size_t)0, stream,
                        (const __nv_bfloat16*)src, lds, (__nv_bfloat16*)dst, ldd, src_of, rows, width, top));
    NIB_LAUNCH_CHECK();
    return 0;
}

// gate_up 1: A = the rows in the grouped order [a_rows, K], W [experts, 2N, K] (gate rows, then up rows), out bfloat16
// [a_rows, N]; 2: the same with W [experts, N, K] (no gate) and relu(.)^2. 0: A [a_rows, K] in the grouped order, W [experts, N, K], out floats: [a_rows, N] in the grouped order, or
// with scatter added into the token's row of [tokens, N] (1: plainly, one choice per token; 2: by reductions in memory).
// The table must have been made for row tiles of `tile_rows` (32 or 128).
NIB_API int nib_moe_gemm_tc(int gate_up, const void* A, int lda, int a_rows, const void* W, int experts, void* out, int ldo, const int* tiles,
                            const int* n_tiles, int max_tiles, const int* src_of, const float* sel_w, int top, int N, int K, int scatter,
                            int tile_rows, int w_out, cudaStream_t stream) {
    NIB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && top > 0 && a_rows >= 0 && experts > 0 && max_tiles >= 0 && scatter >= 0 && scatter <= 2
                && (scatter != 1 || top == 1) && gate_up >= 0 && gate_up <= 2, "experts (tensor cores): bad sizes");
    NIB_REQUIRE(tile_rows == 32 || tile_rows == 128, "experts (tensor cores): row tiles of 32 or 128, not %d", tile_rows);
    if (max_tiles == 0 || a_rows == 0) return 0;
    const int w_rows = gate_up == 1 ? 2 * N : N;
    CUtensorMap mw, ma;
    {
        std::lock_guard<std::mutex> lock(g_expert_map_mutex);
        MapKey key{W, (long long)experts * w_rows, K};
        auto it = g_expert_maps.find(key);
        if (it == g_expert_maps.end()) {
            if (make_map(&mw, W, (long long)experts * w_rows, K, K, BLOCK_F)) return 1;
            if (g_expert_maps.size() > 4096) g_expert_maps.clear();
            g_expert_maps.emplace(key, mw);
        } else {
            mw = it->second;
        }
    }
    if (make_map(&ma, A, a_rows, K, lda, tile_rows)) return 1;
    // A short step's down product: its tiles (about one per expert in use, times the feature tiles) leave SMs idle and each is a
    // long walk over K; K is split so that about as many items as SMs stream the weights, none shorter than four stages.
    int splits = 1;
    if (!gate_up && scatter && tile_rows == 32) {
        const long long tiles_est = (long long)(a_rows < experts ? a_rows : experts) * ceil_div(N, BLOCK_F);
        const int sms = sm_count(), k_blocks = ceil_div(K, BLOCK_K);
        if (tiles_est * 2 <= sms) splits = (int)(sms / tiles_est);
        if (splits > k_blocks / 4) splits = k_blocks / 4;
        if (splits < 1) splits = 1;
    }
#define NIB_MT(TOK, GU) launch_moe_tc<TOK, GU>(mw, ma, out, ldo, tiles, n_tiles, max_tiles, src_of, sel_w, top, N, K, w_rows, scatter, splits, w_out, stream)
    int rc;
    if (tile_rows == 32) rc = gate_up == 1 ? NIB_MT(32, 1) : (gate_up == 2 ? NIB_MT(32, 2) : NIB_MT(32, 0));
    else rc = gate_up == 1 ? NIB_MT(128, 1) : (gate_up == 2 ? NIB_MT(128, 2) : NIB_MT(128, 0));
#undef NIB_MT
    if (rc) return rc;
    NIB_LAUNCH_CHECK();
    return 0;
}
