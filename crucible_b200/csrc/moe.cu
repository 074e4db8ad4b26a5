// Mixture of experts: every token goes through `top` of `E` small gated feed-forwards,
//   y[t] = sum_j weight[t][j] * Wd[e_j] (silu(Wg[e_j] h[t]) * (Wu[e_j] h[t])),
// e_j the experts with the largest router logits of the token (the lower index on equal
// logits) and weight the softmax over those `top` logits alone.
//
// Everything is decided on the device, so a step's launches depend on its shape only:
//   route    one warp per token: the top logits, their softmax, and each (token, choice)
//            pair's place among its expert's pairs (a counter per expert)
//   plan     one block: where each expert's pairs start in the sorted order, the list of
//            row tiles (an expert, a start, a count), and the sorted order itself
//   tiles    gate/up with the gated pair (SiLU, or the capped form), then down times the pair's weight: a block owns a tile of
//            rows of one expert and a tile of columns; rows beyond the tile's count and
//            tiles beyond the plan's count do nothing.  fp32 sums over ascending k, so a
//            pair's result does not depend on which other pairs share its tile.
//   combine  residual[t] += the token's pairs in the order of its choices.
#define CB_PDL_BIT 13      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int TM = 32, TN = 64, TK = 32, THREADS = 128;
constexpr int MAX_PER_LANE = 8;       // experts <= 256, of which a token takes at most 32

// The gated pair of an expert.  limit <= 0: silu(g) * u.  Else the capped pair:
// g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(alpha * g') * (u' + offset).
struct GateRule { float limit, alpha, offset; };
__device__ __forceinline__ float gated_f(float g, float u, const GateRule& p) {
    if (p.limit <= 0.f) return g / (1.0f + expf(-g)) * u;
    g = fminf(g, p.limit);
    u = fminf(fmaxf(u, -p.limit), p.limit);
    return g / (1.0f + expf(-p.alpha * g)) * (u + p.offset);
}

__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 int n_tokens, int E, int top,
                                 int* __restrict__ idx, float* __restrict__ weight,
                                 int* __restrict__ place, int* __restrict__ count) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const int lane = threadIdx.x & 31;
    float v[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? logits[(size_t)t * E + e] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
    }
    float first = 0.f, total = 0.f, mine = 0.f;
    int mine_e = 0;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = j < E ? j : 0;      // nothing comparable left (NaN logits)
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i)
            if (lane + 32 * i == best_e) v[i] = -INFINITY;
        if (j == 0) first = best;
        const float p = expf(best - first);
        total += p;
        if (lane == j) { mine = p; mine_e = best_e; }
    }
    if (lane < top) {
        idx[(size_t)t * top + lane] = mine_e;
        weight[(size_t)t * top + lane] = mine / total;
        place[(size_t)t * top + lane] = atomicAdd(&count[mine_e], 1);
    }
}

// (tile_rows_: rows of a tile: TM for the kernels of this file, 128 for the tensor cores' grouped product)
// plan: [0] number of tiles, [1 .. E+1] each expert's start in the sorted order, then
// max_tiles each of (expert, start, rows).
__global__ void moe_plan_kernel(int* __restrict__ count, int E, int n_pairs, const int* __restrict__ idx,
                                const int* __restrict__ place, int* __restrict__ plan, int max_tiles,
                                int* __restrict__ sorted_pair, int tile_rows_) {
    cb_pdl_trigger();
    cb_pdl_wait();
    int* offsets = plan + 1;
    int* tile_expert = plan + 2 + E;
    int* tile_start = tile_expert + max_tiles;
    int* tile_rows = tile_start + max_tiles;
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            const int n = count[e];
            for (int r = 0; r < n && tiles < max_tiles; r += tile_rows_, ++tiles) {
                tile_expert[tiles] = e;
                tile_start[tiles] = at + r;
                tile_rows[tiles] = min(tile_rows_, n - r);
            }
            at += n;
        }
        offsets[E] = at;
        plan[0] = tiles;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) sorted_pair[offsets[idx[p]] + place[p]] = p;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;      // ready for the next step
}

// GATED: rows are h[token of the pair], W = [gate rows; up rows] of the tile's expert,
//        out[sorted place][n] = silu(gate) * up in T.
// else:  rows are act[sorted place], W = down of the expert, out[pair][n] = weight[pair] * sum, fp32.
template <typename T, bool GATED>
__global__ void __launch_bounds__(THREADS) moe_tile_kernel(
    const T* __restrict__ a, int a_stride, const T* __restrict__ w, long expert_stride, int N, int K,
    const int* __restrict__ plan, int E, int max_tiles, const int* __restrict__ sorted_pair, int top,
    const float* __restrict__ weight, void* __restrict__ out_, int out_stride, GateRule rule) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int* tile_expert = plan + 2 + E;
    const int e = tile_expert[tile], start = tile_expert[max_tiles + tile], rows = tile_expert[2 * max_tiles + tile];
    const int n0 = blockIdx.y * TN;
    __shared__ float sa[TM][TK + 1];
    __shared__ float sw[GATED ? 2 : 1][TN][TK + 1];
    __shared__ int src_row[TM];
    if (threadIdx.x < TM) {
        const int s = start + min((int)threadIdx.x, rows - 1);
        src_row[threadIdx.x] = GATED ? sorted_pair[s] / top : s;
    }
    __syncthreads();
    const T* we = w + (size_t)e * expert_stride;
    const int tr = (threadIdx.x >> 4) * 4, tc = (threadIdx.x & 15) * 4;
    float acc[GATED ? 2 : 1][4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += THREADS) {
            const int r = i / TK, k = i - r * TK;
            sa[r][k] = k0 + k < K ? cb_to_float(a[(size_t)src_row[r] * a_stride + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < TN * TK; i += THREADS) {
            const int c = i / TK, k = i - c * TK;
            const bool in = n0 + c < N && k0 + k < K;
            sw[0][c][k] = in ? cb_to_float(we[(size_t)(n0 + c) * K + k0 + k]) : 0.f;
            if (GATED) sw[1][c][k] = in ? cb_to_float(we[(size_t)(N + n0 + c) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < TK; ++k) {
            float av[4], wv[GATED ? 2 : 1][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = sa[tr + i][k];
                wv[0][i] = sw[0][tc + i][k];
                if (GATED) wv[1][i] = sw[1][tc + i][k];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[0][i][j] = fmaf(av[i], wv[0][j], acc[0][i][j]);
                    if (GATED) acc[1][i][j] = fmaf(av[i], wv[1][j], acc[1][i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (tr + i >= rows) continue;
        const int s = start + tr + i;
        if (GATED) {
            T* dst = reinterpret_cast<T*>(out_) + (size_t)s * out_stride;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n0 + tc + j < N) dst[n0 + tc + j] = cb_from_float<T>(gated_f(acc[0][i][j], acc[GATED ? 1 : 0][i][j], rule));
        } else {
            const int p = sorted_pair[s];
            const float wt = weight[p];
            float* dst = reinterpret_cast<float*>(out_) + (size_t)p * out_stride;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n0 + tc + j < N) dst[n0 + tc + j] = wt * acc[0][i][j];
        }
    }
}

// The same two products for steps of few rows (decoded tokens): the experts' weights are what
// moves, so each weight row is read once, by one warp whose lanes share K in 16-byte pieces, and
// meets every row of its tile (ROWS at a time).  A block owns a tile and a run of output features.
template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
    typedef uint4 Raw;
    static __device__ __forceinline__ Raw fetch(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void put(__nv_bfloat16* p, const Raw& raw) { *reinterpret_cast<uint4*>(p) = raw; }
    static __device__ __forceinline__ void unpack(const Raw& raw, float* v) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
};
template <> struct Vec8<float> {
    struct Raw { float4 a, b; };
    static __device__ __forceinline__ Raw fetch(const float* p) {
        Raw r;
        r.a = *reinterpret_cast<const float4*>(p);
        r.b = *reinterpret_cast<const float4*>(p + 4);
        return r;
    }
    static __device__ __forceinline__ void put(float* p, const Raw& r) {
        *reinterpret_cast<float4*>(p) = r.a;
        *reinterpret_cast<float4*>(p + 4) = r.b;
    }
    static __device__ __forceinline__ void unpack(const Raw& r, float* v) {
        v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
    }
};

extern __shared__ __align__(16) unsigned char moe_rows_staged[];

template <typename T, bool GATED, int ROWS>
__global__ void __launch_bounds__(256, 3) moe_rows_small_kernel(
    const T* __restrict__ a, int a_stride, const T* __restrict__ w, long expert_stride, int N, int K,
    const int* __restrict__ plan, int E, int max_tiles, const int* __restrict__ sorted_pair, int top,
    const float* __restrict__ weight, void* __restrict__ out_, int out_stride, int per_block, GateRule rule) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int tile = blockIdx.x;
    if (tile >= plan[0]) return;
    const int* tile_expert = plan + 2 + E;
    const int e = tile_expert[tile], start = tile_expert[max_tiles + tile], rows = tile_expert[2 * max_tiles + tile];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const T* we = w + (size_t)e * expert_stride;
    const int n_end = min(N, (int)(blockIdx.y + 1) * per_block);
    T* staged = reinterpret_cast<T*>(moe_rows_staged);       // ROWS rows of K: this pass's rows
    for (int r0 = 0; r0 < rows; r0 += ROWS) {
        __syncthreads();
        for (int i = threadIdx.x * 8; i < ROWS * K; i += blockDim.x * 8) {
            const int r = i / K, k = i - r * K;
            const int s = start + min(r0 + r, rows - 1);
            Vec8<T>::put(staged + i, Vec8<T>::fetch(a + (size_t)(GATED ? sorted_pair[s] / top : s) * a_stride + k));
        }
        __syncthreads();
        for (int n = blockIdx.y * per_block + warp; n < n_end; n += n_warps) {
            const T* w0 = we + (size_t)n * K;
            const T* w1 = we + (size_t)(N + n) * K;          // the up row (GATED)
            float acc0[ROWS], acc1[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) acc0[r] = acc1[r] = 0.f;
            // four pieces of a weight row are asked for before the first is used: a warp then has
            // 2 to 4 KB on its way, a block of eight warps what an SM needs to stream
            constexpr int AHEAD = 4;
            for (int k = lane * 8; k < K; k += 256 * AHEAD) {
                typename Vec8<T>::Raw raw0[AHEAD], raw1[AHEAD];
#pragma unroll
                for (int u = 0; u < AHEAD; ++u) {
                    const int kk = k + u * 256;
                    if (kk < K) {
                        raw0[u] = Vec8<T>::fetch(w0 + kk);
                        if (GATED) raw1[u] = Vec8<T>::fetch(w1 + kk);
                    }
                }
#pragma unroll
                for (int u = 0; u < AHEAD; ++u) {
                    const int kk = k + u * 256;
                    if (kk >= K) break;
                    float wv0[8], wv1[8], av[8];
                    Vec8<T>::unpack(raw0[u], wv0);
                    if (GATED) Vec8<T>::unpack(raw1[u], wv1);
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        if (r0 + r >= rows) break;
                        Vec8<T>::unpack(Vec8<T>::fetch(staged + r * K + kk), av);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            acc0[r] = fmaf(av[i], wv0[i], acc0[r]);
                            if (GATED) acc1[r] = fmaf(av[i], wv1[i], acc1[r]);
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r0 + r >= rows) break;
                const float g = cb_warp_sum(acc0[r]);
                const float u = GATED ? cb_warp_sum(acc1[r]) : 0.f;
                if (lane == 0) {
                    const int s = start + r0 + r;
                    if (GATED) {
                        reinterpret_cast<T*>(out_)[(size_t)s * out_stride + n] = cb_from_float<T>(gated_f(g, u, rule));
                    } else {
                        const int p = sorted_pair[s];
                        reinterpret_cast<float*>(out_)[(size_t)p * out_stride + n] = weight[p] * g;
                    }
                }
            }
        }
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ pair_out, int top, float* __restrict__ residual,
                                   int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float sum = 0.f;
        for (int j = 0; j < top; ++j) sum += pair_out[((size_t)t * top + j) * width + i];
        residual[(size_t)t * width + i] += sum;
    }
}

// rows of `h` gathered into the sorted order (for products that want an expert's rows side by side)
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, int h_stride, const int* __restrict__ sorted_pair,
                                  int top, T* __restrict__ out, int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const T* src = h + (size_t)(sorted_pair[blockIdx.x] / top) * h_stride;
    T* dst = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

// pair_out[pair] = weight[pair] * rows[sorted place of the pair]
__global__ void moe_scatter_kernel(const float* __restrict__ rows, const int* __restrict__ sorted_pair,
                                   const float* __restrict__ weight, float* __restrict__ pair_out, int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int p = sorted_pair[blockIdx.x];
    const float wt = weight[p];
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        pair_out[(size_t)p * width + i] = wt * rows[(size_t)blockIdx.x * width + i];
}

}  // namespace

CB_EXPORT int cb_moe_tile_rows() { return TM; }

CB_EXPORT int cb_moe_route(const float* logits, const float* bias, int n_tokens, int E, int top, int* idx,
                           float* weight,
                           int* place, int* count, int* plan, int max_tiles, int* sorted_pair,
                           int tile_rows, void* stream) {
    if (n_tokens <= 0) return 0;
    if (E > 32 * MAX_PER_LANE || top > E || top <= 0 || top > 32) return CB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    cb_launch(moe_route_kernel, dim3((n_tokens + 3) / 4), dim3(128), 0, s, logits, bias, n_tokens, E, top, idx,
              weight, place, count);
    cb_launch(moe_plan_kernel, dim3(1), dim3(256), 0, s, count, E, n_tokens * top, (const int*)idx,
              (const int*)place, plan, max_tiles, sorted_pair, tile_rows > 0 ? tile_rows : TM);
    return cb_last_error();
}

// gated != 0: act[sorted place][N] from h rows; else pair_out[pair][N] from act rows.
CB_EXPORT int cb_moe_tiles(int gated, const void* a, int a_stride, const void* w, long expert_stride,
                           int dtype, int N, int K, const int* plan, int E, int max_tiles,
                           const int* sorted_pair, int top, const float* weight, void* out,
                           int out_stride, float limit, float alpha, float offset, void* stream) {
    if (max_tiles <= 0) return 0;
    const GateRule rule = {limit, alpha, offset};
    const dim3 grid(max_tiles, (N + TN - 1) / TN), block(THREADS);
    cudaStream_t s = (cudaStream_t)stream;
#define CB_MOE(TT, GG)                                                                             \
    cb_launch(moe_tile_kernel<TT, GG>, grid, block, 0, s, (const TT*)a, a_stride, (const TT*)w,    \
              expert_stride, N, K, plan, E, max_tiles, sorted_pair, top, weight, out, out_stride, rule)
    if (dtype == CB_F32) { if (gated) CB_MOE(float, true); else CB_MOE(float, false); }
    else { if (gated) CB_MOE(__nv_bfloat16, true); else CB_MOE(__nv_bfloat16, false); }
#undef CB_MOE
    return cb_last_error();
}

// The same as cb_moe_tiles for steps of few rows; K a multiple of 8 and 16-byte aligned rows.
CB_EXPORT int cb_moe_rows_small(int gated, const void* a, int a_stride, const void* w, long expert_stride,
                                int dtype, int N, int K, const int* plan, int E, int max_tiles,
                                const int* sorted_pair, int top, const float* weight, void* out,
                                int out_stride, float limit, float alpha, float offset, void* stream) {
    if (max_tiles <= 0) return 0;
    const GateRule rule = {limit, alpha, offset};
    if (K % 8 || a_stride % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return CB_ERR_UNSUPPORTED;
    // enough blocks to keep the memory busy: about four to an SM over all tiles
    int chunks = (4 * 148 + max_tiles - 1) / max_tiles;
    int per_block = (N + chunks - 1) / chunks;
    per_block = per_block < 8 ? 8 : per_block;
    const dim3 grid(max_tiles, (N + per_block - 1) / per_block), block(256);
    const size_t smem = (size_t)4 * K * (dtype == CB_F32 ? 4 : 2);      // the staged rows
    if (smem > 64 * 1024) return CB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define CB_MOE(TT, GG)                                                                                  \
    do {                                                                                                \
        if (smem > 48 * 1024) {                                                                         \
            static bool configured = false;                                                             \
            if (!configured) {                                                                          \
                cudaError_t err = cudaFuncSetAttribute(moe_rows_small_kernel<TT, GG, 4>,                \
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); \
                if (err != cudaSuccess) return (int)err;                                                \
                configured = true;                                                                      \
            }                                                                                           \
        }                                                                                               \
        cb_launch(moe_rows_small_kernel<TT, GG, 4>, grid, block, smem, s, (const TT*)a, a_stride,       \
                  (const TT*)w, expert_stride, N, K, plan, E, max_tiles, sorted_pair, top, weight, out, \
                  out_stride, per_block, rule);                                                         \
    } while (0)
    if (dtype == CB_F32) { if (gated) CB_MOE(float, true); else CB_MOE(float, false); }
    else { if (gated) CB_MOE(__nv_bfloat16, true); else CB_MOE(__nv_bfloat16, false); }
#undef CB_MOE
    return cb_last_error();
}

CB_EXPORT int cb_moe_combine(const float* pair_out, int top, float* residual, int n_tokens, int width,
                             void* stream) {
    if (n_tokens <= 0) return 0;
    cb_launch(moe_combine_kernel, dim3(n_tokens), dim3(width >= 1024 ? 256 : 128), 0, (cudaStream_t)stream,
              pair_out, top, residual, width);
    return cb_last_error();
}

CB_EXPORT int cb_moe_gather(const void* h, int h_stride, int dtype, const int* sorted_pair, int top,
                            void* out, int n_pairs, int width, void* stream) {
    if (n_pairs <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(moe_gather_kernel<float>, dim3(n_pairs), dim3(128), 0, s, (const float*)h, h_stride,
                  sorted_pair, top, (float*)out, width);
    else
        cb_launch(moe_gather_kernel<__nv_bfloat16>, dim3(n_pairs), dim3(128), 0, s, (const __nv_bfloat16*)h,
                  h_stride, sorted_pair, top, (__nv_bfloat16*)out, width);
    return cb_last_error();
}

CB_EXPORT int cb_moe_scatter(const float* rows, const int* sorted_pair, const float* weight,
                             float* pair_out, int n_pairs, int width, void* stream) {
    if (n_pairs <= 0) return 0;
    cb_launch(moe_scatter_kernel, dim3(n_pairs), dim3(128), 0, (cudaStream_t)stream, rows, sorted_pair,
              weight, pair_out, width);
    return cb_last_error();
}
