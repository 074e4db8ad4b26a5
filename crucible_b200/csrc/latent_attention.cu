// Attention over a cached latent: a token leaves one row [c | k_rot] in the pages, c the
// RMS-normed latent of `rank` features and k_rot a rotated key part of `rot` features that all
// heads share.  With each head's key matrix folded into its query
//   q'[h] = [ W_uk[h]^T q_plain[h] | rotate(q_rot[h]) ],
// the head's scores over the cache are q'[h] . [c | k_rot], and with the cached row also taken
// as the value, the first `rank` features of the result are sum_j p_j c_j, which the head's
// value matrix takes to its output.  So the attention itself is the paged attention of one
// shared key/value head of size rank + rot.  The kernels here are what surrounds it:
//
//   prepare   per token: RMS norm (fp32) of the latent with its gain, the rotation of the
//             shared key part, the row's write into its page; and the rotation of every
//             head's q_rot into the last `rot` columns of q'.
//   head gate per (token, head): the head's output times sigmoid(logit).
//
// Rotation: of the `rot` features the first `turned` turn (split_halves: feature i pairs with
// i + turned/2; else neighbours 2i, 2i + 1), the rest pass unchanged; the angle is fp32(position)
// * freq[i] as an fp32 product, cos and sin (fp32) times `mscale`.  A launch may do the pages'
// part alone (q null) or the queries' part alone (write 0: a layer that reads another layer's rows).
#define CB_PDL_BIT 15      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

// dkv: T rows [rank + rot]; q: T rows [H][dim + rot]; qx: T rows [H][rank + rot] (only the
// last rot columns of every head are written here); pages: T [page][1][page_tokens][rank + rot].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ dkv, int dkv_stride, const T* __restrict__ q,
                                      int q_stride, T* __restrict__ qx, int qx_stride,
                                      const float* __restrict__ gain, const float* __restrict__ freq,
                                      float mscale, float eps, const int* __restrict__ positions,
                                      const int* __restrict__ row_request,
                                      const int* __restrict__ block_table, int table_stride,
                                      T* __restrict__ pages, int n_heads, int dim, int rank, int rot,
                                      int turned, int page_tokens, int write, int split_halves) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = turned >> 1, still = rot - turned;
    const int step = split_halves ? 1 : 2, apart = split_halves ? half : 1;   // pair j: (j * step, j * step + apart)
    const T* src = dkv + (size_t)t * dkv_stride;
    if (write) {
        const int page = block_table[(size_t)row_request[t] * table_stride + pos / page_tokens];
        T* dst = pages + ((size_t)page * page_tokens + (pos % page_tokens)) * (rank + rot);
        float ss = 0.f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            const float v = cb_to_float(src[i]);
            ss = fmaf(v, v, ss);
        }
        const float r = 1.0f / sqrtf(cb_block_sum(ss, scratch) / (float)rank + eps);
        for (int i = threadIdx.x; i < rank; i += blockDim.x)
            dst[i] = cb_from_float<T>(cb_to_float(src[i]) * r * gain[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf((float)pos * freq[i], &sn, &cs);
            sn *= mscale; cs *= mscale;
            const int ia = rank + i * step, ib = ia + apart;
            const float u = cb_to_float(src[ia]), v = cb_to_float(src[ib]);
            dst[ia] = cb_from_float<T>(u * cs - v * sn);
            dst[ib] = cb_from_float<T>(v * cs + u * sn);
        }
        for (int i = threadIdx.x; i < still; i += blockDim.x) dst[rank + turned + i] = src[rank + turned + i];
    }
    if (q == nullptr) return;
    for (int i = threadIdx.x; i < n_heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        float sn, cs;
        sincosf((float)pos * freq[j], &sn, &cs);
        sn *= mscale; cs *= mscale;
        const T* qr = q + (size_t)t * q_stride + (size_t)h * (dim + rot) + dim;
        T* dq = qx + (size_t)t * qx_stride + (size_t)h * (rank + rot) + rank;
        const int ia = j * step, ib = ia + apart;
        const float u = cb_to_float(qr[ia]), v = cb_to_float(qr[ib]);
        dq[ia] = cb_from_float<T>(u * cs - v * sn);
        dq[ib] = cb_from_float<T>(v * cs + u * sn);
    }
    for (int i = threadIdx.x; i < n_heads * still; i += blockDim.x) {
        const int h = i / still, j = turned + (i - h * still);
        qx[(size_t)t * qx_stride + (size_t)h * (rank + rot) + rank + j] =
            q[(size_t)t * q_stride + (size_t)h * (dim + rot) + dim + j];
    }
}

// x[t][h][:] *= sigmoid(logit[t][h]); the logits are float32 or rows of T (columns of a joint
// projection).  Eight values of T a thread where the rows allow it.
template <typename T, typename L>
__global__ void head_gate_kernel(T* __restrict__ x, int x_stride, const L* __restrict__ logit,
                                 int logit_stride, int n_rows, int n_heads, int E) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    T* xr = x + (size_t)t * x_stride;
    const L* lr = logit + (size_t)t * logit_stride;
    constexpr int VEC = 16 / sizeof(T);
    if (E % VEC == 0 && x_stride % VEC == 0 && ((uintptr_t)x & 15) == 0) {
        for (int i = threadIdx.x * VEC; i < n_heads * E; i += blockDim.x * VEC) {
            const float g = 1.0f / (1.0f + expf(-cb_to_float(lr[i / E])));
            uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
            T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] = cb_from_float<T>(cb_to_float(v[j]) * g);
            *reinterpret_cast<uint4*>(xr + i) = raw;
        }
        return;
    }
    for (int i = threadIdx.x; i < n_heads * E; i += blockDim.x) {
        const float g = 1.0f / (1.0f + expf(-cb_to_float(lr[i / E])));
        xr[i] = cb_from_float<T>(cb_to_float(xr[i]) * g);
    }
}

// x[t][i] *= sigmoid(g[t][i]): a gate with a logit of its own for every feature
template <typename T>
__global__ void rows_gate_kernel(T* __restrict__ x, int x_stride, const T* __restrict__ g, int g_stride,
                                 int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    T* xr = x + (size_t)t * x_stride;
    const T* gr = g + (size_t)t * g_stride;
    // 16 bytes a load where the rows allow it (VEC values of T), the rest one by one
    constexpr int VEC = 16 / sizeof(T);
    const bool wide = ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(gr)) & 15) == 0;
    const int n_vec = wide ? width / VEC : 0;
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        uint4 xv = reinterpret_cast<const uint4*>(xr)[i];
        const uint4 gv = reinterpret_cast<const uint4*>(gr)[i];
        T* xs = reinterpret_cast<T*>(&xv);
        const T* gs = reinterpret_cast<const T*>(&gv);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float s = 1.0f / (1.0f + expf(-cb_to_float(gs[j])));
            xs[j] = cb_from_float<T>(cb_to_float(xs[j]) * s);
        }
        reinterpret_cast<uint4*>(xr)[i] = xv;
    }
    for (int i = n_vec * VEC + threadIdx.x; i < width; i += blockDim.x) {
        const float s = 1.0f / (1.0f + expf(-cb_to_float(gr[i])));
        xr[i] = cb_from_float<T>(cb_to_float(xr[i]) * s);
    }
}

// Per-head products of a step of few rows: out[t][h][n] = sum_k a[t][h][k] * w[h][n][k].
// One warp per (head, output feature): its lanes share K, the weight row is read once and meets
// every row of the step (up to ROWS at a time).  a: rows with a_stride, head h at h * a_head;
// out likewise.  fp32 sums.
template <typename T, int ROWS>
__global__ void heads_linear_small_kernel(const T* __restrict__ a, int a_stride, int a_head,
                                          const T* __restrict__ w, T* __restrict__ out, int out_stride,
                                          int out_head, int n_rows, int n_heads, int N, int K,
                                          const float* __restrict__ gate_logit, int gate_stride,
                                          const T* __restrict__ gate_rows, int gate_rows_stride) {
    // gate_logit (optional): fp32 [rows][heads]; the head's results times sigmoid(logit)
    // gate_rows (optional): T [rows][heads * N]; every result times the sigmoid of its own logit
    cb_pdl_trigger();
    cb_pdl_wait();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= n_heads * N) return;
    const int lane = threadIdx.x & 31;
    const int h = unit / N, n = unit - h * N;
    const T* wr = w + ((size_t)h * N + n) * K;
    for (int t0 = 0; t0 < n_rows; t0 += ROWS) {
        float acc[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
        for (int k = lane; k < K; k += 32) {
            const float wv = cb_to_float(wr[k]);
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (t0 + r < n_rows)
                    acc[r] = fmaf(cb_to_float(a[(size_t)(t0 + r) * a_stride + (size_t)h * a_head + k]), wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float v = cb_warp_sum(acc[r]);
            if (lane == 0 && t0 + r < n_rows) {
                if (gate_logit != nullptr)
                    v *= 1.0f / (1.0f + expf(-gate_logit[(size_t)(t0 + r) * gate_stride + h]));
                if (gate_rows != nullptr)
                    v *= 1.0f / (1.0f + expf(-cb_to_float(gate_rows[(size_t)(t0 + r) * gate_rows_stride + (size_t)h * N + n])));
                out[(size_t)(t0 + r) * out_stride + (size_t)h * out_head + n] = cb_from_float<T>(v);
            }
        }
    }
}

}  // namespace

CB_EXPORT int cb_heads_linear_small(const void* a, int a_stride, int a_head, const void* w, void* out,
                                    int out_stride, int out_head, int dtype, int n_rows, int n_heads,
                                    int N, int K, const float* gate_logit, int gate_stride,
                                    const void* gate_rows, int gate_rows_stride, void* stream) {
    if (n_rows <= 0 || n_heads <= 0 || N <= 0) return 0;
    const int warps = 4;
    const dim3 grid((unsigned)(((long)n_heads * N + warps - 1) / warps)), block(warps * 32);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(heads_linear_small_kernel<float, 8>, grid, block, 0, s, (const float*)a, a_stride, a_head,
                  (const float*)w, (float*)out, out_stride, out_head, n_rows, n_heads, N, K, gate_logit,
                  gate_stride, (const float*)gate_rows, gate_rows_stride);
    else
        cb_launch(heads_linear_small_kernel<__nv_bfloat16, 8>, grid, block, 0, s, (const __nv_bfloat16*)a,
                  a_stride, a_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, out_head, n_rows,
                  n_heads, N, K, gate_logit, gate_stride, (const __nv_bfloat16*)gate_rows, gate_rows_stride);
    return cb_last_error();
}

CB_EXPORT int cb_latent_prepare(const void* dkv, int dkv_stride, const void* q, int q_stride, void* qx,
                                int qx_stride, int dtype, const float* gain, const float* freq,
                                float mscale, float eps, const int* positions, const int* row_request,
                                const int* block_table, int table_stride, void* pages, int n_rows,
                                int n_heads, int dim, int rank, int rot, int turned, int page_tokens,
                                int write, int split_halves, void* stream) {
    if (n_rows <= 0) return 0;
    if (rot < 0 || turned < 0 || turned > rot || (turned & 1) || rank <= 0) return CB_ERR_UNSUPPORTED;
    if ((write && dkv == nullptr) || (!write && q == nullptr)) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(rank >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(latent_prepare_kernel<float>, grid, block, 0, s, (const float*)dkv, dkv_stride,
                  (const float*)q, q_stride, (float*)qx, qx_stride, gain, freq, mscale, eps, positions,
                  row_request, block_table, table_stride, (float*)pages, n_heads, dim, rank, rot,
                  turned, page_tokens, write, split_halves);
    else
        cb_launch(latent_prepare_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)dkv,
                  dkv_stride, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)qx, qx_stride, gain, freq,
                  mscale, eps, positions, row_request, block_table, table_stride, (__nv_bfloat16*)pages,
                  n_heads, dim, rank, rot, turned, page_tokens, write, split_halves);
    return cb_last_error();
}

CB_EXPORT int cb_rows_gate(void* x, int x_stride, const void* g, int g_stride, int dtype, int n_rows,
                           int width, void* stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    const dim3 grid(n_rows), block(width >= 2048 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(rows_gate_kernel<float>, grid, block, 0, s, (float*)x, x_stride, (const float*)g, g_stride, width);
    else
        cb_launch(rows_gate_kernel<__nv_bfloat16>, grid, block, 0, s, (__nv_bfloat16*)x, x_stride,
                  (const __nv_bfloat16*)g, g_stride, width);
    return cb_last_error();
}

// logit_dtype: float32 logits, or logits of the rows' own dtype.
CB_EXPORT int cb_head_gate(void* x, int x_stride, int dtype, const void* logit, int logit_dtype,
                           int logit_stride, int n_rows, int n_heads, int E, void* stream) {
    if (n_rows <= 0) return 0;
    if (logit_dtype != CB_F32 && logit_dtype != dtype) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(n_heads * E >= 2048 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(head_gate_kernel<float, float>, grid, block, 0, s, (float*)x, x_stride, (const float*)logit,
                  logit_stride, n_rows, n_heads, E);
    else if (logit_dtype == CB_F32)
        cb_launch(head_gate_kernel<__nv_bfloat16, float>, grid, block, 0, s, (__nv_bfloat16*)x, x_stride,
                  (const float*)logit, logit_stride, n_rows, n_heads, E);
    else
        cb_launch(head_gate_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, s, (__nv_bfloat16*)x,
                  x_stride, (const __nv_bfloat16*)logit, logit_stride, n_rows, n_heads, E);
    return cb_last_error();
}
