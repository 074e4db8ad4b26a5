// Paged softmax attention whose window keeps the first tokens and whose denominator
// may hold a learned sink.  Two kernels (the preparation in two forms: the one described
// first, and a general one with an RMS norm of q and k, either pairing of the rotation and
// values cached as they are).
//
// (1) Preparation of a step's rows, one block per token.  A row of the joint
//     projection is [q: H*D | k: G*D | v: G*E | ...].  Pairs (2i, 2i+1), i < R/2, of
//     every q and k head turn by the angle position * freq[i] (the angle is an fp32
//     product, its sine and cosine are taken in fp32); features from R on pass.
//     q stays in the row; k goes to the token's place in the key pages; every v
//     head is divided by its root mean square over E (eps under the root) and goes
//     to the value pages.  Keys and values have sizes of their own (D and E):
//     pages are [page][kv head][token][feature] for each.
//
// (2) Attention, one warp per (row, query head), keys one by one in ascending
//     position with a running maximum, fp32 throughout.  A row at position p sees
//     j <= p with p - j < window or j < keep_first, i.e. the ranges
//     [0, min(keep_first, lo)) and [lo, p], lo = max(0, p - window + 1); window 0
//     means every earlier key.  After the keys the sink joins the denominator:
//     l += exp(sink[h] - m), with no value.  With a gate, the head's result is
//     multiplied by sigmoid(gate) and by out_scale before it is stored.
// A row's result depends on its own query and keys only.
#define CB_PDL_BIT 10      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

// key and value sizes up to 32 * PER_LANE: 256 in the usual form, 1,024 in the wide one

template <typename T>
__global__ void rotate_norm_append_kernel(T* __restrict__ proj, int proj_stride,
                                          const float* __restrict__ freq, int rotary_dim,
                                          const int* __restrict__ positions,
                                          const int* __restrict__ row_request,
                                          const int* __restrict__ block_table, int table_stride,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          int n_heads, int n_kv_heads, int key_dim, int value_dim,
                                          int page_tokens, int write_cache, float value_eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    T* row = proj + (size_t)t * proj_stride;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    size_t k_base = 0, v_base = 0;
    const size_t k_head_stride = (size_t)page_tokens * key_dim;
    const size_t v_head_stride = (size_t)page_tokens * value_dim;
    if (write_cache) {
        const int page = block_table[(size_t)row_request[t] * table_stride + pos / page_tokens];
        k_base = (size_t)page * n_kv_heads * k_head_stride + (size_t)(pos % page_tokens) * key_dim;
        v_base = (size_t)page * n_kv_heads * v_head_stride + (size_t)(pos % page_tokens) * value_dim;
    }
    const int n_rot_heads = n_heads + (write_cache ? n_kv_heads : 0);
    for (int i = threadIdx.x; i < n_rot_heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        T* src = row + (size_t)h * key_dim;
        const float angle = (float)pos * freq[j];
        float s, c;
        sincosf(angle, &s, &c);
        const float a = cb_to_float(src[2 * j]), b = cb_to_float(src[2 * j + 1]);
        T* dst = h < n_heads ? src : k_cache + k_base + (size_t)(h - n_heads) * k_head_stride;
        dst[2 * j] = cb_from_float<T>(a * c - b * s);
        dst[2 * j + 1] = cb_from_float<T>(b * c + a * s);
    }
    if (!write_cache) return;
    const int pass = key_dim - rotary_dim;
    for (int i = threadIdx.x; i < n_kv_heads * pass; i += blockDim.x) {
        const int h = i / pass, j = rotary_dim + (i - h * pass);
        k_cache[k_base + (size_t)h * k_head_stride + j] = row[(size_t)(n_heads + h) * key_dim + j];
    }
    // values: a warp per head
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const T* v_src = row + (size_t)(n_heads + n_kv_heads) * key_dim;
    for (int h = warp; h < n_kv_heads; h += n_warps) {
        const T* v = v_src + (size_t)h * value_dim;
        float ss = 0.f;
        for (int e = lane; e < value_dim; e += 32) {
            const float x = cb_to_float(v[e]);
            ss = fmaf(x, x, ss);
        }
        const float r = 1.0f / sqrtf(cb_warp_sum(ss) / (float)value_dim + value_eps);
        T* dst = v_cache + v_base + (size_t)h * v_head_stride;
        for (int e = lane; e < value_dim; e += 32) dst[e] = cb_from_float<T>(cb_to_float(v[e]) * r);
    }
}

// The general preparation: a warp per head of the token's row [q: H*D | k: G*D | v: G*E].
// Every q and k head may first be divided by its root mean square over D (eps under the root)
// and multiplied by a gain over D that all heads share (q_gain / k_gain null: no norm); then
// the first R features turn, as neighbouring pairs (2i, 2i + 1) or as split halves (i, i + R/2),
// by the fp32 angle position * freq[i]; q stays in the row, k goes to the pages.  Values are
// divided by their root mean square when value_eps >= 0 and copied as they are otherwise.
// whole_norm: the root mean square is taken over ALL of the token's q features (and all of its
// k features) at once instead of head by head, and the gains are [H * D] and [G * D].
// Norms, angles and the rotation are fp32; one rounding to T at the end.
template <typename T>
__global__ void norm_rotate_append_kernel(T* __restrict__ proj, int proj_stride,
                                          const float* __restrict__ q_gain,
                                          const float* __restrict__ k_gain, float qk_eps,
                                          const float* __restrict__ freq, int rotary_dim, int split_halves,
                                          const int* __restrict__ positions,
                                          const int* __restrict__ row_request,
                                          const int* __restrict__ block_table, int table_stride,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          int n_heads, int n_kv_heads, int key_dim, int value_dim,
                                          int page_tokens, int write_cache, float value_eps,
                                          int whole_norm) {
    cb_pdl_trigger();
    cb_pdl_wait();
    extern __shared__ float head_rows[];          // a row of key_dim floats per warp, then 2 * warps sums
    const int t = blockIdx.x;
    T* row = proj + (size_t)t * proj_stride;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    size_t k_base = 0, v_base = 0;
    const size_t k_head_stride = (size_t)page_tokens * key_dim;
    const size_t v_head_stride = (size_t)page_tokens * value_dim;
    if (write_cache) {
        const int page = block_table[(size_t)row_request[t] * table_stride + pos / page_tokens];
        k_base = (size_t)page * n_kv_heads * k_head_stride + (size_t)(pos % page_tokens) * key_dim;
        v_base = (size_t)page * n_kv_heads * v_head_stride + (size_t)(pos % page_tokens) * value_dim;
    }
    float* mine = head_rows + (size_t)warp * key_dim;
    const int n_turn_heads = n_heads + (write_cache ? n_kv_heads : 0);
    float r_q = 0.f, r_k = 0.f;
    if (whole_norm) {
        // the sums of squares over all q features and over all k features: every warp adds its
        // share of both (the block's size is a function of the head counts alone, so a row's
        // sum has one order whatever the step holds), then every thread adds the warps' shares
        float* sums = head_rows + (size_t)n_warps * key_dim;
        const int nq = n_heads * key_dim, nk = n_kv_heads * key_dim;
        float sq = 0.f, sk = 0.f;
        for (int f = threadIdx.x; f < nq; f += blockDim.x) {
            const float x = cb_to_float(row[f]);
            sq = fmaf(x, x, sq);
        }
        for (int f = threadIdx.x; f < nk; f += blockDim.x) {
            const float x = cb_to_float(row[nq + f]);
            sk = fmaf(x, x, sk);
        }
        sq = cb_warp_sum(sq);
        sk = cb_warp_sum(sk);
        if (lane == 0) {
            sums[warp] = sq;
            sums[n_warps + warp] = sk;
        }
        __syncthreads();
        sq = sk = 0.f;
        for (int w = 0; w < n_warps; ++w) {
            sq += sums[w];
            sk += sums[n_warps + w];
        }
        r_q = 1.0f / sqrtf(sq / (float)nq + qk_eps);
        r_k = 1.0f / sqrtf(sk / (float)nk + qk_eps);
    }
    for (int h = warp; h < n_turn_heads; h += n_warps) {
        const bool is_q = h < n_heads;
        T* src = row + (size_t)h * key_dim;
        const float* gain = is_q ? q_gain : k_gain;
        if (whole_norm && gain != nullptr) gain += (size_t)(is_q ? h : h - n_heads) * key_dim;
        float ss = 0.f;
        for (int f = lane; f < key_dim; f += 32) {
            const float x = cb_to_float(src[f]);
            mine[f] = x;
            ss = fmaf(x, x, ss);
        }
        if (gain != nullptr) {
            const float r = whole_norm ? (is_q ? r_q : r_k)
                                       : 1.0f / sqrtf(cb_warp_sum(ss) / (float)key_dim + qk_eps);
            for (int f = lane; f < key_dim; f += 32) mine[f] = mine[f] * r * gain[f];
        }
        __syncwarp();
        T* dst = is_q ? src : k_cache + k_base + (size_t)(h - n_heads) * k_head_stride;
        for (int j = lane; j < half; j += 32) {
            const int ia = split_halves ? j : 2 * j, ib = split_halves ? j + half : 2 * j + 1;
            float s, c;
            sincosf((float)pos * freq[j], &s, &c);
            const float a = mine[ia], b = mine[ib];
            dst[ia] = cb_from_float<T>(a * c - b * s);
            dst[ib] = cb_from_float<T>(b * c + a * s);
        }
        for (int f = rotary_dim + lane; f < key_dim; f += 32) dst[f] = cb_from_float<T>(mine[f]);
        __syncwarp();
    }
    if (!write_cache) return;
    const T* v_src = row + (size_t)(n_heads + n_kv_heads) * key_dim;
    for (int h = warp; h < n_kv_heads; h += n_warps) {
        const T* v = v_src + (size_t)h * value_dim;
        T* dst = v_cache + v_base + (size_t)h * v_head_stride;
        if (value_eps >= 0.f) {
            float ss = 0.f;
            for (int e = lane; e < value_dim; e += 32) {
                const float x = cb_to_float(v[e]);
                ss = fmaf(x, x, ss);
            }
            const float r = 1.0f / sqrtf(cb_warp_sum(ss) / (float)value_dim + value_eps);
            for (int e = lane; e < value_dim; e += 32) dst[e] = cb_from_float<T>(cb_to_float(v[e]) * r);
        } else {
            for (int e = lane; e < value_dim; e += 32) dst[e] = v[e];
        }
    }
}

template <typename T, int MAX_PER_LANE>
__global__ void sink_attention_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ gate, int gate_stride,
    T* __restrict__ out, int out_stride, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const float* __restrict__ sinks, const int* __restrict__ positions,
    const int* __restrict__ row_request, const int* __restrict__ block_table, int table_stride,
    int n_rows, int n_heads, int n_kv_heads, int key_dim, int value_dim, int page_tokens,
    float scale, int window, int keep_first, float out_scale, int gate_per_head) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int unit = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (unit >= n_rows * n_heads) return;
    const int lane = threadIdx.x & 31;
    const int t = unit / n_heads, h = unit - t * n_heads;
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)row_request[t] * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kept = keep_first < lo ? keep_first : lo;      // keys [0, kept) and [lo, pos]

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * key_dim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int f = lane + 32 * i;
        qv[i] = f < key_dim ? cb_to_float(qrow[f]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int range = 0; range < 2; ++range) {
        const int from = range == 0 ? 0 : lo, to = range == 0 ? kept : pos + 1;
        for (int j = from; j < to; ++j) {
            const int page = table[j / page_tokens];
            const size_t at = ((size_t)page * n_kv_heads + kvh) * page_tokens + (j % page_tokens);
            const T* kp = k_cache + at * key_dim;
            const T* vp = v_cache + at * value_dim;
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                const int f = lane + 32 * i;
                if (f < key_dim) part = fmaf(qv[i], cb_to_float(kp[f]), part);
            }
            const float s = cb_warp_sum(part) * scale;
            const float m_new = fmaxf(m, s);
            const float corr = expf(m - m_new);
            const float p = expf(s - m_new);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                const int f = lane + 32 * i;
                if (f < value_dim) acc[i] = fmaf(p, cb_to_float(vp[f]), acc[i] * corr);
            }
            m = m_new;
        }
    }
    float corr = 1.f;
    if (sinks != nullptr) {
        const float sk = sinks[h];
        const float m_new = fmaxf(m, sk);
        corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
    }
    const float inv = corr / l;
    T* orow = out + (size_t)t * out_stride + (size_t)h * value_dim;
    const T* grow = gate != nullptr
        ? gate + (size_t)t * gate_stride + (gate_per_head ? (size_t)h : (size_t)h * value_dim) : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int f = lane + 32 * i;
        if (f < value_dim) {
            float o = acc[i] * inv;
            if (grow != nullptr) o *= 1.0f / (1.0f + expf(-cb_to_float(grow[gate_per_head ? 0 : f])));
            orow[f] = cb_from_float<T>(o * out_scale);
        }
    }
}

}  // namespace

CB_EXPORT int cb_rotate_norm_append(void* proj, int proj_stride, int dtype, const float* freq,
                                    int rotary_dim, const int* positions, const int* row_request,
                                    const int* block_table, int table_stride, void* k_cache,
                                    void* v_cache, int n_rows, int n_heads, int n_kv_heads, int key_dim,
                                    int value_dim, int page_tokens, int write_cache, float value_eps,
                                    void* stream) {
    if (n_rows <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > key_dim || (rotary_dim & 1)) return CB_ERR_UNSUPPORTED;
    int threads = ((n_heads + n_kv_heads) * (rotary_dim / 2) + 31) / 32 * 32;
    threads = threads > 256 ? 256 : (threads < 64 ? 64 : threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(rotate_norm_append_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (float*)proj,
                  proj_stride, freq, rotary_dim, positions, row_request, block_table, table_stride,
                  (float*)k_cache, (float*)v_cache, n_heads, n_kv_heads, key_dim, value_dim,
                  page_tokens, write_cache, value_eps);
    else
        cb_launch(rotate_norm_append_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s,
                  (__nv_bfloat16*)proj, proj_stride, freq, rotary_dim, positions, row_request,
                  block_table, table_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads,
                  n_kv_heads, key_dim, value_dim, page_tokens, write_cache, value_eps);
    return cb_last_error();
}

// The general preparation (see norm_rotate_append_kernel): q_gain / k_gain null: no norm of
// q and k; split_halves 0: neighbouring pairs turn, 1: feature i with i + rotary_dim / 2;
// value_eps < 0: values are cached as they are; whole_norm 1: one root mean square over all of
// a token's q features (and one over its k features), gains [H * D] and [G * D].
CB_EXPORT int cb_norm_rotate_append(void* proj, int proj_stride, int dtype, const float* q_gain,
                                    const float* k_gain, float qk_eps, const float* freq,
                                    int rotary_dim, int split_halves, const int* positions,
                                    const int* row_request, const int* block_table, int table_stride,
                                    void* k_cache, void* v_cache, int n_rows, int n_heads,
                                    int n_kv_heads, int key_dim, int value_dim, int page_tokens,
                                    int write_cache, float value_eps, int whole_norm, void* stream) {
    if (n_rows <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > key_dim || (rotary_dim & 1) || key_dim > 4096) return CB_ERR_UNSUPPORTED;
    int warps = n_heads + n_kv_heads;
    warps = warps > 8 ? 8 : warps;
    const size_t smem = ((size_t)warps * key_dim + 2 * warps) * sizeof(float);
    if (smem > 48 * 1024) return CB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(norm_rotate_append_kernel<float>, dim3(n_rows), dim3(warps * 32), smem, s, (float*)proj,
                  proj_stride, q_gain, k_gain, qk_eps, freq, rotary_dim, split_halves, positions,
                  row_request, block_table, table_stride, (float*)k_cache, (float*)v_cache, n_heads,
                  n_kv_heads, key_dim, value_dim, page_tokens, write_cache, value_eps, whole_norm);
    else
        cb_launch(norm_rotate_append_kernel<__nv_bfloat16>, dim3(n_rows), dim3(warps * 32), smem, s,
                  (__nv_bfloat16*)proj, proj_stride, q_gain, k_gain, qk_eps, freq, rotary_dim,
                  split_halves, positions, row_request, block_table, table_stride,
                  (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads, n_kv_heads, key_dim,
                  value_dim, page_tokens, write_cache, value_eps, whole_norm);
    return cb_last_error();
}

CB_EXPORT int cb_sink_attention(const void* q, int q_stride, const void* gate, int gate_stride,
                                void* out, int out_stride, const void* k_cache, const void* v_cache,
                                int dtype, const float* sinks, const int* positions,
                                const int* row_request, const int* block_table, int table_stride,
                                int n_rows, int n_heads, int n_kv_heads, int key_dim, int value_dim,
                                int page_tokens, float scale, int window, int keep_first,
                                float out_scale, int gate_per_head, void* stream) {
    if (n_rows <= 0) return 0;
    if (key_dim > 1024 || value_dim > 1024 || n_heads % n_kv_heads != 0) return CB_ERR_UNSUPPORTED;
    const bool wide = key_dim > 256 || value_dim > 256;
    const int warps = 4;
    const long units = (long)n_rows * n_heads;
    const int blocks = (int)((units + warps - 1) / warps);
    cudaStream_t s = (cudaStream_t)stream;
#define CB_SINK_LAUNCH(TT, PL)                                                                          \
    cb_launch(sink_attention_kernel<TT, PL>, dim3(blocks), dim3(warps * 32), 0, s, (const TT*)q, q_stride, \
              (const TT*)gate, gate_stride, (TT*)out, out_stride, (const TT*)k_cache, (const TT*)v_cache, \
              sinks, positions, row_request, block_table, table_stride, n_rows, n_heads, n_kv_heads,    \
              key_dim, value_dim, page_tokens, scale, window, keep_first, out_scale, gate_per_head)
    if (dtype == CB_F32) {
        if (wide) CB_SINK_LAUNCH(float, 32);
        else CB_SINK_LAUNCH(float, 8);
    } else {
        if (wide) CB_SINK_LAUNCH(__nv_bfloat16, 32);
        else CB_SINK_LAUNCH(__nv_bfloat16, 8);
    }
#undef CB_SINK_LAUNCH
    return cb_last_error();
}
