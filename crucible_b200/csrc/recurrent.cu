// Mixers that carry a matrix of fixed size per head from token to token instead of
// a cache of keys: the gated delta rule, the matrix memory with exponential gates
// (mLSTM), the wkv rule with a decay per key channel and a bonus for the current token,
// and the state-space rule with one decay per head (Mamba-2).  Per request and head the state is S [D][E] in fp32 (mLSTM also n [D] and
// a running maximum m); it lives in the request's state slot and is read at the
// start of a step and written at its end, so a prompt may be cut anywhere.
//
//   delta rule, per token:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                           (the kernel takes both dots from S before the write: see there)
//   mLSTM, per token:       m' = max(f + m, i);  a = exp(f + m - m');  b = exp(i - m');
//                           S <- a S + b k v^T;  n <- a n + b k;
//                           o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
//   wkv, per token:         o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T
//                           (w a vector over the key channels, u a constant per head)
//   state space, per token: S <- a S + (dt k) v^T;  o = S^T q + skip v
//                           (a, dt numbers per head and token, skip a constant per head)
//   retention, per token:   S <- decay S + k v^T;  o = S^T q   (decay a constant per head):
//                           the state-space rule with a = decay, dt = 1 and no skip
//
// Kernels: the preparation of a step's rows (for the delta rule: a short causal
// convolution over time per channel, whose last taps - 1 inputs are state too,
// SiLU, unit vectors per head, and the gates; for the mLSTM: the capped gates), the
// update of the convolution's state, the recurrence itself, and the per-head RMS
// norm with gain and output gate.  Everything after the projections is fp32.
//
// The recurrence walks a request's tokens in order.  8 to 32 lanes share a column of a head's
// S, each with four or eight of its D entries in registers; a block is 128 threads.  A token
// costs one pass over a lane's entries and one shuffle reduction of its sums.
// The tokens' q, k, v and gates are staged in shared memory 16 tokens at a time, by
// asynchronous copies one chunk ahead.
#define CB_PDL_BIT 11      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int RULE_DELTA = 0, RULE_MLSTM = 1, RULE_WKV = 2, RULE_SSD = 3;
constexpr int GATE_SILU = 0, GATE_SIGMOID = 1;
constexpr int THREADS = 128;      // of a recurrence block: 128 / LANES columns of S
constexpr int CHUNK = 16;         // tokens staged at a time

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <int BYTES>
__device__ __forceinline__ void cp_async(float* smem, const float* gmem) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    if (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gmem) : "memory");
}

__device__ __forceinline__ float* state_at(unsigned char* state, long slot_stride, int slot, long off) {
    return reinterpret_cast<float*>(state + (size_t)slot * slot_stride + off);
}

// ---- delta rule: convolution + SiLU, unit q and k, gates ---------------------------------
// proj row: [q: G*D | k: G*D | v: H*E | ...] in T.  conv_w: fp32 [C][taps], the last column
// meets the current token.  The request's state holds the last taps - 1 inputs of every
// channel, oldest first, fp32 [taps-1][C].  gates: fp32 [rows][2H] = [beta logits | rate logits].
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, int proj_stride,
                                     const float* __restrict__ conv_w, int taps,
                                     const float* __restrict__ gates, int gates_stride,
                                     const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias,
                                     const int* __restrict__ row_request,
                                     const int* __restrict__ req_row_start,
                                     const int* __restrict__ req_state_slot, unsigned char* state,
                                     long slot_stride, long tail_off, float* __restrict__ qkv,
                                     float* __restrict__ beta, float* __restrict__ decay, int n_heads,
                                     int n_kv_heads, int key_dim, int value_dim) {
    cb_pdl_trigger();
    cb_pdl_wait();
    extern __shared__ float row[];
    const int t = blockIdx.x;
    const int r = row_request[t];
    const int first = req_row_start[r];
    const int local = t - first;
    const int C = 2 * n_kv_heads * key_dim + n_heads * value_dim;
    const float* tail = state_at(state, slot_stride, req_state_slot[r], tail_off);
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = local - (taps - 1) + j;
            const float x = src >= 0 ? cb_to_float(proj[(size_t)(first + src) * proj_stride + c])
                                     : tail[(size_t)(taps - 1 + src) * C + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        row[c] = silu_f(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    // q heads then k heads: unit vectors; q also times D^-1/2
    const float q_scale = 1.0f / sqrtf((float)key_dim);
    for (int h = warp; h < 2 * n_kv_heads; h += n_warps) {
        float* v = row + (size_t)h * key_dim;
        float ss = 0.f;
        for (int d = lane; d < key_dim; d += 32) ss = fmaf(v[d], v[d], ss);
        float inv = 1.0f / sqrtf(cb_warp_sum(ss) + 1e-6f);
        if (h < n_kv_heads) inv *= q_scale;
        for (int d = lane; d < key_dim; d += 32) v[d] *= inv;
    }
    __syncthreads();
    float* dst = qkv + (size_t)t * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = row[c];
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        const float* g = gates + (size_t)t * gates_stride;
        beta[(size_t)t * n_heads + h] = sigmoid_f(g[h]);
        decay[(size_t)t * n_heads + h] = expf(-expf(a_log[h]) * softplus_f(g[n_heads + h] + dt_bias[h]));
    }
}

// After a step: the convolution's state becomes the last taps - 1 inputs seen.
template <typename T>
__global__ void conv_tail_update_kernel(const T* __restrict__ proj, int proj_stride, int taps, int C,
                                        const int* __restrict__ req_row_start,
                                        const int* __restrict__ req_state_slot, unsigned char* state,
                                        long slot_stride, long tail_off) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int r = blockIdx.x;
    const int first = req_row_start[r], n_new = req_row_start[r + 1] - first;
    float* tail = state_at(state, slot_stride, req_state_slot[r], tail_off);
    const int keep = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        for (int i = 0; i < keep; ++i) {          // ascending: reads run ahead of writes
            const int src = n_new - keep + i;
            tail[(size_t)i * C + c] = src >= 0 ? cb_to_float(proj[(size_t)(first + src) * proj_stride + c])
                                               : tail[(size_t)(i + n_new) * C + c];
        }
    }
}

// ---- mLSTM: q * D^-1/2, k, v to fp32 and the capped log gates -----------------------------
// proj row: [q: H*D | k: H*D | v: H*E | ...]; gates: fp32 [rows][2H] = [input | forget] logits.
template <typename T>
__global__ void mlstm_prepare_kernel(const T* __restrict__ proj, int proj_stride,
                                     const float* __restrict__ gates, int gates_stride,
                                     const float* __restrict__ bias_i,
                                     const float* __restrict__ bias_f, float cap, float* __restrict__ qkv,
                                     float* __restrict__ log_keep, float* __restrict__ log_in,
                                     int n_heads, int key_dim, int value_dim) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    const int nq = n_heads * key_dim, C = 2 * nq + n_heads * value_dim;
    const float q_scale = 1.0f / sqrtf((float)key_dim);
    const T* src = proj + (size_t)t * proj_stride;
    float* dst = qkv + (size_t)t * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float x = cb_to_float(src[c]);
        dst[c] = c < nq ? x * q_scale : x;
    }
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        const float* g = gates + (size_t)t * gates_stride;
        log_in[(size_t)t * n_heads + h] = cap * tanhf((g[h] + bias_i[h]) / cap);
        log_keep[(size_t)t * n_heads + h] = logsigmoid_f(cap * tanhf((g[n_heads + h] + bias_f[h]) / cap));
    }
}

// ---- retention: rotation of q and k, the keys' scale, the heads' fixed decays ---------------
// proj row: [q: H*D | k: H*D | v: H*E | ...].  The first R features of every q and k head turn
// by the fp32 angle position * freq[i], as split halves (i with i + R/2) or as neighbouring
// pairs; k is multiplied by k_scale after the rotation; all of it fp32, written to qkv fp32
// [rows][2*H*D + H*E].  keep[rows][H] receives the head's decay, step[rows][H] ones: what the
// state-space rule of the recurrence reads per token.
template <typename T>
__global__ void retention_prepare_kernel(const T* __restrict__ proj, int proj_stride,
                                         const float* __restrict__ freq, int rotary_dim, int split_halves,
                                         const int* __restrict__ positions,
                                         const float* __restrict__ head_decay, float k_scale,
                                         float* __restrict__ qkv, float* __restrict__ keep,
                                         float* __restrict__ step, int n_heads, int key_dim,
                                         int value_dim) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    const int nq = n_heads * key_dim, C = 2 * nq + n_heads * value_dim;
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[t];
    const T* src = proj + (size_t)t * proj_stride;
    float* dst = qkv + (size_t)t * C;
    // the turning pairs of the 2H heads of q and k
    for (int i = threadIdx.x; i < 2 * n_heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        const int ia = split_halves ? j : 2 * j, ib = split_halves ? j + half : 2 * j + 1;
        float sn, cs;
        sincosf(pos * freq[j], &sn, &cs);
        const float a = cb_to_float(src[(size_t)h * key_dim + ia]), b = cb_to_float(src[(size_t)h * key_dim + ib]);
        const float sc = h < n_heads ? 1.0f : k_scale;
        dst[(size_t)h * key_dim + ia] = (a * cs - b * sn) * sc;
        dst[(size_t)h * key_dim + ib] = (b * cs + a * sn) * sc;
    }
    // the features of q and k that pass unchanged
    const int pass = key_dim - rotary_dim;
    for (int i = threadIdx.x; i < 2 * n_heads * pass; i += blockDim.x) {
        const int h = i / pass, f = rotary_dim + (i - h * pass);
        const float x = cb_to_float(src[(size_t)h * key_dim + f]);
        dst[(size_t)h * key_dim + f] = h < n_heads ? x : x * k_scale;
    }
    for (int c = 2 * nq + threadIdx.x; c < C; c += blockDim.x) dst[c] = cb_to_float(src[c]);
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        keep[(size_t)t * n_heads + h] = head_decay[h];
        step[(size_t)t * n_heads + h] = 1.0f;
    }
}

// ---- the recurrence ----------------------------------------------------------------------
// qkv: fp32 [rows][C] with q heads at q_off, k heads at k_off (both n_qk_heads of D), v heads at
// v_off (n_heads of E).  sc0, sc1: fp32 [rows][H]: (decay, beta) or (log keep, log in).
// State: S at s_off [H][D][E] (kept as [H][E][D], a column's entries side by side, a decode
// step was slower: 0.237 against 0.218 ms); mLSTM: n at n_off [H][D], m at m_off [H].
// A block: COLS columns x LANES lanes; lane `part` of a column owns entries part * P .. part * P + P - 1
// of it.  The staged k and q rows are padded by four floats per part, so that the parts'
// 16-byte reads fall on different banks.
template <int P, int LANES, int RULE>
__global__ void __launch_bounds__(THREADS) matrix_memory_kernel(
    const float* __restrict__ qkv, int C, int q_off, int k_off, int v_off,
    const float* __restrict__ sc0, const float* __restrict__ sc1,
    const int* __restrict__ req_row_start, const int* __restrict__ req_state_slot,
    unsigned char* state, long slot_stride, long s_off, long n_off, long m_off,
    float* __restrict__ out, int n_heads, int n_qk_heads, int D, int E, int w_off,
    const float* __restrict__ per_head) {
    // w_off: wkv's decay vectors in the rows of qkv (one of D per head); per_head: wkv's bonus
    // u [H][D], the state-space rule's skip [H]
    cb_pdl_trigger();
    cb_pdl_wait();
    constexpr int COLS = THREADS / LANES;
    constexpr int PAD = P == 4 ? 8 : 4;       // the parts' 16-byte reads then fall on different banks
    constexpr int PITCH = LANES * (P + PAD);
    constexpr int NVEC = RULE == RULE_WKV ? 3 : 2;      // staged vectors of D per token: k, q (, w)
    constexpr int BUF = CHUNK * (NVEC * PITCH + COLS) + 2 * CHUNK;      // floats of one stage
    extern __shared__ __align__(16) float stage[];
    const int r = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * COLS;
    const int g = head / (n_heads / n_qk_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = col0 + warp * (32 / LANES) + lane / LANES, part = lane % LANES;
    const bool live = col < E;
    const int row0 = req_row_start[r], row1 = req_row_start[r + 1];
    const int slot = req_state_slot[r];
    float* S = state_at(state, slot_stride, slot, s_off) + (size_t)head * D * E;
    float* N = RULE == RULE_MLSTM ? state_at(state, slot_stride, slot, n_off) + (size_t)head * D : nullptr;
    float* M = RULE == RULE_MLSTM ? state_at(state, slot_stride, slot, m_off) + head : nullptr;
    // the padding of the staged rows and the columns beyond E stay zero
    for (int i = threadIdx.x; i < 2 * BUF; i += blockDim.x) stage[i] = 0.f;
    float s[P], n[P];
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < P; ++i) {
        const int d = part * P + i;
        s[i] = (live && d < D) ? S[(size_t)d * E + col] : 0.f;
        n[i] = (RULE == RULE_MLSTM && d < D) ? N[d] : 0.f;
        if (RULE == RULE_WKV) n[i] = d < D ? per_head[(size_t)head * D + d] : 0.f;      // the bonus u
    }
    const float skip = RULE == RULE_SSD ? per_head[head] : 0.f;
    if (RULE == RULE_MLSTM) m = *M;
    __syncthreads();
    // 16-byte copies if every row of q and k starts on a 16-byte boundary
    const bool vec = ((C | q_off | k_off | D | (RULE == RULE_WKV ? w_off : 0)) & 3) == 0;
    // a chunk's q, k, v and gates on their way into one of the two stages (asynchronous
    // copies: the next chunk travels while this one is worked on)
    auto fetch = [&](int base, int buf) {
        float* sk = stage + buf * BUF;
        float* sq = sk + CHUNK * PITCH;
        float* sv = sq + (NVEC - 1) * CHUNK * PITCH;
        float* sw = sq + CHUNK * PITCH;                     // wkv only
        float* s0 = sv + CHUNK * COLS;
        float* s1 = s0 + CHUNK;
        const int cnt = min(CHUNK, row1 - base);
        if (vec) {
            const int per_row = D >> 2;
            for (int i = threadIdx.x; i < cnt * per_row; i += blockDim.x) {
                const int tt = i / per_row, d = (i - tt * per_row) << 2;
                const float* src = qkv + (size_t)(base + tt) * C + (size_t)g * D + d;
                const int at = tt * PITCH + d + (d / P) * PAD;
                cp_async<16>(sk + at, src + k_off);
                cp_async<16>(sq + at, src + q_off);
                if (RULE == RULE_WKV) cp_async<16>(sw + at, src + w_off);
            }
        } else {
            for (int i = threadIdx.x; i < cnt * D; i += blockDim.x) {
                const int tt = i / D, d = i - tt * D;
                const float* src = qkv + (size_t)(base + tt) * C + (size_t)g * D + d;
                const int at = tt * PITCH + d + (d / P) * PAD;
                cp_async<4>(sk + at, src + k_off);
                cp_async<4>(sq + at, src + q_off);
                if (RULE == RULE_WKV) cp_async<4>(sw + at, src + w_off);
            }
        }
        for (int i = threadIdx.x; i < cnt * COLS; i += blockDim.x) {
            const int tt = i / COLS, c = i - tt * COLS;
            if (col0 + c < E)
                cp_async<4>(sv + i, qkv + (size_t)(base + tt) * C + v_off + (size_t)head * E + col0 + c);
        }
        if (RULE != RULE_WKV && threadIdx.x < cnt) {
            cp_async<4>(s0 + threadIdx.x, sc0 + (size_t)(base + threadIdx.x) * n_heads + head);
            cp_async<4>(s1 + threadIdx.x, sc1 + (size_t)(base + threadIdx.x) * n_heads + head);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (row0 < row1) fetch(row0, 0);
    // delta rule: the pending write of the token before; mLSTM: the sums of the token before
    float k_prev[P], g_prev = 1.f, u_prev = 0.f;
#pragma unroll
    for (int i = 0; i < P; ++i) k_prev[i] = 0.f;
    float p_o = 0.f, p_n = 0.f, p_m = 0.f;
    size_t p_at = 0;
    bool pending = false;
    int buf = 0;
    for (int base = row0; base < row1; base += CHUNK, buf ^= 1) {
        const int cnt = min(CHUNK, row1 - base);
        if (base + CHUNK < row1) {
            fetch(base + CHUNK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* sk = stage + buf * BUF;
        const float* sq = sk + CHUNK * PITCH;
        const float* sv = sq + (NVEC - 1) * CHUNK * PITCH;
        const float* sw = sq + CHUNK * PITCH;
        const float* s0 = sv + CHUNK * COLS;
        const float* s1 = s0 + CHUNK;
#pragma unroll 4
        for (int tt = 0; tt < cnt; ++tt) {
            const float4* k4 = reinterpret_cast<const float4*>(sk + tt * PITCH + part * (P + PAD));
            const float4* q4 = reinterpret_cast<const float4*>(sq + tt * PITCH + part * (P + PAD));
            float kk[P], qq[P];
#pragma unroll
            for (int j = 0; j < P / 4; ++j) {
                const float4 a = k4[j], b = q4[j];
                kk[4 * j] = a.x; kk[4 * j + 1] = a.y; kk[4 * j + 2] = a.z; kk[4 * j + 3] = a.w;
                qq[4 * j] = b.x; qq[4 * j + 1] = b.y; qq[4 * j + 2] = b.z; qq[4 * j + 3] = b.w;
            }
            const float v = sv[tt * COLS + (col - col0)];
            const size_t out_at = (size_t)(base + tt) * n_heads * E + (size_t)head * E + col;
            if (RULE == RULE_DELTA) {
                // One pass per token.  The write of the token before (S <- g S + k u^T) is still
                // pending; it is applied on the way, and this token's dots are taken from the
                // result.  With r = S^T k and w = S^T q over S as that write leaves it:
                //   u = beta (v - g r),   o = g w + u (k . q)       [= (g S + k u^T)^T q]
                const float decay = s0[tt], beta = s1[tt];
                float rk[4] = {0.f, 0.f, 0.f, 0.f}, rq[4] = {0.f, 0.f, 0.f, 0.f}, kq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < P; ++i) {
                    s[i] = fmaf(k_prev[i], u_prev, g_prev * s[i]);
                    rk[i & 3] = fmaf(s[i], kk[i], rk[i & 3]);
                    rq[i & 3] = fmaf(s[i], qq[i], rq[i & 3]);
                    kq[i & 3] = fmaf(kk[i], qq[i], kq[i & 3]);
                }
                float r = (rk[0] + rk[1]) + (rk[2] + rk[3]);
                float w = (rq[0] + rq[1]) + (rq[2] + rq[3]);
                float c = (kq[0] + kq[1]) + (kq[2] + kq[3]);
#pragma unroll
                for (int x = 1; x < LANES; x <<= 1) {
                    r += __shfl_xor_sync(0xffffffffu, r, x);
                    w += __shfl_xor_sync(0xffffffffu, w, x);
                    c += __shfl_xor_sync(0xffffffffu, c, x);
                }
                const float u = beta * (v - decay * r);
                if (live && part == 0) out[out_at] = fmaf(u, c, decay * w);
#pragma unroll
                for (int i = 0; i < P; ++i) k_prev[i] = kk[i];
                g_prev = decay;
                u_prev = u;
            } else if (RULE == RULE_WKV || RULE == RULE_SSD) {
                // As below: the update needs no sum over a column; a token's sum is reduced and
                // stored under the next token's pass.
                float oc[4] = {0.f, 0.f, 0.f, 0.f};
                if (RULE == RULE_WKV) {
                    const float4* w4 = reinterpret_cast<const float4*>(sw + tt * PITCH + part * (P + PAD));
                    float ww[P];
#pragma unroll
                    for (int j = 0; j < P / 4; ++j) {
                        const float4 a = w4[j];
                        ww[4 * j] = a.x; ww[4 * j + 1] = a.y; ww[4 * j + 2] = a.z; ww[4 * j + 3] = a.w;
                    }
#pragma unroll
                    for (int i = 0; i < P; ++i) {
                        const float kv = __fmul_rn(kk[i], v);
                        oc[i & 3] = fmaf(fmaf(n[i], kv, s[i]), qq[i], oc[i & 3]);
                        s[i] = fmaf(ww[i], s[i], kv);
                    }
                } else {
                    const float a = s0[tt], dv = __fmul_rn(s1[tt], v);
#pragma unroll
                    for (int i = 0; i < P; ++i) {
                        s[i] = fmaf(kk[i], dv, __fmul_rn(a, s[i]));
                        oc[i & 3] = fmaf(s[i], qq[i], oc[i & 3]);
                    }
                }
                if (pending) {
#pragma unroll
                    for (int x = 1; x < LANES; x <<= 1) p_o += __shfl_xor_sync(0xffffffffu, p_o, x);
                    if (live && part == 0) out[p_at] = __fadd_rn(p_o, p_n);
                }
                p_o = (oc[0] + oc[1]) + (oc[2] + oc[3]);
                p_n = __fmul_rn(skip, v);      // never fused with the sum: every token rounds alike
                p_at = out_at;
                pending = true;
            } else {
                // The state's update needs no sum over a column, so tokens follow one another
                // without waiting for a shuffle: a token's sums are reduced, divided and stored
                // while the next token's pass runs.
                const float f = s0[tt], in = s1[tt];
                const float m_new = fmaxf(f + m, in);
                const float a = expf(f + m - m_new), b = expf(in - m_new);
                m = m_new;
                const float bv = b * v;
                float oc[4] = {0.f, 0.f, 0.f, 0.f}, nc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < P; ++i) {
                    s[i] = fmaf(kk[i], bv, a * s[i]);
                    n[i] = fmaf(b, kk[i], a * n[i]);
                    oc[i & 3] = fmaf(s[i], qq[i], oc[i & 3]);
                    nc[i & 3] = fmaf(n[i], qq[i], nc[i & 3]);
                }
                if (pending) {
#pragma unroll
                    for (int x = 1; x < LANES; x <<= 1) {
                        p_o += __shfl_xor_sync(0xffffffffu, p_o, x);
                        p_n += __shfl_xor_sync(0xffffffffu, p_n, x);
                    }
                    if (live && part == 0) out[p_at] = p_o / (fmaxf(fabsf(p_n), expf(-p_m)) + 1e-6f);
                }
                p_o = (oc[0] + oc[1]) + (oc[2] + oc[3]);
                p_n = (nc[0] + nc[1]) + (nc[2] + nc[3]);
                p_m = m;
                p_at = out_at;
                pending = true;
            }
        }
        __syncthreads();          // the stage is free for the chunk after next
    }
    if (RULE == RULE_DELTA) {
#pragma unroll
        for (int i = 0; i < P; ++i) s[i] = fmaf(k_prev[i], u_prev, g_prev * s[i]);      // the last token's write
    } else if ((RULE == RULE_WKV || RULE == RULE_SSD) && pending) {
#pragma unroll
        for (int x = 1; x < LANES; x <<= 1) p_o += __shfl_xor_sync(0xffffffffu, p_o, x);
        if (live && part == 0) out[p_at] = __fadd_rn(p_o, p_n);
    } else if (pending) {
#pragma unroll
        for (int x = 1; x < LANES; x <<= 1) {
            p_o += __shfl_xor_sync(0xffffffffu, p_o, x);
            p_n += __shfl_xor_sync(0xffffffffu, p_n, x);
        }
        if (live && part == 0) out[p_at] = p_o / (fmaxf(fabsf(p_n), expf(-p_m)) + 1e-6f);
    }
#pragma unroll
    for (int i = 0; i < P; ++i) {
        const int d = part * P + i;
        if (live && d < D) S[(size_t)d * E + col] = s[i];
        if (RULE == RULE_MLSTM && blockIdx.z == 0 && col == 0 && d < D) N[d] = n[i];
    }
    if (RULE == RULE_MLSTM && blockIdx.z == 0 && threadIdx.x == 0) *M = m;
}

// ---- wkv: the mixes of a token with the token before it ------------------------------------
// h: T rows [rows][width].  mu: fp32 [n_mix][width].  out: T [n_mix][rows][width]:
//   out[s][t] = h[t] + (h[t-1] - h[t]) * mu[s]      (fp32 arithmetic, rounded once)
// h[t-1] of a portion's first row is the request's state (fp32 [width], zeros at a sequence's
// start); the block of that row reads it and then leaves the portion's last row there.
template <typename T>
__global__ void shift_mix_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ mu,
                                 int n_mix, const int* __restrict__ row_request,
                                 const int* __restrict__ req_row_start,
                                 const int* __restrict__ req_state_slot, unsigned char* state,
                                 long slot_stride, long prev_off, T* __restrict__ out, int n_rows,
                                 int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    const int r = row_request[t];
    const int row0 = req_row_start[r], row1 = req_row_start[r + 1];
    float* kept = state_at(state, slot_stride, req_state_slot[r], prev_off);
    const T* cur = h + (size_t)t * h_stride;
    const T* before = t > row0 ? h + (size_t)(t - 1) * h_stride : nullptr;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = cb_to_float(cur[i]);
        const float d = (before != nullptr ? cb_to_float(before[i]) : kept[i]) - x;
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * n_rows + t) * width + i] = cb_from_float<T>(fmaf(d, mu[(size_t)s * width + i], x));
    }
    if (t == row0) {
        // each thread rewrites only the entries it has read itself
        const T* last = h + (size_t)(row1 - 1) * h_stride;
        for (int i = threadIdx.x; i < width; i += blockDim.x) kept[i] = cb_to_float(last[i]);
    }
}

// ---- wkv: r, k, v to fp32 and the decay w = exp(-exp(logit + w0)) ---------------------------
// rkv: T [3][rows][H*D] (r, k, v one after the other); logit: fp32 [rows][H*D]; qkv: fp32
// [rows][4*H*D] = [r | k | v | w].
template <typename T>
__global__ void wkv_prepare_kernel(const T* __restrict__ rkv, long plane_stride,
                                   const float* __restrict__ logit, const float* __restrict__ w0,
                                   float* __restrict__ qkv, int HD) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    float* dst = qkv + (size_t)t * 4 * HD;
    for (int c = threadIdx.x; c < 3 * HD; c += blockDim.x) {
        const int plane = c / HD;
        dst[c] = cb_to_float(rkv[(size_t)plane * plane_stride + (size_t)t * HD + (c - plane * HD)]);
    }
    for (int c = threadIdx.x; c < HD; c += blockDim.x)
        dst[3 * HD + c] = expf(-expf(logit[(size_t)t * HD + c] + w0[c]));
}

// ---- state space: convolution with bias + SiLU over [x | B | C], step size and decay --------
// proj: T rows whose columns conv_at .. conv_at + C - 1 are the convolution's channels; conv_w:
// fp32 [C][taps], the last column meets the current token; conv_b: fp32 [C].  The request's
// state holds the last taps - 1 inputs of every channel, oldest first, fp32 [taps-1][C].
// gates: fp32 [rows][H] step-size logits: dt = softplus(logit + dt_bias), decay = exp(-exp(A_log) dt).
template <typename T>
__global__ void ssd_prepare_kernel(const T* __restrict__ proj, int proj_stride, int conv_at,
                                   const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                                   int taps, const float* __restrict__ gates, int gates_stride,
                                   const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                   const int* __restrict__ row_request,
                                   const int* __restrict__ req_row_start,
                                   const int* __restrict__ req_state_slot, unsigned char* state,
                                   long slot_stride, long tail_off, float* __restrict__ xbc,
                                   float* __restrict__ decay, float* __restrict__ step, int n_heads,
                                   int C) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    const int r = row_request[t];
    const int first = req_row_start[r];
    const int local = t - first;
    const float* tail = state_at(state, slot_stride, req_state_slot[r], tail_off);
    float* dst = xbc + (size_t)t * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = conv_b != nullptr ? conv_b[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = local - (taps - 1) + j;
            const float x = src >= 0 ? cb_to_float(proj[(size_t)(first + src) * proj_stride + conv_at + c])
                                     : tail[(size_t)(taps - 1 + src) * C + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        dst[c] = silu_f(acc);
    }
    for (int h = threadIdx.x; h < n_heads; h += blockDim.x) {
        const float dt = softplus_f(gates[(size_t)t * gates_stride + h] + dt_bias[h]);
        step[(size_t)t * n_heads + h] = dt;
        decay[(size_t)t * n_heads + h] = expf(-expf(a_log[h]) * dt);
    }
}

// ---- output gate, then RMS norm in equal parts of a row, then gain ---------------------------
// y: fp32 [rows][width]; gate: T rows; out[t] = unit_rms_per_part(y[t] * silu(gate[t])) * gain.
// One block per (row, part); the block size is a function of the part's width alone.
template <typename T>
__global__ void gate_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate,
                                       int gate_stride, const float* __restrict__ gain,
                                       T* __restrict__ out, int out_stride, int width, int parts,
                                       float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x / parts, part = blockIdx.x - t * parts;
    const int n = width / parts, at = part * n;
    const float* src = y + (size_t)t * width + at;
    const T* g = gate + (size_t)t * gate_stride + at;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = src[i] * silu_f(cb_to_float(g[i]));
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(cb_block_sum(ss, scratch) / (float)n + eps);
    T* dst = out + (size_t)t * out_stride + at;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        dst[i] = cb_from_float<T>(src[i] * silu_f(cb_to_float(g[i])) * r * gain[at + i]);
}

// ---- per-head RMS norm, gain and output gate ----------------------------------------------
// o: fp32 [rows][H*E].  gain: [E] shared by the heads (gain_head_stride 0) or [H*E], or null
// (a norm without a weight).
// gate: T rows (the joint projection) at a column offset.  out: T rows at a column offset.
template <typename T, int GATE>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gain,
                                      int gain_head_stride, const T* __restrict__ gate, int gate_stride,
                                      T* __restrict__ out, int out_stride, int n_rows, int n_heads,
                                      int E, float eps, float out_scale) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= n_rows * n_heads) return;
    const int lane = threadIdx.x & 31;
    const int t = unit / n_heads, h = unit - t * n_heads;
    const float* src = o + (size_t)t * n_heads * E + (size_t)h * E;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) ss = fmaf(src[e], src[e], ss);
    const float r = 1.0f / sqrtf(cb_warp_sum(ss) / (float)E + eps);
    const T* grow = gate + (size_t)t * gate_stride + (size_t)h * E;
    T* dst = out + (size_t)t * out_stride + (size_t)h * E;
    const float* gn = gain != nullptr ? gain + (size_t)h * gain_head_stride : nullptr;
    for (int e = lane; e < E; e += 32) {
        const float z = cb_to_float(grow[e]);
        const float gt = GATE == GATE_SILU ? silu_f(z) : sigmoid_f(z);
        const float normed = gn != nullptr ? src[e] * r * gn[e] : src[e] * r;
        dst[e] = cb_from_float<T>(normed * gt * out_scale);
    }
}

template <int P, int LANES, int RULE>
int launch_memory_as(const float* qkv, int C, int q_off, int k_off, int v_off, const float* sc0,
                     const float* sc1, const int* req_row_start, const int* req_state_slot,
                     unsigned char* state, long slot_stride, long s_off, long n_off, long m_off, float* out,
                     int n_requests, int n_heads, int n_qk_heads, int D, int E, int w_off,
                     const float* per_head, cudaStream_t s) {
    constexpr int COLS = THREADS / LANES, PAD = P == 4 ? 8 : 4, NVEC = RULE == RULE_WKV ? 3 : 2;
    const dim3 grid(n_requests, n_heads, (E + COLS - 1) / COLS), block(THREADS);
    const size_t smem = 2 * (size_t)(CHUNK * (NVEC * LANES * (P + PAD) + COLS) + 2 * CHUNK) * sizeof(float);
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(matrix_memory_kernel<P, LANES, RULE>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
    }
    cb_launch(matrix_memory_kernel<P, LANES, RULE>, grid, block, smem, s, qkv, C, q_off, k_off, v_off, sc0,
              sc1, req_row_start, req_state_slot, state, slot_stride, s_off, n_off, m_off, out, n_heads,
              n_qk_heads, D, E, w_off, per_head);
    return cb_last_error();
}

// Eight lanes to a column.  More lanes (16 or 32, four entries each) were slower: at width
// 2,048 a 2,048-token prompt's recurrence took 1.16 ms instead of 0.61, a batch-8 decode step
// 0.46 ms instead of 0.33 (four times the warps, each repeating the loads of k and q and two
// more shuffle rounds).
template <int RULE>
int launch_memory(const float* qkv, int C, int q_off, int k_off, int v_off, const float* sc0,
                  const float* sc1, const int* req_row_start, const int* req_state_slot,
                  unsigned char* state, long slot_stride, long s_off, long n_off, long m_off, float* out,
                  int n_requests, int n_heads, int n_qk_heads, int D, int E, int w_off,
                  const float* per_head, cudaStream_t s) {
#define CB_MEM(PP, LL)                                                                              \
    return launch_memory_as<PP, LL, RULE>(qkv, C, q_off, k_off, v_off, sc0, sc1, req_row_start,     \
                                          req_state_slot, state, slot_stride, s_off, n_off, m_off,  \
                                          out, n_requests, n_heads, n_qk_heads, D, E, w_off,        \
                                          per_head, s)
    if (D <= 32) CB_MEM(4, 8);
    if (D <= 64) CB_MEM(8, 8);
    if (D <= 128) CB_MEM(16, 8);
    if (D <= 256) CB_MEM(32, 8);
#undef CB_MEM
    return CB_ERR_UNSUPPORTED;
}

}  // namespace

CB_EXPORT int cb_delta_prepare(const void* proj, int proj_stride, int dtype, const float* conv_w,
                               int taps, const float* gates, int gates_stride, const float* a_log,
                               const float* dt_bias,
                               const int* row_request, const int* req_row_start,
                               const int* req_state_slot, void* state, long slot_stride, long tail_off,
                               float* qkv, float* beta, float* decay, int n_rows, int n_heads,
                               int n_kv_heads, int key_dim, int value_dim, void* stream) {
    if (n_rows <= 0) return 0;
    const int C = 2 * n_kv_heads * key_dim + n_heads * value_dim;
    if (taps < 1 || C > 12000 || n_heads % n_kv_heads != 0) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(C <= 256 ? 128 : (C >= 2048 ? 1024 : (C / 2 + 31) / 32 * 32));
    const size_t smem = (size_t)C * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(delta_prepare_kernel<float>, grid, block, smem, s, (const float*)proj, proj_stride,
                  conv_w, taps, gates, gates_stride, a_log, dt_bias, row_request, req_row_start, req_state_slot,
                  (unsigned char*)state, slot_stride, tail_off, qkv, beta, decay, n_heads, n_kv_heads,
                  key_dim, value_dim);
    else
        cb_launch(delta_prepare_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)proj,
                  proj_stride, conv_w, taps, gates, gates_stride, a_log, dt_bias, row_request, req_row_start,
                  req_state_slot, (unsigned char*)state, slot_stride, tail_off, qkv, beta, decay,
                  n_heads, n_kv_heads, key_dim, value_dim);
    return cb_last_error();
}

CB_EXPORT int cb_conv_tail_update(const void* proj, int proj_stride, int dtype, int taps, int C,
                                  const int* req_row_start, const int* req_state_slot, void* state,
                                  long slot_stride, long tail_off, int n_requests, void* stream) {
    if (n_requests <= 0 || taps <= 1) return 0;
    const dim3 grid(n_requests, (C + 127) / 128), block(128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(conv_tail_update_kernel<float>, grid, block, 0, s, (const float*)proj, proj_stride,
                  taps, C, req_row_start, req_state_slot, (unsigned char*)state, slot_stride, tail_off);
    else
        cb_launch(conv_tail_update_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)proj,
                  proj_stride, taps, C, req_row_start, req_state_slot, (unsigned char*)state,
                  slot_stride, tail_off);
    return cb_last_error();
}

CB_EXPORT int cb_mlstm_prepare(const void* proj, int proj_stride, int dtype, const float* gates,
                               int gates_stride, const float* bias_i, const float* bias_f, float cap, float* qkv,
                               float* log_keep, float* log_in, int n_rows, int n_heads, int key_dim,
                               int value_dim, void* stream) {
    if (n_rows <= 0) return 0;
    const int C = n_heads * (2 * key_dim + value_dim);
    const dim3 grid(n_rows), block(C <= 512 ? 128 : (C >= 4096 ? 1024 : (C / 4 + 31) / 32 * 32));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(mlstm_prepare_kernel<float>, grid, block, 0, s, (const float*)proj, proj_stride,
                  gates, gates_stride, bias_i, bias_f, cap, qkv, log_keep, log_in, n_heads, key_dim, value_dim);
    else
        cb_launch(mlstm_prepare_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)proj,
                  proj_stride, gates, gates_stride, bias_i, bias_f, cap, qkv, log_keep, log_in, n_heads,
                  key_dim, value_dim);
    return cb_last_error();
}

// split_halves 0: neighbouring pairs turn, 1: feature i with i + rotary_dim / 2.
CB_EXPORT int cb_retention_prepare(const void* proj, int proj_stride, int dtype, const float* freq,
                                   int rotary_dim, int split_halves, const int* positions,
                                   const float* head_decay, float k_scale, float* qkv, float* keep,
                                   float* step, int n_rows, int n_heads, int key_dim, int value_dim,
                                   void* stream) {
    if (n_rows <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > key_dim || (rotary_dim & 1) || (rotary_dim && freq == nullptr))
        return CB_ERR_UNSUPPORTED;
    const int C = n_heads * (2 * key_dim + value_dim);
    const dim3 grid(n_rows), block(C <= 512 ? 128 : (C >= 4096 ? 1024 : (C / 4 + 31) / 32 * 32));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(retention_prepare_kernel<float>, grid, block, 0, s, (const float*)proj, proj_stride, freq,
                  rotary_dim, split_halves, positions, head_decay, k_scale, qkv, keep, step, n_heads,
                  key_dim, value_dim);
    else
        cb_launch(retention_prepare_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)proj,
                  proj_stride, freq, rotary_dim, split_halves, positions, head_decay, k_scale, qkv, keep,
                  step, n_heads, key_dim, value_dim);
    return cb_last_error();
}

// rule 0: the delta rule (sc0 decay, sc1 beta); rule 1: mLSTM (sc0 log keep, sc1 log in);
// rule 2: wkv (decay vectors at w_off in the rows, per_head the bonus [H][D]);
// rule 3: state space (sc0 decay, sc1 step size, per_head the skip [H]).
CB_EXPORT int cb_matrix_memory(int rule, const float* qkv, int C, int q_off, int k_off, int v_off,
                               const float* sc0, const float* sc1, const int* req_row_start,
                               const int* req_state_slot, void* state, long slot_stride, long s_off,
                               long n_off, long m_off, float* out, int n_requests, int n_heads,
                               int n_qk_heads, int key_dim, int value_dim, int w_off,
                               const float* per_head, void* stream) {
    if (n_requests <= 0) return 0;
    if (n_heads % n_qk_heads != 0) return CB_ERR_UNSUPPORTED;
    if ((rule == RULE_WKV || rule == RULE_SSD) && per_head == nullptr) return CB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define CB_RULE(RR)                                                                                  \
    if (rule == RR)                                                                                  \
        return launch_memory<RR>(qkv, C, q_off, k_off, v_off, sc0, sc1, req_row_start,               \
                                 req_state_slot, (unsigned char*)state, slot_stride, s_off, n_off,   \
                                 m_off, out, n_requests, n_heads, n_qk_heads, key_dim, value_dim,    \
                                 w_off, per_head, s)
    CB_RULE(RULE_DELTA);
    CB_RULE(RULE_MLSTM);
    CB_RULE(RULE_WKV);
    CB_RULE(RULE_SSD);
#undef CB_RULE
    return CB_ERR_UNSUPPORTED;
}

// gate_kind 0: SiLU, 1: sigmoid.
CB_EXPORT int cb_head_norm_gate(const float* o, const float* gain, int gain_head_stride,
                                const void* gate, int gate_stride, void* out, int out_stride, int dtype,
                                int gate_kind, int n_rows, int n_heads, int value_dim, float eps,
                                float out_scale, void* stream) {
    if (n_rows <= 0) return 0;
    const int warps = 4;
    const long units = (long)n_rows * n_heads;
    const dim3 grid((unsigned)((units + warps - 1) / warps)), block(warps * 32);
    cudaStream_t s = (cudaStream_t)stream;
#define CB_HNG(TT, GG)                                                                             \
    cb_launch(head_norm_gate_kernel<TT, GG>, grid, block, 0, s, o, gain, gain_head_stride,         \
              (const TT*)gate, gate_stride, (TT*)out, out_stride, n_rows, n_heads, value_dim, eps, \
              out_scale)
    if (dtype == CB_F32) {
        if (gate_kind == GATE_SILU) CB_HNG(float, GATE_SILU); else CB_HNG(float, GATE_SIGMOID);
    } else {
        if (gate_kind == GATE_SILU) CB_HNG(__nv_bfloat16, GATE_SILU); else CB_HNG(__nv_bfloat16, GATE_SIGMOID);
    }
#undef CB_HNG
    return cb_last_error();
}

CB_EXPORT int cb_shift_mix(const void* h, int h_stride, int dtype, const float* mu, int n_mix,
                           const int* row_request, const int* req_row_start, const int* req_state_slot,
                           void* state, long slot_stride, long prev_off, void* out, int n_rows, int width,
                           void* stream) {
    if (n_rows <= 0) return 0;
    const dim3 grid(n_rows), block(width >= 1024 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(shift_mix_kernel<float>, grid, block, 0, s, (const float*)h, h_stride, mu, n_mix,
                  row_request, req_row_start, req_state_slot, (unsigned char*)state, slot_stride, prev_off,
                  (float*)out, n_rows, width);
    else
        cb_launch(shift_mix_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)h, h_stride, mu,
                  n_mix, row_request, req_row_start, req_state_slot, (unsigned char*)state, slot_stride,
                  prev_off, (__nv_bfloat16*)out, n_rows, width);
    return cb_last_error();
}

CB_EXPORT int cb_wkv_prepare(const void* rkv, long rkv_stride, int dtype, const float* logit,
                             const float* w0, float* qkv, int n_rows, int HD, void* stream) {
    if (n_rows <= 0) return 0;
    const dim3 grid(n_rows), block(HD >= 1024 ? 512 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(wkv_prepare_kernel<float>, grid, block, 0, s, (const float*)rkv, rkv_stride, logit, w0,
                  qkv, HD);
    else
        cb_launch(wkv_prepare_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)rkv,
                  rkv_stride, logit, w0, qkv, HD);
    return cb_last_error();
}

CB_EXPORT int cb_ssd_prepare(const void* proj, int proj_stride, int conv_at, int dtype,
                             const float* conv_w, const float* conv_b, int taps, const float* gates,
                             int gates_stride, const float* a_log, const float* dt_bias,
                             const int* row_request, const int* req_row_start, const int* req_state_slot,
                             void* state, long slot_stride, long tail_off, float* xbc, float* decay,
                             float* step, int n_rows, int n_heads, int C, void* stream) {
    if (n_rows <= 0) return 0;
    if (taps < 1) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(C <= 256 ? 128 : (C >= 2048 ? 1024 : (C / 2 + 31) / 32 * 32));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(ssd_prepare_kernel<float>, grid, block, 0, s, (const float*)proj, proj_stride, conv_at,
                  conv_w, conv_b, taps, gates, gates_stride, a_log, dt_bias, row_request, req_row_start,
                  req_state_slot, (unsigned char*)state, slot_stride, tail_off, xbc, decay, step, n_heads, C);
    else
        cb_launch(ssd_prepare_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)proj,
                  proj_stride, conv_at, conv_w, conv_b, taps, gates, gates_stride, a_log, dt_bias,
                  row_request, req_row_start, req_state_slot, (unsigned char*)state, slot_stride, tail_off,
                  xbc, decay, step, n_heads, C);
    return cb_last_error();
}

CB_EXPORT int cb_gate_group_norm(const float* y, const void* gate, int gate_stride, const float* gain,
                                 void* out, int out_stride, int dtype, int n_rows, int width, int parts,
                                 float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (parts <= 0 || width % parts) return CB_ERR_UNSUPPORTED;
    const int n = width / parts;
    const dim3 grid((unsigned)((long)n_rows * parts)), block(n >= 1024 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(gate_group_norm_kernel<float>, grid, block, 0, s, y, (const float*)gate, gate_stride, gain,
                  (float*)out, out_stride, width, parts, eps);
    else
        cb_launch(gate_group_norm_kernel<__nv_bfloat16>, grid, block, 0, s, y, (const __nv_bfloat16*)gate,
                  gate_stride, gain, (__nv_bfloat16*)out, out_stride, width, parts, eps);
    return cb_last_error();
}
