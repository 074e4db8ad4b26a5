// Elementwise activations between two products: out = act(z), rows of T with a stride each.
//   0 squared ReLU: max(z, 0)^2      1 tanh      2 GELU (tanh form)      3 SiLU
// fp32 arithmetic, rounded once.
// And the gated pair of a feed-forward, out = gate_act(g) * up(u) over rows [g: F | u: F]:
//   silu:    g / (1 + exp(-g)) * u
//   capped:  g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(alpha * g') * (u' + offset)
#define CB_PDL_BIT 14      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int ACT_RELU2 = 0, ACT_TANH = 1, ACT_GELU_TANH = 2, ACT_SILU = 3;

template <int KIND>
__device__ __forceinline__ float act_f(float z) {
    if (KIND == ACT_RELU2) { const float r = fmaxf(z, 0.f); return r * r; }
    if (KIND == ACT_TANH) return tanhf(z);
    if (KIND == ACT_GELU_TANH)
        return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.0f + expf(-z));
}

template <typename TI, typename TO, int KIND>
__global__ void activation_kernel(const TI* __restrict__ z, int z_stride, TO* __restrict__ out,
                                  int out_stride, int n_rows, int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const size_t total = (size_t)n_rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width, c = i - t * width;
        out[t * out_stride + c] = cb_from_float<TO>(act_f<KIND>(cb_to_float(z[t * z_stride + c])));
    }
}

// limit <= 0: the silu pair; else the capped one.
__device__ __forceinline__ float glu_f(float g, float u, float limit, float alpha, float offset) {
    if (limit <= 0.f) return g / (1.0f + expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + offset);
}

template <typename T>
__global__ void glu_kernel(const T* __restrict__ both, int both_stride, T* __restrict__ out, int out_stride,
                           int n_rows, int width, float limit, float alpha, float offset) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const size_t total = (size_t)n_rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / width, c = i - t * width;
        const T* row = both + t * both_stride;
        out[t * out_stride + c] = cb_from_float<T>(glu_f(cb_to_float(row[c]), cb_to_float(row[width + c]),
                                                         limit, alpha, offset));
    }
}

template <typename TI, typename TO>
int launch(int kind, const void* z, int z_stride, void* out, int out_stride, int n_rows, int width,
           cudaStream_t s) {
    const size_t total = (size_t)n_rows * width;
    const dim3 grid((unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256)), block(256);
#define CB_ACT(KK)                                                                                  \
    cb_launch(activation_kernel<TI, TO, KK>, grid, block, 0, s, (const TI*)z, z_stride, (TO*)out,   \
              out_stride, n_rows, width)
    if (kind == ACT_RELU2) CB_ACT(ACT_RELU2);
    else if (kind == ACT_TANH) CB_ACT(ACT_TANH);
    else if (kind == ACT_GELU_TANH) CB_ACT(ACT_GELU_TANH);
    else if (kind == ACT_SILU) CB_ACT(ACT_SILU);
    else return CB_ERR_UNSUPPORTED;
#undef CB_ACT
    return cb_last_error();
}

}  // namespace

CB_EXPORT int cb_activation(int kind, const void* z, int z_stride, int in_dtype, void* out, int out_stride,
                            int out_dtype, int n_rows, int width, void* stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == CB_F32 && out_dtype == CB_F32)
        return launch<float, float>(kind, z, z_stride, out, out_stride, n_rows, width, s);
    if (in_dtype == CB_F32)
        return launch<float, __nv_bfloat16>(kind, z, z_stride, out, out_stride, n_rows, width, s);
    if (out_dtype == CB_F32)
        return launch<__nv_bfloat16, float>(kind, z, z_stride, out, out_stride, n_rows, width, s);
    return launch<__nv_bfloat16, __nv_bfloat16>(kind, z, z_stride, out, out_stride, n_rows, width, s);
}

// out[T, F] = pair(both[T, 0:F], both[T, F:2F]); limit <= 0: silu(g) * u, else the capped pair.
CB_EXPORT int cb_glu(const void* both, int both_stride, void* out, int out_stride, int dtype, int n_rows,
                     int width, float limit, float alpha, float offset, void* stream) {
    if (n_rows <= 0 || width <= 0) return 0;
    const size_t total = (size_t)n_rows * width;
    const dim3 grid((unsigned)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256)), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(glu_kernel<float>, grid, block, 0, s, (const float*)both, both_stride, (float*)out, out_stride,
                  n_rows, width, limit, alpha, offset);
    else
        cb_launch(glu_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)both, both_stride,
                  (__nv_bfloat16*)out, out_stride, n_rows, width, limit, alpha, offset);
    return cb_last_error();
}
