// Elementwise activations between two products: out = act(z), rows of T with a stride each.
//   0 squared ReLU: max(z, 0)^2      1 tanh      2 GELU (tanh form)      3 SiLU
// fp32 arithmetic, rounded once.
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
