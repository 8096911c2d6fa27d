// PolyNorm, an activation of a feed-forward: for a token's vector z of ff values
//     act(z) = a N(z) + b N(z^2) + c N(z^3) + e,   N(v) = v / sqrt(mean(v^2) + eps),
// with powers taken element by element and four learned numbers (a, b, c, e).
// One block per token: the sums of z^2, z^4 and z^6 in fp32 in one pass, then the
// result in a second.  The block's size is a function of ff alone.
#define CB_PDL_BIT 12      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

template <typename T>
__global__ void polynorm_kernel(const T* __restrict__ z, int z_stride, const float* __restrict__ coef,
                                T* __restrict__ out, int out_stride, int ff, float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float scratch[32];
    const T* row = z + (size_t)blockIdx.x * z_stride;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < ff; i += blockDim.x) {
        const float v = cb_to_float(row[i]);
        const float v2 = v * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v2 * v, v2 * v, s6);
    }
    const float t2 = cb_block_sum(s2, scratch);
    const float t4 = cb_block_sum(s4, scratch);
    const float t6 = cb_block_sum(s6, scratch);
    const float r1 = coef[0] / sqrtf(t2 / (float)ff + eps);
    const float r2 = coef[1] / sqrtf(t4 / (float)ff + eps);
    const float r3 = coef[2] / sqrtf(t6 / (float)ff + eps);
    const float e = coef[3];
    T* dst = out + (size_t)blockIdx.x * out_stride;
    for (int i = threadIdx.x; i < ff; i += blockDim.x) {
        const float v = cb_to_float(row[i]);
        const float v2 = v * v;
        dst[i] = cb_from_float<T>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))));
    }
}

}  // namespace

CB_EXPORT int cb_polynorm(const void* z, int z_stride, const float* coef, void* out, int out_stride,
                          int dtype, int n_rows, int ff, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    const dim3 grid(n_rows), block(ff <= 256 ? 64 : (ff >= 4096 ? 1024 : (ff / 4 + 31) / 32 * 32));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(polynorm_kernel<float>, grid, block, 0, s, (const float*)z, z_stride, coef,
                  (float*)out, out_stride, ff, eps);
    else
        cb_launch(polynorm_kernel<__nv_bfloat16>, grid, block, 0, s, (const __nv_bfloat16*)z, z_stride,
                  coef, (__nv_bfloat16*)out, out_stride, ff, eps);
    return cb_last_error();
}
