// A residual kept as several streams (hyper-connections).  The residual of a step is
// fp32 [tokens, S, width].  A sublayer reads one mixture of the streams,
//     u = sum_s a[s] x_s,
// through an RMSNorm, and its result y comes back into every stream at once,
//     x_t <- sum_s m[s][t] x_s + b[t] y      (all t from the old x_s).
// Kernels: the embedding row normalised and copied to every stream; the read
// (mixture + norm); the write, which can also do the next sublayer's read in the
// same pass over the token's row; and the sum of the streams at chosen rows.
// All arithmetic is fp32; T is the type the normalised rows leave in.  A block's
// size is a function of the width alone, so a row's sums are added in the same
// order whatever else the step holds.
#define CB_PDL_BIT 9      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

// half a thread per feature, so a decode step's few rows still have many loads in flight
__host__ __device__ inline int threads_for(int width) {
    const int t = ((width + 1) / 2 + 31) / 32 * 32;
    return t < 64 ? 64 : (t > 512 ? 512 : t);      // 512: the write kernel holds every stream of a feature in registers
}

// x0 = rmsnorm(table[id]) * gain, written to all S streams of the token
template <typename T>
__global__ void embed_norm_streams_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                          const float* __restrict__ gain, float* __restrict__ out,
                                          int width, int vocab, int n_streams, float eps,
                                          const int* __restrict__ device_tokens) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && device_tokens != nullptr) id = device_tokens[-id - 1];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* row = table + (size_t)id * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = cb_to_float(row[i]);
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(cb_block_sum(ss, scratch) / (float)width + eps);
    float* dst = out + (size_t)t * n_streams * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = cb_to_float(row[i]) * r * gain[i];
        for (int s = 0; s < n_streams; ++s) dst[(size_t)s * width + i] = v;
    }
}

// h = rmsnorm(sum_s a[s] x_s) * gain
template <typename T>
__global__ void streams_read_kernel(const float* __restrict__ x, const float* __restrict__ a,
                                    const float* __restrict__ gain, T* __restrict__ h, int width,
                                    int n_streams, float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    extern __shared__ float u[];
    __shared__ float scratch[32];
    const float* row = x + (size_t)blockIdx.x * n_streams * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_streams; ++s) v = fmaf(a[s], row[(size_t)s * width + i], v);
        u[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float r = 1.0f / sqrtf(cb_block_sum(ss, scratch) / (float)width + eps);
    T* dst = h + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = cb_from_float<T>(u[i] * r * gain[i]);
}

// x_t <- sum_s m[s][t] x_s + b[t] y; with NEXT also h = rmsnorm(sum_t a2[t] x_t) * gain2
template <typename T, bool NEXT>
__global__ void streams_write_kernel(float* __restrict__ x, const float* __restrict__ y,
                                     const float* __restrict__ m, const float* __restrict__ b,
                                     int width, int n_streams, const float* __restrict__ a2,
                                     const float* __restrict__ gain2, T* __restrict__ h, float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    extern __shared__ float u[];
    __shared__ float scratch[32];
    __shared__ float sm[MAX_STREAMS * MAX_STREAMS], sb[MAX_STREAMS], sa[MAX_STREAMS];
    if (threadIdx.x < n_streams * n_streams) sm[threadIdx.x] = m[threadIdx.x];
    if (threadIdx.x < n_streams) {
        sb[threadIdx.x] = b[threadIdx.x];
        sa[threadIdx.x] = NEXT ? a2[threadIdx.x] : 0.f;
    }
    __syncthreads();
    float* row = x + (size_t)blockIdx.x * n_streams * width;
    const float* yrow = y + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float old[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < n_streams ? row[(size_t)s * width + i] : 0.f;
        const float yi = yrow[i];
        float next = 0.f;
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) {
            if (t < n_streams) {
                float v = 0.f;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s)
                    if (s < n_streams) v = fmaf(sm[s * n_streams + t], old[s], v);
                v = fmaf(sb[t], yi, v);
                row[(size_t)t * width + i] = v;
                if (NEXT) next = fmaf(sa[t], v, next);
            }
        }
        if (NEXT) {
            u[i] = next;
            ss = fmaf(next, next, ss);
        }
    }
    if (NEXT) {
        const float r = 1.0f / sqrtf(cb_block_sum(ss, scratch) / (float)width + eps);
        T* dst = h + (size_t)blockIdx.x * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            dst[i] = cb_from_float<T>(u[i] * r * gain2[i]);
    }
}

__global__ void streams_sum_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                        float* __restrict__ out, int width, int n_streams) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const float* row = x + (size_t)rows[blockIdx.x] * n_streams * width;
    float* dst = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_streams; ++s) v += row[(size_t)s * width + i];
        dst[i] = v;
    }
}

}  // namespace

CB_EXPORT int cb_embed_norm_streams(const void* table, int table_dtype, const int* ids,
                                    const float* gain, float* out, int n_rows, int width, int vocab,
                                    int n_streams, float eps, const int* device_tokens, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > MAX_STREAMS) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(threads_for(width));
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == CB_F32)
        cb_launch(embed_norm_streams_kernel<float>, grid, block, 0, s, (const float*)table, ids, gain,
                  out, width, vocab, n_streams, eps, device_tokens);
    else
        cb_launch(embed_norm_streams_kernel<__nv_bfloat16>, grid, block, 0, s,
                  (const __nv_bfloat16*)table, ids, gain, out, width, vocab, n_streams, eps,
                  device_tokens);
    return cb_last_error();
}

CB_EXPORT int cb_streams_read(const float* x, const float* a, const float* gain, void* h, int h_dtype,
                              int n_rows, int width, int n_streams, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > MAX_STREAMS || width > 12000) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(threads_for(width));
    const size_t smem = (size_t)width * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype == CB_F32)
        cb_launch(streams_read_kernel<float>, grid, block, smem, s, x, a, gain, (float*)h, width,
                  n_streams, eps);
    else
        cb_launch(streams_read_kernel<__nv_bfloat16>, grid, block, smem, s, x, a, gain,
                  (__nv_bfloat16*)h, width, n_streams, eps);
    return cb_last_error();
}

// a2 null: only the write.  Otherwise the next sublayer's read leaves in h.
CB_EXPORT int cb_streams_write(float* x, const float* y, const float* m, const float* b, int n_rows,
                               int width, int n_streams, const float* a2, const float* gain2, void* h,
                               int h_dtype, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_streams < 1 || n_streams > MAX_STREAMS || width > 12000) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_rows), block(threads_for(width));
    cudaStream_t s = (cudaStream_t)stream;
    if (a2 == nullptr) {
        cb_launch(streams_write_kernel<float, false>, grid, block, 0, s, x, y, m, b, width, n_streams,
                  (const float*)nullptr, (const float*)nullptr, (float*)nullptr, eps);
    } else {
        const size_t smem = (size_t)width * sizeof(float);
        if (h_dtype == CB_F32)
            cb_launch(streams_write_kernel<float, true>, grid, block, smem, s, x, y, m, b, width,
                      n_streams, a2, gain2, (float*)h, eps);
        else
            cb_launch(streams_write_kernel<__nv_bfloat16, true>, grid, block, smem, s, x, y, m, b,
                      width, n_streams, a2, gain2, (__nv_bfloat16*)h, eps);
    }
    return cb_last_error();
}

CB_EXPORT int cb_streams_sum_rows(const float* x, const int* rows, float* out, int n_out, int width,
                                  int n_streams, void* stream) {
    if (n_out <= 0) return 0;
    cb_launch(streams_sum_rows_kernel, dim3(n_out), dim3(threads_for(width)), 0, (cudaStream_t)stream,
              x, rows, out, width, n_streams);
    return cb_last_error();
}
