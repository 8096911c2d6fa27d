// Token embedding with a scale, a hashed bigram row and a learned position row:
//   x[t] = table[token] * scale + bigram[row(previous token, token)] + positions[p]
// row(a, b) = (a * mul_prev + b * mul_cur) mod buckets; the first token of a sequence
// (position 0) takes row `buckets`, the one after the hashed rows.  Either addend may be
// absent (null table).  The sum is fp32 and goes into the fp32 residual.
//
// The previous token of a portion's first row was fed by an earlier step: it lives in the
// request's state slot as one int32, the token + 1 (0: none yet; a slot is handed out
// zeroed).  The block of a request's first row reads it and then leaves the portion's last
// token there; no other block touches that word.
#define CB_PDL_BIT 12      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

__device__ __forceinline__ int resolve_token(int id, const int* device_tokens, int vocab) {
    if (id < 0 && device_tokens != nullptr) id = device_tokens[-id - 1];
    return id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
}

template <typename T>
__global__ void hashed_embedding_kernel(const T* __restrict__ table, const T* __restrict__ bigram,
                                        const T* __restrict__ pos_table, const int* __restrict__ ids,
                                        const int* __restrict__ positions,
                                        const int* __restrict__ row_request,
                                        const int* __restrict__ req_row_start,
                                        const int* __restrict__ req_state_slot, unsigned char* state,
                                        long slot_stride, float* __restrict__ out, int width, int vocab,
                                        float scale, int buckets, long long mul_prev, long long mul_cur,
                                        int max_positions, const int* __restrict__ device_tokens) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    const int r = row_request[t];
    const int row0 = req_row_start[r], row1 = req_row_start[r + 1];
    const int tok = resolve_token(ids[t], device_tokens, vocab);
    const int p = positions[t];
    int* last = state != nullptr
        ? reinterpret_cast<int*>(state + (size_t)req_state_slot[r] * slot_stride) : nullptr;
    long long brow = buckets;
    if (bigram != nullptr && p > 0) {
        int prev = 0;
        if (t > row0) prev = resolve_token(ids[t - 1], device_tokens, vocab);
        else if (last != nullptr) prev = max(*last - 1, 0);
        brow = ((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets;
        if (brow < 0) brow += buckets;
    }
    const T* e = table + (size_t)tok * width;
    const T* b = bigram != nullptr ? bigram + (size_t)brow * width : nullptr;
    const int pp = p < max_positions ? p : max_positions - 1;      // the host refuses longer contexts
    const T* q = pos_table != nullptr ? pos_table + (size_t)pp * width : nullptr;
    float* dst = out + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = cb_to_float(e[i]) * scale;
        if (b != nullptr) v += cb_to_float(b[i]);
        if (q != nullptr) v += cb_to_float(q[i]);
        dst[i] = v;
    }
    if (t == row0 && last != nullptr) {
        __syncthreads();          // every thread of this block has read the old word
        if (threadIdx.x == 0) *last = resolve_token(ids[row1 - 1], device_tokens, vocab) + 1;
    }
}

}  // namespace

CB_EXPORT int cb_hashed_embedding(const void* table, const void* bigram, const void* pos_table, int dtype,
                                  const int* ids, const int* positions, const int* row_request,
                                  const int* req_row_start, const int* req_state_slot, void* state,
                                  long slot_stride, float* out, int n_rows, int width, int vocab,
                                  float scale, int buckets, long long mul_prev, long long mul_cur,
                                  int max_positions, const int* device_tokens, void* stream) {
    if (n_rows <= 0) return 0;
    if (bigram != nullptr && buckets <= 0) return CB_ERR_UNSUPPORTED;
    const int threads = width >= 256 ? 256 : 64;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(hashed_embedding_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (const float*)table,
                  (const float*)bigram, (const float*)pos_table, ids, positions, row_request, req_row_start,
                  req_state_slot, (unsigned char*)state, slot_stride, out, width, vocab, scale, buckets,
                  mul_prev, mul_cur, max_positions, device_tokens);
    else
        cb_launch(hashed_embedding_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s,
                  (const __nv_bfloat16*)table, (const __nv_bfloat16*)bigram, (const __nv_bfloat16*)pos_table,
                  ids, positions, row_request, req_row_start, req_state_slot, (unsigned char*)state,
                  slot_stride, out, width, vocab, scale, buckets, mul_prev, mul_cur, max_positions,
                  device_tokens);
    return cb_last_error();
}
