// Minimal gated recurrence (minGRU): gates that read only the current token, one state value per channel,
// carried in 32-bit between steps:
//
//   z = sigmoid(zr + bz)      u = xr + bx      cand = u + 1/2 (u >= 0),  sigmoid(u) (u < 0)
//   s <- (1 - z) * s + z * cand                 out = s * silu(gr)
//
// zr, xr, gr are the three column blocks of one projection [N, 3W].  One thread per (request, channel)
// walks the request's rows in order.  Gates, candidate and state are 32-bit; `out` is rounded to the
// model's dtype.
#include "common.cuh"

template <typename T>
__global__ void min_gru_kernel(T* __restrict__ out, const T* __restrict__ zxg, int in_stride, const float* __restrict__ bz,
                               const float* __restrict__ bx, float* __restrict__ state, const int* __restrict__ cu_q,
                               const int* __restrict__ slot_ids, int W, int write_state, int num_slots,
                               int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int start = cu_q[seq], end = cu_q[seq + 1];
    if (end <= start) return;
    const int slot = zai_checked_slot(slot_ids[seq], num_slots, status);
    float s = state[(size_t)slot * W + c];
    const float b_z = bz ? bz[c] : 0.f, b_x = bx ? bx[c] : 0.f;
#pragma unroll 4
    for (int t = start; t < end; ++t) {
        const T* row = zxg + (size_t)t * in_stride;
        const float zr = to_float(row[c]) + b_z, u = to_float(row[W + c]) + b_x, gr = to_float(row[2 * W + c]);
        const float z = 1.f / (1.f + expf(-zr));
        const float cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
        s = (1.f - z) * s + z * cand;
        out[(size_t)t * W + c] = from_float<T>(s * (gr / (1.f + expf(-gr))));
    }
    if (write_state) state[(size_t)slot * W + c] = s;
}

ZAI_API int zai_min_gru(void* out, const void* zxg, int in_stride, int dtype, const float* bz, const float* bx, float* state,
                        const int* cu_q, const int* slot_ids, int N, int n_seqs, int W, int write_state, int num_slots,
                        int* status, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0 || W <= 0) return ZAI_OK;
    const int threads = 128;
    const unsigned cb = (unsigned)((W + threads - 1) / threads);
    if (cb > 65535) return ZAI_BAD_SIZE;
    ZAI_DISPATCH(dtype, return launch_pdl(min_gru_kernel<T>, dim3(n_seqs, cb), dim3(threads), 0, stream, (T*)out, (const T*)zxg,
        in_stride, bz, bx, state, cu_q, slot_ids, W, write_state, num_slots, status));
}
