// Short causal depthwise convolution over time with a per-request history, an optional bias and an
// optional SiLU:
//
//   y[t, c] = act( b[c] + sum_{j < L} w[c, j] * u[t - (L-1) + j, c] ),   u = history ++ x
//
// Tap L-1 multiplies the current token.  The history is the last L-1 inputs of the request (zero for
// a new request), kept in 32-bit [slots, L-1, C], oldest first.  x may be a column slice of a wider
// matrix (its row stride is given).  Sums and the activation are 32-bit; y is rounded to the model's
// dtype.  A step of prompt portions runs two kernels (all outputs read the old history, then the
// history is replaced); a step of single tokens runs one.
#include "common.cuh"

#define ZAI_CONV_MAX_TAPS 16

template <typename T>
__global__ void causal_conv_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ x, int x_stride,
                                   const float* __restrict__ taps, const float* __restrict__ bias,
                                   const float* __restrict__ state, const int* __restrict__ seq_idx,
                                   const int* __restrict__ cu_q, const int* __restrict__ slot_ids, int C, int L, int act,
                                   int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = seq_idx[t], start = cu_q[s];
    const int slot = zai_checked_slot(slot_ids[s], num_slots, status);
    const float* hist = state + (size_t)slot * (L - 1) * C;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < L; ++j) {
        const int tt = t - (L - 1) + j;
        const float u = tt >= start ? to_float(x[(size_t)tt * x_stride + c]) : hist[(size_t)(L - 1 + tt - start) * C + c];
        acc += taps[(size_t)c * L + j] * u;
    }
    if (act) acc = acc / (1.f + expf(-acc));
    out[(size_t)t * out_stride + c] = from_float<T>(acc);
}

// history <- the last L-1 rows of (history ++ the request's rows of this step)
template <typename T>
__global__ void causal_conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                         const int* __restrict__ cu_q, const int* __restrict__ slot_ids, int C, int L,
                                         int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int start = cu_q[s], n = cu_q[s + 1] - start;
    if (n <= 0) return;
    const int slot = zai_checked_slot(slot_ids[s], num_slots, status);
    float* hist = state + (size_t)slot * (L - 1) * C;
    for (int i = 0; i < L - 1; ++i) {                 // reads run ahead of writes: row n+i > i
        const int src = n + i;
        hist[(size_t)i * C + c] = src < L - 1 ? hist[(size_t)src * C + c]
                                              : to_float(x[(size_t)(start + src - (L - 1)) * x_stride + c]);
    }
}

// every request brings one token: output and history in one pass
template <typename T>
__global__ void causal_conv_single_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ x, int x_stride,
                                          const float* __restrict__ taps, const float* __restrict__ bias,
                                          float* __restrict__ state, const int* __restrict__ slot_ids, int C, int L,
                                          int act, int write_state, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int slot = zai_checked_slot(slot_ids[s], num_slots, status);
    float* hist = state + (size_t)slot * (L - 1) * C;
    const float cur = to_float(x[(size_t)s * x_stride + c]);
    float acc = (bias ? bias[c] : 0.f) + taps[(size_t)c * L + (L - 1)] * cur;
    for (int j = 0; j < L - 1; ++j) {
        const float u = hist[(size_t)j * C + c];
        acc += taps[(size_t)c * L + j] * u;
        if (write_state && j > 0) hist[(size_t)(j - 1) * C + c] = u;
    }
    if (write_state && L > 1) hist[(size_t)(L - 2) * C + c] = cur;
    if (act) acc = acc / (1.f + expf(-acc));
    out[(size_t)s * out_stride + c] = from_float<T>(acc);
}

ZAI_API int zai_causal_conv(void* out, int out_stride, const void* x, int x_stride, int dtype, const float* taps,
                            const float* bias, float* state, const int* seq_idx, const int* cu_q, const int* slot_ids,
                            int N, int S, int C, int L, int act, int single_tokens, int write_state, int num_slots,
                            int* status, cudaStream_t stream) {
    if (N <= 0 || C <= 0) return ZAI_OK;
    if (L < 1 || L > ZAI_CONV_MAX_TAPS || C > 65535 * 128) return ZAI_BAD_SIZE;
    const int threads = 128;
    const unsigned cb = (unsigned)((C + threads - 1) / threads);
    if (single_tokens && N == S) {
        ZAI_DISPATCH(dtype, return launch_pdl(causal_conv_single_kernel<T>, dim3(S, cb), dim3(threads), 0, stream, (T*)out,
            out_stride, (const T*)x, x_stride, taps, bias, state, slot_ids, C, L, act, write_state, num_slots, status));
    }
    int rc;
    ZAI_DISPATCH(dtype, rc = launch_pdl(causal_conv_kernel<T>, dim3(N, cb), dim3(threads), 0, stream, (T*)out, out_stride,
        (const T*)x, x_stride, taps, bias, (const float*)state, seq_idx, cu_q, slot_ids, C, L, act, num_slots, status));
    if (rc != 0 || !write_state || L == 1) return rc;
    ZAI_DISPATCH(dtype, return launch_pdl(causal_conv_state_kernel<T>, dim3(S, cb), dim3(threads), 0, stream, (const T*)x,
        x_stride, state, cu_q, slot_ids, C, L, num_slots, status));
}
