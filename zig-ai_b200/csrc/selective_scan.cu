// Selective scan (the Mamba recurrence) over the rows of a step, with the per-request state carried
// in 32-bit between steps:
//
//   dt[t, c]  = softplus( sum_r Wdt[c, r] * p[t, r] + bdt[c] )                 p = [dt_in: R | B: S | C: S] per token
//   h[c, n]  <- exp(dt[t, c] * A[c, n]) * h[c, n] + dt[t, c] * x[t, c] * B[t, n]        A = -exp(A_log)
//   y[t, c]   = ( sum_n h[c, n] * C[t, n] + D[c] * x[t, c] ) * silu(z[t, c])
//
// Everything but the stored activations (x, p, z, y in the model's dtype) is 32-bit: the step size, the
// decay, the state and the sums.  G lanes of a warp share a channel, each with K of its S states in
// registers; the R-term product for the step size is split over the same lanes.  A block walks the
// tokens of one request in order, so a row's result does not depend on what else is in the batch.
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T, int K, int G>
__global__ void __launch_bounds__(128) selective_scan_kernel(
    T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ proj, int proj_stride, const T* __restrict__ z,
    int z_stride, const T* __restrict__ w_dt, const float* __restrict__ b_dt, const float* __restrict__ a_log,
    const float* __restrict__ d_skip, float* __restrict__ state, const int* __restrict__ cu_q,
    const int* __restrict__ slot_ids, int I, int S, int R, int write_state, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x;
    const int g = threadIdx.x % G;
    int c = blockIdx.y * (128 / G) + threadIdx.x / G;
    const bool live = c < I;
    if (!live) c = I - 1;                              // (keeps the lane in the shuffles; it stores nothing)
    const int start = cu_q[seq], end = cu_q[seq + 1];
    if (end <= start) return;
    const int slot = zai_checked_slot(slot_ids[seq], num_slots, status);
    float* st = state + ((size_t)slot * I + c) * S;
    float h[K], a[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const int n = g + k * G;
        h[k] = n < S ? st[n] : 0.f;
        a[k] = n < S ? -expf(a_log[(size_t)c * S + n]) : 0.f;
    }
    const float bias = b_dt[c], dsk = d_skip[c];
    const T* wrow = w_dt + (size_t)c * R;
    for (int t = start; t < end; ++t) {
        const T* p = proj + (size_t)t * proj_stride;
        float acc = 0.f;
        for (int r = g; r < R; r += G) acc += to_float(wrow[r]) * to_float(p[r]);
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        const float dt = softplus_f(acc + bias);
        const float xv = to_float(x[(size_t)t * I + c]);
        const float dx = dt * xv;
        float out = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int n = g + k * G;
            if (n < S) {
                h[k] = expf(dt * a[k]) * h[k] + dx * to_float(p[R + n]);
                out += h[k] * to_float(p[R + S + n]);
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
        if (g == 0 && live) {
            const float zv = to_float(z[(size_t)t * z_stride + c]);
            y[(size_t)t * I + c] = from_float<T>((out + dsk * xv) * (zv / (1.f + expf(-zv))));
        }
    }
    if (write_state && live) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int n = g + k * G;
            if (n < S) st[n] = h[k];
        }
    }
}

template <typename T, int K, int G>
static int launch_scan(void* y, const void* x, const void* proj, int proj_stride, const void* z, int z_stride, const void* w_dt,
                       const float* b_dt, const float* a_log, const float* d_skip, float* state, const int* cu_q,
                       const int* slot_ids, int n_seqs, int I, int S, int R, int write_state, int num_slots, int* status,
                       cudaStream_t stream) {
    const int per_block = 128 / G;
    const unsigned cb = (unsigned)((I + per_block - 1) / per_block);
    if (cb > 65535) return ZAI_BAD_SIZE;
    return launch_pdl(selective_scan_kernel<T, K, G>, dim3(n_seqs, cb), dim3(128), 0, stream, (T*)y, (const T*)x, (const T*)proj,
                      proj_stride, (const T*)z, z_stride, (const T*)w_dt, b_dt, a_log, d_skip, state, cu_q, slot_ids, I, S, R,
                      write_state, num_slots, status);
}

// y [N, I]; x [N, I]; proj [N, proj_stride] (dt_in | B | C); z [N, z_stride]; w_dt [I, R]; state [slots, I, S].
ZAI_API int zai_selective_scan(void* y, const void* x, const void* proj, int proj_stride, const void* z, int z_stride, int dtype,
                               const void* w_dt, const float* b_dt, const float* a_log, const float* d_skip, float* state,
                               const int* cu_q, const int* slot_ids, int N, int n_seqs, int I, int S, int R, int write_state,
                               int num_slots, int* status, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0) return ZAI_OK;
    if (I < 1 || S < 1 || S > 256 || R < 1) return ZAI_BAD_SIZE;
#define ZAI_SCAN(KK, GG) ZAI_DISPATCH(dtype, return launch_scan<T, KK, GG>(y, x, proj, proj_stride, z, z_stride, w_dt, b_dt, a_log, \
        d_skip, state, cu_q, slot_ids, n_seqs, I, S, R, write_state, num_slots, status, stream))
    if (S <= 4) ZAI_SCAN(1, 4);
    if (S <= 8) ZAI_SCAN(2, 4);
    if (S <= 16) ZAI_SCAN(4, 4);
    if (S <= 32) ZAI_SCAN(8, 4);
    if (S <= 64) ZAI_SCAN(8, 8);
    if (S <= 128) ZAI_SCAN(8, 16);
    ZAI_SCAN(8, 32);
#undef ZAI_SCAN
}
