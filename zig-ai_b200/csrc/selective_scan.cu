// Selective scan (the Mamba recurrence) over the rows of a step, with the per-request state carried
// in 32-bit between steps:
//
//   dt[t, c]  = softplus( sum_r Wdt[c, r] * p[t, r] + bdt[c] )                 p = [dt_in: R | B: S | C: S] per token
//   h[c, n]  <- exp(dt[t, c] * A[c, n]) * h[c, n] + dt[t, c] * x[t, c] * B[t, n]        A = -exp(A_log)
//   y[t, c]   = ( sum_n h[c, n] * C[t, n] + D[c] * x[t, c] ) * silu(z[t, c])
//
// Everything but the stored activations (x, p, z, y in the model's dtype) is 32-bit: the step size, the
// decay, the state and the sums.  The products dt_in . Wdt^T of all rows are one matrix product made beforehand
// (on the tensor cores where the model is bfloat16).  A lane holds K consecutive states of a channel in registers:
// a whole channel where S <= 16, else G lanes of a warp share it.  Rows are taken two or four at a time: the loads,
// step sizes and decays of the group do not depend on the state and are in flight together, only the state's own
// multiply-adds wait for one another.
//
// Two ways through a step:
//   * one pass (steps of single tokens and short portions): a block walks one request's rows in order;
//   * three passes (long portions): the rows of every request are cut into chunks of `chunk` tokens.
//     Pass 1 walks every chunk from a zero state and keeps its end state E and its summed step sizes
//     (the chunk's decay is exp(A * sum dt)); pass 2 carries the state across the chunks of a request,
//     h_in(j+1) = exp(A sum_j) h_in(j) + E_j, starting from the stored state, and stores the request's new
//     state; pass 3 walks every chunk again from its h_in and writes y.  The recurrence is linear in h, so
//     this is the same sum in another order (a difference of rounding only), and all chunks run at once.
#include "common.cuh"

// Exponentials and the softplus: exact library functions where the model is 32-bit; where activations are
// bfloat16 the hardware approximations (relative error about 2^-21, far below the 2^-9 of a stored activation).
template <typename T> __device__ __forceinline__ float exp_for(float v) { return expf(v); }
template <> __device__ __forceinline__ float exp_for<bf16>(float v) { return __expf(v); }
template <typename T> __device__ __forceinline__ float softplus_for(float v) { return v > 20.f ? v : log1pf(expf(v)); }
template <> __device__ __forceinline__ float softplus_for<bf16>(float v) { return v > 20.f ? v : __logf(1.f + __expf(v)); }
template <typename T> __device__ __forceinline__ float silu_for(float v) { return v / (1.f + expf(-v)); }
template <> __device__ __forceinline__ float silu_for<bf16>(float v) { return __fdividef(v, 1.f + __expf(-v)); }

// The chunk with index b among all chunks of the step (requests in order, each cut into chunks of Lc rows).
__device__ __forceinline__ bool zai_find_chunk(const int* __restrict__ cu_q, int n_seqs, int Lc, int b, int& seq, int& t0,
                                               int& t1) {
    for (int s = 0; s < n_seqs; ++s) {
        const int a = cu_q[s], e = cu_q[s + 1];
        const int nc = (e - a + Lc - 1) / Lc;
        if (b < nc) {
            seq = s;
            t0 = a + b * Lc;
            t1 = min(t0 + Lc, e);
            return true;
        }
        b -= nc;
    }
    return false;
}

// K consecutive values as 32-bit; `vec`: the address is a multiple of 8 bytes and K of four (16-bit values, 8 bytes a load)
template <int K>
__device__ __forceinline__ void load_run(const float* p, float (&d)[K], int n_valid, bool vec) {
#pragma unroll
    for (int k = 0; k < K; ++k) d[k] = k < n_valid ? p[k] : 0.f;
}
template <int K>
__device__ __forceinline__ void load_run(const bf16* p, float (&d)[K], int n_valid, bool vec) {
    if (K % 4 == 0 && vec && n_valid == K) {
#pragma unroll
        for (int k = 0; k < K; k += 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(p + k);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            d[k] = a.x; d[k + 1] = a.y; d[k + 2] = b.x; d[k + 3] = b.y;
        }
    } else {
#pragma unroll
        for (int k = 0; k < K; ++k) d[k] = k < n_valid ? __bfloat162float(p[k]) : 0.f;
    }
}

__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

// Walks rows [t0, t1) of one request for channel c; this lane holds the states g*K .. g*K + K - 1 (with 16 states
// or fewer one lane holds a channel's whole state: nothing is exchanged between lanes, and the rows' B and C are
// the same addresses for every lane of a warp).  `dt_raw` [N, I] holds the step sizes' products dt_in . Wdt^T in
// 32-bit (a matrix product made beforehand).  EMIT: writes y.  U rows are in flight together.  PREFETCH: the rows
// are first asked into L1 (one trip to memory for a chunk, not one per group of rows).
// dt_in . wrow over R terms, split over the G lanes of the channel (16 bytes a load where rows are aligned)
template <typename T, int G>
__device__ __forceinline__ float step_size_product(const T* __restrict__ wrow, const T* __restrict__ prow, int R, int g, bool vec) {
    float s = 0.f;
    if (sizeof(T) == 2 && vec) {
        for (int r = g * 8; r < R; r += G * 8) {
            const uint4 wv = *reinterpret_cast<const uint4*>(wrow + r), pv = *reinterpret_cast<const uint4*>(prow + r);
            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
            const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&pv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(wp[e]), b = __bfloat1622float2(pp[e]);
                s += a.x * b.x + a.y * b.y;
            }
        }
    } else {
        for (int r = g; r < R; r += G) s += to_float(wrow[r]) * to_float(prow[r]);
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return s;
}

template <typename T, int K, int G, bool EMIT, int U, bool PREFETCH>
__device__ __forceinline__ void scan_walk(float (&h)[K], const float (&a)[K], int t0, int t1, int c, int g, bool live,
                                          T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ proj, int proj_stride,
                                          const T* __restrict__ z, int z_stride, const float* __restrict__ dt_raw,
                                          const T* __restrict__ wrow, float bias, float dsk, int I, int S, int R, float* sum_dt) {
    if (PREFETCH) {
        const int c0 = blockIdx.y * (128 / G);
        for (int tt = t0 + threadIdx.x; tt < t1; tt += 128) {
            const T* p = proj + (size_t)tt * proj_stride + R;
            for (int o = 0; o < (int)(2 * S * sizeof(T)); o += 128) prefetch_l1(reinterpret_cast<const char*>(p) + o);
            for (int o = 0; o < 128 / G; o += 32) {
                prefetch_l1(dt_raw + (size_t)tt * I + c0 + o);
                if (o % 64 == 0) {
                    prefetch_l1(x + (size_t)tt * I + c0 + o);
                    if (EMIT) prefetch_l1(z + (size_t)tt * z_stride + c0 + o);
                }
            }
        }
    }
    const int n_mine = max(min(S - g * K, K), 0);
    const bool vec = sizeof(T) == 2 && ((proj_stride | R | S) & 3) == 0 && (reinterpret_cast<uintptr_t>(proj) & 7) == 0;
    float total = 0.f;
    for (int t = t0; t < t1; t += U) {
        float dt[U], xv[U], zv[U], bv[U][K], cv[U][K];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool on = t + u < t1;
            const int tt = on ? t + u : t;
            const T* p = proj + (size_t)tt * proj_stride + R + g * K;
            if (dt_raw) {
                dt[u] = on ? dt_raw[(size_t)tt * I + c] : 0.f;
            } else {                                   // (single-token steps: the product is summed here, no launch for it)
                const bool vec8 = ((proj_stride | R) & 7) == 0 && ((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(wrow)) & 15) == 0;
                dt[u] = step_size_product<T, G>(wrow, proj + (size_t)tt * proj_stride, R, g, vec8);
            }
            xv[u] = on ? to_float(x[(size_t)tt * I + c]) : 0.f;
            zv[u] = (EMIT && on) ? to_float(z[(size_t)tt * z_stride + c]) : 0.f;
            load_run<K>(p, bv[u], on ? n_mine : 0, vec);
            if (EMIT) load_run<K>(p + S, cv[u], on ? n_mine : 0, vec);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) dt[u] = softplus_for<T>(dt[u] + bias);
        float out[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            out[u] = 0.f;
            if (t + u < t1) {
                const float dx = dt[u] * xv[u];
                total += dt[u];
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    h[k] = exp_for<T>(dt[u] * a[k]) * h[k] + dx * bv[u][k];
                    if (EMIT) out[u] += h[k] * cv[u][k];
                }
            }
        }
        if (EMIT) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float s = out[u];
#pragma unroll
                for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (g == 0 && live && t + u < t1) y[(size_t)(t + u) * I + c] = from_float<T>((s + dsk * xv[u]) * silu_for<T>(zv[u]));
            }
        }
    }
    if (sum_dt) *sum_dt = total;
}

// a lane's K states from / to memory (16 bytes a time where the run is aligned)
template <int K>
__device__ __forceinline__ void state_io(float* st, float (&h)[K], int n_valid, bool store) {
    if (K % 4 == 0 && n_valid == K && (reinterpret_cast<uintptr_t>(st) & 15) == 0) {
#pragma unroll
        for (int k = 0; k < K; k += 4) {
            float4* p = reinterpret_cast<float4*>(st + k);
            if (store) *p = make_float4(h[k], h[k + 1], h[k + 2], h[k + 3]);
            else { const float4 v = *p; h[k] = v.x; h[k + 1] = v.y; h[k + 2] = v.z; h[k + 3] = v.w; }
        }
    } else {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            if (k < n_valid) { if (store) st[k] = h[k]; else h[k] = st[k]; }
            else if (!store) h[k] = 0.f;
        }
    }
}

// ---- one pass: a block walks one request's rows (U = 1: every request brings one token)
template <typename T, int K, int G, int U>
__global__ void __launch_bounds__(128) selective_scan_kernel(
    T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ proj, int proj_stride, const T* __restrict__ z,
    int z_stride, const float* __restrict__ dt_raw, const T* __restrict__ w_dt, const float* __restrict__ b_dt,
    const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state, const int* __restrict__ cu_q,
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
    const int n_mine = max(min(S - g * K, K), 0);
    float* st = state + ((size_t)slot * I + c) * S + g * K;
    float h[K], a[K];
    state_io<K>(st, h, n_mine, false);
#pragma unroll
    for (int k = 0; k < K; ++k) a[k] = k < n_mine ? -expf(a_log[(size_t)c * S + g * K + k]) : 0.f;
    scan_walk<T, K, G, true, U, false>(h, a, start, end, c, g, live, y, x, proj, proj_stride, z, z_stride, dt_raw,
                                       w_dt + (size_t)c * R, b_dt[c], d_skip[c], I, S, R, nullptr);
    if (write_state && live) state_io<K>(st, h, n_mine, true);
}

// ---- three passes.  ends [chunks, I, S]: a chunk's end state from zero, then (after pass 2) its start state;
// sums [chunks, I]: its summed step sizes.
template <typename T, int K, int G, bool EMIT>
__global__ void __launch_bounds__(128) selective_scan_chunk_kernel(
    T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ proj, int proj_stride, const T* __restrict__ z,
    int z_stride, const float* __restrict__ dt_raw, const float* __restrict__ b_dt, const float* __restrict__ a_log,
    const float* __restrict__ d_skip, float* __restrict__ ends, float* __restrict__ sums, const int* __restrict__ cu_q,
    int n_seqs, int Lc, int I, int S, int R) {
    pdl_trigger();
    pdl_wait();
    int seq, t0, t1;
    if (!zai_find_chunk(cu_q, n_seqs, Lc, blockIdx.x, seq, t0, t1)) return;
    const int g = threadIdx.x % G;
    int c = blockIdx.y * (128 / G) + threadIdx.x / G;
    const bool live = c < I;
    if (!live) c = I - 1;
    const int n_mine = max(min(S - g * K, K), 0);
    float* e = ends + ((size_t)blockIdx.x * I + c) * S + g * K;
    float h[K], a[K];
    if (EMIT) state_io<K>(e, h, n_mine, false);
#pragma unroll
    for (int k = 0; k < K; ++k) {
        if (!EMIT) h[k] = 0.f;
        a[k] = k < n_mine ? -expf(a_log[(size_t)c * S + g * K + k]) : 0.f;
    }
    float total = 0.f;
    scan_walk<T, K, G, EMIT, (K > 8 ? 2 : 4), true>(h, a, t0, t1, c, g, live, y, x, proj, proj_stride, z, z_stride, dt_raw,
                                                    (const T*)nullptr, b_dt[c], d_skip[c], I, S, R, &total);
    if (!EMIT && live) {
        state_io<K>(e, h, n_mine, true);
        if (g == 0) sums[(size_t)blockIdx.x * I + c] = total;
    }
}

// pass 2: one thread per (channel, state) carries the state across every request's chunks
__global__ void selective_scan_carry_kernel(float* __restrict__ ends, const float* __restrict__ sums,
                                            const float* __restrict__ a_log, float* __restrict__ state,
                                            const int* __restrict__ cu_q, const int* __restrict__ slot_ids, int n_seqs, int Lc,
                                            int I, int S, int write_state, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= I * S) return;
    const int c = idx / S;
    const float a = -expf(a_log[idx]);
    int chunk = 0;
    for (int s = 0; s < n_seqs; ++s) {
        const int len = cu_q[s + 1] - cu_q[s];
        if (len <= 0) continue;
        const int nc = (len + Lc - 1) / Lc;
        const int slot = zai_checked_slot(slot_ids[s], num_slots, status);
        float* st = state + (size_t)slot * I * S + idx;
        float h = *st;
        for (int j = 0; j < nc; ++j, ++chunk) {
            float* e = ends + (size_t)chunk * I * S + idx;
            const float h_in = h;
            h = expf(a * sums[(size_t)chunk * I + c]) * h + *e;
            *e = h_in;
        }
        if (write_state) *st = h;
    }
}

template <typename T, int K, int G>
static int launch_scan(void* y, const void* x, const void* proj, int proj_stride, const void* z, int z_stride, const float* dt_raw,
                       const void* w_dt, const float* b_dt, const float* a_log, const float* d_skip, float* state, const int* cu_q,
                       const int* slot_ids, int n_seqs, int I, int S, int R, int write_state, int num_slots, int* status,
                       float* ends, float* sums, int chunk, int max_chunks, int single_tokens, cudaStream_t stream) {
    const int per_block = 128 / G;
    const unsigned cb = (unsigned)((I + per_block - 1) / per_block);
    if (cb > 65535) return ZAI_BAD_SIZE;
    if (single_tokens)
        return launch_pdl(selective_scan_kernel<T, K, G, 1>, dim3(n_seqs, cb), dim3(128), 0, stream, (T*)y, (const T*)x,
                          (const T*)proj, proj_stride, (const T*)z, z_stride, dt_raw, (const T*)w_dt, b_dt, a_log, d_skip, state,
                          cu_q, slot_ids, I, S, R, write_state, num_slots, status);
    if (!dt_raw) return ZAI_BAD_SIZE;
    if (!ends || chunk <= 0)
        return launch_pdl(selective_scan_kernel<T, K, G, (K > 8 ? 2 : 4)>, dim3(n_seqs, cb), dim3(128), 0, stream, (T*)y,
                          (const T*)x, (const T*)proj, proj_stride, (const T*)z, z_stride, dt_raw, (const T*)w_dt, b_dt, a_log, d_skip,
                          state, cu_q, slot_ids, I, S, R, write_state, num_slots, status);
    int rc = launch_pdl(selective_scan_chunk_kernel<T, K, G, false>, dim3(max_chunks, cb), dim3(128), 0, stream, (T*)y,
                        (const T*)x, (const T*)proj, proj_stride, (const T*)z, z_stride, dt_raw, b_dt, a_log, d_skip, ends,
                        sums, cu_q, n_seqs, chunk, I, S, R);
    if (rc) return rc;
    rc = launch_pdl(selective_scan_carry_kernel, dim3((I * S + 127) / 128), dim3(128), 0, stream, ends, (const float*)sums, a_log,
                    state, cu_q, slot_ids, n_seqs, chunk, I, S, write_state, num_slots, status);
    if (rc) return rc;
    return launch_pdl(selective_scan_chunk_kernel<T, K, G, true>, dim3(max_chunks, cb), dim3(128), 0, stream, (T*)y, (const T*)x,
                      (const T*)proj, proj_stride, (const T*)z, z_stride, dt_raw, b_dt, a_log, d_skip, ends, sums, cu_q,
                      n_seqs, chunk, I, S, R);
}

// y [N, I]; x [N, I]; proj [N, proj_stride] (dt_in | B | C, of which B and C are read here); z [N, z_stride];
// dt_raw [N, I]: the products dt_in . w_dt^T in 32-bit (a matrix product made beforehand), or null in a step of single
// tokens, which then sums them from w_dt [I, R] itself; state [slots, I, S].
// With `ends` [max_chunks, I, S] and `sums` [max_chunks, I] (32-bit scratch) and chunk > 0 the step runs in three
// passes over chunks of `chunk` rows; max_chunks >= the number of chunks of the step (N / chunk + n_seqs covers it).
// single_tokens: every request brings one row (a leaner kernel).
ZAI_API int zai_selective_scan(void* y, const void* x, const void* proj, int proj_stride, const void* z, int z_stride, int dtype,
                               const float* dt_raw, const void* w_dt, const float* b_dt, const float* a_log, const float* d_skip,
                               float* state,
                               const int* cu_q, const int* slot_ids, int N, int n_seqs, int I, int S, int R, int write_state,
                               int num_slots, int* status, float* ends, float* sums, int chunk, int max_chunks,
                               int single_tokens, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0) return ZAI_OK;
    if (I < 1 || S < 1 || S > 256 || R < 1 || (!dt_raw && !w_dt)) return ZAI_BAD_SIZE;
#define ZAI_SCAN(KK, GG) ZAI_DISPATCH(dtype, return launch_scan<T, KK, GG>(y, x, proj, proj_stride, z, z_stride, dt_raw, w_dt, b_dt, a_log, \
        d_skip, state, cu_q, slot_ids, n_seqs, I, S, R, write_state, num_slots, status, ends, sums, chunk, max_chunks, \
        single_tokens && N == n_seqs, stream))
    if (S <= 4) ZAI_SCAN(4, 1);
    if (S <= 8) ZAI_SCAN(8, 1);
    if (S <= 16) ZAI_SCAN(16, 1);
    if (S <= 32) ZAI_SCAN(16, 2);
    if (S <= 64) ZAI_SCAN(16, 4);
    if (S <= 128) ZAI_SCAN(16, 8);
    ZAI_SCAN(16, 16);
#undef ZAI_SCAN
}
