// Minimal gated recurrence (minGRU): gates that read only the current token, one state value per channel,
// carried in 32-bit between steps:
//
//   z = sigmoid(zr + bz)      u = xr + bx      cand = u + 1/2 (u >= 0),  sigmoid(u) (u < 0)
//   s <- (1 - z) * s + z * cand                 out = s * silu(gr)
//
// zr, xr, gr are the three column blocks of one projection [N, 3W].  One thread per (request, channel)
// walks the request's rows in order, eight at a time (the gates of the eight do not depend on the state).
// Gates, candidate and state are 32-bit; `out` is rounded to the model's dtype.
#include "common.cuh"

#define ZAI_GRU_U 8             // tokens whose gates are in flight together

// Walks rows [t0, t1) of one request for channel c from state s; EMIT writes out.  `decay` (if not null)
// receives the product of (1 - z) over the rows.
template <typename T, bool EMIT>
__device__ __forceinline__ float min_gru_walk(float s, int t0, int t1, int c, T* __restrict__ out, const T* __restrict__ zxg,
                                              int in_stride, float b_z, float b_x, int W, float* decay) {
    float prod = 1.f;
    for (int t = t0; t < t1; t += ZAI_GRU_U) {
        float zr[ZAI_GRU_U], u[ZAI_GRU_U], gr[ZAI_GRU_U];
#pragma unroll
        for (int i = 0; i < ZAI_GRU_U; ++i) {
            const T* row = zxg + (size_t)min(t + i, t1 - 1) * in_stride;
            zr[i] = to_float(row[c]) + b_z;
            u[i] = to_float(row[W + c]) + b_x;
            gr[i] = EMIT ? to_float(row[2 * W + c]) : 0.f;
        }
        float z[ZAI_GRU_U], zc[ZAI_GRU_U];
#pragma unroll
        for (int i = 0; i < ZAI_GRU_U; ++i) {
            z[i] = 1.f / (1.f + expf(-zr[i]));
            zc[i] = z[i] * (u[i] >= 0.f ? u[i] + 0.5f : 1.f / (1.f + expf(-u[i])));
            if (EMIT) gr[i] = gr[i] / (1.f + expf(-gr[i]));
        }
#pragma unroll
        for (int i = 0; i < ZAI_GRU_U; ++i) {
            if (t + i < t1) {
                s = (1.f - z[i]) * s + zc[i];
                prod *= 1.f - z[i];
                if (EMIT) out[(size_t)(t + i) * W + c] = from_float<T>(s * gr[i]);
            }
        }
    }
    if (decay) *decay = prod;
    return s;
}

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
    const float s = min_gru_walk<T, true>(state[(size_t)slot * W + c], start, end, c, out, zxg, in_stride, bz ? bz[c] : 0.f,
                                          bx ? bx[c] : 0.f, W, nullptr);
    if (write_state) state[(size_t)slot * W + c] = s;
}

// ---- long portions in three passes over chunks of Lc rows (the recurrence is linear in the state): every chunk
// from a zero state (its end value and its decay), the carry across a request's chunks, every chunk again
// from its start value.  ends, decays: [chunks, W] 32-bit scratch.
__device__ __forceinline__ bool zai_find_chunk(const int* __restrict__ cu_q, int n_seqs, int Lc, int b, int& seq, int& t0, int& t1) {
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

template <typename T, bool EMIT>
__global__ void min_gru_chunk_kernel(T* __restrict__ out, const T* __restrict__ zxg, int in_stride, const float* __restrict__ bz,
                                     const float* __restrict__ bx, float* __restrict__ ends, float* __restrict__ decays,
                                     const int* __restrict__ cu_q, int n_seqs, int Lc, int W) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    int seq, t0, t1;
    if (c >= W || !zai_find_chunk(cu_q, n_seqs, Lc, blockIdx.x, seq, t0, t1)) return;
    const size_t at = (size_t)blockIdx.x * W + c;
    float decay;
    const float s = min_gru_walk<T, EMIT>(EMIT ? ends[at] : 0.f, t0, t1, c, out, zxg, in_stride, bz ? bz[c] : 0.f,
                                          bx ? bx[c] : 0.f, W, &decay);
    if (!EMIT) {
        ends[at] = s;
        decays[at] = decay;
    }
}

__global__ void min_gru_carry_kernel(float* __restrict__ ends, const float* __restrict__ decays, float* __restrict__ state,
                                     const int* __restrict__ cu_q, const int* __restrict__ slot_ids, int n_seqs, int Lc, int W,
                                     int write_state, int num_slots, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    int chunk = 0;
    for (int s = 0; s < n_seqs; ++s) {
        const int len = cu_q[s + 1] - cu_q[s];
        if (len <= 0) continue;
        const int nc = (len + Lc - 1) / Lc;
        const int slot = zai_checked_slot(slot_ids[s], num_slots, status);
        float h = state[(size_t)slot * W + c];
        for (int j = 0; j < nc; ++j, ++chunk) {
            const size_t at = (size_t)chunk * W + c;
            const float h_in = h;
            h = decays[at] * h + ends[at];
            ends[at] = h_in;
        }
        if (write_state) state[(size_t)slot * W + c] = h;
    }
}

ZAI_API int zai_min_gru(void* out, const void* zxg, int in_stride, int dtype, const float* bz, const float* bx, float* state,
                        const int* cu_q, const int* slot_ids, int N, int n_seqs, int W, int write_state, int num_slots,
                        int* status, float* ends, float* decays, int chunk, int max_chunks, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0 || W <= 0) return ZAI_OK;
    const int threads = 128;
    const unsigned cb = (unsigned)((W + threads - 1) / threads);
    if (cb > 65535) return ZAI_BAD_SIZE;
    if (!ends || chunk <= 0) {
        ZAI_DISPATCH(dtype, return launch_pdl(min_gru_kernel<T>, dim3(n_seqs, cb), dim3(threads), 0, stream, (T*)out, (const T*)zxg,
            in_stride, bz, bx, state, cu_q, slot_ids, W, write_state, num_slots, status));
    }
    int rc;
    ZAI_DISPATCH(dtype, rc = launch_pdl(min_gru_chunk_kernel<T, false>, dim3(max_chunks, cb), dim3(threads), 0, stream, (T*)out,
        (const T*)zxg, in_stride, bz, bx, ends, decays, cu_q, n_seqs, chunk, W));
    if (rc) return rc;
    rc = launch_pdl(min_gru_carry_kernel, dim3(cb), dim3(threads), 0, stream, ends, (const float*)decays, state, cu_q, slot_ids,
                    n_seqs, chunk, W, write_state, num_slots, status);
    if (rc) return rc;
    ZAI_DISPATCH(dtype, return launch_pdl(min_gru_chunk_kernel<T, true>, dim3(max_chunks, cb), dim3(threads), 0, stream, (T*)out,
        (const T*)zxg, in_stride, bz, bx, ends, decays, cu_q, n_seqs, chunk, W));
}
