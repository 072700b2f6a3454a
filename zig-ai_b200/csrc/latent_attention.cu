// Causal attention of many heads over one shared cached vector per position (latent attention with the key and
// value expansions folded into the query and the output):
//
//   cached row j = [c_j (R values) | r_j (Dr values)]          pages [num_pages, page_size, R + Dr]
//   s_j = (q_lat . c_j + q_rot . r_j) * scale                  for cached positions j <= pos, same request
//   o   = sum_j softmax(s)_j c_j                               [R] per row and head
//
// A block owns one row of the step and up to LA_WARPS heads (one warp a head).  The cached rows are brought into
// shared memory 32 at a time, once for all heads of the block, as 32-bit values; lane j of every warp scores key j
// (rows are padded by one word, so the lanes read different banks), the warp keeps an online softmax, and every lane
// sums its share of the output dimensions.  Scores, weights and sums are 32-bit.  Keys are always visited from
// position 0 in steps of 32, so a row's result does not depend on how the request was cut into steps or on its batch.
#include "common.cuh"

#define LA_WARPS 8
#define LA_KEYS 32

template <typename T, int MAXR>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(
    T* __restrict__ out, const T* __restrict__ q_lat, const T* __restrict__ q_rot, const T* __restrict__ pages,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ positions, const int* __restrict__ seq_idx,
    int page_size, int H, int R, int Dr, float scale, int num_pages, int* __restrict__ status) {
    extern __shared__ float smem[];
    const int W = R + Dr, WP = W + 1;
    float* qs = smem;                                   // [LA_WARPS][W]  the block's queries, scaled
    float* ks = smem + (size_t)LA_WARPS * W;            // [LA_KEYS][WP]  a tile of cached rows
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y * LA_WARPS + warp;
    const bool live = h < H;
    const int pos = positions[t];
    const ZaiTableRow table{block_table + (size_t)seq_idx[t] * table_width, table_width, num_pages, status};
    if (live) {
        const T* a = q_lat + ((size_t)t * H + h) * R;
        const T* b = q_rot + ((size_t)t * H + h) * Dr;
        float* q = qs + (size_t)warp * W;
        for (int d = lane; d < R; d += 32) q[d] = to_float(a[d]) * scale;
        for (int d = lane; d < Dr; d += 32) q[R + d] = to_float(b[d]) * scale;
    }
    const int kend = pos + 1;
    float m = -INFINITY, l = 0.f;
    float acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
    for (int base = 0; base < kend; base += LA_KEYS) {
        const int n = min(LA_KEYS, kend - base);
        __syncthreads();                                // the tile before this one has been read by every warp
        for (int j = warp; j < n; j += LA_WARPS) {
            const int key = base + j;
            const int page = table.page(key / page_size);
            const T* src = pages + ((size_t)page * page_size + key % page_size) * W;
            float* dst = ks + (size_t)j * WP;
            for (int d = lane; d < W; d += 32) dst[d] = to_float(src[d]);
        }
        __syncthreads();
        if (!live) continue;
        const float* q = qs + (size_t)warp * W;
        float s = -INFINITY;
        if (lane < n) {
            const float* k = ks + (size_t)lane * WP;
            float d0 = 0.f, d1 = 0.f;
            int d = 0;
            for (; d + 1 < W; d += 2) {
                d0 += q[d] * k[d];
                d1 += q[d + 1] * k[d + 1];
            }
            if (d < W) d0 += q[d] * k[d];
            s = d0 + d1;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = lane < n ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);             // m = -inf at first: 0
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] *= corr;
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* v = ks + (size_t)jj * WP;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int d = lane + 32 * r;
                if (d < R) acc[r] += pj * v[d];
            }
        }
        m = m_new;
    }
    if (!live) return;
    const float inv = 1.f / l;
    T* orow = out + ((size_t)t * H + h) * R;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < R) orow[d] = from_float<T>(acc[r] * inv);
    }
}

template <typename T, int MAXR>
static int launch_latent(void* out, const void* q_lat, const void* q_rot, const void* pages, const int* block_table, int table_width,
                         const int* positions, const int* seq_idx, int page_size, int N, int H, int R, int Dr, float scale,
                         int num_pages, int* status, cudaStream_t stream) {
    const int W = R + Dr;
    const size_t smem = ((size_t)LA_WARPS * W + (size_t)LA_KEYS * (W + 1)) * sizeof(float);
    static unsigned long long done = 0;
    if (smem > 48 * 1024 && zai_first_on_device(&done))
        cudaFuncSetAttribute(latent_attention_kernel<T, MAXR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return launch_pdl(latent_attention_kernel<T, MAXR>, dim3(N, (H + LA_WARPS - 1) / LA_WARPS), dim3(LA_WARPS * 32), smem, stream,
                      (T*)out, (const T*)q_lat, (const T*)q_rot, (const T*)pages, block_table, table_width, positions, seq_idx,
                      page_size, H, R, Dr, scale, num_pages, status);
}

// out [N, H, R], q_lat [N, H, R], q_rot [N, H, Dr], pages [num_pages, page_size, R + Dr], all in `dtype`.
ZAI_API int zai_latent_attention(void* out, const void* q_lat, const void* q_rot, const void* pages, int dtype, const int* block_table,
                                 int table_width, const int* positions, const int* seq_idx, int page_size, int N, int H, int R,
                                 int Dr, float scale, int num_pages, int* status, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (H < 1 || R < 1 || R > 1024 || Dr < 0 || H > 65535 * LA_WARPS) return ZAI_BAD_SIZE;
    if (((size_t)LA_WARPS * (R + Dr) + (size_t)LA_KEYS * (R + Dr + 1)) * sizeof(float) > 200 * 1024) return ZAI_BAD_SIZE;
#define LA_GO(MAXR)                                                                                                            \
    ZAI_DISPATCH(dtype, return (launch_latent<T, MAXR>(out, q_lat, q_rot, pages, block_table, table_width, positions, seq_idx, \
                                                       page_size, N, H, R, Dr, scale, num_pages, status, stream)))
    if (R <= 128) LA_GO(4);
    else if (R <= 256) LA_GO(8);
    else if (R <= 512) LA_GO(16);
    else LA_GO(32);
#undef LA_GO
    return launch_status();
}
