// Layer norm with weight and bias, fused with the residual addition before it:
//   h += delta;  out = (h - mean(h)) * rsqrt(mean((h - mean(h))^2) + eps) * gamma + beta
// The residual stream h is 32-bit, and so are the sum, both means and the scaling; only `out` is rounded
// to the model's dtype.  The variance is the mean of the squared deviations (a second pass over the row,
// which the block keeps in registers or re-reads), not E[x^2] - E[x]^2.  The order of the reductions depends
// only on the row width, so a row's result does not depend on what else is in the batch.
#include "common.cuh"

__device__ __forceinline__ void ln_load4(const float* p, float (&d)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
}
__device__ __forceinline__ void ln_load4(const bf16* p, float (&d)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    d[0] = a.x; d[1] = a.y; d[2] = b.x; d[3] = b.y;
}
__device__ __forceinline__ void ln_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void ln_store4(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// Any width: the row is read again for the second mean and for the output.
template <typename T>
__global__ void add_layernorm_kernel(float* __restrict__ h, const T* __restrict__ delta, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, T* __restrict__ out, float eps, int H) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = h[base + c];
        if (delta) {
            v += to_float(delta[base + c]);
            h[base + c] = v;
        }
        s += v;
    }
    const float mean = block_sum(s, red) / (float)H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float d = h[base + c] - mean;
        ss += d * d;
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[base + c] = from_float<T>((h[base + c] - mean) * inv * gamma[c] + beta[c]);
}

// Rows with H a multiple of 4 and at most 4 * 256 * VEC: each thread keeps its 4 * VEC values in registers, so the
// row is read once.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) add_layernorm_vec_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                                                const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                T* __restrict__ out, float eps, int H) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float v[VEC][4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = (threadIdx.x + i * 256) * 4;
        v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
        if (c < H) {
            ln_load4(h + base + c, v[i]);
            if (delta) {
                float d[4];
                ln_load4(delta + base + c, d);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[i][e] += d[e];
                ln_store4(h + base + c, v[i][0], v[i][1], v[i][2], v[i][3]);
            }
            s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
        }
    }
    const float mean = block_sum(s, red) / (float)H;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = (threadIdx.x + i * 256) * 4;
        if (c < H) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v[i][e] -= mean;
                ss += v[i][e] * v[i][e];
            }
        }
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = (threadIdx.x + i * 256) * 4;
        if (c < H) {
            float g[4], b[4];
            ln_load4(gamma + c, g);
            ln_load4(beta + c, b);
            ln_store4(out + base + c, v[i][0] * inv * g[0] + b[0], v[i][1] * inv * g[1] + b[1], v[i][2] * inv * g[2] + b[2],
                      v[i][3] * inv * g[3] + b[3]);
        }
    }
}

// h [N, H] 32-bit (updated in place if delta is given), delta [N, H] in `dtype` or null, gamma and beta [H] 32-bit,
// out [N, H] in `dtype`.
ZAI_API int zai_add_layernorm(float* h, const void* delta, const float* gamma, const float* beta, void* out, int dtype,
                              float eps, int N, int H, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (H < 1) return ZAI_BAD_SIZE;
    if (H % 4 == 0 && H <= 4096) {
        if (H <= 1024) {
            ZAI_DISPATCH(dtype, return launch_pdl(add_layernorm_vec_kernel<T, 1>, dim3(N), dim3(256), 0, stream, h, (const T*)delta,
                                                  gamma, beta, (T*)out, eps, H));
        } else if (H <= 2048) {
            ZAI_DISPATCH(dtype, return launch_pdl(add_layernorm_vec_kernel<T, 2>, dim3(N), dim3(256), 0, stream, h, (const T*)delta,
                                                  gamma, beta, (T*)out, eps, H));
        } else {
            ZAI_DISPATCH(dtype, return launch_pdl(add_layernorm_vec_kernel<T, 4>, dim3(N), dim3(256), 0, stream, h, (const T*)delta,
                                                  gamma, beta, (T*)out, eps, H));
        }
    }
    ZAI_DISPATCH(dtype, return launch_pdl(add_layernorm_kernel<T>, dim3(N), dim3(256), 0, stream, h, (const T*)delta, gamma, beta,
                                          (T*)out, eps, H));
    return launch_status();
}
