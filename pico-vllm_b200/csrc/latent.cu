// Kernels of the latent-attention mixer: what stands between its matrix products.
//
// A token's down projection row holds, side by side, the query latent (q_rank), the key/value latent
// (kv_rank; absent in a layer that reads another layer's cache) and one gate logit per head.
// latent_norm_store_kernel, one block per token:
//   c_q  = u_q / sqrt(mean(u_q^2) + eps) * w_q                -> cq [T, q_rank]       (activation type)
//   c    = u_kv / sqrt(mean(u_kv^2) + eps) * w_kv             -> the token's cache row (cache type), zero
//                                                                beyond kv_rank up to the row's width
//   gate = 1 / (1 + exp(-u_g))                                -> gate [T, heads]      (float32)
// All arithmetic in float32.  A token whose slot is negative stores nothing (padding rows).
//
// head_scale_kernel: o[t, h, :] *= gate[t, h]  (the per-head output gate).
#include "common.cuh"

template <typename TA>
__global__ void latent_norm_store_kernel(const TA* __restrict__ proj, int proj_stride, int q_off, int q_rank,
                                         const float* __restrict__ wq, TA* __restrict__ cq, int kv_off, int kv_rank,
                                         const float* __restrict__ wkv, const int* __restrict__ slots,
                                         TA* __restrict__ cache, int cache_row, int g_off, int heads,
                                         float* __restrict__ gate, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const TA* row = proj + (size_t)t * proj_stride;
    {   // query latent
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_f32(row[q_off + i]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq[(size_t)t * q_rank + i] = from_f32<TA>(to_f32(row[q_off + i]) * inv * wq[i]);
    }
    if (kv_rank > 0) {   // key/value latent into its cache row
        const int slot = slots ? slots[t] : -1;     // the same for every thread of the block
        if (slot >= 0) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
                const float v = to_f32(row[kv_off + i]);
                ss += v * v;
            }
            ss = block_sum(ss, scratch);
            const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
            TA* dst = cache + (size_t)slot * cache_row;
            for (int i = threadIdx.x; i < cache_row; i += blockDim.x)
                dst[i] = i < kv_rank ? from_f32<TA>(to_f32(row[kv_off + i]) * inv * wkv[i]) : from_f32<TA>(0.f);
        }
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x)
        gate[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-to_f32(row[g_off + h])));
}

// proj [T, >= all offsets] with row stride proj_stride; cq [T, q_rank]; cache rows of cache_row elements
// (>= kv_rank); slots int32 [T] or nullptr with kv_rank 0; gate float32 [T, heads].
PICO_API int pico_latent_norm_store(const void* proj, int proj_stride, int q_off, int q_rank, const float* wq, void* cq,
                                    int kv_off, int kv_rank, const float* wkv, const int* slots, void* cache,
                                    int cache_row, int g_off, int heads, float* gate, float eps, int T, int dtype,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (q_rank <= 0 || heads <= 0 || kv_rank < 0 || (kv_rank > 0 && (cache_row < kv_rank || !cache || !wkv)))
        return PICO_ERR_SIZE;
    const int widest = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = widest <= 128 ? 64 : (widest <= 1024 ? 128 : 256);
    if (dtype == PICO_F32)
        pico_launch((latent_norm_store_kernel<float>), dim3(T), dim3(threads), 0, stream, (const float*)proj, proj_stride,
                    q_off, q_rank, wq, (float*)cq, kv_off, kv_rank, wkv, slots, (float*)cache, cache_row, g_off, heads,
                    gate, eps);
    else if (dtype == PICO_BF16)
        pico_launch((latent_norm_store_kernel<bf16>), dim3(T), dim3(threads), 0, stream, (const bf16*)proj, proj_stride,
                    q_off, q_rank, wq, (bf16*)cq, kv_off, kv_rank, wkv, slots, (bf16*)cache, cache_row, g_off, heads,
                    gate, eps);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

template <typename TA>
__global__ void head_scale_kernel(TA* __restrict__ o, const float* __restrict__ gate, int head_width, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        o[idx] = from_f32<TA>(to_f32(o[idx]) * gate[idx / head_width]);
}

// o [T, heads * head_width] contiguous, gate float32 [T, heads]: o[t, h, :] *= gate[t, h].
PICO_API int pico_head_scale(void* o, const float* gate, int T, int heads, int head_width, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || head_width <= 0) return PICO_ERR_SIZE;
    const size_t total = (size_t)T * heads * head_width;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_F32)
        pico_launch((head_scale_kernel<float>), dim3(blocks), dim3(256), 0, stream, (float*)o, gate, head_width, total);
    else if (dtype == PICO_BF16)
        pico_launch((head_scale_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (bf16*)o, gate, head_width, total);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
