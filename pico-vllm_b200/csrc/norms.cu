// Norm -> residual add -> norm in one pass over a row, for layers that norm a sublayer's output before it
// is added to the residual stream and norm the stream again for the next sublayer.
//
//   d' = N_post(d)            (optional; N_post is an RMS norm or a mean-centred norm with a weight)
//   x  = x + d'               (float32 residual stream, written back unless rows are picked)
//   y  = N(x)                 (optional; the same two kinds)
//
// RMS:      u / sqrt(mean(u^2) + eps) * w
// centred:  (u - mean u) / sqrt(mean((u - mean u)^2) + eps) * w     (two passes over the row held in
//           shared memory: the mean first, then the mean of the squared deviations)
// All arithmetic in float32; d and y are in the activation type.
#include "common.cuh"

enum { NORM_NONE = 0, NORM_RMS = 1, NORM_CENTRED = 2 };

// Normalises vals[0..H) in place (every thread of the block takes part); w may be nullptr (no weight).
__device__ __forceinline__ void norm_row_inplace(float* vals, int H, int kind, const float* __restrict__ w, float eps,
                                                 float* scratch) {
    float mean = 0.f;
    if (kind == NORM_CENTRED) {
        float s = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) s += vals[i];
        mean = block_sum(s, scratch) / (float)H;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = vals[i] - mean;
        ss += d * d;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) vals[i] = (vals[i] - mean) * inv * (w ? w[i] : 1.f);
}

template <typename TA>
__global__ void post_add_norm_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                     const float* __restrict__ post_w, int post_kind, float post_eps,
                                     const float* __restrict__ w, int kind, float eps, TA* __restrict__ out,
                                     const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float vals[];  // H floats, then 33 of scratch
    float* scratch = vals + H;
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    if (delta) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) vals[i] = to_f32(delta[src + i]);
        if (post_kind != NORM_NONE) {
            __syncthreads();
            norm_row_inplace(vals, H, post_kind, post_w, post_eps, scratch);
        }
        // each thread touches the same elements in every loop: no barrier needed between them
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = x[src + i] + vals[i];
            if (!rows) x[src + i] = v;
            vals[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) vals[i] = x[src + i];
    }
    if (!out || kind == NORM_NONE) return;
    __syncthreads();
    norm_row_inplace(vals, H, kind, w, eps, scratch);
    TA* dst = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_f32<TA>(vals[i]);
}

// x float32 [*, H]; delta [*, H] or nullptr; out [R, H] or nullptr; rows int32 [R] or nullptr.
PICO_API int pico_post_add_norm(float* x, const void* delta, const float* post_w, int post_kind, float post_eps,
                                const float* w, int kind, float eps, void* out, const int* rows, int R, int H,
                                int act_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (post_kind < 0 || post_kind > 2 || kind < 0 || kind > 2) return PICO_ERR_SIZE;
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return PICO_ERR_SIZE;
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 2048) threads = 128;
    else if (H > 4096) threads = 512;
#define LAUNCH_PAN(TA)                                                                                                  \
    do {                                                                                                                \
        if (smem > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(post_add_norm_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        pico_launch((post_add_norm_kernel<TA>), dim3(R), dim3(threads), smem, stream, x, (const TA*)delta, post_w,      \
                    post_kind, post_eps, w, kind, eps, (TA*)out, rows, H);                                              \
    } while (0)
    if (act_dtype == PICO_F32) LAUNCH_PAN(float);
    else if (act_dtype == PICO_BF16) LAUNCH_PAN(bf16);
    else return PICO_ERR_DTYPE;
#undef LAUNCH_PAN
    return pico_launch_status();
}

// ---------------------------------------------------------------- logits: scale and soft cap
// y = y * scale, then y = cap * tanh(y / cap) when cap > 0.  In place on float32 logits [R, V] (row stride given).
__global__ void scale_softcap_kernel(float* __restrict__ y, int V, int row_stride, size_t total, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / V;
        float* p = y + r * (size_t)row_stride + (idx - r * V);
        float v = *p * scale;
        if (cap > 0.f) v = cap * tanhf(v / cap);
        *p = v;
    }
}

PICO_API int pico_scale_softcap(float* y, int R, int V, int row_stride, float scale, float cap, cudaStream_t stream) {
    if (R <= 0 || V <= 0) return 0;
    const size_t total = (size_t)R * V;
    const long long cap_blocks = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap_blocks ? cap_blocks : (long long)want);
    pico_launch(scale_softcap_kernel, dim3(blocks), dim3(256), 0, stream, y, V, row_stride, total, scale, cap);
    return pico_launch_status();
}
