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

enum { NORM_NONE = 0, NORM_RMS = 1, NORM_CENTRED = 2, NORM_COPY = 3 };   // COPY: no norm, but the row is written out in the activation type

// Four elements of the activation type from / to memory in one access.
template <typename TA> struct Row4;
template <> struct Row4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Row4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// Normalises vals[0..H) in place (every thread of the block takes part); w may be nullptr (no weight).  A thread
// touches the same elements in every loop of this file (element i, or with VEC the four elements of vector i, for
// i = thread, thread + threads, ...), so loops over the row need no barrier between them.
template <bool VEC>
__device__ __forceinline__ void norm_row_inplace(float* vals, int H, int kind, const float* __restrict__ w, float eps,
                                                 float* scratch) {
    const int n = VEC ? H >> 2 : H;
    float mean = 0.f;
    if (kind == NORM_CENTRED) {
        float s = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            if (VEC) {
                const float4 v = *reinterpret_cast<const float4*>(vals + 4 * i);
                s += (v.x + v.y) + (v.z + v.w);
            } else {
                s += vals[i];
            }
        }
        mean = block_sum(s, scratch) / (float)H;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (VEC) {
            const float4 v = *reinterpret_cast<const float4*>(vals + 4 * i);
            const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
            ss += (a * a + b * b) + (c * c + d * d);
        } else {
            const float d = vals[i] - mean;
            ss += d * d;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll 4
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (VEC) {
            float4 v = *reinterpret_cast<const float4*>(vals + 4 * i);
            const float4 g = w ? *reinterpret_cast<const float4*>(w + 4 * i) : make_float4(1.f, 1.f, 1.f, 1.f);
            v.x = (v.x - mean) * inv * g.x;
            v.y = (v.y - mean) * inv * g.y;
            v.z = (v.z - mean) * inv * g.z;
            v.w = (v.w - mean) * inv * g.w;
            *reinterpret_cast<float4*>(vals + 4 * i) = v;
        } else {
            vals[i] = (vals[i] - mean) * inv * (w ? w[i] : 1.f);
        }
    }
}

// VEC: H is a multiple of 4 and every access moves four elements.  The loops that read global memory write shared
// memory only, and the residual stream is written back in a loop of its own: the loads of a row are all in flight
// together instead of waiting for one another (a row is a few accesses per thread, each a trip to DRAM).
template <typename TA, bool VEC>
__global__ void post_add_norm_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                     const float* __restrict__ post_w, int post_kind, float post_eps,
                                     const float* __restrict__ w, int kind, float eps, TA* __restrict__ out,
                                     const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float vals[];  // H floats, then 33 of scratch
    float* scratch = vals + ((H + 3) & ~3);
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    const int n = VEC ? H >> 2 : H;
    if (delta) {
#pragma unroll 4
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            if (VEC) *reinterpret_cast<float4*>(vals + 4 * i) = Row4<TA>::load(delta + src + 4 * i);
            else vals[i] = to_f32(delta[src + i]);
        }
        if (post_kind != NORM_NONE) norm_row_inplace<VEC>(vals, H, post_kind, post_w, post_eps, scratch);
#pragma unroll 4
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            if (VEC) {
                float4 v = *reinterpret_cast<const float4*>(vals + 4 * i);
                const float4 a = *reinterpret_cast<const float4*>(x + src + 4 * i);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                *reinterpret_cast<float4*>(vals + 4 * i) = v;
            } else {
                vals[i] += x[src + i];
            }
        }
        if (!rows) {
#pragma unroll 4
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                if (VEC) *reinterpret_cast<float4*>(x + src + 4 * i) = *reinterpret_cast<const float4*>(vals + 4 * i);
                else x[src + i] = vals[i];
            }
        }
    } else {
#pragma unroll 4
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            if (VEC) *reinterpret_cast<float4*>(vals + 4 * i) = *reinterpret_cast<const float4*>(x + src + 4 * i);
            else vals[i] = x[src + i];
        }
    }
    if (!out || kind == NORM_NONE) return;
    if (kind != NORM_COPY) norm_row_inplace<VEC>(vals, H, kind, w, eps, scratch);
    else __syncthreads();
    TA* dst = out + (size_t)r * H;
#pragma unroll 4
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (VEC) Row4<TA>::store(dst + 4 * i, *reinterpret_cast<const float4*>(vals + 4 * i));
        else dst[i] = from_f32<TA>(vals[i]);
    }
}

// The same work with a warp per row and the row in registers (H a multiple of 4, at most 128 * VPL elements): every
// load of a row - what is added and the stream - is issued before anything is waited for, the sums
// go through shuffles, and nothing passes through shared memory or a block barrier.  Four rows a block.
template <int VPL>
__device__ __forceinline__ void norm_regs(float4 (&v)[VPL], const float* __restrict__ w, int n4, int lane, int H, int kind,
                                          float eps) {
    float mean = 0.f;
    if (kind == NORM_CENTRED) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < VPL; ++k)
            if (lane + 32 * k < n4) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        mean = warp_sum(s) / (float)H;
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k)
        if (lane + 32 * k < n4) {
            const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
            ss += (a * a + b * b) + (c * c + d * d);
        }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)H + eps);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {     // the weights are shared by all rows: these loads hit the caches
        const float4 g = w && lane + 32 * k < n4 ? *reinterpret_cast<const float4*>(w + 4 * (lane + 32 * k))
                                                 : make_float4(1.f, 1.f, 1.f, 1.f);
        v[k].x = (v[k].x - mean) * inv * g.x;
        v[k].y = (v[k].y - mean) * inv * g.y;
        v[k].z = (v[k].z - mean) * inv * g.z;
        v[k].w = (v[k].w - mean) * inv * g.w;
    }
}

template <typename TA, int VPL>
__global__ void __launch_bounds__(128) post_add_norm_warp_kernel(float* __restrict__ x, const TA* __restrict__ delta,
                                                                 const float* __restrict__ post_w, int post_kind,
                                                                 float post_eps, const float* __restrict__ w, int kind,
                                                                 float eps, TA* __restrict__ out,
                                                                 const int* __restrict__ rows, int R, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= R) return;
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    const int n4 = H >> 2;
    const bool norm_out = out && kind != NORM_NONE;
    const bool norm_in = delta && post_kind != NORM_NONE;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 d[VPL], a[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const int i = lane + 32 * k;
        const bool ok = i < n4;
        d[k] = ok && delta ? Row4<TA>::load(delta + src + 4 * i) : zero;
        a[k] = ok ? *reinterpret_cast<const float4*>(x + src + 4 * i) : zero;
    }
    if (norm_in) norm_regs<VPL>(d, post_w, n4, lane, H, post_kind, post_eps);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        a[k].x += d[k].x; a[k].y += d[k].y; a[k].z += d[k].z; a[k].w += d[k].w;
        if (delta && !rows && lane + 32 * k < n4) *reinterpret_cast<float4*>(x + src + 4 * (lane + 32 * k)) = a[k];
    }
    if (!norm_out) return;
    if (kind != NORM_COPY) norm_regs<VPL>(a, w, n4, lane, H, kind, eps);
    TA* dst = out + (size_t)r * H;
#pragma unroll
    for (int k = 0; k < VPL; ++k)
        if (lane + 32 * k < n4) Row4<TA>::store(dst + 4 * (lane + 32 * k), a[k]);
}

template <typename TA>
static void launch_pan_warp(int vpl, dim3 grid, cudaStream_t stream, float* x, const void* delta, const float* post_w,
                            int post_kind, float post_eps, const float* w, int kind, float eps, void* out, const int* rows,
                            int R, int H) {
#define PAN_WARP(V)                                                                                                       \
    pico_launch((post_add_norm_warp_kernel<TA, V>), grid, dim3(128), 0, stream, x, (const TA*)delta, post_w, post_kind,    \
                post_eps, w, kind, eps, (TA*)out, rows, R, H)
    if (vpl <= 1) PAN_WARP(1);
    else if (vpl <= 2) PAN_WARP(2);
    else if (vpl <= 4) PAN_WARP(4);
    else if (vpl <= 6) PAN_WARP(6);
    else if (vpl <= 8) PAN_WARP(8);
    else if (vpl <= 12) PAN_WARP(12);
    else PAN_WARP(16);
#undef PAN_WARP
}

// x float32 [*, H]; delta [*, H] or nullptr; out [R, H] or nullptr; rows int32 [R] or nullptr.
PICO_API int pico_post_add_norm(float* x, const void* delta, const float* post_w, int post_kind, float post_eps,
                                const float* w, int kind, float eps, void* out, const int* rows, int R, int H,
                                int act_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (post_kind < 0 || post_kind > 2 || kind < 0 || kind > 3) return PICO_ERR_SIZE;
    if (act_dtype != PICO_F32 && act_dtype != PICO_BF16) return PICO_ERR_DTYPE;
    if (H % 4 == 0 && H <= 2048) {       // a warp per row, the row in registers
        const int vpl = (H / 4 + 31) / 32;
        const dim3 grid((R + 3) / 4);
        if (act_dtype == PICO_F32)
            launch_pan_warp<float>(vpl, grid, stream, x, delta, post_w, post_kind, post_eps, w, kind, eps, out, rows, R, H);
        else
            launch_pan_warp<bf16>(vpl, grid, stream, x, delta, post_w, post_kind, post_eps, w, kind, eps, out, rows, R, H);
        return pico_launch_status();
    }
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (smem > 200 * 1024) return PICO_ERR_SIZE;
    int threads = 256;
    if (H <= 256) threads = 64;
    else if (H <= 2048) threads = 128;
    else if (H > 4096) threads = 512;
#define LAUNCH_PAN(TA, V4)                                                                                                \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(post_add_norm_kernel<TA, V4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        pico_launch((post_add_norm_kernel<TA, V4>), dim3(R), dim3(threads), smem, stream, x, (const TA*)delta, post_w,    \
                    post_kind, post_eps, w, kind, eps, (TA*)out, rows, H);                                                \
    } while (0)
    const bool v4 = H % 4 == 0;
    if (act_dtype == PICO_F32) {
        if (v4) LAUNCH_PAN(float, true); else LAUNCH_PAN(float, false);
    } else if (act_dtype == PICO_BF16) {
        if (v4) LAUNCH_PAN(bf16, true); else LAUNCH_PAN(bf16, false);
    } else
        return PICO_ERR_DTYPE;
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
