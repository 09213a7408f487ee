// Per-head RMS norm of queries and keys, rotary position encoding on the first rot_dim dimensions of every
// head, and the store of keys and values into cache pages, one kernel.
//
//   row of a token: [ q heads (nh x hd) | k heads (nkv x hd) | v heads (nkv x hd, absent when the values are the keys) ]
//   u  = row + bias                                                     (float32 from here on)
//   v  = the v head of the row, or - values_from_keys - the k head u itself, before norm and rotation
//   u' = u / sqrt(mean(u^2) + eps) * w_q (or w_k), one weight of hd elements shared by the heads  (skipped without weights);
//        the mean is over norm_dim <= hd elements: a head padded with zeros to the next size the attention kernels take
//   dims i and i + rot_dim/2 (i < rot_dim/2) turn by the angle position * inv_freq[i]; cos and sin are multiplied
//   by `mult` (a position scaling's attention factor; 1 without); dims from rot_dim on pass unchanged
//   q' is written back in place; k' and v go to their pages and are not written back.
//
// A block per token; its warps take the heads in turn, a lane holds dims lane, lane + 32, ... (hd <= 256).
// Angles, sines, the norm and the rotation are float32 whatever the storage type.
#include "common.cuh"

#define QKN_MAX_DPL 8

template <typename TA>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_kernel(TA* __restrict__ qkv, int row_stride, const float* __restrict__ bias,
                          const int* __restrict__ positions, const float* __restrict__ inv_freq, float mult,
                          const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                          const int* __restrict__ slots, TA* __restrict__ k_pages, TA* __restrict__ v_pages, int nh,
                          int nkv, int hd, int norm_dim, int rot_half, int page_size, int values_from_keys) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float qsm[];          // cos[rot_half], sin[rot_half], then hd floats per warp
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;                    // a padding row
    float* cs = qsm;
    for (int i = threadIdx.x; i < rot_half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c * mult;
        cs[rot_half + i] = s * mult;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* mine = qsm + 2 * rot_half + warp * hd;
    TA* row = qkv + (size_t)t * row_stride;
    const int slot = slots ? slots[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    const int rot_dim = 2 * rot_half;
    const int heads = nh + (slot >= 0 ? nkv : 0);
    for (int head = warp; head < heads; head += nwarps) {
        const bool is_q = head < nh;
        const int kh = head - nh;
        const int c0 = head * hd;
        float u[QKN_MAX_DPL];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < QKN_MAX_DPL; ++j) {
            const int d = lane + 32 * j;
            u[j] = 0.f;
            if (d < hd) {
                u[j] = to_f32(row[c0 + d]) + (bias ? bias[c0 + d] : 0.f);
                ss += u[j] * u[j];
            }
        }
        TA* kdst = is_q ? nullptr : k_pages + (((size_t)page * nkv + kh) * page_size + off) * hd;
        if (!is_q && values_from_keys) {
            TA* vdst = v_pages + (((size_t)page * nkv + kh) * page_size + off) * hd;
#pragma unroll
            for (int j = 0; j < QKN_MAX_DPL; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) vdst[d] = from_f32<TA>(u[j]);
            }
        }
        const float* w = is_q ? q_w : k_w;
        if (w) {
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)norm_dim + eps);
#pragma unroll
            for (int j = 0; j < QKN_MAX_DPL; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) u[j] = u[j] * inv * w[d];
            }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < QKN_MAX_DPL; ++j) {
            const int d = lane + 32 * j;
            if (d < hd) mine[d] = u[j];
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < QKN_MAX_DPL; ++j) {
            const int d = lane + 32 * j;
            if (d >= hd) continue;
            float y = u[j];
            if (d < rot_half) y = u[j] * cs[d] - mine[d + rot_half] * cs[rot_half + d];
            else if (d < rot_dim) y = u[j] * cs[d - rot_half] + mine[d - rot_half] * cs[d];
            if (is_q) row[c0 + d] = from_f32<TA>(y);
            else kdst[d] = from_f32<TA>(y);
        }
    }
    if (slot >= 0 && !values_from_keys) {
        const int v0 = (nh + nkv) * hd;
        for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
            const int kh = idx / hd, d = idx - kh * hd;
            const float v = to_f32(row[v0 + idx]) + (bias ? bias[v0 + idx] : 0.f);
            v_pages[(((size_t)page * nkv + kh) * page_size + off) * hd + d] = from_f32<TA>(v);
        }
    }
}

// qkv: [T, row_stride] rows as described above; bias float32 over the q, k (and v) columns or nullptr; q_w, k_w float32
// [hd] or nullptr (no norm); inv_freq float32 [rot_dim / 2]; slots int32 [T] (page * page_size + offset, -1: no store)
// or nullptr (only q is treated); pages [num_pages, nkv, page_size, hd].
PICO_API int pico_qk_norm_rope_store(void* qkv, int row_stride, const float* bias, const int* positions,
                                     const float* inv_freq, float mult, const float* q_w, const float* k_w, float eps,
                                     const int* slots, void* k_pages, void* v_pages, int T, int nh, int nkv, int hd,
                                     int norm_dim, int rot_dim, int page_size, int values_from_keys, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd < 1 || hd > 32 * QKN_MAX_DPL || rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || nh < 1 || nkv < 0 || norm_dim < 1 ||
        norm_dim > hd)
        return PICO_ERR_SIZE;
    const int heads = nh + nkv;
    const int warps = heads < 8 ? heads : 8;
    const size_t smem = ((size_t)rot_dim + (size_t)warps * hd) * sizeof(float);
    if (dtype == PICO_F32)
        pico_launch((qk_norm_rope_store_kernel<float>), dim3(T), dim3(warps * 32), smem, stream, (float*)qkv, row_stride,
                    bias, positions, inv_freq, mult, q_w, k_w, eps, slots, (float*)k_pages, (float*)v_pages, nh, nkv, hd,
                    norm_dim, rot_dim / 2, page_size, values_from_keys);
    else if (dtype == PICO_BF16)
        pico_launch((qk_norm_rope_store_kernel<bf16>), dim3(T), dim3(warps * 32), smem, stream, (bf16*)qkv, row_stride,
                    bias, positions, inv_freq, mult, q_w, k_w, eps, slots, (bf16*)k_pages, (bf16*)v_pages, nh, nkv, hd,
                    norm_dim, rot_dim / 2, page_size, values_from_keys);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}

// o[t, c] *= sigmoid(g[t, c]) for c < n: an output gate whose logits lie in rows of their own stride (a slice of a wider
// projection buffer), float32 inside.
template <typename TA>
__global__ void sigmoid_gate_kernel(TA* __restrict__ o, const TA* __restrict__ g, int g_stride, int n, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int c = (int)(idx - t * n);
        const float z = to_f32(g[t * g_stride + c]);
        o[idx] = from_f32<TA>(to_f32(o[idx]) / (1.0f + expf(-z)));
    }
}

PICO_API int pico_sigmoid_gate(void* o, const void* g, int g_stride, int T, int n, int dtype, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    const size_t total = (size_t)T * n;
    const long long cap = 16LL * pico_num_sms();
    const size_t want = (total + 255) / 256;
    const int blocks = (int)((long long)want > cap ? cap : (long long)want);
    if (dtype == PICO_F32)
        pico_launch((sigmoid_gate_kernel<float>), dim3(blocks), dim3(256), 0, stream, (float*)o, (const float*)g, g_stride, n, total);
    else if (dtype == PICO_BF16)
        pico_launch((sigmoid_gate_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (bf16*)o, (const bf16*)g, g_stride, n, total);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
