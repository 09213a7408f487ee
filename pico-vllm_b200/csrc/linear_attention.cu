// Linear attention with one decay per head and a state per request, and the gated norm that follows it.
//
//   per head:  S_t = decay * S_(t-1) + k_t v_t^T   (S: [d, dv], float32, kept per request between steps)
//              o_t = S_t^T q_t
//   q, k, v are slices of a token's projection row, optionally passed through silu on the way in (float32).
//
// decay_linear_attention_kernel: the columns of S evolve independently of each other (column j needs k_t, q_t and the
// scalar v_t[j]), so a block takes 32 columns of one head of one segment, a warp four of them, and a lane the rows
// lane, lane + 32, ... of those four columns in registers.  The tokens of the segment are walked in order, eight at a
// time: their q and k (all rows) and v (the block's columns) are staged in shared memory as float32; per token a
// lane updates its 4 x DPL state elements and leaves its partial dot products in shared memory; after the eight
// tokens the lanes add the 32 partials of each (token, column) - no shuffle chain per token.  The state is stored
// transposed, [request slot, head, dv, d], so that a warp's loads and stores of a column are contiguous.
// Prompt portions and single tokens take this one kernel: a segment of one token is a decode step.  Long portions run as
// chunks side by side (three passes, below).
//
// gated_rms_norm_kernel: y = x / sqrt(mean(x^2) + eps) * w * sigmoid(g) over a whole row (all heads side by side),
// x float32, y in the activation type.
#include "common.cuh"

#define LA_TOK 8          // tokens staged at a time
#define LA_COLS 4         // columns of the state per warp
#define LA_WARPS 8

__device__ __forceinline__ float la_act(float z, int act) { return act == 1 ? z / (1.0f + expf(-z)) : z; }

// Long portions: the tokens of a segment are cut into chunks of `chunk` tokens that run side by side.
//   pass A (STATE_ONLY): every chunk from a zero state, no outputs: L_c = sum_j decay^(n_c-1-j) k_j v_j^T
//   pass B (scan):       S_0 = the request's state; start_c = S_c; S_(c+1) = decay^(n_c) S_c + L_c; the request's
//                        state becomes the last S.  L_c is replaced by start_c in place.
//   pass C:              every chunk again, from start_c, with outputs.
// Only the order of the float32 additions differs from the token-by-token walk.  With chunk == 0 a block walks its whole
// segment from the request's state and writes the state back (single tokens, short portions).
// Chunk c of segment s is block z = s * max_chunks + c; its place in `chunk_state` is (chunks of the segments before s) + c.
__device__ __forceinline__ int la_chunk_base(const int* __restrict__ cu_q, int seg, int chunk) {
    int base = 0;
    for (int s = 0; s < seg; ++s) base += (cu_q[s + 1] - cu_q[s] + chunk - 1) / chunk;
    return base;
}

template <typename TA, int DPL, bool STATE_ONLY>
__global__ void __launch_bounds__(LA_WARPS * 32)
decay_linear_attention_kernel(const TA* __restrict__ proj, int row_stride, int q_off, int k_off, int v_off,
                              const float* __restrict__ decay, float* __restrict__ state,
                              const int* __restrict__ seg_slots, const int* __restrict__ cu_q,
                              const int* __restrict__ positions, float* __restrict__ out, int H, int d, int dv, int act,
                              int chunk, int max_chunks, float* __restrict__ chunk_state) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float lsm[];
    const int dp = (d + 3) & ~3;
    float* qs = lsm;                                   // [LA_TOK][dp]
    float* ks = qs + LA_TOK * dp;                      // [LA_TOK][dp]
    float* vs = ks + LA_TOK * dp;                      // [LA_TOK][LA_WARPS * LA_COLS]
    float* part = vs + LA_TOK * LA_WARPS * LA_COLS;    // [LA_WARPS][LA_TOK][32][LA_COLS]
    const int seg = chunk > 0 ? blockIdx.z / max_chunks : blockIdx.z, ci = chunk > 0 ? blockIdx.z % max_chunks : 0;
    const int h = blockIdx.y, col_base = blockIdx.x * (LA_WARPS * LA_COLS);
    int t_begin = cu_q[seg], t_end = cu_q[seg + 1];
    if (t_end <= t_begin || positions[t_begin] < 0) return;      // an empty or a padding segment
    if (chunk > 0) {
        t_begin += ci * chunk;
        if (t_begin >= t_end) return;
        t_end = min(t_end, t_begin + chunk);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = col_base + warp * LA_COLS;
    const float a = decay[h];
    float* st = chunk > 0 ? chunk_state + ((size_t)(la_chunk_base(cu_q, seg, chunk) + ci) * H + h) * (size_t)dv * d
                          : state + ((size_t)seg_slots[seg] * H + h) * (size_t)dv * d;
    float S[DPL][LA_COLS];
#pragma unroll
    for (int r = 0; r < DPL; ++r)
#pragma unroll
        for (int c = 0; c < LA_COLS; ++c) {
            const int i = lane + 32 * r, j = col0 + c;
            S[r][c] = (!STATE_ONLY && i < d && j < dv) ? st[(size_t)j * d + i] : 0.f;
        }
    float* mypart = part + (size_t)warp * LA_TOK * 32 * LA_COLS;
    // The next eight tokens' q, k and v are asked for before the current eight are worked on and wait in registers
    // (thread x holds elements x, x + 256, ... of the [8][d] tiles, DPL of them, and one v): the trip to memory hides
    // behind the arithmetic instead of standing between two barriers.
    TA rq[DPL], rk[DPL], rv;
    auto fetch = [&](int t0) {
        const int nt = min(LA_TOK, t_end - t0);
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            const int idx = threadIdx.x + e * (LA_WARPS * 32);
            const int tt = idx / d, i = idx - tt * d;
            if (tt < nt) {
                const TA* row = proj + (size_t)(t0 + tt) * row_stride + (size_t)h * d + i;
                if (!STATE_ONLY) rq[e] = row[q_off];
                rk[e] = row[k_off];
            }
        }
        const int tt = threadIdx.x / (LA_WARPS * LA_COLS), j = col_base + threadIdx.x % (LA_WARPS * LA_COLS);
        if (tt < nt && j < dv) rv = proj[(size_t)(t0 + tt) * row_stride + v_off + (size_t)h * dv + j];
    };
    fetch(t_begin);
    for (int t0 = t_begin; t0 < t_end; t0 += LA_TOK) {
        const int nt = min(LA_TOK, t_end - t0);
        __syncthreads();                               // everyone is done with the tokens before
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            const int idx = threadIdx.x + e * (LA_WARPS * 32);
            const int tt = idx / d, i = idx - tt * d;
            if (tt < nt) {
                if (!STATE_ONLY) qs[tt * dp + i] = la_act(to_f32(rq[e]), act);
                ks[tt * dp + i] = la_act(to_f32(rk[e]), act);
            }
        }
        {
            const int tt = threadIdx.x / (LA_WARPS * LA_COLS), j = col_base + threadIdx.x % (LA_WARPS * LA_COLS);
            if (tt < nt) vs[threadIdx.x] = j < dv ? la_act(to_f32(rv), act) : 0.f;
        }
        __syncthreads();
        if (t0 + LA_TOK < t_end) fetch(t0 + LA_TOK);
        for (int tt = 0; tt < nt; ++tt) {
            const float4 v4 = *reinterpret_cast<const float4*>(vs + tt * LA_WARPS * LA_COLS + warp * LA_COLS);
            const float vv[LA_COLS] = {v4.x, v4.y, v4.z, v4.w};
            float p[LA_COLS] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < DPL; ++r) {
                const int i = lane + 32 * r;
                const float kk = i < d ? ks[tt * dp + i] : 0.f;
                const float qq = (!STATE_ONLY && i < d) ? qs[tt * dp + i] : 0.f;
#pragma unroll
                for (int c = 0; c < LA_COLS; ++c) {
                    S[r][c] = fmaf(a, S[r][c], kk * vv[c]);
                    if (!STATE_ONLY) p[c] = fmaf(S[r][c], qq, p[c]);
                }
            }
            if (!STATE_ONLY)
                *reinterpret_cast<float4*>(mypart + ((size_t)tt * 32 + lane) * LA_COLS) = make_float4(p[0], p[1], p[2], p[3]);
        }
        if (!STATE_ONLY) {
            __syncwarp();
            // lane -> (token lane / 4, column lane % 4): the sum of the 32 lanes' partials, read in a rotated order so that
            // the 32 reads of a step fall into 32 banks
            const int tt = lane >> 2, c = lane & 3;
            if (tt < nt) {
                float acc = 0.f;
#pragma unroll 8
                for (int l = 0; l < 32; ++l) acc += mypart[((size_t)tt * 32 + ((l + tt) & 31)) * LA_COLS + c];
                const int j = col0 + c;
                if (j < dv) out[(size_t)(t0 + tt) * ((size_t)H * dv) + (size_t)h * dv + j] = acc;
            }
            __syncwarp();
        }
    }
    if (STATE_ONLY || chunk == 0) {
#pragma unroll
        for (int r = 0; r < DPL; ++r)
#pragma unroll
            for (int c = 0; c < LA_COLS; ++c) {
                const int i = lane + 32 * r, j = col0 + c;
                if (i < d && j < dv) st[(size_t)j * d + i] = S[r][c];
            }
    }
}

// Pass B: a thread per state element of one (segment, head); walks the segment's chunks in order.
__global__ void __launch_bounds__(256)
decay_linear_scan_kernel(const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ seg_slots,
                         const int* __restrict__ cu_q, const int* __restrict__ positions, int H, int per_head, int chunk,
                         float* __restrict__ chunk_state) {
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int t_begin = cu_q[seg], t_end = cu_q[seg + 1];
    if (e >= per_head || t_end <= t_begin || positions[t_begin] < 0) return;
    const int n_chunks = (t_end - t_begin + chunk - 1) / chunk;
    const float a = decay[h];
    float a_full = 1.f;                                 // decay^chunk by repeated multiplication, as the token walk does
    for (int i = 0; i < chunk; ++i) a_full *= a;
    float* sp = state + ((size_t)seg_slots[seg] * H + h) * (size_t)per_head + e;
    float* cs = chunk_state + ((size_t)la_chunk_base(cu_q, seg, chunk) * H + h) * (size_t)per_head + e;
    const int n_last = t_end - t_begin - (n_chunks - 1) * chunk;
    float a_last = 1.f;
    for (int i = 0; i < n_last; ++i) a_last *= a;
    const size_t step = (size_t)H * per_head;
    float S = *sp;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {          // the loads of eight chunks are in flight together
        float local[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) local[k] = c0 + k < n_chunks ? cs[(size_t)(c0 + k) * step] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (c0 + k < n_chunks) {
                cs[(size_t)(c0 + k) * step] = S;
                S = fmaf(c0 + k == n_chunks - 1 ? a_last : a_full, S, local[k]);
            }
    }
    *sp = S;
}

// proj: [T, row_stride] rows; a token's q of head h at q_off + h*d, k at k_off + h*d, v at v_off + h*dv.  decay float32
// [H]; state float32 [slots, H, dv, d]; seg_slots int32 [S]; cu_q int32 [S + 1]; positions int32 [T] (a segment whose
// first position is negative is padding and is skipped); out float32 [T, H * dv].  act: 0 none, 1 silu.
// chunk > 0: the chunked form, for max_q_len (the longest segment) tokens; chunk_state float32 with room for
// (T / chunk + S) x H x dv x d elements.
PICO_API int pico_decay_linear_attention(const void* proj, int row_stride, int q_off, int k_off, int v_off,
                                         const float* decay, float* state, const int* seg_slots, const int* cu_q,
                                         const int* positions, float* out, int S, int H, int d, int dv, int act,
                                         int chunk, int max_q_len, float* chunk_state, int dtype, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || d < 1 || d > 256 || dv < 1 || (act != 0 && act != 1)) return PICO_ERR_SIZE;
    if (chunk < 0 || (chunk > 0 && (!chunk_state || max_q_len < 1))) return PICO_ERR_SIZE;
    const int max_chunks = chunk > 0 ? (max_q_len + chunk - 1) / chunk : 1;
    if ((long long)S * max_chunks > 65535) return PICO_ERR_SIZE;
    const int dpl = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8;
    const int dp = (d + 3) & ~3;
    const size_t smem = ((size_t)2 * LA_TOK * dp + LA_TOK * LA_WARPS * LA_COLS + (size_t)LA_WARPS * LA_TOK * 32 * LA_COLS) * sizeof(float);
    const dim3 grid((dv + LA_WARPS * LA_COLS - 1) / (LA_WARPS * LA_COLS), H, S * max_chunks);
#define LA_LAUNCH(TA, DPL, SO)                                                                                           \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(decay_linear_attention_kernel<TA, DPL, SO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                             \
        pico_launch((decay_linear_attention_kernel<TA, DPL, SO>), grid, dim3(LA_WARPS * 32), smem, stream,               \
                    (const TA*)proj, row_stride, q_off, k_off, v_off, decay, state, seg_slots, cu_q, positions, out, H, d, \
                    dv, act, chunk, max_chunks, chunk_state);                                                            \
    } while (0)
#define LA_BY_DPL(TA, SO)                                                                                                \
    do {                                                                                                                 \
        if (dpl == 1) LA_LAUNCH(TA, 1, SO); else if (dpl == 2) LA_LAUNCH(TA, 2, SO); else if (dpl == 4) LA_LAUNCH(TA, 4, SO); \
        else LA_LAUNCH(TA, 8, SO);                                                                                       \
    } while (0)
    if (dtype != PICO_F32 && dtype != PICO_BF16) return PICO_ERR_DTYPE;
    if (chunk > 0) {
        if (dtype == PICO_F32) LA_BY_DPL(float, true); else LA_BY_DPL(bf16, true);
        const int per_head = d * dv;
        pico_launch(decay_linear_scan_kernel, dim3((per_head + 255) / 256, H, S), dim3(256), 0, stream, decay, state, seg_slots,
                    cu_q, positions, H, per_head, chunk, chunk_state);
    }
    if (dtype == PICO_F32) LA_BY_DPL(float, false); else LA_BY_DPL(bf16, false);
#undef LA_BY_DPL
#undef LA_LAUNCH
    return pico_launch_status();
}

// A block per row.  x float32 [T, N]; w float32 [N] or nullptr; g (gate logits, activation type) in rows of g_stride
// elements, or nullptr; y [T, N] in the activation type.
template <typename TA>
__global__ void __launch_bounds__(256) gated_rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             const TA* __restrict__ g, int g_stride, float eps,
                                                             TA* __restrict__ y, int N) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const size_t t = blockIdx.x;
    const float* row = x + t * N;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss += row[i] * row[i];
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float v = row[i] * inv * (w ? w[i] : 1.0f);
        if (g) v /= 1.0f + expf(-to_f32(g[t * g_stride + i]));
        y[t * N + i] = from_f32<TA>(v);
    }
}

PICO_API int pico_gated_rms_norm(const float* x, const float* w, const void* g, int g_stride, float eps, void* y, int T,
                                 int N, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N < 1) return PICO_ERR_SIZE;
    const int threads = N >= 1024 ? 256 : 128;
    if (dtype == PICO_F32)
        pico_launch((gated_rms_norm_kernel<float>), dim3(T), dim3(threads), 0, stream, x, w, (const float*)g, g_stride, eps,
                    (float*)y, N);
    else if (dtype == PICO_BF16)
        pico_launch((gated_rms_norm_kernel<bf16>), dim3(T), dim3(threads), 0, stream, x, w, (const bf16*)g, g_stride, eps,
                    (bf16*)y, N);
    else
        return PICO_ERR_DTYPE;
    return pico_launch_status();
}
