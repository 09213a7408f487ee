// Linear attention with one decay per head and a state per request, and the gated norm that follows it.
//
//   per head:  S_t = decay * S_(t-1) + k_t v_t^T   (S: [d, dv], float32, kept per request between steps)
//              o_t = S_t^T q_t
//   q, k, v are slices of a token's projection row, optionally passed through silu on the way in (float32).
//
// decay_linear_attention_kernel: the columns of S evolve independently of each other (column j needs k_t, q_t and the
// scalar v_t[j]), so a block takes 64 columns of one head of one segment, a warp eight of them, and a lane the rows
// lane, lane + 32, ... of those eight columns in registers.  The tokens of the segment are walked in order, eight at a
// time: their q and k (all rows) and v (the block's columns) are staged in shared memory as float32; per token a
// lane updates its 8 x DPL state elements and leaves its partial dot products in shared memory; after the eight
// tokens the lanes add the 32 partials of each (token, column) - no shuffle chain per token.  The state is stored
// transposed, [request slot, head, dv, d], so that a warp's loads and stores of a column are contiguous.
// Prompt portions and single tokens take this one kernel: a segment of one token is a decode step.  Long portions run as
// chunks side by side (three passes, below).
//
// gated_rms_norm_kernel: y = x / sqrt(mean(x^2) + eps) * w * sigmoid(g) over a whole row (all heads side by side),
// x float32, y in the activation type; a warp per row.
#include "common.cuh"

#define LA_TOK 8          // tokens staged at a time
#define LA_COLS 8         // columns of the state per warp
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

// EXACT: d == 32 * DPL and dv is a multiple of the block's columns: no element of a tile lies outside.
template <typename TA, int DPL, bool STATE_ONLY, bool EXACT>
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
            S[r][c] = (!STATE_ONLY && (EXACT || (i < d && j < dv))) ? st[(size_t)j * d + i] : 0.f;
        }
    float* mypart = part + (size_t)warp * LA_TOK * 32 * LA_COLS;
    // The next eight tokens' q, k and v are asked for before the current eight are worked on and wait in registers
    // (thread x holds elements x, x + 256, ... of the [8][d] tiles, DPL of them, and one v): the trip to memory hides
    // behind the arithmetic instead of standing between two barriers.
    constexpr int NV = LA_TOK * LA_COLS / 32;           // v elements of the [8][block's columns] tile per thread
    TA rq[DPL], rk[DPL], rv[NV];
    int e_tt[DPL], e_src[DPL], e_dst[DPL];             // which token and element of the tiles this thread carries: the same every round
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
        const int idx = threadIdx.x + e * (LA_WARPS * 32);
        e_tt[e] = idx / d;
        const int i = idx - e_tt[e] * d;
        e_src[e] = e_tt[e] * row_stride + h * d + i;
        e_dst[e] = e_tt[e] * dp + i;
    }
    auto fetch = [&](int t0) {
        const int nt = min(LA_TOK, t_end - t0);
        const TA* base = proj + (size_t)t0 * row_stride;
#pragma unroll
        for (int e = 0; e < DPL; ++e)
            if (e_tt[e] < nt) {
                if (!STATE_ONLY) rq[e] = base[e_src[e] + q_off];
                rk[e] = base[e_src[e] + k_off];
            }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = threadIdx.x + e * (LA_WARPS * 32);
            const int v_tt = idx / (LA_WARPS * LA_COLS), v_j = col_base + idx % (LA_WARPS * LA_COLS);
            if (v_tt < nt && (EXACT || v_j < dv)) rv[e] = base[v_tt * row_stride + v_off + h * dv + v_j];
        }
    };
    fetch(t_begin);
    for (int t0 = t_begin; t0 < t_end; t0 += LA_TOK) {
        const int nt = min(LA_TOK, t_end - t0);
        __syncthreads();                               // everyone is done with the tokens before
#pragma unroll
        for (int e = 0; e < DPL; ++e)
            if (e_tt[e] < nt) {
                if (!STATE_ONLY) qs[e_dst[e]] = la_act(to_f32(rq[e]), act);
                ks[e_dst[e]] = la_act(to_f32(rk[e]), act);
            }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = threadIdx.x + e * (LA_WARPS * 32);
            const int v_tt = idx / (LA_WARPS * LA_COLS), v_j = col_base + idx % (LA_WARPS * LA_COLS);
            if (v_tt < nt) vs[idx] = (EXACT || v_j < dv) ? la_act(to_f32(rv[e]), act) : 0.f;
        }
        __syncthreads();
        if (t0 + LA_TOK < t_end) fetch(t0 + LA_TOK);
        auto token = [&](int tt) {
            const float4 va = *reinterpret_cast<const float4*>(vs + tt * LA_WARPS * LA_COLS + warp * LA_COLS);
            const float4 vb = *reinterpret_cast<const float4*>(vs + tt * LA_WARPS * LA_COLS + warp * LA_COLS + 4);
            const float vv[LA_COLS] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
            float p[LA_COLS];
#pragma unroll
            for (int c = 0; c < LA_COLS; ++c) p[c] = 0.f;
#pragma unroll
            for (int r = 0; r < DPL; ++r) {
                const int i = lane + 32 * r;
                const float kk = (EXACT || i < d) ? ks[tt * dp + i] : 0.f;
                const float qq = (!STATE_ONLY && (EXACT || i < d)) ? qs[tt * dp + i] : 0.f;
#pragma unroll
                for (int c = 0; c < LA_COLS; ++c) {
                    S[r][c] = fmaf(a, S[r][c], kk * vv[c]);
                    if (!STATE_ONLY) p[c] = fmaf(S[r][c], qq, p[c]);
                }
            }
            if (!STATE_ONLY) {
                float* dst = mypart + ((size_t)tt * 32 + lane) * LA_COLS;
                *reinterpret_cast<float4*>(dst) = make_float4(p[0], p[1], p[2], p[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(p[4], p[5], p[6], p[7]);
            }
        };
        if (nt == LA_TOK) {
#pragma unroll
            for (int tt = 0; tt < LA_TOK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        if (!STATE_ONLY) {
            __syncwarp();
            // lane -> (tokens lane / 8 and lane / 8 + 4, column lane % 8): the sum of the 32 lanes' partials, read in a rotated
            // order so that the 32 reads of a step fall into 32 banks
            const int t4 = lane >> 3, c = lane & 7;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 8
            for (int l = 0; l < 32; ++l) {
                const int ll = (l + t4) & 31;
                acc0 += mypart[((size_t)t4 * 32 + ll) * LA_COLS + c];
                acc1 += mypart[((size_t)(t4 + 4) * 32 + ll) * LA_COLS + c];
            }
            const int j = col0 + c;
            if (EXACT || j < dv) {
                if (t4 < nt) out[(size_t)(t0 + t4) * ((size_t)H * dv) + (size_t)h * dv + j] = acc0;
                if (t4 + 4 < nt) out[(size_t)(t0 + t4 + 4) * ((size_t)H * dv) + (size_t)h * dv + j] = acc1;
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
                if (EXACT || (i < d && j < dv)) st[(size_t)j * d + i] = S[r][c];
            }
    }
}

// q, k and v of every token through the activation, once, as float32 rows [q heads | k heads | v heads]: the chunked
// form stages every token's q and k eight times (four column blocks, two passes) and would apply the activation each time.
template <typename TA>
__global__ void la_prepare_kernel(const TA* __restrict__ proj, int row_stride, int q_off, int k_off, int v_off, int nqk, int nv,
                                  int act, size_t total, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = 2 * nqk + nv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n;
        const int c = (int)(idx - t * n);
        const int src = c < nqk ? q_off + c : c < 2 * nqk ? k_off + (c - nqk) : v_off + (c - 2 * nqk);
        out[idx] = la_act(to_f32(proj[t * row_stride + src]), act);
    }
}

// The same for bfloat16 rows with 16-byte loads: a thread takes eight neighbouring columns (every offset, size and stride a
// multiple of 8, so that the eight lie in one of q, k, v and on a 16-byte boundary).
__global__ void la_prepare_bf16x8_kernel(const bf16* __restrict__ proj, int row_stride, int q_off, int k_off, int v_off,
                                         int nqk, int nv, int act, size_t total8, float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int n8 = (2 * nqk + nv) / 8;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / n8;
        const int c = (int)(idx - t * n8) * 8;
        const int src = c < nqk ? q_off + c : c < 2 * nqk ? k_off + (c - nqk) : v_off + (c - 2 * nqk);
        const uint4 raw = *reinterpret_cast<const uint4*>(proj + t * row_stride + src);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float f[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 v = __bfloat1622float2(h2[k]);
            f[2 * k] = la_act(v.x, act);
            f[2 * k + 1] = la_act(v.y, act);
        }
        float4* dst = reinterpret_cast<float4*>(out + t * (size_t)(n8 * 8) + c);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
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
// (T / chunk + S) x H x dv x d elements; prepared (optional) float32 with room for T x H x (2 d + dv) elements.
PICO_API int pico_decay_linear_attention(const void* proj, int row_stride, int q_off, int k_off, int v_off,
                                         const float* decay, float* state, const int* seg_slots, const int* cu_q,
                                         const int* positions, float* out, int S, int H, int d, int dv, int act,
                                         int chunk, int max_q_len, float* chunk_state, float* prepared, int T, int dtype,
                                         cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H < 1 || H > 65535 || S > 65535 || d < 1 || d > 256 || dv < 1 || (act != 0 && act != 1)) return PICO_ERR_SIZE;
    if (chunk < 0 || (chunk > 0 && (!chunk_state || max_q_len < 1))) return PICO_ERR_SIZE;
    const int max_chunks = chunk > 0 ? (max_q_len + chunk - 1) / chunk : 1;
    if ((long long)S * max_chunks > 65535) return PICO_ERR_SIZE;
    const int dpl = d <= 32 ? 1 : d <= 64 ? 2 : d <= 128 ? 4 : 8;
    const int dp = (d + 3) & ~3;
    const bool exact = d == 32 * dpl && dv % (LA_WARPS * LA_COLS) == 0;
    const size_t smem = ((size_t)2 * LA_TOK * dp + LA_TOK * LA_WARPS * LA_COLS + (size_t)LA_WARPS * LA_TOK * 32 * LA_COLS) * sizeof(float);
    const dim3 grid((dv + LA_WARPS * LA_COLS - 1) / (LA_WARPS * LA_COLS), H, S * max_chunks);
#define LA_LAUNCH(TA, DPL, SO, EX)                                                                                       \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(decay_linear_attention_kernel<TA, DPL, SO, EX>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                             \
        pico_launch((decay_linear_attention_kernel<TA, DPL, SO, EX>), grid, dim3(LA_WARPS * 32), smem, stream,           \
                    (const TA*)proj, row_stride, q_off, k_off, v_off, decay, state, seg_slots, cu_q, positions, out, H, d, \
                    dv, act, chunk, max_chunks, chunk_state);                                                            \
    } while (0)
#define LA_BY_EX(TA, DPL, SO)                                                                                            \
    do {                                                                                                                 \
        if (exact) LA_LAUNCH(TA, DPL, SO, true); else LA_LAUNCH(TA, DPL, SO, false);                                     \
    } while (0)
#define LA_BY_DPL(TA, SO)                                                                                                \
    do {                                                                                                                 \
        if (dpl == 1) LA_BY_EX(TA, 1, SO); else if (dpl == 2) LA_BY_EX(TA, 2, SO); else if (dpl == 4) LA_BY_EX(TA, 4, SO); \
        else LA_BY_EX(TA, 8, SO);                                                                                        \
    } while (0)
    if (dtype != PICO_F32 && dtype != PICO_BF16) return PICO_ERR_DTYPE;
    if (chunk > 0 && prepared) {
        // the activation once, into float32 rows; the passes below then read those rows as they are
        const int nqk = H * d, nv = H * dv;
        const size_t total = (size_t)T * (2 * nqk + nv);
        const long long cap = 16LL * pico_num_sms();
        const size_t want = (total + 255) / 256;
        const int blocks = (int)((long long)want > cap ? cap : (long long)want);
        const bool vec8 = dtype == PICO_BF16 && nqk % 8 == 0 && nv % 8 == 0 && row_stride % 8 == 0 && q_off % 8 == 0 &&
                          k_off % 8 == 0 && v_off % 8 == 0 && ((uintptr_t)proj & 15) == 0 && ((uintptr_t)prepared & 15) == 0;
        if (dtype == PICO_F32)
            pico_launch((la_prepare_kernel<float>), dim3(blocks), dim3(256), 0, stream, (const float*)proj, row_stride, q_off,
                        k_off, v_off, nqk, nv, act, total, prepared);
        else if (vec8) {
            const size_t want8 = (total / 8 + 255) / 256;
            pico_launch(la_prepare_bf16x8_kernel, dim3((int)((long long)want8 > cap ? cap : (long long)want8)), dim3(256), 0, stream,
                        (const bf16*)proj, row_stride, q_off, k_off, v_off, nqk, nv, act, total / 8, prepared);
        } else
            pico_launch((la_prepare_kernel<bf16>), dim3(blocks), dim3(256), 0, stream, (const bf16*)proj, row_stride, q_off,
                        k_off, v_off, nqk, nv, act, total, prepared);
        proj = prepared;
        row_stride = 2 * nqk + nv;
        q_off = 0, k_off = nqk, v_off = 2 * nqk;
        act = 0;
        dtype = PICO_F32;
    }
    if (chunk > 0) {
        if (dtype == PICO_F32) LA_BY_DPL(float, true); else LA_BY_DPL(bf16, true);
        const int per_head = d * dv;
        pico_launch(decay_linear_scan_kernel, dim3((per_head + 255) / 256, H, S), dim3(256), 0, stream, decay, state, seg_slots,
                    cu_q, positions, H, per_head, chunk, chunk_state);
    }
    if (dtype == PICO_F32) LA_BY_DPL(float, false); else LA_BY_DPL(bf16, false);
#undef LA_BY_DPL
#undef LA_BY_EX
#undef LA_LAUNCH
    return pico_launch_status();
}

// A warp per row, eight rows a block: the row is read twice (the second time from the caches), every load of a pass is
// independent of the others, sums go through shuffles; no shared memory, no block barrier.  x float32 [T, N]; w float32 [N]
// or nullptr; g (gate logits, activation type) in rows of g_stride elements, or nullptr; y [T, N] in the activation type.
// VEC: N is a multiple of 4 and x rows are read as float4.
template <typename TA, bool VEC>
__global__ void __launch_bounds__(256) gated_rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             const TA* __restrict__ g, int g_stride, float eps,
                                                             TA* __restrict__ y, int T, int N) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t t = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= (size_t)T) return;
    const float* row = x + t * N;
    float ss = 0.f;
    if (VEC) {
#pragma unroll 4
        for (int i = lane * 4; i < N; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
    } else {
        for (int i = lane; i < N; i += 32) ss += row[i] * row[i];
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)N + eps);
    const TA* gr = g ? g + t * g_stride : nullptr;
    TA* yr = y + t * N;
    if (VEC) {
#pragma unroll 2
        for (int i = lane * 4; i < N; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            const float4 ww = w ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
            float o[4] = {v.x * inv * ww.x, v.y * inv * ww.y, v.z * inv * ww.z, v.w * inv * ww.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (gr) o[k] /= 1.0f + expf(-to_f32(gr[i + k]));
                yr[i + k] = from_f32<TA>(o[k]);
            }
        }
    } else {
        for (int i = lane; i < N; i += 32) {
            float v = row[i] * inv * (w ? w[i] : 1.0f);
            if (gr) v /= 1.0f + expf(-to_f32(gr[i]));
            yr[i] = from_f32<TA>(v);
        }
    }
}

// A block per row, every access four elements wide (N, g_stride and the pointers allow it): a thread's float4 loads of x
// and its loads of the gate logits and the weight are all asked for before anything is waited for - a row of a few
// thousand elements is one or two trips to memory, which is what a step of a handful of tokens is made of.
template <typename TA>
__global__ void __launch_bounds__(256) gated_rms_norm_row4_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                  const TA* __restrict__ g, int g_stride, float eps,
                                                                  TA* __restrict__ y, int N) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    constexpr int MAXV = 4;                              // float4 per thread: N <= 4 * 256 * MAXV
    const size_t t = blockIdx.x;
    const float* row = x + t * N;
    const TA* gr = g ? g + t * g_stride : nullptr;
    float4 v[MAXV], ww[MAXV], gg[MAXV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int i = (threadIdx.x + k * 256) * 4;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < N) {
            v[k] = *reinterpret_cast<const float4*>(row + i);
            ww[k] = w ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
            if (gr) gg[k] = make_float4(to_f32(gr[i]), to_f32(gr[i + 1]), to_f32(gr[i + 2]), to_f32(gr[i + 3]));
        }
        ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)N + eps);
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int i = (threadIdx.x + k * 256) * 4;
        if (i >= N) continue;
        float o[4] = {v[k].x * inv * ww[k].x, v[k].y * inv * ww[k].y, v[k].z * inv * ww[k].z, v[k].w * inv * ww[k].w};
        if (gr) {
            o[0] /= 1.0f + expf(-gg[k].x);
            o[1] /= 1.0f + expf(-gg[k].y);
            o[2] /= 1.0f + expf(-gg[k].z);
            o[3] /= 1.0f + expf(-gg[k].w);
        }
        TA* dst = y + t * N + i;
#pragma unroll
        for (int e = 0; e < 4; ++e) dst[e] = from_f32<TA>(o[e]);
    }
}

PICO_API int pico_gated_rms_norm(const float* x, const float* w, const void* g, int g_stride, float eps, void* y, int T,
                                 int N, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N < 1) return PICO_ERR_SIZE;
    const dim3 grid((T + 7) / 8);
    const bool vec = N % 4 == 0;
    if (vec && N <= 4096 && T <= 4096) {             // few rows: a block per row
        if (dtype == PICO_F32)
            pico_launch((gated_rms_norm_row4_kernel<float>), dim3(T), dim3(256), 0, stream, x, w, (const float*)g, g_stride, eps,
                        (float*)y, N);
        else if (dtype == PICO_BF16)
            pico_launch((gated_rms_norm_row4_kernel<bf16>), dim3(T), dim3(256), 0, stream, x, w, (const bf16*)g, g_stride, eps,
                        (bf16*)y, N);
        else
            return PICO_ERR_DTYPE;
        return pico_launch_status();
    }
#define GN_LAUNCH(TA, V)                                                                                              \
    pico_launch((gated_rms_norm_kernel<TA, V>), grid, dim3(256), 0, stream, x, w, (const TA*)g, g_stride, eps, (TA*)y, T, N)
    if (dtype == PICO_F32) {
        if (vec) GN_LAUNCH(float, true); else GN_LAUNCH(float, false);
    } else if (dtype == PICO_BF16) {
        if (vec) GN_LAUNCH(bf16, true); else GN_LAUNCH(bf16, false);
    } else
        return PICO_ERR_DTYPE;
#undef GN_LAUNCH
    return pico_launch_status();
}
