// Linear recurrences with a matrix state per request and head, carried from
// token to token in float32:
//
//   retention        S_t = decay_h S_{t-1} + k_t v_t^T                      o_t = S_t^T q_t
//   delta rule       S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T
//                                                                           o_t = S_t^T r_t
//   gated memory     m_t = max(f_t + m_{t-1}, i_t)   (m_0 = 0)
//                    S_t = e^(f_t + m_{t-1} - m_t) S_{t-1} + e^(i_t - m_t) k_t v_t^T,  n_t likewise with k_t alone
//                                        o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
//   wkv              o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_{t-1} + k_t v_t^T
//                    (the output reads the OLD state; the bonus u counts the current token only;
//                    w = exp(-exp(w_raw + w_bias)) per head, key channel and token)
//   state space     S_t = exp(-exp(A_h) dt_t) S_{t-1} + dt_t B_t x_t^T,   y_t = S_t^T C_t + D_h x_t
//                    (the selective state space recurrence in its dual, matrix-state form: x, B and C
//                    pass a short causal convolution and silu first; dt = softplus(dt_raw + bias); the
//                    heads of a group share B and C; then the gate silu(z), a root-mean-square division
//                    in equal parts of the row, a weight)
//
// S is [key dim, value dim].  Retention rotates q and k by the step's (cos, sin)
// table (pair (i, i + rot/2), the first `rot` dims) and scales k afterwards; its
// decay is one number per head.  The delta rule's decay and removal rate are per
// key channel and token: w = exp(-exp(-1/2) sigmoid(w_raw + w_bias)), a =
// sigmoid(a_raw + a_bias), u = k / sqrt(sum k^2 + 1e-6); both of its terms read the
// old state.  After the recurrence each head's o is divided by its root mean
// square (eps inside the root), optionally multiplied by a weight, gated by
// silu or sigmoid of a projection, scaled by out_scale and stored in the compute
// type for the output projection.
//
// The gated memory (the matrix memory of the xLSTM) has a log input gate i = cap tanh((x_i + b_i) / cap)
// and a log forget gate f = logsigmoid(cap tanh((x_f + b_f) / cap)) per head and token, q scaled by
// q_scale.  Its n is carried as one more value column of S whose value is 1 in every token, so that
// n_t . q_t is that column's output; the running maximum m is kept per head beside S (one copy per
// slice of value columns, so that the blocks of a head do not share a word).  The state of a slot is
// [heads][dim][v_dim + 4] (columns v_dim + 1 .. v_dim + 3 stay zero) followed by [heads][slices] of m.
//
// Everything that enters the recurrence is formed in float32 from the
// projections (which arrive in the compute type); the state never leaves float32.
//
// (The state space layer's convolution is a kernel of its own before them, and the inputs its slot keeps
// are written by one after them.)
// Three kernels per step.  (1) prepare: a warp per (token, head) forms the token's vectors in
// float32 (q/r, k, and for the delta rule w, a * u, u) in a workspace; fully parallel over the
// step's tokens.  (2) scan: a block per (entry, head, slice of 32 value columns) -- the columns
// of S evolve independently -- walks the entry's tokens in order; a thread owns one column and
// at most 32 key rows of it (every P-th row) in registers (P = 1, 2, 4, 8 or 16 threads per column, neighbours in a
// warp, their partial sums met by shuffles); the token vectors come through shared memory in
// batches.  The state is read from and written back to its slot once per launch; a decoded token
// is a batch of one.  (3) finish: a warp per (token, head) divides by the root mean square,
// applies weight, gate and scale and stores in the compute type.  The order of every sum depends
// on the sizes only.
#include "common.cuh"
#include <math.h>
#include <algorithm>

#ifndef KIPP_SSD_WIDE
#define KIPP_SSD_WIDE 1
#endif
namespace {
constexpr int MAX_CHUNK = 32;

struct ScanArgs {
    void* out; long long ld_out;           // [T, heads * v_dim] compute type
    const void* proj; long long ld_proj;   // [T, ...] compute type: the fused projections
    int q_off, k_off, v_off, g_off, a_off; // column offsets of r/q, k, v, gate, removal rate in proj
    const void* w_raw; long long ld_w;     // delta: [T, heads * dim] compute type
    const float* a_bias;                   // delta: [heads * dim]
    const float* w_bias;                   // delta: [heads * dim]
    const float* norm_w;                   // [heads * v_dim] or null
    const float* decay;                    // retention: [heads]
    const float* cos_sin; int rot;         // retention: [T, rot / 2, 2] or null
    float* state;                          // [slots, heads, dim, v_dim]
    const int* q_start; const int* slots;
    int heads, dim, v_dim, batch;
    float k_scale, eps, out_scale;
    int gate;                              // 0 none, 1 silu, 2 sigmoid
    // gated memory: columns of the two gates in proj, their biases [heads], the cap, the scale of q
    int i_off, f_off;
    const float* i_bias; const float* f_bias;
    float gate_cap, q_scale;
    long long slot_stride;                 // floats per slot of `state` (0: heads * dim * v_dim)
    const float* bonus;                    // wkv: u [heads * dim]
    // state space: columns of z, of the convolved channels [x: heads * v_dim | B: groups * dim | C: groups * dim]
    // and of dt in proj; the convolution [channels, taps] with its bias; per head dt's bias, A (as its
    // logarithm) and D; the slot keeps the last taps - 1 inputs of every channel behind S
    int z_off, xbc_off, dt_off, taps, groups, norm_groups;
    const float* conv_w; const float* conv_b;
    const float* dt_bias; const float* a_log; const float* d_skip;
    const int* entry_of_token;
};
enum { RETENTION = 0, DELTA_RULE = 1, GATED_MEMORY = 2, WKV = 3, SSD = 4 };
// vectors per token besides v, extra floats after them, extra value columns
template <int KIND> struct Rec {
    static constexpr int NV = KIND == DELTA_RULE ? 5 : KIND == WKV ? 3 : 2;     // wkv: r, k, w
    static constexpr int XG = KIND == GATED_MEMORY || KIND == WKV || KIND == SSD ? 4 : 0;   // (i, f, 0, 0), wkv's (sum u k r, 0, 0, 0) or the state space's (decay, dt, 0, 0), after the vectors
    static constexpr int XV = KIND == GATED_MEMORY ? 4 : 0;     // value columns (1, 0, 0, 0) after v
};
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// (1) the token vectors: one record of NV * D + V floats per (head, token), heads outermost so that
// a head's consecutive tokens are neighbours: NV = 5 (delta: r, k, w, a*u, u) or 2 (q, k), then v
template <typename T, int KIND>
__global__ void __launch_bounds__(128)
recurrent_prepare_kernel(const ScanArgs a, float* __restrict__ vec, int tokens) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr bool DELTA = KIND == DELTA_RULE;
    constexpr int NV = Rec<KIND>::NV, XG = Rec<KIND>::XG, XV = Rec<KIND>::XV;
    const int lane = threadIdx.x & 31;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)tokens * a.heads) return;
    const size_t row = (size_t)(wg / a.heads);
    const int h = (int)(wg % a.heads), D = a.dim;
    const T* pr = static_cast<const T*>(a.proj) + row * a.ld_proj;
    const int rec = NV * D + XG + a.v_dim + XV;
    float* dst = vec + ((size_t)h * tokens + row) * rec;
    for (int c = lane; c < a.v_dim; c += 32) dst[NV * D + XG + c] = to_f32(pr[a.v_off + h * a.v_dim + c]);
    if (KIND == GATED_MEMORY) {
        if (lane < XV) dst[NV * D + XG + a.v_dim + lane] = lane == 0 ? 1.f : 0.f;
        if (lane == 0) {
            const float cap = a.gate_cap;
            dst[NV * D] = cap * tanhf((to_f32(pr[a.i_off + h]) + a.i_bias[h]) / cap);
            dst[NV * D + 1] = log_sigmoid(cap * tanhf((to_f32(pr[a.f_off + h]) + a.f_bias[h]) / cap));
            dst[NV * D + 2] = 0.f;
            dst[NV * D + 3] = 0.f;
        }
        for (int d = lane; d < D; d += 32) {
            dst[d] = to_f32(pr[a.q_off + h * D + d]) * a.q_scale;
            dst[D + d] = to_f32(pr[a.k_off + h * D + d]);
        }
    } else if (KIND == WKV) {
        const T* w_raw = static_cast<const T*>(a.w_raw);
        float bonus = 0.f;
        for (int d = lane; d < D; d += 32) {
            const int c = h * D + d;
            const float r = to_f32(pr[a.q_off + c]), k = to_f32(pr[a.k_off + c]);
            const float wr = to_f32(w_raw[row * a.ld_w + c]) + a.w_bias[c];
            dst[d] = r;
            dst[D + d] = k;
            dst[2 * D + d] = expf(-expf(wr));
            bonus = fmaf(a.bonus[c] * k, r, bonus);
        }
        bonus = warp_sum(bonus);
        if (lane < XG) dst[NV * D + lane] = lane == 0 ? bonus : 0.f;
    } else if (DELTA) {
        const T* w_raw = static_cast<const T*>(a.w_raw);
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float k = to_f32(pr[a.k_off + h * D + d]);
            ss = fmaf(k, k, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + 1e-6f);
        for (int d = lane; d < D; d += 32) {
            const int c = h * D + d;
            const float k = to_f32(pr[a.k_off + c]);
            const float u = k * inv;
            const float rate = sigmoidf_(to_f32(pr[a.a_off + c]) + a.a_bias[c]);
            const float wr = to_f32(w_raw[row * a.ld_w + c]) + a.w_bias[c];
            dst[d] = to_f32(pr[a.q_off + c]);
            dst[D + d] = k;
            dst[2 * D + d] = expf(-0.6065306597126334f * sigmoidf_(wr));
            dst[3 * D + d] = rate * u;
            dst[4 * D + d] = u;
        }
    } else {
        const int half = a.rot / 2;
        const float2* cs = a.cos_sin ? reinterpret_cast<const float2*>(a.cos_sin) + row * half : nullptr;
        for (int d = lane; d < D; d += 32) {
            const int c = h * D + d;
            float q = to_f32(pr[a.q_off + c]), k = to_f32(pr[a.k_off + c]);
            if (cs != nullptr && d < a.rot) {
                const bool low = d < half;
                const float2 t = cs[low ? d : d - half];
                const float q2 = to_f32(pr[a.q_off + h * D + (low ? d + half : d - half)]);
                const float k2 = to_f32(pr[a.k_off + h * D + (low ? d + half : d - half)]);
                // low: u cos - v sin; high: v cos + u sin (u the low half, v the high one)
                q = low ? q * t.x - q2 * t.y : q * t.x + q2 * t.y;
                k = low ? k * t.x - k2 * t.y : k * t.x + k2 * t.y;
            }
            dst[d] = q;
            dst[D + d] = k * a.k_scale;
        }
    }
}

// (2) the recurrence; raw o goes to o_raw [T, heads * v_dim] float32.  The records of a batch of
// tokens come into shared memory by asynchronous copies, the next batch while this one is walked.
constexpr int VS = 32;                     // value columns per block
__device__ __forceinline__ void load_batch(float* __restrict__ tv, float* __restrict__ vv, const float* __restrict__ rec0,
                                           int rec, int nvd, int nb, int slice, int V, bool async, int threads) {
    // rec0: the record of the batch's first token; the vectors' part [nvd] and this slice's values
    if (async) {
        const int c4 = nvd / 4;
        for (int i = threadIdx.x; i < nb * c4; i += threads) {
            const int tt = i / c4, c = i % c4;
            cp_async16(smem_address(tv + (size_t)tt * nvd + c * 4), rec0 + (size_t)tt * rec + c * 4, 16);
        }
        for (int i = threadIdx.x; i < nb * (VS / 4); i += threads) {
            const int tt = i / (VS / 4), c = i % (VS / 4), col = slice * VS + c * 4;
            const bool ok = col < V;                    // V is a multiple of 4 here: a chunk is whole or absent
            cp_async16(smem_address(vv + (size_t)tt * VS + c * 4), ok ? rec0 + (size_t)tt * rec + nvd + col : rec0, ok ? 16 : 0);
        }
    } else {
        for (int i = threadIdx.x; i < nb * nvd; i += threads) tv[i] = rec0[(size_t)(i / nvd) * rec + i % nvd];
        for (int i = threadIdx.x; i < nb * VS; i += threads) {
            const int col = slice * VS + i % VS;
            vv[i] = col < V ? rec0[(size_t)(i / VS) * rec + nvd + col] : 0.f;
        }
    }
    cp_async_commit();
}

// VEC: the head's key size is a multiple of 4: a thread's rows come in groups of four neighbours
// (rows 4 (p + P g) .. + 3), read with one 16-byte load per vector.
template <typename T, int KIND, int P, int CHUNK, bool VEC>
__global__ void __launch_bounds__(VS * P)
recurrent_scan_kernel(const ScanArgs a, const float* __restrict__ vec, float* __restrict__ o_raw, int v_slices,
                      int tokens) {
    extern __shared__ __align__(16) float smem[];
    constexpr bool DELTA = KIND == DELTA_RULE;
    constexpr int NV = Rec<KIND>::NV;
    // V counts the value columns of the state: those of v and, for the gated memory, n's and its padding
    const int D = a.dim, V = a.v_dim + Rec<KIND>::XV, TB = a.batch;
    const int nvd = NV * D + Rec<KIND>::XG, rec = nvd + V;
    // two buffers of [TB][NV][D] vectors followed by [TB][VS] values; their addresses are formed
    // from the shared base each time (a table of pointers would turn the loads into generic ones)
    const int buf_floats = TB * (nvd + VS);
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int slice = blockIdx.x % v_slices, eh = blockIdx.x / v_slices;
    const int e = eh / a.heads, h = eh % a.heads;
    const int row0 = a.q_start[e], n_tok = a.q_start[e + 1] - row0;
    const int p = tid % P, cl = tid / P, col = slice * VS + cl;
    // the key rows of a column are dealt out to its P threads in turn (thread p has rows p, p + P, ..., or
    // groups of four rows in turn): the threads of a column then read neighbouring words of a token's
    // vectors, which no bank serves twice
    auto row_of = [p](int i) { return VEC ? 4 * (p + P * (i >> 2)) + (i & 3) : p + P * i; };
    const bool live = col < V;
    float* slot_base = a.state + (size_t)a.slots[e] * (size_t)(a.slot_stride > 0 ? a.slot_stride : (long long)a.heads * D * V);
    float* S_slot = slot_base + (size_t)h * D * V;
    // the gated memory's running maximum: this block's own copy
    float* m_slot = slot_base + (size_t)a.heads * D * V + (size_t)h * v_slices + slice;
    float m_run = KIND == GATED_MEMORY ? *m_slot : 0.f;
    const float* recs = vec + ((size_t)h * tokens + row0) * rec;
    // 16-byte copies need every record and every part of it on a 16-byte boundary
    const bool async = nvd % 4 == 0 && V % 4 == 0;

    float S[CHUNK];
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) S[i] = (live && row_of(i) < D) ? S_slot[(size_t)row_of(i) * V + col] : 0.f;
    const float decay = DELTA || KIND == WKV ? 0.f : a.decay[h];

    load_batch(smem, smem + TB * nvd, recs, rec, nvd, min(TB, n_tok), slice, V, async, VS * P);
    int buf = 0;
    for (int t0 = 0; t0 < n_tok; t0 += TB, buf ^= 1) {
        const int nb = min(TB, n_tok - t0);
        if (t0 + TB < n_tok)
            load_batch(smem + (buf ^ 1) * buf_floats, smem + (buf ^ 1) * buf_floats + TB * nvd,
                              recs + (size_t)(t0 + TB) * rec, rec, nvd, min(TB, n_tok - t0 - TB), slice, V, async, VS * P);
        else
            cp_async_commit();
        cp_async_wait<1>();                 // this batch has landed; the next one may still be on its way
        __syncthreads();
        const float* tvb = smem + buf * buf_floats;
        const float* vvb = tvb + TB * nvd;
        for (int tt = 0; tt < nb; ++tt) {
            const float v = vvb[tt * VS + cl];
            const float* base = tvb + tt * nvd + p;
            float us = 0.f, keep = 0.f, take = 0.f;
            if (KIND == GATED_MEMORY) {
                const float gi = tvb[tt * nvd + NV * D], gf = tvb[tt * nvd + NV * D + 1];
                const float m_new = fmaxf(gf + m_run, gi);
                keep = expf(gf + m_run - m_new);
                take = expf(gi - m_new);
                m_run = m_new;
            }
            if (KIND == SSD) {
                keep = tvb[tt * nvd + NV * D];          // exp(-exp(A) dt)
                take = tvb[tt * nvd + NV * D + 1];      // dt
            }
            const float* tok = tvb + tt * nvd;
            if (DELTA) {
                if (VEC) {
#pragma unroll
                    for (int g = 0; g < CHUNK / 4; ++g) {
                        const int r = 4 * (p + P * g);
                        if (r < D) {
                            const float4 u4 = *reinterpret_cast<const float4*>(tok + 4 * D + r);
                            us = fmaf(u4.x, S[4 * g], us); us = fmaf(u4.y, S[4 * g + 1], us);
                            us = fmaf(u4.z, S[4 * g + 2], us); us = fmaf(u4.w, S[4 * g + 3], us);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < CHUNK; ++i)
                        if (p + P * i < D) us = fmaf(base[4 * D + P * i], S[i], us);
                }
#pragma unroll
                for (int x = P / 2; x > 0; x >>= 1) us += __shfl_xor_sync(0xffffffffu, us, x);
            }
            float o = 0.f;
            const float tv = take * v;                  // (gated memory, state space: the input's weight on this column's value)
            if (VEC && KIND == SSD) {
                // the state space layer's heads are tall (128 rows and more): a group's four rows are a short chain
                // of their own, and the groups' sums meet at the end (an order fixed by the sizes)
                float og[CHUNK / 4];
#pragma unroll
                for (int g = 0; g < CHUNK / 4; ++g) {
                    og[g] = 0.f;
                    const int r = 4 * (p + P * g);
                    if (r < D) {
                        const float4 q4 = *reinterpret_cast<const float4*>(tok + r);
                        const float4 k4 = *reinterpret_cast<const float4*>(tok + D + r);
                        const float s0 = fmaf(k4.x, tv, keep * S[4 * g]), s1 = fmaf(k4.y, tv, keep * S[4 * g + 1]);
                        const float s2 = fmaf(k4.z, tv, keep * S[4 * g + 2]), s3 = fmaf(k4.w, tv, keep * S[4 * g + 3]);
                        S[4 * g] = s0; S[4 * g + 1] = s1; S[4 * g + 2] = s2; S[4 * g + 3] = s3;
                        og[g] = fmaf(s3, q4.w, fmaf(s2, q4.z, fmaf(s1, q4.y, s0 * q4.x)));
                    }
                }
#pragma unroll
                for (int g = 0; g < CHUNK / 4; ++g) o += og[g];
            } else if (VEC) {
#pragma unroll
                for (int g = 0; g < CHUNK / 4; ++g) {
                    const int r = 4 * (p + P * g);
                    if (r < D) {
                        float qq[4], kk[4], ww[4], aa[4];
                        *reinterpret_cast<float4*>(qq) = *reinterpret_cast<const float4*>(tok + r);
                        *reinterpret_cast<float4*>(kk) = *reinterpret_cast<const float4*>(tok + D + r);
                        if (DELTA || KIND == WKV) *reinterpret_cast<float4*>(ww) = *reinterpret_cast<const float4*>(tok + 2 * D + r);
                        if (DELTA) *reinterpret_cast<float4*>(aa) = *reinterpret_cast<const float4*>(tok + 3 * D + r);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float s;
                            if (DELTA) s = fmaf(kk[j], v, fmaf(-aa[j], us, ww[j] * S[4 * g + j]));
                            else if (KIND == GATED_MEMORY || KIND == SSD) s = fmaf(kk[j], tv, keep * S[4 * g + j]);
                            else if (KIND == WKV) s = fmaf(kk[j], v, ww[j] * S[4 * g + j]);
                            else s = fmaf(kk[j], v, decay * S[4 * g + j]);
                            o = fmaf(KIND == WKV ? S[4 * g + j] : s, qq[j], o);      // wkv reads the old state
                            S[4 * g + j] = s;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < CHUNK; ++i) {
                    if (p + P * i < D) {
                        float s;
                        if (DELTA) s = fmaf(base[D + P * i], v, fmaf(-base[3 * D + P * i], us, base[2 * D + P * i] * S[i]));
                        else if (KIND == GATED_MEMORY || KIND == SSD) s = fmaf(base[D + P * i], tv, keep * S[i]);
                        else if (KIND == WKV) s = fmaf(base[D + P * i], v, base[2 * D + P * i] * S[i]);
                        else s = fmaf(base[D + P * i], v, decay * S[i]);
                        o = fmaf(KIND == WKV ? S[i] : s, base[P * i], o);
                        S[i] = s;
                    }
                }
            }
#pragma unroll
            for (int x = P / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (KIND == WKV) o = fmaf(tok[NV * D], v, o);                   // the current token's own pair, weighted by u
            if (KIND == GATED_MEMORY && col == a.v_dim + 1) o = m_run;      // the column after n's carries m_t to the finish
            if (live && p == 0) o_raw[(size_t)(row0 + t0 + tt) * (a.heads * V) + h * V + col] = o;
        }
        __syncthreads();                    // the buffer is free for the batch after the next
    }
#pragma unroll
    for (int i = 0; i < CHUNK; ++i)
        if (live && row_of(i) < D) S_slot[(size_t)row_of(i) * V + col] = S[i];
    if (KIND == GATED_MEMORY && tid == 0) *m_slot = m_run;
}

// (3) per-head root-mean-square division, weight, gate, scale
template <typename T, int KIND>
__global__ void __launch_bounds__(128)
recurrent_finish_kernel(const ScanArgs a, const float* __restrict__ o_raw, int tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)tokens * a.heads) return;
    const size_t row = (size_t)(wg / a.heads);
    const int h = (int)(wg % a.heads), V = a.v_dim;
    const int VX = V + Rec<KIND>::XV;
    const float* o = o_raw + row * (a.heads * VX) + h * VX;
    const T* proj = static_cast<const T*>(a.proj);
    T* out = static_cast<T*>(a.out);
    // the gated memory divides by max(|n . q|, e^(-m)) + 1e-6 first
    const float den = KIND == GATED_MEMORY ? 1.0f / (fmaxf(fabsf(o[V]), expf(-o[V + 1])) + 1e-6f) : 1.f;
    float ss = 0.f;
    for (int c = lane; c < V; c += 32) {
        const float y = o[c] * den;
        ss = fmaf(y, y, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)V + a.eps);
    for (int c = lane; c < V; c += 32) {
        const int hc = h * V + c;
        float y = o[c] * den * inv;
        if (a.norm_w != nullptr) y *= a.norm_w[hc];
        if (a.gate != 0) {
            const float g = to_f32(proj[row * a.ld_proj + a.g_off + hc]);
            y *= a.gate == 1 ? g * sigmoidf_(g) : sigmoidf_(g);
        }
        out[row * a.ld_out + hc] = from_f32<T>(y * a.out_scale);
    }
}

// The state space layer's causal convolution: a thread per (token, channel) sums taps inputs (the
// step's own rows, and before the portion's first token the rows the slot keeps, zeros at a
// sequence's start), adds the bias and applies silu; the result stays float32, [tokens, channels].
constexpr int MAX_TAPS = 16;
template <typename T>
__global__ void __launch_bounds__(256)
ssd_conv_kernel(const ScanArgs a, float* __restrict__ conv_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, taps = a.taps;
    const int channels = a.heads * a.v_dim + 2 * a.groups * a.dim;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int e = a.entry_of_token[row], first = a.q_start[e];
    const T* proj = static_cast<const T*>(a.proj);
    const float* kept = a.state + (size_t)a.slots[e] * (size_t)a.slot_stride + (size_t)a.heads * a.dim * a.v_dim;   // [taps - 1][channels]
    float acc = a.conv_b[c];
    for (int j = 0; j < taps; ++j) {
        const int r = row - (taps - 1 - j);                         // the row that meets tap j
        const float in = r >= first ? to_f32(proj[(size_t)r * a.ld_proj + a.xbc_off + c])
                                    : kept[(size_t)(taps - 1 + r - first) * channels + c];
        acc = fmaf(a.conv_w[(size_t)c * taps + j], in, acc);
    }
    conv_out[(size_t)row * channels + c] = acc / (1.0f + expf(-acc));
}

// The state space layer's token vectors.  A warp per (token, head) copies its group's C and B and its own
// x out of the convolved row and forms dt = softplus(dt_raw + bias) without a clamp: the record
// [C, B, (exp(-exp(A) dt), dt, 0, 0), x].
template <typename T>
__global__ void __launch_bounds__(128)
ssd_prepare_kernel(const ScanArgs a, const float* __restrict__ conv_out, float* __restrict__ vec, int tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)tokens * a.heads) return;
    const int row = (int)(wg / a.heads), h = (int)(wg % a.heads);
    const int D = a.dim, V = a.v_dim;
    const int inner = a.heads * V, channels = inner + 2 * a.groups * D;
    const int g = h / (a.heads / a.groups);
    const float* cv = conv_out + (size_t)row * channels;
    const T* proj = static_cast<const T*>(a.proj);
    const int rec = 2 * D + 4 + V;
    float* dst = vec + ((size_t)h * tokens + row) * rec;
    for (int d = lane; d < D; d += 32) {
        dst[d] = cv[inner + a.groups * D + g * D + d];              // C: what reads the state
        dst[D + d] = cv[inner + g * D + d];                          // B: what writes it
    }
    for (int c = lane; c < V; c += 32) dst[2 * D + 4 + c] = cv[h * V + c];
    if (lane == 0) {
        const float raw = to_f32(proj[(size_t)row * a.ld_proj + a.dt_off + h]) + a.dt_bias[h];
        const float dt = fmaxf(raw, 0.f) + log1pf(expf(-fabsf(raw)));       // softplus, exact at both ends
        dst[2 * D] = expf(-expf(a.a_log[h]) * dt);
        dst[2 * D + 1] = dt;
        dst[2 * D + 2] = 0.f;
        dst[2 * D + 3] = 0.f;
    }
}

// After the scan: y = (o + D_h x) * silu(z), divided by the root mean square of its part of the row
// (norm_groups equal parts of heads * v_dim), times the weight.  A block per (token, part).
template <typename T>
__global__ void __launch_bounds__(128)
ssd_finish_kernel(const ScanArgs a, const float* __restrict__ conv_out, const float* __restrict__ o_raw) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x / a.norm_groups;
    const int part = blockIdx.x % a.norm_groups, V = a.v_dim, inner = a.heads * V, n = inner / a.norm_groups;
    const int channels = inner + 2 * a.groups * a.dim;
    const T* proj = static_cast<const T*>(a.proj) + row * a.ld_proj;
    auto value = [&](int ch) {
        const float x = conv_out[row * channels + ch];
        const float z = to_f32(proj[a.z_off + ch]);
        return fmaf(a.d_skip[ch / V], x, o_raw[row * inner + ch]) * (z / (1.0f + expf(-z)));
    };
    // a thread's first values stay in registers between the two passes (all of them for parts of up to 1,024)
    constexpr int HELD = 8;
    float held[HELD];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < HELD; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        held[k] = i < n ? value(part * n + i) : 0.f;
        ss = fmaf(held[k], held[k], ss);
    }
    for (int i = threadIdx.x + HELD * blockDim.x; i < n; i += blockDim.x) {
        const float y = value(part * n + i);
        ss = fmaf(y, y, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + a.eps);
    T* out = static_cast<T*>(a.out) + row * a.ld_out;
#pragma unroll
    for (int k = 0; k < HELD; ++k) {
        const int i = threadIdx.x + k * blockDim.x, ch = part * n + i;
        if (i < n) out[ch] = from_f32<T>(held[k] * inv * (a.norm_w ? a.norm_w[ch] : 1.f));
    }
    for (int i = threadIdx.x + HELD * blockDim.x; i < n; i += blockDim.x) {
        const int ch = part * n + i;
        out[ch] = from_f32<T>(value(ch) * inv * (a.norm_w ? a.norm_w[ch] : 1.f));
    }
}

// The slot keeps the last taps - 1 inputs of every convolved channel: the portion's last rows, and
// where the portion is shorter than that, the rows kept before move up.  A thread per (entry,
// channel) reads what it needs first and writes then.
template <typename T>
__global__ void __launch_bounds__(256)
ssd_conv_keep_kernel(const ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, first = a.q_start[e], n = a.q_start[e + 1] - first, keep = a.taps - 1;
    const int channels = a.heads * a.v_dim + 2 * a.groups * a.dim;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (n <= 0 || c >= channels) return;
    const T* proj = static_cast<const T*>(a.proj);
    float* kept = a.state + (size_t)a.slots[e] * (size_t)a.slot_stride + (size_t)a.heads * a.dim * a.v_dim;
    float rows[MAX_TAPS - 1];
#pragma unroll
    for (int r = 0; r < MAX_TAPS - 1; ++r) {
        if (r >= keep) break;
        const int k = n - keep + r;                                // row of the portion, or (negative) a row kept before
        rows[r] = k >= 0 ? to_f32(proj[(size_t)(first + k) * a.ld_proj + a.xbc_off + c]) : kept[(size_t)(keep + k) * channels + c];
    }
#pragma unroll
    for (int r = 0; r < MAX_TAPS - 1; ++r) {
        if (r >= keep) break;
        kept[(size_t)r * channels + c] = rows[r];
    }
}

template <typename T, int DELTA, int P, bool VEC>
int launch_scan_rows(const ScanArgs& b, const float* vec, float* o_raw, int slices, int tokens, dim3 grid, size_t smem,
                     cudaStream_t stream) {
    const int chunk = (b.dim + P - 1) / P;
    if (chunk <= 8) return kipp_launch(recurrent_scan_kernel<T, DELTA, P, 8, VEC>, grid, dim3(VS * P), smem, stream, 1, b, vec, o_raw, slices, tokens);
    if (chunk <= 16) return kipp_launch(recurrent_scan_kernel<T, DELTA, P, 16, VEC>, grid, dim3(VS * P), smem, stream, 1, b, vec, o_raw, slices, tokens);
    if (chunk <= 24) return kipp_launch(recurrent_scan_kernel<T, DELTA, P, 24, VEC>, grid, dim3(VS * P), smem, stream, 1, b, vec, o_raw, slices, tokens);
    return kipp_launch(recurrent_scan_kernel<T, DELTA, P, 32, VEC>, grid, dim3(VS * P), smem, stream, 1, b, vec, o_raw, slices, tokens);
}
template <typename T, int DELTA, int P>
int launch_scan_chunk(const ScanArgs& b, const float* vec, float* o_raw, int slices, int tokens, dim3 grid, size_t smem,
                      cudaStream_t stream) {
    // groups of four rows per 16-byte load where the key size allows (every vector of a record then
    // starts on a 16-byte boundary)
    return b.dim % 4 == 0 ? launch_scan_rows<T, DELTA, P, true>(b, vec, o_raw, slices, tokens, grid, smem, stream)
                          : launch_scan_rows<T, DELTA, P, false>(b, vec, o_raw, slices, tokens, grid, smem, stream);
}

// scratch: float32 [heads][tokens][NV * dim + v_dim] for the records, then [tokens][heads * v_dim] for raw o
// conv_out: float32 [tokens, channels] for the state space layer's convolved rows (null for the other kinds)
template <typename T, int DELTA>
int launch_scan(const ScanArgs& a, int entries, int tokens, float* scratch, cudaStream_t stream, float* conv_out = nullptr) {
    const int D = a.dim, V = a.v_dim + Rec<DELTA>::XV;
    constexpr int NV = Rec<DELTA>::NV, XG = Rec<DELTA>::XG;
    // threads per column: runs of 8 key rows where the head allows (short chains of dependent
    // multiply-adds, more warps per block), at most 8 threads (16 only where a head has more than 256 key rows)
    int P = 1;
    while (P < 8 && (D + P - 1) / P > 8) P *= 2;
    if ((D + P - 1) / P > MAX_CHUNK) P = 16;
    if (DELTA == SSD && D > 64 && KIPP_SSD_WIDE) P = 16;
    if ((D + P - 1) / P > MAX_CHUNK || scratch == nullptr) return KIPP_ERR_ARG;
    const size_t per_token = ((size_t)NV * D + XG + VS) * sizeof(float);
    int batch = (int)std::min<size_t>(32, (20 * 1024) / per_token);       // two buffers of at most 20 KB
    if (batch < 1) return KIPP_ERR_ARG;
    ScanArgs b = a;
    b.batch = batch;
    float* vec = scratch;
    float* o_raw = scratch + (size_t)tokens * a.heads * (NV * D + XG + V);
    const long long warps = (long long)tokens * a.heads;
    const dim3 wgrid((unsigned)((warps + 3) / 4));
    int rc = 0;
    const int channels = DELTA == SSD ? a.heads * a.v_dim + 2 * a.groups * a.dim : 0;
    if (DELTA == SSD) {
        if (conv_out == nullptr) return KIPP_ERR_ARG;
        rc = kipp_launch(ssd_conv_kernel<T>, dim3((unsigned)tokens, (unsigned)((channels + 255) / 256)), dim3(256), 0, stream, 1, b,
                         conv_out);
        if (rc) return rc;
        rc = kipp_launch(ssd_prepare_kernel<T>, wgrid, dim3(128), 0, stream, 1, b, (const float*)conv_out, vec, tokens);
    } else {
        rc = kipp_launch(recurrent_prepare_kernel<T, DELTA>, wgrid, dim3(128), 0, stream, 1, b, vec, tokens);
    }
    if (rc) return rc;
    const int slices = (V + VS - 1) / VS;
    const dim3 grid((unsigned)(entries * a.heads * slices));
    const size_t smem = 2 * per_token * batch;
    switch (P) {
    case 1: rc = launch_scan_chunk<T, DELTA, 1>(b, vec, o_raw, slices, tokens, grid, smem, stream); break;
    case 2: rc = launch_scan_chunk<T, DELTA, 2>(b, vec, o_raw, slices, tokens, grid, smem, stream); break;
    case 4: rc = launch_scan_chunk<T, DELTA, 4>(b, vec, o_raw, slices, tokens, grid, smem, stream); break;
    case 8: rc = launch_scan_chunk<T, DELTA, 8>(b, vec, o_raw, slices, tokens, grid, smem, stream); break;
    default: rc = launch_scan_chunk<T, DELTA, 16>(b, vec, o_raw, slices, tokens, grid, smem, stream); break;
    }
    if (rc) return rc;
    if (DELTA == SSD) {
        const long long parts = (long long)tokens * b.norm_groups;
        if (parts > 0x7fffffffLL) return KIPP_ERR_ARG;
        const int per_part = a.heads * a.v_dim / b.norm_groups;
        rc = kipp_launch(ssd_finish_kernel<T>, dim3((unsigned)parts), dim3(per_part >= 128 ? 128 : (per_part + 31) / 32 * 32), 0,
                         stream, 1, b, (const float*)conv_out, (const float*)o_raw);
        if (rc || b.taps <= 1) return rc;
        return kipp_launch(ssd_conv_keep_kernel<T>, dim3((unsigned)entries, (unsigned)((channels + 255) / 256)), dim3(256), 0,
                           stream, 1, b);
    }
    return kipp_launch(recurrent_finish_kernel<T, DELTA>, wgrid, dim3(128), 0, stream, 1, b, (const float*)o_raw, tokens);
}

template <typename T>
__global__ void __launch_bounds__(128)
token_shift_mix_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ h, const float* __restrict__ mu,
                       const float* __restrict__ prev, long long slot_stride, const int* __restrict__ q_start,
                       const int* __restrict__ entry_of_token, const int* __restrict__ slots, int hidden, int n_mix) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, e = entry_of_token[t];
    const bool inside = t > q_start[e];
    const T* above = h + (size_t)(inside ? t - 1 : t) * hidden;
    const float* kept = prev + (size_t)slots[e] * slot_stride;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float hv = to_f32(h[(size_t)t * hidden + i]);
        const float d = (inside ? to_f32(above[i]) : kept[i]) - hv;
        for (int s = 0; s < n_mix; ++s)
            out[(size_t)s * out_stride + (size_t)t * hidden + i] = from_f32<T>(fmaf(d, mu[(size_t)s * hidden + i], hv));
    }
}
template <typename T>
__global__ void __launch_bounds__(128)
token_shift_keep_kernel(float* __restrict__ prev, long long slot_stride, const T* __restrict__ h,
                        const int* __restrict__ q_start, const int* __restrict__ slots, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x, last = q_start[e + 1] - 1;
    if (last < q_start[e]) return;
    float* dst = prev + (size_t)slots[e] * slot_stride;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(h[(size_t)last * hidden + i]);
}

template <typename T>
__global__ void tanh_rows_kernel(T* __restrict__ out, long long ld_out, const T* __restrict__ in, long long ld_in,
                                 int rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const long long r = i / cols, c = i % cols;
    out[r * ld_out + c] = from_f32<T>(tanhf(to_f32(in[r * ld_in + c])));
}
}  // namespace

// Whether the scan kernels take a head of these sizes.
extern "C" int kipp_recurrent_scan_ok(int dim, int v_dim, int kind) {
    if (dim <= 0 || v_dim <= 0 || dim > 16 * MAX_CHUNK || kind < 0 || kind > 4) return 0;
    return (((kind == DELTA_RULE ? 5 : kind == WKV ? 3 : 2) * (size_t)dim + 4 + VS) * sizeof(float)) <= 20 * 1024 ? 1 : 0;
}
// float32 values of scratch a scan of `tokens` tokens needs.
extern "C" long long kipp_recurrent_scratch_floats(int tokens, int heads, int dim, int v_dim, int kind) {
    const long long x = kind == GATED_MEMORY ? 4 : 0, g = kind == WKV || kind == SSD ? 4 : 0;
    return (long long)tokens * heads * ((kind == DELTA_RULE ? 5 : kind == WKV ? 3 : 2) * (long long)dim + x + g + 2 * ((long long)v_dim + x));
}
// float32 values of state one request slot of the gated memory holds: S with n's column and its
// padding, then one running maximum per head and slice of value columns.
extern "C" long long kipp_gated_memory_state_floats(int heads, int dim, int v_dim) {
    return (long long)heads * dim * (v_dim + 4) + (long long)heads * ((v_dim + 4 + VS - 1) / VS);
}

extern "C" int kipp_retention_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype,
                                   int q_off, int k_off, int v_off, int g_off, float* state, const float* decay,
                                   const float* cos_sin, int rot, const int* q_start, const int* slots, int entries,
                                   int tokens, int heads, int dim, int v_dim, float k_scale, float eps,
                                   float out_scale, int gate, float* scratch, void* stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, v_dim, 0) || heads <= 0 || rot < 0 || rot > dim || (rot & 1)) return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
    a.decay = decay; a.cos_sin = rot > 0 ? cos_sin : nullptr; a.rot = rot; a.state = state;
    a.q_start = q_start; a.slots = slots; a.heads = heads; a.dim = dim; a.v_dim = v_dim;
    a.k_scale = k_scale; a.eps = eps; a.out_scale = out_scale; a.gate = gate;
    if (dtype == KIPP_DT_F32) return launch_scan<float, RETENTION>(a, entries, tokens, scratch, (cudaStream_t)stream);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, RETENTION>(a, entries, tokens, scratch, (cudaStream_t)stream);
    return KIPP_ERR_DTYPE;
}

extern "C" int kipp_delta_rule_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype,
                                    int r_off, int k_off, int v_off, int g_off, int a_off, const void* w_raw,
                                    long long ld_w, const float* a_bias, const float* w_bias, const float* norm_w,
                                    float* state, const int* q_start, const int* slots, int entries, int tokens,
                                    int heads, int dim, float eps, float out_scale, int gate, float* scratch,
                                    void* stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, dim, 1) || heads <= 0 || a_bias == nullptr || w_bias == nullptr)
        return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.q_off = r_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off; a.a_off = a_off;
    a.w_raw = w_raw; a.ld_w = ld_w; a.a_bias = a_bias; a.w_bias = w_bias; a.norm_w = norm_w;
    a.state = state; a.q_start = q_start; a.slots = slots; a.heads = heads; a.dim = dim; a.v_dim = dim;
    a.k_scale = 1.f; a.eps = eps; a.out_scale = out_scale; a.gate = gate;
    if (dtype == KIPP_DT_F32) return launch_scan<float, DELTA_RULE>(a, entries, tokens, scratch, (cudaStream_t)stream);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, DELTA_RULE>(a, entries, tokens, scratch, (cudaStream_t)stream);
    return KIPP_ERR_DTYPE;
}

// The gated matrix memory (see the head of this file): q, k [heads, dim], v and the output gate
// [heads, v_dim] and the two gates' pre-activations [heads] are columns of proj; the state of a slot
// is kipp_gated_memory_state_floats floats.
extern "C" int kipp_gated_memory_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype,
                                      int q_off, int k_off, int v_off, int g_off, int i_off, int f_off,
                                      const float* i_bias, const float* f_bias, const float* norm_w, float* state,
                                      const int* q_start, const int* slots, int entries, int tokens, int heads,
                                      int dim, int v_dim, float gate_cap, float q_scale, float eps, float out_scale,
                                      int gate, float* scratch, void* stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, v_dim, GATED_MEMORY) || heads <= 0 || i_bias == nullptr || f_bias == nullptr ||
        !(gate_cap > 0.f))
        return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off; a.i_off = i_off; a.f_off = f_off;
    a.i_bias = i_bias; a.f_bias = f_bias; a.norm_w = norm_w; a.gate_cap = gate_cap; a.q_scale = q_scale;
    a.state = state; a.q_start = q_start; a.slots = slots; a.heads = heads; a.dim = dim; a.v_dim = v_dim;
    a.k_scale = 1.f; a.eps = eps; a.out_scale = out_scale; a.gate = gate;
    a.slot_stride = kipp_gated_memory_state_floats(heads, dim, v_dim);
    if (dtype == KIPP_DT_F32) return launch_scan<float, GATED_MEMORY>(a, entries, tokens, scratch, (cudaStream_t)stream);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, GATED_MEMORY>(a, entries, tokens, scratch, (cudaStream_t)stream);
    return KIPP_ERR_DTYPE;
}

// The wkv recurrence (see the head of this file): r, k, v and the output gate [heads, dim] are columns of
// proj, the decay's pre-activation is w_raw [T, heads * dim]; `bonus` is u [heads * dim].  The state of a
// slot is `slot_stride` floats of which the first heads * dim * dim are S.
extern "C" int kipp_wkv_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int r_off,
                             int k_off, int v_off, int g_off, const void* w_raw, long long ld_w, const float* w_bias,
                             const float* bonus, const float* norm_w, float* state, long long slot_stride,
                             const int* q_start, const int* slots, int entries, int tokens, int heads, int dim,
                             float eps, float out_scale, int gate, float* scratch, void* stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, dim, WKV) || heads <= 0 || w_bias == nullptr || bonus == nullptr || w_raw == nullptr ||
        slot_stride < (long long)heads * dim * dim)
        return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.q_off = r_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
    a.w_raw = w_raw; a.ld_w = ld_w; a.w_bias = w_bias; a.bonus = bonus; a.norm_w = norm_w;
    a.state = state; a.slot_stride = slot_stride; a.q_start = q_start; a.slots = slots;
    a.heads = heads; a.dim = dim; a.v_dim = dim;
    a.k_scale = 1.f; a.eps = eps; a.out_scale = out_scale; a.gate = gate;
    if (dtype == KIPP_DT_F32) return launch_scan<float, WKV>(a, entries, tokens, scratch, (cudaStream_t)stream);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, WKV>(a, entries, tokens, scratch, (cudaStream_t)stream);
    return KIPP_ERR_DTYPE;
}

// float32 values of state one request slot of the state space layer holds: S [heads, dim, v_dim], then the
// last taps - 1 inputs of the heads * v_dim + 2 * groups * dim convolved channels.
extern "C" long long kipp_ssd_state_floats(int heads, int groups, int dim, int v_dim, int taps) {
    return (long long)heads * dim * v_dim + (long long)(taps > 1 ? taps - 1 : 0) * ((long long)heads * v_dim + 2LL * groups * dim);
}

// The state space layer (see the head of this file).  proj [T, ...] holds z [heads * v_dim] at z_off, the
// channels to convolve [x | B | C] at xbc_off and dt [heads] at dt_off; conv_w [channels, taps] (the last
// tap meets the current token), conv_b [channels], dt_bias, a_log, d_skip [heads], norm_w [heads * v_dim]
// (or null) float32; `dim` is the size of B and C (the state's rows).  A slot is kipp_ssd_state_floats floats.
// conv_out: float32 [tokens, channels] of scratch for the convolved rows.  At most 16 taps.
extern "C" int kipp_ssd_max_taps() { return 16; }
extern "C" int kipp_ssd_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int z_off,
                             int xbc_off, int dt_off, const float* conv_w, const float* conv_b, int taps,
                             const float* dt_bias, const float* a_log, const float* d_skip, const float* norm_w,
                             int norm_groups, float* state, long long slot_stride, const int* q_start,
                             const int* entry_of_token, const int* slots, int entries, int tokens, int heads, int groups,
                             int dim, int v_dim, float eps, float* scratch, float* conv_out, void* stream) {
    if (entries <= 0 || tokens <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, v_dim, SSD) || heads <= 0 || groups <= 0 || heads % groups || taps < 1 || taps > MAX_TAPS ||
        norm_groups <= 0 || (heads * v_dim) % norm_groups || conv_w == nullptr || conv_b == nullptr || dt_bias == nullptr ||
        a_log == nullptr || d_skip == nullptr || entry_of_token == nullptr ||
        slot_stride < kipp_ssd_state_floats(heads, groups, dim, v_dim, taps))
        return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.z_off = z_off; a.xbc_off = xbc_off; a.dt_off = dt_off; a.taps = taps; a.groups = groups; a.norm_groups = norm_groups;
    a.conv_w = conv_w; a.conv_b = conv_b; a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip; a.norm_w = norm_w;
    a.state = state; a.slot_stride = slot_stride; a.q_start = q_start; a.entry_of_token = entry_of_token; a.slots = slots;
    a.heads = heads; a.dim = dim; a.v_dim = v_dim; a.eps = eps; a.k_scale = 1.f; a.out_scale = 1.f;
    if (dtype == KIPP_DT_F32) return launch_scan<float, SSD>(a, entries, tokens, scratch, (cudaStream_t)stream, conv_out);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, SSD>(a, entries, tokens, scratch, (cudaStream_t)stream, conv_out);
    return KIPP_ERR_DTYPE;
}

// Token shift: out[s][t, :] = h[t, :] + (h'[t, :] - h[t, :]) * mu[s, :] for s < n_mix, with h' the row of
// the token before in the same sequence: the row above inside a step's portion, the row the
// sequence's slot keeps (prev[slot * slot_stride ...], float32, zeros at admission) for the portion's
// first token.  kipp_token_shift_keep then stores the portion's last row in the slot.
extern "C" int kipp_token_shift_mix(void* out, long long out_stride, const void* h, const float* mu, const float* prev,
                                    long long slot_stride, const int* q_start, const int* entry_of_token,
                                    const int* slots, int dtype, int tokens, int hidden, int n_mix, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || n_mix <= 0 || n_mix > 8 || prev == nullptr || mu == nullptr) return KIPP_ERR_ARG;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(token_shift_mix_kernel<float>, dim3((unsigned)tokens), dim3(128), 0, (cudaStream_t)stream, 1,
                           (float*)out, out_stride, (const float*)h, mu, prev, slot_stride, q_start, entry_of_token, slots,
                           hidden, n_mix);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(token_shift_mix_kernel<bf16>, dim3((unsigned)tokens), dim3(128), 0, (cudaStream_t)stream, 1,
                           (bf16*)out, out_stride, (const bf16*)h, mu, prev, slot_stride, q_start, entry_of_token, slots,
                           hidden, n_mix);
    return KIPP_ERR_DTYPE;
}
extern "C" int kipp_token_shift_keep(float* prev, long long slot_stride, const void* h, const int* q_start,
                                     const int* slots, int dtype, int entries, int hidden, void* stream) {
    if (entries <= 0) return 0;
    if (hidden <= 0 || prev == nullptr) return KIPP_ERR_ARG;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(token_shift_keep_kernel<float>, dim3((unsigned)entries), dim3(128), 0, (cudaStream_t)stream, 1,
                           prev, slot_stride, (const float*)h, q_start, slots, hidden);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(token_shift_keep_kernel<bf16>, dim3((unsigned)entries), dim3(128), 0, (cudaStream_t)stream, 1,
                           prev, slot_stride, (const bf16*)h, q_start, slots, hidden);
    return KIPP_ERR_DTYPE;
}

// out[r, c] = tanh(in[r, c]) in the compute type (the bottleneck of a low-rank projection).
extern "C" int kipp_tanh_rows(void* out, long long ld_out, const void* in, long long ld_in, int dtype, int rows,
                              int cols, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const long long n = (long long)rows * cols;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == KIPP_DT_F32)
        return kipp_launch(tanh_rows_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, 1, (float*)out, ld_out,
                           (const float*)in, ld_in, rows, cols);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(tanh_rows_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, 1, (bf16*)out, ld_out,
                           (const bf16*)in, ld_in, rows, cols);
    return KIPP_ERR_DTYPE;
}
