// A feed-forward made of many small experts of which every token uses a few.
//
//   route     z = W_r h + b in float32 (a warp per expert); the `top` largest logits are chosen (the
//             lower index on a tie) and their weights are the softmax over the chosen logits only;
//   lists     the (token, choice) pairs sorted by expert, cut into tiles of 64 rows that belong to
//             one expert each; everything on the device, so that a step's launches do not depend
//             on the routing (a captured graph replays them);
//   products  per tile: rows gathered from the tokens' input times the expert's up projection,
//             with the activation, into a hidden buffer in sorted order; then the hidden rows
//             times the expert's down projection into one float32 row per pair;
//   combine   y[t] += sum over the token's choices, in the order of their rank, of weight x row.
//
// A second way of routing (kipp_moe_route_scores): scores s = softmax(z) over ALL outputs of the
// router; the choice by s + correction (a learned number per output that steers the choice only); the
// weights are the chosen scores divided by their sum, times a scale.  The last outputs of the router
// may be identity experts, which hand the token's input on: their pairs carry a negative expert id,
// the lists and products leave them out, and the combine adds weight x input for them.
//
// In bfloat16 (sizes that are multiples of 8) the two products take another road: the pairs' input
// rows are copied into a buffer sorted by expert in which every expert's rows are padded to whole
// tiles (padded lists, gather), and each projection is ONE grouped product on the tcgen05 kernels
// of gemm_tc.cu, whose token tiles then meet one expert's weights each: tiles of 128 rows on the
// prompt kernel for prompt-sized steps, of 16 rows on the few-token kernel otherwise.  The
// products of this file (CUDA cores) serve float32 and the other sizes.
//
// A pair's row is computed from its own token alone, in an order of sums that depends on the
// sizes only: the result does not depend on which other tokens share its tile.
#include "common.cuh"
#include <math.h>
#include <limits.h>

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// Four values of a row from element i on (i a multiple of 4, the row 8- or 16-byte aligned).
__device__ __forceinline__ void load4(float (&x)[4], const float* row, int i) {
    const float4 v = *reinterpret_cast<const float4*>(row + i);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void load4(float (&x)[4], const bf16* row, int i) {
    const uint2 v = *reinterpret_cast<const uint2*>(row + i);
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
}

// A block per TOK tokens.  Warp w forms the logits of experts w, w + warps, ...: a lane sums its
// share of the row in rising order (four neighbouring elements at a time where the row's size and
// place allow: `vec`), then the lanes are summed; a router row is read once for all TOK tokens.
// The order of a token's sums depends on the sizes only, not on TOK or on the other tokens.
// Then warp j chooses for token j.
template <typename T, int TOK>
__global__ void __launch_bounds__(512)
moe_route_kernel(int* __restrict__ expert_of, float* __restrict__ weight_of, const T* __restrict__ h, long long ldh,
                 const float* __restrict__ router, const float* __restrict__ bias, int tokens, int hidden, int experts,
                 int top, int vec, int by_scores, int real_experts, float weight_scale) {
    extern __shared__ float z_all[];                      // [TOK][experts], and [TOK][experts] scores when by_scores
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int t0 = blockIdx.x * TOK;
    const T* rows[TOK];
#pragma unroll
    for (int j = 0; j < TOK; ++j) rows[j] = h + (size_t)min(t0 + j, tokens - 1) * ldh;
    for (int e = warp; e < experts; e += warps) {
        const float* w = router + (size_t)e * hidden;
        float acc[TOK];
#pragma unroll
        for (int j = 0; j < TOK; ++j) acc[j] = 0.f;
        if (vec) {
#pragma unroll 4
            for (int i = 4 * lane; i < hidden; i += 128) {
                float wv[4];
                load4(wv, w, i);
#pragma unroll
                for (int j = 0; j < TOK; ++j) {
                    float x[4];
                    load4(x, rows[j], i);
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[j] = fmaf(wv[u], x[u], acc[j]);
                }
            }
        } else {
#pragma unroll 4
            for (int i = lane; i < hidden; i += 32) {
                const float wv = w[i];
#pragma unroll
                for (int j = 0; j < TOK; ++j) acc[j] = fmaf(wv, to_f32(rows[j][i]), acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < TOK; ++j) {
            const float sum = warp_sum(acc[j]);
            if (lane == 0) z_all[(size_t)j * experts + e] = sum + (bias && !by_scores ? bias[e] : 0.f);
        }
    }
    __syncthreads();
    for (int j = warp; j < TOK; j += warps) {
        const int t = t0 + j;
        if (t >= tokens) continue;
        float* z = z_all + (size_t)j * experts;
        float* score = z_all + (size_t)(TOK + j) * experts;
        if (by_scores) {
            // s = softmax(z) over all outputs; what is compared is s + correction
            float top_z = -INFINITY;
            for (int e = lane; e < experts; e += 32) top_z = fmaxf(top_z, z[e]);
            top_z = warp_max(top_z);
            float sum = 0.f;
            for (int e = lane; e < experts; e += 32) {
                const float w = expf(z[e] - top_z);
                score[e] = w;
                sum += w;
            }
            sum = warp_sum(sum);
            const float inv = 1.0f / sum;
            for (int e = lane; e < experts; e += 32) {
                const float sc = score[e] * inv;
                score[e] = sc;
                z[e] = sc + (bias ? bias[e] : 0.f);
            }
            __syncwarp();
        }
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int idx = INT_MAX;
            for (int e = lane; e < experts; e += 32) {
                const float v = z[e];
                if (v > best) { best = v; idx = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
            }
            if (idx >= experts) { idx = k; best = 0.f; }      // logits that are no numbers: still a valid expert
            if (lane == 0) {
                // an identity expert (an output behind the real experts) is marked by a negative id
                expert_of[(size_t)t * top + k] = idx < real_experts ? idx : -1 - (idx - real_experts);
                weight_of[(size_t)t * top + k] = by_scores ? score[idx] : best;
                z[idx] = -INFINITY;
            }
            __syncwarp();
        }
        if (lane == 0 && by_scores) {
            float* w = weight_of + (size_t)t * top;
            float sum = 0.f;
            for (int k = 0; k < top; ++k) sum += w[k];
            const float f = weight_scale / (sum + 1e-20f);
            for (int k = 0; k < top; ++k) w[k] *= f;
        } else if (lane == 0) {
            float* w = weight_of + (size_t)t * top;
            const float m = w[0];                            // the largest of the chosen
            float sum = 0.f;
            for (int k = 0; k < top; ++k) { w[k] = expf(w[k] - m); sum += w[k]; }
            const float inv = 1.0f / sum;
            for (int k = 0; k < top; ++k) w[k] *= inv;
        }
    }
}

// tile_info: (expert, first row in the sorted list, rows) per tile
__global__ void __launch_bounds__(1024)
moe_lists_kernel(int* __restrict__ sorted_pair, int* __restrict__ tile_info, int* __restrict__ n_tiles,
                 const int* __restrict__ expert_of, int pairs, int experts) {
    extern __shared__ int lists[];                        // counts [experts], cursor [experts]
    int* counts = lists;
    int* cursor = lists + experts;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x)
        if (expert_of[p] >= 0) atomicAdd(&counts[expert_of[p]], 1);      // (a negative id: a pair without an expert's product)
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, nt = 0;
        for (int e = 0; e < experts; ++e) {
            cursor[e] = off;
            for (int r0 = 0; r0 < counts[e]; r0 += BM) {
                tile_info[3 * nt] = e;
                tile_info[3 * nt + 1] = off + r0;
                tile_info[3 * nt + 2] = min(BM, counts[e] - r0);
                ++nt;
            }
            off += counts[e];
        }
        *n_tiles = nt;
    }
    __syncthreads();
    // a pair's place among its expert's rows is whatever the race gives: its row's value does not depend on it
    for (int p = threadIdx.x; p < pairs; p += blockDim.x)
        if (expert_of[p] >= 0) sorted_pair[atomicAdd(&cursor[expert_of[p]], 1)] = p;
}

// The pairs sorted by expert with every expert's rows padded to whole tiles of `tile_rows`:
// place_of_pair [pairs] (a pair's row among the padded rows), expert_of_tile [tiles], n_tiles [1].
__global__ void __launch_bounds__(1024)
moe_padded_lists_kernel(int* __restrict__ place_of_pair, int* __restrict__ expert_of_tile, int* __restrict__ n_tiles,
                        const int* __restrict__ expert_of, int pairs, int experts, int tile_rows) {
    extern __shared__ int lists[];                        // counts [experts], cursor [experts]
    int* counts = lists;
    int* cursor = lists + experts;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x)
        if (expert_of[p] >= 0) atomicAdd(&counts[expert_of[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int nt = 0;
        for (int e = 0; e < experts; ++e) {
            cursor[e] = nt * tile_rows;
            for (int r0 = 0; r0 < counts[e]; r0 += tile_rows) expert_of_tile[nt++] = e;
        }
        *n_tiles = nt;
    }
    __syncthreads();
    // a pair's place among its expert's rows is whatever the race gives: its row's value does not depend on it
    for (int p = threadIdx.x; p < pairs; p += blockDim.x)
        place_of_pair[p] = expert_of[p] >= 0 ? atomicAdd(&cursor[expert_of[p]], 1) : -1;
}

// dst[place_of_pair[p], :] = src[p / top, :], 16 bytes per thread and step (bfloat16 rows of 8 n elements).
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long ld_src16, int row16,
                       const int* __restrict__ place_of_pair, int pairs, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (p >= pairs) return;
    if (place_of_pair[p] < 0) return;                    // a pair without an expert's product
    const uint4* from = src + (size_t)(p / top) * ld_src16;
    uint4* to = dst + (size_t)place_of_pair[p] * row16;
    for (int i = threadIdx.x & 31; i < row16; i += 32) to[i] = from[i];
}

struct GemmArgs {
    void* out; long long ldo;
    const void* a; long long lda;
    const void* w; long long w_expert;      // elements between two experts' matrices [N, K]
    int N, K, top, gather, scatter, act;
    const int* sorted_pair; const int* tile_info; const int* n_tiles;
};

// CUDA cores: a block of 256 threads per 64 x 64 tile, each thread 4 x 4 results.
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const GemmArgs g) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int arow[BM], orow[BM];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    if (tile >= *g.n_tiles) return;
    const int e = g.tile_info[3 * tile], r0 = g.tile_info[3 * tile + 1], rows = g.tile_info[3 * tile + 2];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    if (tid < BM) {
        const int pair = tid < rows ? g.sorted_pair[r0 + tid] : -1;
        arow[tid] = pair < 0 ? -1 : (g.gather ? pair / g.top : r0 + tid);
        orow[tid] = pair < 0 ? -1 : (g.scatter ? pair : r0 + tid);
    }
    __syncthreads();
    const T* A = static_cast<const T*>(g.a);
    const T* W = static_cast<const T*>(g.w) + (size_t)e * g.w_expert;
    const int n0 = blockIdx.x * BN, N = g.N, K = g.K;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const int ar = arow[lrow];
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i, wn = n0 + lrow;
            As[lk + i][lrow] = (ar >= 0 && k < K) ? to_f32(A[(size_t)ar * g.lda + k]) : 0.f;
            Ws[lk + i][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float x[TM], y[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) x[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) y[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(x[i], y[j], acc[i][j]);
        }
        __syncthreads();
    }
    TO* out = static_cast<TO*>(g.out);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int orw = orow[ty * TM + i];
        if (orw < 0) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) out[(size_t)orw * g.ldo + n] = from_f32<TO>(g.act >= 0 ? kipp_activation(acc[i][j], g.act) : acc[i][j]);
        }
    }
}

__global__ void __launch_bounds__(512)
moe_combine_kernel(float* __restrict__ y, const float* __restrict__ rows, const float* __restrict__ weight_of, int hidden,
                   int top, const int* __restrict__ place_of_pair) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float* w = weight_of + (size_t)t * top;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const size_t row = place_of_pair ? (size_t)place_of_pair[(size_t)t * top + k] : (size_t)t * top + k;
            acc = fmaf(w[k], rows[row * hidden + i], acc);
        }
        y[(size_t)t * hidden + i] += acc;
    }
}

// The combine where some pairs are identity experts (expert_of < 0): their row is the token's input.
template <typename T>
__global__ void __launch_bounds__(512)
moe_combine_identity_kernel(float* __restrict__ y, const float* __restrict__ rows, const float* __restrict__ weight_of,
                            const int* __restrict__ expert_of, const T* __restrict__ h, long long ldh, int hidden, int top,
                            const int* __restrict__ place_of_pair) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float* w = weight_of + (size_t)t * top;
    const int* ex = expert_of + (size_t)t * top;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            if (ex[k] < 0) {
                acc = fmaf(w[k], to_f32(h[(size_t)t * ldh + i]), acc);
            } else {
                const size_t row = place_of_pair ? (size_t)place_of_pair[(size_t)t * top + k] : (size_t)t * top + k;
                acc = fmaf(w[k], rows[row * hidden + i], acc);
            }
        }
        y[(size_t)t * hidden + i] += acc;
    }
}
}  // namespace

// Tiles a step of `pairs` (token, choice) pairs over `experts` experts can need at most.
extern "C" int kipp_moe_max_tiles(int pairs, int experts) { return (pairs + BM - 1) / BM + experts; }

// expert_of, weight_of [tokens, top]: the chosen experts in the order of their logits and their weights.
static int moe_route_any(int* expert_of, float* weight_of, const void* h, long long ldh, int dtype, const float* router,
                         const float* bias, int tokens, int hidden, int experts, int top, int by_scores, int real_experts,
                         float weight_scale, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || experts <= 0 || top <= 0 || top > experts || experts > 2048) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t es = dtype == KIPP_DT_F32 ? 4 : 2;
    const int vec = hidden % 4 == 0 && ldh % 4 == 0 && ((uintptr_t)h % (4 * es)) == 0 && ((uintptr_t)router & 15) == 0;
    // many tokens: four per block share a read of the router; few: a warp per expert, up to sixteen
    const int tok = tokens >= 256 ? 4 : 1;
    const int warps = tok == 4 ? 8 : (experts >= 16 ? 16 : experts > 8 ? 8 : 4);
    const dim3 grid((unsigned)((tokens + tok - 1) / tok)), block((unsigned)(32 * warps));
    const size_t smem = (size_t)(by_scores ? 2 : 1) * tok * experts * sizeof(float);
    if (dtype == KIPP_DT_F32) {
        if (tok == 4)
            return kipp_launch(moe_route_kernel<float, 4>, grid, block, smem, s, 1, expert_of, weight_of, (const float*)h,
                               ldh, router, bias, tokens, hidden, experts, top, vec, by_scores, real_experts, weight_scale);
        return kipp_launch(moe_route_kernel<float, 1>, grid, block, smem, s, 1, expert_of, weight_of, (const float*)h, ldh,
                           router, bias, tokens, hidden, experts, top, vec, by_scores, real_experts, weight_scale);
    }
    if (dtype == KIPP_DT_BF16) {
        if (tok == 4)
            return kipp_launch(moe_route_kernel<bf16, 4>, grid, block, smem, s, 1, expert_of, weight_of, (const bf16*)h, ldh,
                               router, bias, tokens, hidden, experts, top, vec, by_scores, real_experts, weight_scale);
        return kipp_launch(moe_route_kernel<bf16, 1>, grid, block, smem, s, 1, expert_of, weight_of, (const bf16*)h, ldh,
                           router, bias, tokens, hidden, experts, top, vec, by_scores, real_experts, weight_scale);
    }
    return KIPP_ERR_DTYPE;
}
extern "C" int kipp_moe_route(int* expert_of, float* weight_of, const void* h, long long ldh, int dtype, const float* router,
                              const float* bias, int tokens, int hidden, int experts, int top, void* stream) {
    return moe_route_any(expert_of, weight_of, h, ldh, dtype, router, bias, tokens, hidden, experts, top, 0, experts, 1.f, stream);
}
// Routing by scores: s = softmax(W_r h) over `outputs` router rows, the `top` largest of s + correction
// (correction null: of s), weights s / (sum of the chosen + 1e-20) * weight_scale.  Outputs from
// `experts` on are identity experts: expert_of holds -1 - (output - experts) for them.
extern "C" int kipp_moe_route_scores(int* expert_of, float* weight_of, const void* h, long long ldh, int dtype,
                                     const float* router, const float* correction, int tokens, int hidden, int outputs,
                                     int experts, int top, float weight_scale, void* stream) {
    if (experts < 0 || experts > outputs) return KIPP_ERR_ARG;
    return moe_route_any(expert_of, weight_of, h, ldh, dtype, router, correction, tokens, hidden, outputs, top, 1, experts,
                         weight_scale, stream);
}

// sorted_pair [pairs], tile_info [3 x kipp_moe_max_tiles], n_tiles [1]
extern "C" int kipp_moe_lists(int* sorted_pair, int* tile_info, int* n_tiles, const int* expert_of, int pairs, int experts,
                              void* stream) {
    if (pairs <= 0) return 0;
    if (experts <= 0 || experts > 2048) return KIPP_ERR_ARG;
    return kipp_launch(moe_lists_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int), (cudaStream_t)stream, 1,
                       sorted_pair, tile_info, n_tiles, expert_of, pairs, experts);
}

// One product of every tile: out rows = act(A rows x W[expert]^T).  gather: a row of A is the pair's
// token (else its place in the sorted list); scatter: a row of out is the pair (else its place in the
// sorted list).  A and W in `dtype`; out in `out_dtype`.  On the CUDA cores: float32, and sizes the
// grouped tensor-core products cannot take.
extern "C" int kipp_moe_gemm(void* out, int out_dtype, long long ldo, const void* a, long long lda, const void* w,
                             long long w_expert, int dtype, int N, int K, int top, int gather, int scatter, int act,
                             const int* sorted_pair, const int* tile_info, const int* n_tiles, int pairs, int experts,
                             void* stream) {
    if (pairs <= 0) return 0;
    if (N <= 0 || K <= 0 || top <= 0 || experts <= 0) return KIPP_ERR_ARG;
    GemmArgs g;
    g.out = out; g.ldo = ldo; g.a = a; g.lda = lda; g.w = w; g.w_expert = w_expert;
    g.N = N; g.K = K; g.top = top; g.gather = gather; g.scatter = scatter; g.act = act;
    g.sorted_pair = sorted_pair; g.tile_info = tile_info; g.n_tiles = n_tiles;
    const int tiles = kipp_moe_max_tiles(pairs, experts);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)tiles);
    if (dtype == KIPP_DT_F32 && out_dtype == KIPP_DT_F32) return kipp_launch(moe_gemm_kernel<float, float>, grid, dim3(256), 0, s, 1, g);
    if (dtype == KIPP_DT_BF16 && out_dtype == KIPP_DT_BF16) return kipp_launch(moe_gemm_kernel<bf16, bf16>, grid, dim3(256), 0, s, 1, g);
    if (dtype == KIPP_DT_BF16 && out_dtype == KIPP_DT_F32) return kipp_launch(moe_gemm_kernel<bf16, float>, grid, dim3(256), 0, s, 1, g);
    return KIPP_ERR_DTYPE;
}

// y[t, :] += sum_k weight_of[t, k] * rows[r, :], k in order; r = t * top + k, or place_of_pair[t * top + k] if given.
extern "C" int kipp_moe_combine(float* y, const float* rows, const float* weight_of, int tokens, int hidden, int top,
                                const int* place_of_pair, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || top <= 0) return KIPP_ERR_ARG;
    // (an element's steps wait for one another, the loads behind the store before them: few elements per thread)
    return kipp_launch(moe_combine_kernel, dim3((unsigned)tokens), dim3(hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128), 0,
                       (cudaStream_t)stream, 1, y, rows, weight_of, hidden, top, place_of_pair);
}

// The same where pairs with expert_of < 0 stand for the token's own input h [tokens, ldh] (`dtype`).
extern "C" int kipp_moe_combine_identity(float* y, const float* rows, const float* weight_of, const int* expert_of,
                                         const void* h, long long ldh, int dtype, int tokens, int hidden, int top,
                                         const int* place_of_pair, void* stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || top <= 0 || expert_of == nullptr || h == nullptr) return KIPP_ERR_ARG;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(moe_combine_identity_kernel<float>, dim3((unsigned)tokens), dim3(hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128), 0, (cudaStream_t)stream, 1, y,
                           rows, weight_of, expert_of, (const float*)h, ldh, hidden, top, place_of_pair);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(moe_combine_identity_kernel<bf16>, dim3((unsigned)tokens), dim3(hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128), 0, (cudaStream_t)stream, 1, y,
                           rows, weight_of, expert_of, (const bf16*)h, ldh, hidden, top, place_of_pair);
    return KIPP_ERR_DTYPE;
}

// Tiles of `tile_rows` rows that `pairs` pairs over `experts` experts can need at most when every
// expert's rows are padded to whole tiles.
extern "C" int kipp_moe_max_padded_tiles(int pairs, int experts, int tile_rows) {
    return pairs / tile_rows + (experts < pairs ? experts : pairs);
}

// place_of_pair [pairs], expert_of_tile [kipp_moe_max_padded_tiles], n_tiles [1]
extern "C" int kipp_moe_padded_lists(int* place_of_pair, int* expert_of_tile, int* n_tiles, const int* expert_of, int pairs,
                                     int experts, int tile_rows, void* stream) {
    if (pairs <= 0) return 0;
    if (experts <= 0 || experts > 2048 || tile_rows <= 0) return KIPP_ERR_ARG;
    return kipp_launch(moe_padded_lists_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int), (cudaStream_t)stream,
                       1, place_of_pair, expert_of_tile, n_tiles, expert_of, pairs, experts, tile_rows);
}

// dst[place_of_pair[p], 0 .. hidden) = src[p / top, 0 .. hidden), bfloat16, hidden and ld_src multiples of 8.
extern "C" int kipp_moe_gather_rows(void* dst, const void* src, long long ld_src, const int* place_of_pair, int pairs,
                                    int top, int hidden, void* stream) {
    if (pairs <= 0) return 0;
    if (hidden <= 0 || hidden % 8 || ld_src % 8 || top <= 0 || (((uintptr_t)dst | (uintptr_t)src) & 15)) return KIPP_ERR_ARG;
    return kipp_launch(moe_gather_rows_kernel, dim3((unsigned)((pairs + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, 1,
                       (uint4*)dst, (const uint4*)src, ld_src / 8, hidden / 8, place_of_pair, pairs, top);
}
