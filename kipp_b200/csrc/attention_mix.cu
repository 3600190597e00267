// Paged attention whose heads talk to one another before the softmax, with a
// window that keeps the first tokens of a sequence, and with value heads of a
// size of their own.
//
// For a query at position p the visible keys are j <= p with p - j < window
// (window 0: every j <= p) or j < keep_first; kept keys stay at their true
// positions.  Scores: s[h][j] = scale * (q_h . k_{g(h)}[j]) with g(h) = h /
// (n_q / n_kv); if a mixing matrix M [n_q, n_q] is given the softmax of head h
// runs over sum_g M[h][g] s[g][j].  o_h = softmax . v_{g(h)}, times out_scale.
// Because every head's score of a (query, key) pair is needed to mix one of
// them, a unit of work holds all heads of its query.
//
// Scores, the mix, the softmax and the weighted sum are float32 in both element
// types.  Keys are walked in tiles of 32 aligned to absolute positions (first
// the kept tokens the window has left behind, then the window), so the order of
// every sum depends on the token's own position only: not on how the prompt was
// cut, on the batch, or on the pages.
//
// Options beside the mix (MixExtras, all off by default), each of which needs all heads of a
// query in one place or changes what a key row holds:
//   sink            a learned number per head joins the softmax's denominator as e^sink: it has no
//                   key and no value, is not scaled, and counts once (after the runs are merged);
//   key_maps        every head has several score maps (n_q counts the maps, head by head); a key
//                   row of a kv head holds key_maps keys of head_dim side by side, and all maps of
//                   a head read the same values;
//   diff            with two maps per head the output is o = a1 - lambda a2, divided by its root
//                   mean square over the value size and multiplied by diff_scale;
//   values_in_keys  the value of a key is the first v_dim elements of its key row (a latent that is
//                   both key and value; there are no value pages);
//   gate            head h of token t is multiplied by sigmoid(gate[t, gate_off + h]);
//   chunk           instead of a window: the positions are cut into blocks of `chunk` counted from
//                   position 0 of the sequence, and a query sees the keys j <= p of its own block.
//
// attention_mix_kernel: one block per token (and, in steps of few tokens, per run of
// SPLIT_TILES key tiles of that token: the runs' partial results -- maximum, sum and
// unnormalised output per head -- are merged in run order by attention_mix_merge_kernel; how a
// token's keys are cut into runs depends on its own position only).  Per tile the block gathers
// the keys and values of every key/value head from the pages into shared memory with 16-byte
// loads, forms all heads' scores from there, mixes and masks them, advances the softmax of each
// head, and adds the weighted values.  Any sizes, both element types.
#include "common.cuh"
#include <math.h>
#include <algorithm>

namespace {
constexpr int KT = 32;             // keys per tile
constexpr int THREADS = 256;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<bf16> { static constexpr int N = 8; };

__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const float* __restrict__ row, int n, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int d = 0; d < n; d += 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + d);
            acc = fmaf(qs[d], v.x, acc); acc = fmaf(qs[d + 1], v.y, acc);
            acc = fmaf(qs[d + 2], v.z, acc); acc = fmaf(qs[d + 3], v.w, acc);
        }
    } else {
        for (int d = 0; d < n; ++d) acc = fmaf(qs[d], row[d], acc);
    }
    return acc;
}
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const bf16* __restrict__ row, int n, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int d = 0; d < n; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + d);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc = fmaf(qs[d + 2 * i], __low2float(p[i]), acc);
                acc = fmaf(qs[d + 2 * i + 1], __high2float(p[i]), acc);
            }
        }
    } else {
        for (int d = 0; d < n; ++d) acc = fmaf(qs[d], __bfloat162float(row[d]), acc);
    }
    return acc;
}

// The visible keys of position p as two runs: [0, kept) and [first, p].
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
    return chunk > 0 ? pos - pos % chunk : (window > 0 ? max(0, pos - window + 1) : 0);
}
__device__ __forceinline__ void visible_runs(int pos, int window, int keep_first, int chunk, int& first, int& kept) {
    first = first_visible(pos, window, chunk);
    kept = chunk > 0 ? 0 : min(keep_first, first);
}

constexpr int SPLIT_TILES = 2;     // key tiles per run when a step's tokens are cut into runs

// The layout is the host's AttentionExtras (kernels.hpp).
struct MixExtras {
    const float* sink;         // [n_q] or null
    int key_maps;              // score maps per head (at least 1)
    int values_in_keys;
    int diff;                  // 1: two maps per head are combined (key_maps must be 2)
    float lambda, diff_eps, diff_scale;
    const void* gate;          // [tokens, ld_gate] in the compute type, or null
    long long ld_gate;
    int gate_off;
    int chunk;                 // > 0: blocks of this many positions bound what a query sees (no window then)
    float softcap;             // > 0: a scaled score s becomes softcap * tanh(s / softcap) (before mix, mask and softmax)
};

__device__ __forceinline__ float sigmoid_(float x) { return 1.0f / (1.0f + expf(-x)); }
// the scaled score, capped where the mixer asks for it
__device__ __forceinline__ float capped(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

// The factor that turns a head's unnormalised sum (maximum m, sum of weights l) into its output:
// with a sink the denominator also holds e^sink.
__device__ __forceinline__ float softmax_factor(float m, float l, const float* sink, int h) {
    if (sink == nullptr) return l > 0.f ? 1.0f / l : 0.f;
    const float s = sink[h], top = fmaxf(m, s);
    const float w = m == -INFINITY ? 0.f : expf(m - top);
    return w / (l * w + expf(s - top));
}

// heads [nh][v_dim] (float32, shared memory, already divided by their denominators): heads
// h_first .. h_first + nh - 1 of the token -> their part of the token's row of the output: the maps
// of a head combined (h_first and nh are even then), the gate, the scale.
template <typename T>
__device__ __forceinline__ void finish_heads(T* __restrict__ out, const float* __restrict__ heads, int t, int n_q,
                                             int v_dim, float out_scale, const MixExtras& ex, int threads,
                                             int h_first, int nh) {
    const T* gate = static_cast<const T*>(ex.gate);
    if (!ex.diff) {
        for (int e = threadIdx.x; e < nh * v_dim; e += threads) {
            const int h = h_first + e / v_dim;
            float y = heads[e] * out_scale;
            if (gate != nullptr) y *= sigmoid_(to_f32(gate[(size_t)t * ex.ld_gate + ex.gate_off + h]));
            out[((size_t)t * n_q + h_first) * v_dim + e] = from_f32<T>(y);
        }
        return;
    }
    const int lane = threadIdx.x & 31, n_out = n_q / 2;
    for (int hl = threadIdx.x >> 5; hl < nh / 2; hl += threads >> 5) {
        const int h = h_first / 2 + hl;
        const float* a1 = heads + (size_t)(2 * hl) * v_dim;
        const float* a2 = a1 + v_dim;
        float ss = 0.f;
        for (int d = lane; d < v_dim; d += 32) {
            const float o = fmaf(-ex.lambda, a2[d], a1[d]);
            ss = fmaf(o, o, ss);
        }
        ss = warp_sum(ss);
        float f = ex.diff_scale * out_scale / sqrtf(ss / (float)v_dim + ex.diff_eps);
        if (gate != nullptr) f *= sigmoid_(to_f32(gate[(size_t)t * ex.ld_gate + ex.gate_off + h]));
        for (int d = lane; d < v_dim; d += 32)
            out[((size_t)t * n_out + h) * v_dim + d] = from_f32<T>(fmaf(-ex.lambda, a2[d], a1[d]) * f);
    }
}

// Rows of `elems` elements from the pages into shared memory (row stride ld), 16 bytes at a time
// where the sizes allow; rows of keys that are not visible become zeros.
template <typename T>
__device__ __forceinline__ void stage_rows(T* __restrict__ dst, int ld, const T* __restrict__ pages, int elems,
                                           int n_kv, int g0, int ng, int page_size, const int* pg, const int* sl,
                                           bool vec) {
    // (a row of the pages has `elems` elements)
    // kv heads g0 .. g0 + ng - 1; row (g - g0) * KT + key of dst
    constexpr int VEC = Vec<T>::N;
    if (vec) {
        // asynchronous copies: every chunk of the tile is in flight at once (the caller waits);
        // eight threads per row (row = kv head x key), each every eighth 16-byte chunk
        const int chunks = elems / VEC;
        for (int rr = threadIdx.x >> 3; rr < ng * KT; rr += THREADS / 8) {
            const int jj = rr & (KT - 1), g = g0 + rr / KT;
            const bool ok = pg[jj] >= 0;
            const T* src = ok ? pages + (((size_t)pg[jj] * n_kv + g) * page_size + sl[jj]) * elems : pages;
            const uint32_t to = smem_address(dst + (size_t)rr * ld);
            for (int c = threadIdx.x & 7; c < chunks; c += 8) cp_async16(to + c * 16, ok ? src + c * VEC : src, ok ? 16 : 0);
        }
    } else {
        for (int i = threadIdx.x; i < ng * KT * elems; i += THREADS) {
            const int c = i % elems, jj = (i / elems) % KT, g = g0 + i / (elems * KT);
            dst[(size_t)(i / elems) * ld + c] =
                pg[jj] >= 0 ? pages[(((size_t)pg[jj] * n_kv + g) * page_size + sl[jj]) * elems + c] : from_f32<T>(0.f);
        }
    }
}

template <typename T> __host__ __device__ constexpr int row_pad() { return 16 / (int)sizeof(T); }   // 16 bytes: no bank conflicts between rows

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_mix_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pages,
                     const T* __restrict__ v_pages, const float* __restrict__ head_mix,
                     const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                     const int* __restrict__ block_table, int table_width, int page_size, int n_q, int n_kv,
                     int head_dim, int v_dim, float scale, int window, int keep_first, float out_scale,
                     int split, float* __restrict__ partial, int kv_stage, int* __restrict__ status,
                     const MixExtras ex) {
    // kv_stage: kv heads whose keys (then values) of a tile are in shared memory at a time; all of
    // them where they fit, else the tile is walked in passes over groups of kv heads
    extern __shared__ __align__(16) float smem[];
    const int maps = ex.key_maps, k_row = maps * head_dim;          // a key row holds the keys of all maps
    const int ldk = k_row + row_pad<T>(), ldv = v_dim + row_pad<T>();
    float* qs = smem;                              // [n_q][head_dim]
    float* mix = qs + n_q * head_dim;              // [n_q][n_q]
    float* sraw = mix + n_q * n_q;                 // [n_q][KT]
    float* pw = sraw + n_q * KT;                   // [n_q][KT]
    float* acc = pw + n_q * KT;                    // [n_q][v_dim]
    float* m_run = acc + n_q * v_dim;              // [n_q]
    float* l_run = m_run + n_q;                    // [n_q]
    float* corr = l_run + n_q;                     // [n_q]
    int* pg = reinterpret_cast<int*>(corr + n_q);  // [KT] page of key, -1 = not visible
    int* sl = pg + KT;                             // [KT] slot in page
    const size_t head_floats = ((size_t)n_q * head_dim + (size_t)n_q * n_q + 2 * (size_t)n_q * KT + (size_t)n_q * v_dim +
                                3 * (size_t)n_q + 2 * KT + 3) / 4 * 4;
    T* ktile = reinterpret_cast<T*>(smem + head_floats);           // [kv_stage][KT][ldk]
    T* vtile = ktile + (size_t)kv_stage * KT * ldk;                // [kv_stage][KT][ldv]
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = blockIdx.x;
    const int pos = positions[t];
    int first, kept;
    visible_runs(pos, window, keep_first, ex.chunk, first, kept);
    const int kept_tiles = (kept + KT - 1) / KT;
    const int win0 = first / KT;
    const int n_tiles = kept_tiles + pos / KT - win0 + 1;
    const int it0 = split ? blockIdx.y * SPLIT_TILES : 0;
    if (it0 >= n_tiles) return;                    // this token has fewer runs than the step's longest
    const int it1 = split ? min(n_tiles, it0 + SPLIT_TILES) : n_tiles;
    const int* table = block_table + (size_t)entry_of_token[t] * table_width;
    const int group = n_q / n_kv;                                   // score maps per kv head
    constexpr int VEC = Vec<T>::N;
    const bool kvec = k_row % VEC == 0 && (((uintptr_t)k_pages) & 15) == 0;
    const bool kdot = kvec && head_dim % VEC == 0;
    const bool vvec = v_dim % VEC == 0 && (((uintptr_t)v_pages) & 15) == 0;

    for (int i = tid; i < n_q * head_dim; i += THREADS) qs[i] = to_f32(q[(size_t)t * n_q * head_dim + i]);
    if (head_mix != nullptr)
        for (int i = tid; i < n_q * n_q; i += THREADS) mix[i] = head_mix[i];
    for (int i = tid; i < n_q * v_dim; i += THREADS) acc[i] = 0.f;
    for (int i = tid; i < n_q; i += THREADS) { m_run[i] = -INFINITY; l_run[i] = 0.f; corr[i] = 1.f; }

    for (int it = it0; it < it1; ++it) {
        const bool in_kept = it < kept_tiles;
        const int j0 = in_kept ? it * KT : (win0 + it - kept_tiles) * KT;
        const int lo = in_kept ? 0 : first, hi = in_kept ? kept : pos + 1;
        __syncthreads();
        if (tid < KT) {
            const int j = j0 + tid;
            int page = -1;
            if (j >= lo && j < hi) {
                page = j / page_size < table_width ? table[j / page_size] : -1;
                if (page < 0) atomicExch(status, 3);          // a needed key is not mapped
            }
            pg[tid] = page;
            sl[tid] = j % page_size;
        }
        __syncthreads();
        for (int g0 = 0; g0 < n_kv; g0 += kv_stage) {
            const int ng = min(kv_stage, n_kv - g0);
            if (g0 > 0) __syncthreads();                           // the pass before has read its keys
            stage_rows(ktile, ldk, k_pages, k_row, n_kv, g0, ng, page_size, pg, sl, kvec);
            if (g0 + ng >= n_kv && kv_stage >= n_kv && !ex.values_in_keys)   // one pass: the values can come at once
                stage_rows(vtile, ldv, v_pages, v_dim, n_kv, 0, n_kv, page_size, pg, sl, vvec);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
            for (int idx = tid; idx < ng * group * KT; idx += THREADS) {
                const int hl = idx / KT, jj = idx % KT, h = g0 * group + hl;
                sraw[h * KT + jj] = capped(dot_row(qs + h * head_dim, ktile + ((size_t)(hl / group) * KT + jj) * ldk + (h % maps) * head_dim,
                                            head_dim, kdot) * scale, ex.softcap);
            }
        }
        __syncthreads();
        for (int h = warp; h < n_q; h += THREADS / 32) {
            float s;
            if (head_mix != nullptr) {
                s = 0.f;
                for (int g = 0; g < n_q; ++g) s = fmaf(mix[h * n_q + g], sraw[g * KT + lane], s);
            } else {
                s = sraw[h * KT + lane];
            }
            if (pg[lane] < 0) s = -INFINITY;
            const float m_old = m_run[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            float p = 0.f, c = 1.f;
            if (m_new != -INFINITY) {
                p = s == -INFINITY ? 0.f : expf(s - m_new);
                c = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            }
            const float psum = warp_sum(p);
            pw[h * KT + lane] = p;
            __syncwarp();
            if (lane == 0) {
                l_run[h] = l_run[h] * c + psum;
                m_run[h] = m_new;
                corr[h] = c;
            }
        }
        __syncthreads();
        // rows of keys that are not visible hold zeros and have weight zero: no branch
        for (int g0 = 0; g0 < n_kv; g0 += kv_stage) {
            const int ng = min(kv_stage, n_kv - g0);
            if (kv_stage < n_kv) {                                  // several passes: this group's values now
                __syncthreads();
                stage_rows(vtile, ldv, v_pages, v_dim, n_kv, g0, ng, page_size, pg, sl, vvec);
                cp_async_commit();
                cp_async_wait<0>();
                __syncthreads();
            }
            for (int el = tid; el < ng * group * v_dim; el += THREADS) {
                const int hl = el / v_dim, d = el % v_dim, h = g0 * group + hl, e = h * v_dim + d;
                // (values that are the head of their key row are read where the keys were staged)
                const int ldx = ex.values_in_keys ? ldk : ldv;
                const T* vcol = (ex.values_in_keys ? ktile : vtile) + (size_t)(hl / group) * KT * ldx + d;
                const float* ph = pw + h * KT;
                float a0 = acc[e] * corr[h], a1 = 0.f;
#pragma unroll 8
                for (int jj = 0; jj < KT; jj += 2) {
                    a0 = fmaf(ph[jj], to_f32(vcol[(size_t)jj * ldx]), a0);
                    a1 = fmaf(ph[jj + 1], to_f32(vcol[(size_t)(jj + 1) * ldx]), a1);
                }
                acc[e] = a0 + a1;
            }
        }
    }
    __syncthreads();
    if (split) {
        // this run's maximum, sum and unnormalised output per head: [token][run][head][2 + v_dim]
        float* dst = partial + ((size_t)t * gridDim.y + blockIdx.y) * n_q * (v_dim + 2);
        for (int e = tid; e < n_q * v_dim; e += THREADS) dst[(size_t)(e / v_dim) * (v_dim + 2) + 2 + e % v_dim] = acc[e];
        for (int h = tid; h < n_q; h += THREADS) {
            dst[(size_t)h * (v_dim + 2)] = m_run[h];
            dst[(size_t)h * (v_dim + 2) + 1] = l_run[h];
        }
        return;
    }
    for (int e = tid; e < n_q * v_dim; e += THREADS) {
        const int h = e / v_dim;
        acc[e] *= softmax_factor(m_run[h], l_run[h], ex.sink, h);
    }
    __syncthreads();
    finish_heads(out, acc, t, n_q, v_dim, out_scale, ex, THREADS, 0, n_q);
}

// The runs of a token merged in run order: o = sum_r acc_r e^(m_r - M) / sum_r l_r e^(m_r - M).  A block
// takes MERGE_HEADS heads of a token: a warp per head forms the runs' weights once, then every
// thread sums its elements over the runs.
constexpr int MERGE_HEADS = 2;
template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_mix_merge_kernel(T* __restrict__ out, const float* __restrict__ partial, const int* __restrict__ positions,
                           int n_q, int v_dim, int window, int keep_first, int max_runs, float out_scale,
                           const MixExtras ex) {
    extern __shared__ __align__(16) float merged[];                 // [MERGE_HEADS][v_dim], weights [MERGE_HEADS][max_runs], factors
    float* wts = merged + MERGE_HEADS * v_dim;
    float* fac = wts + MERGE_HEADS * max_runs;
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, pos = positions[t], h_first = blockIdx.y * MERGE_HEADS;
    const int nh = min(MERGE_HEADS, n_q - h_first);
    int first, kept;
    visible_runs(pos, window, keep_first, ex.chunk, first, kept);
    const int n_tiles = (kept + KT - 1) / KT + pos / KT - first / KT + 1;
    const int runs = min(max_runs, (n_tiles + SPLIT_TILES - 1) / SPLIT_TILES);
    const float* src = partial + (size_t)t * max_runs * n_q * (v_dim + 2);
    const int lane = threadIdx.x & 31;
    for (int hl = threadIdx.x >> 5; hl < nh; hl += THREADS / 32) {
        const int h = h_first + hl;
        float m = -INFINITY;
        for (int r = lane; r < runs; r += 32) m = fmaxf(m, src[((size_t)r * n_q + h) * (v_dim + 2)]);
        m = warp_max(m);
        float l = 0.f;
        for (int r = lane; r < runs; r += 32) {
            const float* p = src + ((size_t)r * n_q + h) * (v_dim + 2);
            const float w = p[0] == -INFINITY ? 0.f : expf(p[0] - m);
            wts[hl * max_runs + r] = w;
            l = fmaf(p[1], w, l);
        }
        l = warp_sum(l);
        if (lane == 0) fac[hl] = softmax_factor(m, l, ex.sink, h);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nh * v_dim; e += THREADS) {
        const int hl = e / v_dim, d = e % v_dim;
        const float* p = src + (size_t)(h_first + hl) * (v_dim + 2) + 2 + d;
        float o = 0.f;
        for (int r = 0; r < runs; ++r) o = fmaf(p[(size_t)r * n_q * (v_dim + 2)], wts[hl * max_runs + r], o);
        merged[e] = o * fac[hl];
    }
    __syncthreads();
    finish_heads(out, merged, t, n_q, v_dim, out_scale, ex, THREADS, h_first, nh);
}

// Launches the merge of `runs` runs per token.
template <typename T>
int launch_merge(void* out, const float* partial, const int* positions, int tokens, int n_q, int v_dim, int window,
                 int keep_first, int runs, float out_scale, const MixExtras& ex, cudaStream_t s) {
    const size_t smem = ((size_t)MERGE_HEADS * (v_dim + runs + 1) + 3) * sizeof(float);
    auto merge = attention_mix_merge_kernel<T>;
    static size_t allowed = 0;
    if (smem > 48 * 1024 && smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(merge, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
        allowed = smem;
    }
    const dim3 grid((unsigned)tokens, (unsigned)((n_q + MERGE_HEADS - 1) / MERGE_HEADS));
    return kipp_launch(merge, grid, dim3(THREADS), smem, s, 1, (T*)out, partial, positions, n_q, v_dim, window, keep_first,
                       runs, out_scale, ex);
}

template <typename T>
int launch_mix(void* out, const void* q, const void* k_pages, const void* v_pages, const float* head_mix,
               const int* positions, const int* entry_of_token, const int* block_table, int table_width, int page_size,
               int tokens, int n_q, int n_kv, int head_dim, int v_dim, float scale, int window, int keep_first,
               float out_scale, int runs, float* partial, int* status, const MixExtras& ex, cudaStream_t s) {
    const size_t head_floats = ((size_t)n_q * head_dim + (size_t)n_q * n_q + 2 * (size_t)n_q * KT + (size_t)n_q * v_dim +
                                3 * (size_t)n_q + 2 * KT + 3) / 4 * 4;
    // kv heads staged at a time: all of them within about 100 KB of shared memory, else as many as fit
    const size_t per_kv = (size_t)KT * ((size_t)ex.key_maps * head_dim + row_pad<T>() +
                                        (ex.values_in_keys ? 0 : v_dim + row_pad<T>())) * sizeof(T);
    const size_t head_bytes = head_floats * sizeof(float), budget = 100 * 1024;
    int kv_stage = n_kv;
    if (head_bytes + per_kv * n_kv > budget)
        kv_stage = (int)std::max<size_t>(1, std::min<size_t>((size_t)n_kv, budget > head_bytes ? (budget - head_bytes) / per_kv : 1));
    const size_t smem = head_bytes + per_kv * kv_stage;
    if (smem > 200 * 1024) return KIPP_ERR_ARG;
    if (ex.values_in_keys && kv_stage < n_kv) return KIPP_ERR_ARG;     // the keys of a tile must still be there
    auto kernel = attention_mix_kernel<T>;
    static size_t allowed = 0;
    if (smem > 48 * 1024 && smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
        allowed = smem;
    }
    const int split = runs > 1 ? 1 : 0;
    int rc = kipp_launch(kernel, dim3((unsigned)tokens, (unsigned)(split ? runs : 1)), dim3(THREADS), smem, s, 1, (T*)out,
                         (const T*)q, (const T*)k_pages, (const T*)v_pages, head_mix, positions, entry_of_token,
                         block_table, table_width, page_size, n_q, n_kv, head_dim, v_dim, scale, window, keep_first,
                         out_scale, split, partial, kv_stage, status, ex);
    if (rc || !split) return rc;
    return launch_merge<T>(out, partial, positions, tokens, n_q, v_dim, window, keep_first, runs, out_scale, ex, s);
}

// ---------------------------------------------------------------------------
// Prompt portions in bfloat16 on the tensor cores (mma.sync m16n8k16).  A block of 8 warps
// takes 8 consecutive queries of one entry (work item = (entry, first token)) and ALL heads.  The
// products are formed transposed so that the 8 queries are the instruction's N: per tile of 32
// keys  S^T[key][query] = K Q^T  for every head (keys as M, head_dim as K), the scores go to
// shared memory in float32, are mixed over the heads and masked per (query, key), each (head,
// query) row takes its softmax step in a warp (lane = key), and  O^T[value dim][query] +=
// V^T P^T  (value dims as M, keys as K) adds to accumulators that stay in the registers of the
// warp that owns the head.  The weights P keep float32 precision through the 16-bit product:
// P = hi + lo with hi = bf16(P), lo = bf16(P - hi), two products into the same accumulator.
// K and V tiles share one buffer: V is fetched (asynchronously) while the softmax runs.
// Of the options of MixExtras it takes score maps (a key row holds the keys of a head's maps side by
// side; with two maps a warp owns both maps of its heads, so that it combines them from its own
// registers), the sink and the gate; not values that lie in their key rows.
constexpr int QB = 8;
constexpr int MMA_THREADS = 256;

__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct MmaSmem {
    int ldq, ldkv, lds, ldp;
    size_t qs, kv, phi, plo, sraw, mix, m_run, l_run, corr, pg, bytes;     // byte offsets
    // k_row: elements of a key row (head_dim x score maps per head)
    __host__ __device__ MmaSmem(int n_q, int n_kv, int head_dim, int v_dim, int k_row) {
        ldq = head_dim + 8;
        ldkv = (k_row > v_dim ? k_row : v_dim) + 8;
        lds = KT + 1;
        ldp = KT + 8;
        size_t at = 0;
        qs = at; at += (size_t)n_q * QB * ldq * 2;
        kv = at; at += (size_t)n_kv * KT * ldkv * 2;
        phi = at; at += (size_t)n_q * QB * ldp * 2;
        plo = at; at += (size_t)n_q * QB * ldp * 2;
        sraw = at; at += (size_t)n_q * QB * lds * 4;
        mix = at; at += (size_t)n_q * n_q * 4;
        m_run = at; at += (size_t)n_q * QB * 4;
        l_run = at; at += (size_t)n_q * QB * 4;
        corr = at; at += (size_t)n_q * QB * 4;
        pg = at; at += 2 * KT * 4;
        bytes = at;
    }
};

template <int HPW, int VB>
__global__ void __launch_bounds__(MMA_THREADS)
attention_mix_mma_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                         const bf16* __restrict__ v_pages, const float* __restrict__ head_mix,
                         const int* __restrict__ work, const int* __restrict__ q_start,
                         const int* __restrict__ context_len, const int* __restrict__ block_table, int table_width,
                         int page_size, int n_q_all, int n_kv_all, int head_dim, int v_dim, float scale, int window,
                         int keep_first, float out_scale, int* __restrict__ status, const MixExtras ex, int kv_per_block) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int maps = ex.key_maps, k_row = maps * head_dim;
    // Without a mix the kv heads need nothing of one another: blockIdx.y takes kv_per_block of them with
    // their query heads (n_q, n_kv and every head index below are the block's own; h_first and g_first
    // lead back to the model's).  With a mix one block holds them all.
    const int group = n_q_all / n_kv_all;
    const int g_first = blockIdx.y * kv_per_block, h_first = g_first * group;
    const int n_kv = min(kv_per_block, n_kv_all - g_first), n_q = n_kv * group;
    const MmaSmem L(kv_per_block * group, kv_per_block, head_dim, v_dim, k_row);
    // the heads a warp owns: warp, warp + 8, ...; with two maps per head both maps of heads warp, warp + 8, ...
    const bool pairs = maps == 2;
#define KIPP_OWNED_HEAD(hh) (pairs ? 2 * (warp + 8 * ((hh) >> 1)) + ((hh) & 1) : warp + 8 * (hh))
    bf16* qs = reinterpret_cast<bf16*>(raw + L.qs);
    bf16* kv = reinterpret_cast<bf16*>(raw + L.kv);
    bf16* phi = reinterpret_cast<bf16*>(raw + L.phi);
    bf16* plo = reinterpret_cast<bf16*>(raw + L.plo);
    float* sraw = reinterpret_cast<float*>(raw + L.sraw);
    float* mix = reinterpret_cast<float*>(raw + L.mix);
    float* m_run = reinterpret_cast<float*>(raw + L.m_run);
    float* l_run = reinterpret_cast<float*>(raw + L.l_run);
    float* corr = reinterpret_cast<float*>(raw + L.corr);
    int* pg = reinterpret_cast<int*>(raw + L.pg);
    int* sl = pg + KT;
    const int ldq = L.ldq, ldkv = L.ldkv, lds = L.lds, ldp = L.ldp;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;                      // fragment coordinates
    const int e = work[2 * blockIdx.x], t0 = work[2 * blockIdx.x + 1];
    const int row0 = q_start[e] + t0;
    const int n_tok = min(QB, q_start[e + 1] - row0);
    const int pos0 = context_len[e] + t0;                           // position of the block's first query
    const int pos_hi = pos0 + n_tok - 1;
    const int* table = block_table + (size_t)e * table_width;

    // the block's queries (zero rows beyond the entry's end), the mix, the running softmax state
    const int qchunks = head_dim / 8;
    for (int i = tid; i < n_q * QB * qchunks; i += MMA_THREADS) {
        const int c = i % qchunks, r = (i / qchunks) % QB, h = i / (qchunks * QB);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_tok) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + r) * n_q_all + h_first + h) * head_dim + c * 8);
        *reinterpret_cast<uint4*>(qs + ((size_t)h * QB + r) * ldq + c * 8) = v;
    }
    if (head_mix != nullptr)                                        // transposed: mix[g][h], the heads a lane mixes side by side
        for (int i = tid; i < n_q * n_q; i += MMA_THREADS) mix[(i % n_q) * n_q + i / n_q] = head_mix[i];
    for (int i = tid; i < n_q * QB; i += MMA_THREADS) { m_run[i] = -INFINITY; l_run[i] = 0.f; corr[i] = 1.f; }
    float o[HPW][VB][4];
#pragma unroll
    for (int a = 0; a < HPW; ++a)
#pragma unroll
        for (int b = 0; b < VB; ++b) o[a][b][0] = o[a][b][1] = o[a][b][2] = o[a][b][3] = 0.f;

    // key tiles any query of the block sees: the kept tokens that lie before the window's first
    // tile, then the window's tiles (a kept token inside those is met there)
    const int first_lo = first_visible(pos0, window, ex.chunk);
    const int kept_hi = window > 0 && ex.chunk == 0 ? min(keep_first, pos_hi + 1) : 0;
    const int win0 = first_lo / KT;
    const int kept_only = min((kept_hi + KT - 1) / KT, win0);
    const int n_tiles = kept_only + pos_hi / KT - win0 + 1;
    const int kchunks = k_row / 8, vchunks = v_dim / 8;
    for (int it = 0; it < n_tiles; ++it) {
        const int j0 = it < kept_only ? it * KT : (win0 + it - kept_only) * KT;
        __syncthreads();                                            // the tile before is done with kv and P
        if (tid < KT) {
            const int j = j0 + tid;
            int page = -1;
            if (j <= pos_hi && (j >= first_lo || j < kept_hi)) {    // a key some query of the block may see
                page = j / page_size < table_width ? table[j / page_size] : -1;
                if (page < 0) atomicExch(status, 3);
            }
            pg[tid] = page;
            sl[tid] = j % page_size;
        }
        __syncthreads();
        // eight threads per row of the tile (row = kv head x key), each every eighth 16-byte chunk
        for (int rr = tid >> 3; rr < n_kv * KT; rr += MMA_THREADS / 8) {
            const int jj = rr & (KT - 1), g = rr / KT;
            const bool ok = pg[jj] >= 0;
            const bf16* src = ok ? k_pages + (((size_t)pg[jj] * n_kv_all + g_first + g) * page_size + sl[jj]) * k_row : k_pages;
            const uint32_t dst = smem_address(kv + (size_t)rr * ldkv);
            for (int c = tid & 7; c < kchunks; c += 8) cp_async16(dst + c * 16, ok ? src + c * 8 : src, ok ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        // ---- S^T = K Q^T for the heads this warp owns
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const int h = KIPP_OWNED_HEAD(hh);
            if (h >= n_q) break;
            const bf16* kg = kv + (size_t)(h / group) * KT * ldkv + (h % maps) * head_dim;
            const bf16* qh = qs + (size_t)h * QB * ldq;
            float c[2][4];
#pragma unroll
            for (int mb = 0; mb < 2; ++mb) c[mb][0] = c[mb][1] = c[mb][2] = c[mb][3] = 0.f;
            for (int k0 = 0; k0 < head_dim; k0 += 16) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(qh + (size_t)gid * ldq + k0 + tig * 2);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(qh + (size_t)gid * ldq + k0 + 8 + tig * 2);
#pragma unroll
                for (int mb = 0; mb < 2; ++mb) {
                    const bf16* kr = kg + (size_t)(mb * 16 + gid) * ldkv + k0 + tig * 2;
                    uint32_t a[4];
                    a[0] = *reinterpret_cast<const uint32_t*>(kr);
                    a[1] = *reinterpret_cast<const uint32_t*>(kr + 8 * ldkv);
                    a[2] = *reinterpret_cast<const uint32_t*>(kr + 8);
                    a[3] = *reinterpret_cast<const uint32_t*>(kr + 8 * ldkv + 8);
                    mma_16816(c[mb], a, b0, b1);
                }
            }
            float* sh = sraw + (size_t)h * QB * lds;
#pragma unroll
            for (int mb = 0; mb < 2; ++mb) {
                const int key = mb * 16 + gid;
                sh[(tig * 2) * lds + key] = capped(c[mb][0] * scale, ex.softcap);
                sh[(tig * 2 + 1) * lds + key] = capped(c[mb][1] * scale, ex.softcap);
                sh[(tig * 2) * lds + key + 8] = capped(c[mb][2] * scale, ex.softcap);
                sh[(tig * 2 + 1) * lds + key + 8] = capped(c[mb][3] * scale, ex.softcap);
            }
        }
        __syncthreads();                                            // all scores are there; K is no longer needed
        for (int rr = tid >> 3; rr < n_kv * KT; rr += MMA_THREADS / 8) {
            const int jj = rr & (KT - 1), g = rr / KT;
            const bool ok = pg[jj] >= 0;
            const bf16* src = ok ? v_pages + (((size_t)pg[jj] * n_kv_all + g_first + g) * page_size + sl[jj]) * v_dim : v_pages;
            const uint32_t dst = smem_address(kv + (size_t)rr * ldkv);
            for (int c = tid & 7; c < vchunks; c += 8) cp_async16(dst + c * 16, ok ? src + c * 8 : src, ok ? 16 : 0);
        }
        cp_async_commit();
        // ---- mix, mask, softmax step: warp = query, lane = key, four heads at a time: the four
        // rows share each score they mix, and their chains of dependent shuffles overlap
        constexpr int RI = 4;
        static_assert(MMA_THREADS / 32 == QB, "one warp per query of the block");
        const int r = warp, pos = pos0 + r, j = j0 + lane;
        const bool vis = r < n_tok && pg[lane] >= 0 && j <= pos &&
                         (ex.chunk > 0 ? j >= pos - pos % ex.chunk : (window == 0 || pos - j < window || j < keep_first));
        for (int h0 = 0; h0 < n_q; h0 += RI) {
            float sv[RI], m_old[RI], mx[RI], p[RI], c[RI], ps[RI];
            int rows[RI];
#pragma unroll
            for (int i = 0; i < RI; ++i) {
                rows[i] = min(h0 + i, n_q - 1) * QB + r;               // a head beyond the last repeats it (not stored)
                sv[i] = 0.f;
            }
            if (head_mix != nullptr) {
                const bool four = (n_q & 3) == 0;
                for (int g = 0; g < n_q; ++g) {
                    const float sg = sraw[((size_t)g * QB + r) * lds + lane];
                    if (four) {
                        const float4 m4 = *reinterpret_cast<const float4*>(mix + g * n_q + h0);
                        sv[0] = fmaf(m4.x, sg, sv[0]); sv[1] = fmaf(m4.y, sg, sv[1]);
                        sv[2] = fmaf(m4.z, sg, sv[2]); sv[3] = fmaf(m4.w, sg, sv[3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < RI; ++i) sv[i] = fmaf(mix[g * n_q + min(h0 + i, n_q - 1)], sg, sv[i]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < RI; ++i) sv[i] = sraw[(size_t)rows[i] * lds + lane];
            }
#pragma unroll
            for (int i = 0; i < RI; ++i) {
                if (!vis) sv[i] = -INFINITY;
                m_old[i] = m_run[rows[i]];
                mx[i] = sv[i];
            }
#pragma unroll
            for (int x = 16; x > 0; x >>= 1) {
#pragma unroll
                for (int i = 0; i < RI; ++i) mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], x));
            }
#pragma unroll
            for (int i = 0; i < RI; ++i) {
                mx[i] = fmaxf(mx[i], m_old[i]);
                p[i] = 0.f;
                c[i] = 1.f;
                if (mx[i] != -INFINITY) {
                    p[i] = sv[i] == -INFINITY ? 0.f : expf(sv[i] - mx[i]);
                    c[i] = m_old[i] == -INFINITY ? 0.f : expf(m_old[i] - mx[i]);
                }
                ps[i] = p[i];
            }
#pragma unroll
            for (int x = 16; x > 0; x >>= 1) {
#pragma unroll
                for (int i = 0; i < RI; ++i) ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], x);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < RI; ++i) {
                if (h0 + i >= n_q) continue;
                const int row = rows[i];
                const bf16 hi = __float2bfloat16_rn(p[i]);
                phi[(size_t)row * ldp + lane] = hi;
                plo[(size_t)row * ldp + lane] = __float2bfloat16_rn(p[i] - __bfloat162float(hi));
                if (lane == 0) {
                    l_run[row] = l_run[row] * c[i] + ps[i];
                    m_run[row] = mx[i];
                    corr[row] = c[i];
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();                                            // V has landed, the weights are written
        // ---- O^T += V^T P^T for the heads this warp owns
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const int h = KIPP_OWNED_HEAD(hh);
            if (h >= n_q) break;
            const bf16* vg = kv + (size_t)(h / group) * KT * ldkv;
            const float c0 = corr[h * QB + tig * 2], c1 = corr[h * QB + tig * 2 + 1];
            uint32_t bh[2][2], bl[2][2];
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const size_t at = ((size_t)h * QB + gid) * ldp + ks * 16 + tig * 2;
                bh[ks][0] = *reinterpret_cast<const uint32_t*>(phi + at);
                bh[ks][1] = *reinterpret_cast<const uint32_t*>(phi + at + 8);
                bl[ks][0] = *reinterpret_cast<const uint32_t*>(plo + at);
                bl[ks][1] = *reinterpret_cast<const uint32_t*>(plo + at + 8);
            }
#pragma unroll
            for (int vb = 0; vb < VB; ++vb) {
                if (vb * 16 >= v_dim) break;
                float* acc = o[hh][vb];
                acc[0] *= c0; acc[1] *= c1; acc[2] *= c0; acc[3] *= c1;
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const unsigned short* v0 = reinterpret_cast<const unsigned short*>(vg) + (size_t)(ks * 16 + tig * 2) * ldkv + vb * 16 + gid;
                    uint32_t a[4];
                    a[0] = (uint32_t)v0[0] | ((uint32_t)v0[ldkv] << 16);
                    a[1] = (uint32_t)v0[8] | ((uint32_t)v0[ldkv + 8] << 16);
                    a[2] = (uint32_t)v0[8 * ldkv] | ((uint32_t)v0[9 * ldkv] << 16);
                    a[3] = (uint32_t)v0[8 * ldkv + 8] | ((uint32_t)v0[9 * ldkv + 8] << 16);
                    mma_16816(acc, a, bh[ks][0], bh[ks][1]);
                    mma_16816(acc, a, bl[ks][0], bl[ks][1]);
                }
            }
        }
    }
    __syncthreads();
    const bf16* gate = static_cast<const bf16*>(ex.gate);
    if (ex.diff) {
        // both maps of a head are this warp's: o = a1 - lambda a2 over the head's value dims, which lie
        // in this thread (value blocks) and in the lanes of equal tig (gid), per query
#pragma unroll
        for (int hh = 0; hh + 1 < HPW; hh += 2) {
            const int h = KIPP_OWNED_HEAD(hh);
            if (h + 1 >= n_q) break;
            float f1[2], f2[2], ss[2] = {0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                f1[c] = softmax_factor(m_run[h * QB + tig * 2 + c], l_run[h * QB + tig * 2 + c], ex.sink, h_first + h);
                f2[c] = softmax_factor(m_run[(h + 1) * QB + tig * 2 + c], l_run[(h + 1) * QB + tig * 2 + c], ex.sink, h_first + h + 1);
            }
#pragma unroll
            for (int vb = 0; vb < VB; ++vb) {
                if (vb * 16 >= v_dim) break;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float d = fmaf(-ex.lambda, o[hh + 1][vb][i] * f2[i & 1], o[hh][vb][i] * f1[i & 1]);
                    o[hh][vb][i] = d;
                    ss[i & 1] = fmaf(d, d, ss[i & 1]);
                }
            }
#pragma unroll
            for (int x = 4; x < 32; x <<= 1) {
                ss[0] += __shfl_xor_sync(0xffffffffu, ss[0], x);
                ss[1] += __shfl_xor_sync(0xffffffffu, ss[1], x);
            }
            const int n_out = n_q_all / 2, ho = (h_first + h) / 2;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                if (tig * 2 + c >= n_tok) continue;
                const int row = row0 + tig * 2 + c;
                float f = ex.diff_scale * out_scale / sqrtf(ss[c] / (float)v_dim + ex.diff_eps);
                if (gate != nullptr) f *= sigmoid_(to_f32(gate[(size_t)row * ex.ld_gate + ex.gate_off + ho]));
                bf16* dst = out + ((size_t)row * n_out + ho) * v_dim;
#pragma unroll
                for (int vb = 0; vb < VB; ++vb) {
                    if (vb * 16 >= v_dim) break;
                    dst[vb * 16 + gid] = __float2bfloat16_rn(o[hh][vb][c] * f);
                    dst[vb * 16 + gid + 8] = __float2bfloat16_rn(o[hh][vb][2 + c] * f);
                }
            }
        }
        return;
    }
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int h = KIPP_OWNED_HEAD(hh);
        if (h >= n_q) break;
        const int hm = h_first + h;                                     // the head's index in the model
        float i0 = softmax_factor(m_run[h * QB + tig * 2], l_run[h * QB + tig * 2], ex.sink, hm) * out_scale;
        float i1 = softmax_factor(m_run[h * QB + tig * 2 + 1], l_run[h * QB + tig * 2 + 1], ex.sink, hm) * out_scale;
        if (gate != nullptr) {
            if (tig * 2 < n_tok) i0 *= sigmoid_(to_f32(gate[(size_t)(row0 + tig * 2) * ex.ld_gate + ex.gate_off + hm]));
            if (tig * 2 + 1 < n_tok) i1 *= sigmoid_(to_f32(gate[(size_t)(row0 + tig * 2 + 1) * ex.ld_gate + ex.gate_off + hm]));
        }
#pragma unroll
        for (int vb = 0; vb < VB; ++vb) {
            if (vb * 16 >= v_dim) break;
            const int vd = vb * 16 + gid;
            if (tig * 2 < n_tok) {
                bf16* dst = out + ((size_t)(row0 + tig * 2) * n_q_all + hm) * v_dim;
                dst[vd] = __float2bfloat16_rn(o[hh][vb][0] * i0);
                dst[vd + 8] = __float2bfloat16_rn(o[hh][vb][2] * i0);
            }
            if (tig * 2 + 1 < n_tok) {
                bf16* dst = out + ((size_t)(row0 + tig * 2 + 1) * n_q_all + hm) * v_dim;
                dst[vd] = __float2bfloat16_rn(o[hh][vb][1] * i1);
                dst[vd + 8] = __float2bfloat16_rn(o[hh][vb][3] * i1);
            }
        }
    }
#undef KIPP_OWNED_HEAD
}

template <int HPW, int VB, typename... Args>
int launch_mix_mma(size_t smem, int items, int head_blocks, cudaStream_t s, Args... args) {
    auto kernel = attention_mix_mma_kernel<HPW, VB>;
    static size_t allowed = 0;
    if (smem > 48 * 1024 && smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
        allowed = smem;
    }
    return kipp_launch(kernel, dim3((unsigned)items, (unsigned)head_blocks), dim3(MMA_THREADS), smem, s, 1, args...);
}

// ---------------------------------------------------------------------------
// One key row per token that all heads share and that also holds the value (values_in_keys with
// one kv head: a latent), in bfloat16 on the tensor cores (mma.sync m16n8k16).  The heads need
// nothing of one another here, so the 16 rows of the instruction's M are 16 HEADS of one token: a
// block of 4 warps takes (token, group of 16 heads[, run of key tiles]).  Per tile of 32 keys:
// S[16 heads][32 keys] = Q K^T (each warp 8 keys, head_dim as K), scores to shared memory in
// float32, a softmax step per head row (lane = key), then O[16][v_dim] += P V with the value
// columns dealt out to the warps (VB tiles of 8 columns each, accumulators in registers).  The
// weights keep float32 precision through the 16-bit product (P = hi + lo, as above).  Tiles are
// aligned to absolute positions and cut into the same runs as the CUDA-core kernel's, so the
// same merge kernel finishes a step of few tokens; a prompt's tokens walk all their tiles and
// finish (sink, gate, scale) from their registers.
constexpr int SK_ROWS = 16, SK_THREADS = 128;

struct SharedKeySmem {
    int ldq, lds, ldp;
    size_t qs, ks, phi, plo, sraw, m_run, l_run, corr, pg, bytes;
    __host__ __device__ SharedKeySmem(int head_dim) {
        ldq = head_dim + 8;
        lds = KT + 1;
        ldp = KT + 8;
        size_t at = 0;
        qs = at; at += (size_t)SK_ROWS * ldq * 2;
        ks = at; at += (size_t)KT * ldq * 2;
        phi = at; at += (size_t)SK_ROWS * ldp * 2;
        plo = at; at += (size_t)SK_ROWS * ldp * 2;
        sraw = at; at += (size_t)SK_ROWS * lds * 4;
        m_run = at; at += SK_ROWS * 4;
        l_run = at; at += SK_ROWS * 4;
        corr = at; at += SK_ROWS * 4;
        pg = at; at += 2 * KT * 4;
        bytes = at;
    }
};

template <int VB>
__global__ void __launch_bounds__(SK_THREADS)
attention_shared_key_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ k_pages,
                            const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                            const int* __restrict__ block_table, int table_width, int page_size, int n_q,
                            int head_dim, int v_dim, float scale, int window, float out_scale, int split,
                            float* __restrict__ partial, int* __restrict__ status, const MixExtras ex) {
    extern __shared__ __align__(16) unsigned char raw[];
    const SharedKeySmem L(head_dim);
    bf16* qs = reinterpret_cast<bf16*>(raw + L.qs);
    bf16* ks = reinterpret_cast<bf16*>(raw + L.ks);
    bf16* phi = reinterpret_cast<bf16*>(raw + L.phi);
    bf16* plo = reinterpret_cast<bf16*>(raw + L.plo);
    float* sraw = reinterpret_cast<float*>(raw + L.sraw);
    float* m_run = reinterpret_cast<float*>(raw + L.m_run);
    float* l_run = reinterpret_cast<float*>(raw + L.l_run);
    float* corr = reinterpret_cast<float*>(raw + L.corr);
    int* pg = reinterpret_cast<int*>(raw + L.pg);
    int* sl = pg + KT;
    const int ldq = L.ldq, lds = L.lds, ldp = L.ldp;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int t = blockIdx.x, h0 = blockIdx.y * SK_ROWS;
    const int pos = positions[t];
    const int first = first_visible(pos, window, ex.chunk);
    const int win0 = first / KT;
    const int n_tiles = pos / KT - win0 + 1;
    const int it0 = split ? blockIdx.z * SPLIT_TILES : 0;
    if (it0 >= n_tiles) return;
    const int it1 = split ? min(n_tiles, it0 + SPLIT_TILES) : n_tiles;
    const int* table = block_table + (size_t)entry_of_token[t] * table_width;

    const int chunks = head_dim / 8;
    for (int i = tid; i < SK_ROWS * chunks; i += SK_THREADS) {
        const int c = i % chunks, r = i / chunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (h0 + r < n_q) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * n_q + h0 + r) * head_dim + c * 8);
        *reinterpret_cast<uint4*>(qs + (size_t)r * ldq + c * 8) = v;
    }
    if (tid < SK_ROWS) { m_run[tid] = -INFINITY; l_run[tid] = 0.f; corr[tid] = 1.f; }
    float o[VB][4];
#pragma unroll
    for (int b = 0; b < VB; ++b) o[b][0] = o[b][1] = o[b][2] = o[b][3] = 0.f;
    const int col0 = warp * VB * 8;                                 // this warp's value columns

    for (int it = it0; it < it1; ++it) {
        const int j0 = (win0 + it) * KT;
        __syncthreads();                                            // the tile before is done with K and P
        if (tid < KT) {
            const int j = j0 + tid;
            int page = -1;
            if (j >= first && j <= pos) {
                page = j / page_size < table_width ? table[j / page_size] : -1;
                if (page < 0) atomicExch(status, 3);
            }
            pg[tid] = page;
            sl[tid] = j % page_size;
        }
        __syncthreads();
        for (int rr = tid >> 2; rr < KT; rr += SK_THREADS / 4) {    // four threads per key row
            const bool ok = pg[rr] >= 0;
            const bf16* src = ok ? k_pages + ((size_t)pg[rr] * page_size + sl[rr]) * head_dim : k_pages;
            const uint32_t dst = smem_address(ks + (size_t)rr * ldq);
            for (int c = tid & 3; c < chunks; c += 4) cp_async16(dst + c * 16, ok ? src + c * 8 : src, ok ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        // ---- S = Q K^T: this warp's 8 keys
        {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const bf16* kr = ks + (size_t)(warp * 8 + gid) * ldq + tig * 2;
            const bf16* qa = qs + (size_t)gid * ldq + tig * 2;
            for (int k0 = 0; k0 < head_dim; k0 += 16) {
                uint32_t a[4];
                a[0] = *reinterpret_cast<const uint32_t*>(qa + k0);
                a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * ldq + k0);
                a[2] = *reinterpret_cast<const uint32_t*>(qa + k0 + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * ldq + k0 + 8);
                mma_16816(c, a, *reinterpret_cast<const uint32_t*>(kr + k0), *reinterpret_cast<const uint32_t*>(kr + k0 + 8));
            }
            const int key = warp * 8 + tig * 2;
            sraw[gid * lds + key] = capped(c[0] * scale, ex.softcap);
            sraw[gid * lds + key + 1] = capped(c[1] * scale, ex.softcap);
            sraw[(gid + 8) * lds + key] = capped(c[2] * scale, ex.softcap);
            sraw[(gid + 8) * lds + key + 1] = capped(c[3] * scale, ex.softcap);
        }
        __syncthreads();
        // ---- a softmax step for four head rows per warp (lane = key)
        {
            const bool vis = pg[lane] >= 0;
            float sv[4], mx[4], p[4], ps[4], m_old[4], cf[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = warp * 4 + i;
                sv[i] = vis ? sraw[r * lds + lane] : -INFINITY;
                m_old[i] = m_run[r];
                mx[i] = sv[i];
            }
#pragma unroll
            for (int x = 16; x > 0; x >>= 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], x));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                mx[i] = fmaxf(mx[i], m_old[i]);
                p[i] = 0.f;
                cf[i] = 1.f;
                if (mx[i] != -INFINITY) {
                    p[i] = sv[i] == -INFINITY ? 0.f : expf(sv[i] - mx[i]);
                    cf[i] = m_old[i] == -INFINITY ? 0.f : expf(m_old[i] - mx[i]);
                }
                ps[i] = p[i];
            }
#pragma unroll
            for (int x = 16; x > 0; x >>= 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], x);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = warp * 4 + i;
                const bf16 hi = __float2bfloat16_rn(p[i]);
                phi[r * ldp + lane] = hi;
                plo[r * ldp + lane] = __float2bfloat16_rn(p[i] - __bfloat162float(hi));
                if (lane == 0) {
                    l_run[r] = l_run[r] * cf[i] + ps[i];
                    m_run[r] = mx[i];
                    corr[r] = cf[i];
                }
            }
        }
        __syncthreads();
        // ---- O += P V: the value of a key is the head of its row
        {
            const float c0 = corr[gid], c1 = corr[gid + 8];
            uint32_t ah[2][4], al[2][4];
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
                const int at = gid * ldp + s2 * 16 + tig * 2;
                ah[s2][0] = *reinterpret_cast<const uint32_t*>(phi + at);
                ah[s2][1] = *reinterpret_cast<const uint32_t*>(phi + at + 8 * ldp);
                ah[s2][2] = *reinterpret_cast<const uint32_t*>(phi + at + 8);
                ah[s2][3] = *reinterpret_cast<const uint32_t*>(phi + at + 8 * ldp + 8);
                al[s2][0] = *reinterpret_cast<const uint32_t*>(plo + at);
                al[s2][1] = *reinterpret_cast<const uint32_t*>(plo + at + 8 * ldp);
                al[s2][2] = *reinterpret_cast<const uint32_t*>(plo + at + 8);
                al[s2][3] = *reinterpret_cast<const uint32_t*>(plo + at + 8 * ldp + 8);
            }
#pragma unroll
            for (int b = 0; b < VB; ++b) {
                const int col = col0 + b * 8;
                if (col >= v_dim) break;
                o[b][0] *= c0; o[b][1] *= c0; o[b][2] *= c1; o[b][3] *= c1;
#pragma unroll
                for (int s2 = 0; s2 < 2; ++s2) {
                    const unsigned short* v0 = reinterpret_cast<const unsigned short*>(ks) + (size_t)(s2 * 16 + tig * 2) * ldq + col + gid;
                    const uint32_t b0 = (uint32_t)v0[0] | ((uint32_t)v0[ldq] << 16);
                    const uint32_t b1 = (uint32_t)v0[8 * ldq] | ((uint32_t)v0[9 * ldq] << 16);
                    mma_16816(o[b], ah[s2], b0, b1);
                    mma_16816(o[b], al[s2], b0, b1);
                }
            }
        }
    }
    __syncthreads();
    // rows gid and gid + 8 are heads h0 + gid and h0 + gid + 8; a thread holds columns col + 2 tig, + 1
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = gid + 8 * half, h = h0 + r;
        if (h >= n_q) continue;
        if (split) {
            float* dst = partial + (((size_t)t * gridDim.z + blockIdx.z) * n_q + h) * (v_dim + 2);
            if (warp == 0 && tig == 0) { dst[0] = m_run[r]; dst[1] = l_run[r]; }
#pragma unroll
            for (int b = 0; b < VB; ++b) {
                const int col = col0 + b * 8 + tig * 2;
                if (col0 + b * 8 >= v_dim) break;
                dst[2 + col] = o[b][2 * half];
                dst[2 + col + 1] = o[b][2 * half + 1];
            }
        } else {
            float f = softmax_factor(m_run[r], l_run[r], ex.sink, h) * out_scale;
            if (ex.gate != nullptr)
                f *= sigmoid_(to_f32(static_cast<const bf16*>(ex.gate)[(size_t)t * ex.ld_gate + ex.gate_off + h]));
            bf16* dst = out + ((size_t)t * n_q + h) * v_dim;
#pragma unroll
            for (int b = 0; b < VB; ++b) {
                const int col = col0 + b * 8 + tig * 2;
                if (col0 + b * 8 >= v_dim) break;
                *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[b][2 * half] * f, o[b][2 * half + 1] * f);
            }
        }
    }
}

template <int VB>
int launch_shared_key(void* out, const void* q, const void* k_pages, const int* positions, const int* entry_of_token,
                      const int* block_table, int table_width, int page_size, int tokens, int n_q, int head_dim,
                      int v_dim, float scale, int window, float out_scale, int runs, float* partial, int* status,
                      const MixExtras& ex, cudaStream_t s) {
    const size_t smem = SharedKeySmem(head_dim).bytes;
    auto kernel = attention_shared_key_kernel<VB>;
    static size_t allowed = 0;
    if (smem > 48 * 1024 && smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
        allowed = smem;
    }
    const int split = runs > 1 ? 1 : 0;
    const dim3 grid((unsigned)tokens, (unsigned)((n_q + SK_ROWS - 1) / SK_ROWS), (unsigned)(split ? runs : 1));
    int rc = kipp_launch(kernel, grid, dim3(SK_THREADS), smem, s, 1, (bf16*)out, (const bf16*)q, (const bf16*)k_pages,
                         positions, entry_of_token, block_table, table_width, page_size, n_q, head_dim, v_dim, scale,
                         window, out_scale, split, partial, status, ex);
    if (rc || !split) return rc;
    return launch_merge<bf16>(out, partial, positions, tokens, n_q, v_dim, window, 0, runs, out_scale, ex, s);
}
}  // namespace

// Whether the tensor-core kernel for one shared key row per token takes these sizes (bfloat16 only).
extern "C" int kipp_attention_shared_key_ok(int n_q, int head_dim, int v_dim) {
    if (n_q <= 0 || head_dim <= 0 || v_dim <= 0 || head_dim % 16 || v_dim % 8 || v_dim > head_dim || v_dim > 512) return 0;
    return SharedKeySmem(head_dim).bytes <= 200 * 1024 ? 1 : 0;
}

// n_q heads over one key row of head_dim per token whose first v_dim elements are its value.
// extras: sink and gate of MixExtras (values_in_keys is what this kernel is; no maps, no mix).
extern "C" int kipp_attention_shared_key(void* out, const void* q, const void* k_pages, const int* positions,
                                         const int* entry_of_token, const int* block_table, int table_width,
                                         int page_size, int tokens, int n_q, int head_dim, int v_dim, float scale,
                                         int window, float out_scale, int runs, float* partial, const void* extras,
                                         int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (!kipp_attention_shared_key_ok(n_q, head_dim, v_dim) || page_size <= 0 || window < 0 || runs < 1 ||
        (runs > 1 && partial == nullptr) || runs > 65535)
        return KIPP_ERR_ARG;
    if ((((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)out) & 15) != 0) return -3;
    MixExtras ex = {};
    ex.key_maps = 1;
    if (extras != nullptr) ex = *static_cast<const MixExtras*>(extras);
    if (ex.key_maps != 1 || ex.diff) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int vb = (v_dim + 31) / 32;
#define KIPP_SHARED_KEY(V)                                                                                            \
    return launch_shared_key<V>(out, q, k_pages, positions, entry_of_token, block_table, table_width, page_size,      \
                                tokens, n_q, head_dim, v_dim, scale, window, out_scale, runs, partial, status, ex, s)
    if (vb <= 1) KIPP_SHARED_KEY(1);
    if (vb <= 2) KIPP_SHARED_KEY(2);
    if (vb <= 4) KIPP_SHARED_KEY(4);
    if (vb <= 8) KIPP_SHARED_KEY(8);
    KIPP_SHARED_KEY(16);
#undef KIPP_SHARED_KEY
}

// Whether the tensor-core prompt kernel takes these sizes (bfloat16 only).
// kv heads a block of the tensor-core prompt kernel takes with their query heads (0: the kernel
// does not take these sizes): at most 32 score maps and 220 KB of shared memory; with a mix all of them.
extern "C" int kipp_attention_mix_mma_kv_per_block(int n_q, int n_kv, int head_dim, int v_dim, int maps, int mixed) {
    if (n_q <= 0 || n_kv <= 0 || n_q % n_kv || maps < 1 || maps > 2 || (n_q / n_kv) % maps) return 0;
    if (head_dim <= 0 || v_dim <= 0 || head_dim % 16 || v_dim % 16 || v_dim > 128) return 0;
    const int group = n_q / n_kv;
    for (int kvs = mixed ? n_kv : std::min(n_kv, 32 / std::max(group, 1)); kvs >= (mixed ? n_kv : 1); --kvs)
        if (kvs * group <= 32 && MmaSmem(kvs * group, kvs, head_dim, v_dim, maps * head_dim).bytes <= 220 * 1024) return kvs;
    return 0;
}
extern "C" int kipp_attention_mix_mma_maps_ok(int n_q, int n_kv, int head_dim, int v_dim, int maps) {
    return kipp_attention_mix_mma_kv_per_block(n_q, n_kv, head_dim, v_dim, maps, 1) > 0 ? 1 : 0;
}
extern "C" int kipp_attention_mix_mma_ok(int n_q, int n_kv, int head_dim, int v_dim) {
    return kipp_attention_mix_mma_maps_ok(n_q, n_kv, head_dim, v_dim, 1);
}
extern "C" int kipp_attention_mix_mma_tile() { return QB; }

// work: (entry, first token) per block of 8 tokens, over every entry of the step.  extras: score
// maps, their combination, sink and gate of MixExtras, or null.
extern "C" int kipp_attention_mix_mma_ex(void* out, const void* q, const void* k_pages, const void* v_pages,
                                         const float* head_mix, const int* work, int n_items, const int* q_start,
                                         const int* context_len, const int* block_table, int table_width,
                                         int page_size, int n_q, int n_kv, int head_dim, int v_dim, float scale,
                                         int window, int keep_first, float out_scale, const void* extras, int* status,
                                         void* stream) {
    if (n_items <= 0) return 0;
    MixExtras ex = {};
    ex.key_maps = 1;
    if (extras != nullptr) ex = *static_cast<const MixExtras*>(extras);
    if (ex.values_in_keys || (ex.diff && ex.key_maps != 2) || (ex.key_maps > 1 && head_mix != nullptr)) return KIPP_ERR_ARG;
    const int kvs = kipp_attention_mix_mma_kv_per_block(n_q, n_kv, head_dim, v_dim, ex.key_maps, head_mix != nullptr);
    if (kvs <= 0 || page_size <= 0 || window < 0 || keep_first < 0) return KIPP_ERR_ARG;
    if ((((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) != 0) return -3;
    const int n_q_blk = kvs * (n_q / n_kv), head_blocks = (n_kv + kvs - 1) / kvs;
    const size_t smem = MmaSmem(n_q_blk, kvs, head_dim, v_dim, ex.key_maps * head_dim).bytes;
    cudaStream_t s = (cudaStream_t)stream;
    // heads per warp; with two maps per head a warp owns whole heads, two maps each
    const int hpw = ex.key_maps == 2 ? 2 * ((n_q_blk / 2 + 7) / 8) : (n_q_blk + 7) / 8, vb = (v_dim + 15) / 16;
#define KIPP_MIX_MMA(H, V)                                                                                             \
    return launch_mix_mma<H, V>(smem, n_items, head_blocks, s, (bf16*)out, (const bf16*)q, (const bf16*)k_pages,       \
                                (const bf16*)v_pages, head_mix, work, q_start, context_len, block_table, table_width,  \
                                page_size, n_q, n_kv, head_dim, v_dim, scale, window, keep_first, out_scale, status, ex, \
                                kvs)
    if (hpw <= 1) { if (vb <= 2) KIPP_MIX_MMA(1, 2); if (vb <= 4) KIPP_MIX_MMA(1, 4); KIPP_MIX_MMA(1, 8); }
    if (hpw <= 2) { if (vb <= 2) KIPP_MIX_MMA(2, 2); if (vb <= 4) KIPP_MIX_MMA(2, 4); KIPP_MIX_MMA(2, 8); }
    if (vb <= 2) KIPP_MIX_MMA(4, 2);
    if (vb <= 4) KIPP_MIX_MMA(4, 4);
    KIPP_MIX_MMA(4, 8);
#undef KIPP_MIX_MMA
}
extern "C" int kipp_attention_mix_mma(void* out, const void* q, const void* k_pages, const void* v_pages,
                                      const float* head_mix, const int* work, int n_items, const int* q_start,
                                      const int* context_len, const int* block_table, int table_width,
                                      int page_size, int n_q, int n_kv, int head_dim, int v_dim, float scale,
                                      int window, int keep_first, float out_scale, int* status, void* stream) {
    return kipp_attention_mix_mma_ex(out, q, k_pages, v_pages, head_mix, work, n_items, q_start, context_len, block_table,
                                     table_width, page_size, n_q, n_kv, head_dim, v_dim, scale, window, keep_first,
                                     out_scale, nullptr, status, stream);
}

// Runs a step of `tokens` tokens is cut into (1: every token walks its keys in one block): few
// tokens with many keys are cut so that the GPU has blocks to run.  max_keys bounds the context.
extern "C" int kipp_attention_mix_runs(int tokens, int window, int keep_first, int max_keys) {
    if (tokens <= 0 || tokens > 64) return 1;
    const int win_tiles = window > 0 ? std::min((window - 1) / KT + 2, max_keys / KT + 1) : max_keys / KT + 1;
    const int kept_tiles = window > 0 ? (std::min(keep_first, max_keys) + KT - 1) / KT : 0;
    return std::max(1, (win_tiles + kept_tiles + SPLIT_TILES - 1) / SPLIT_TILES);
}
// float32 values of scratch a step cut into `runs` runs needs.
extern "C" long long kipp_attention_mix_scratch_floats(int tokens, int runs, int n_q, int v_dim) {
    return runs > 1 ? (long long)tokens * runs * n_q * (v_dim + 2) : 0;
}

// `extras`: the options of MixExtras, or null for none.  n_q counts score maps (heads x key_maps);
// out is [tokens, n_q, v_dim], or [tokens, n_q / 2, v_dim] when the maps of a head are combined.
extern "C" int kipp_attention_mix_ex(void* out, const void* q, const void* k_pages, const void* v_pages, int dtype,
                                     const float* head_mix, const int* positions, const int* entry_of_token,
                                     const int* block_table, int table_width, int page_size, int tokens, int n_q,
                                     int n_kv, int head_dim, int v_dim, float scale, int window, int keep_first,
                                     float out_scale, int runs, float* partial, const void* extras, int* status,
                                     void* stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || v_dim <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || page_size <= 0 || window < 0 ||
        keep_first < 0 || runs < 1 || (runs > 1 && partial == nullptr))
        return KIPP_ERR_ARG;
    MixExtras ex = {};
    ex.key_maps = 1;
    if (extras != nullptr) ex = *static_cast<const MixExtras*>(extras);
    if (ex.key_maps < 1 || (n_q / n_kv) % ex.key_maps || (ex.diff && ex.key_maps != 2) ||
        (ex.values_in_keys && v_dim > ex.key_maps * head_dim) || ex.chunk < 0 || (ex.chunk > 0 && window > 0))
        return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KIPP_DT_F32)
        return launch_mix<float>(out, q, k_pages, v_pages, head_mix, positions, entry_of_token, block_table, table_width,
                                 page_size, tokens, n_q, n_kv, head_dim, v_dim, scale, window, keep_first, out_scale, runs,
                                 partial, status, ex, s);
    if (dtype == KIPP_DT_BF16)
        return launch_mix<bf16>(out, q, k_pages, v_pages, head_mix, positions, entry_of_token, block_table, table_width,
                                page_size, tokens, n_q, n_kv, head_dim, v_dim, scale, window, keep_first, out_scale, runs,
                                partial, status, ex, s);
    return KIPP_ERR_DTYPE;
}

extern "C" int kipp_attention_mix(void* out, const void* q, const void* k_pages, const void* v_pages, int dtype,
                                  const float* head_mix, const int* positions, const int* entry_of_token,
                                  const int* block_table, int table_width, int page_size, int tokens, int n_q,
                                  int n_kv, int head_dim, int v_dim, float scale, int window, int keep_first,
                                  float out_scale, int runs, float* partial, int* status, void* stream) {
    return kipp_attention_mix_ex(out, q, k_pages, v_pages, dtype, head_mix, positions, entry_of_token, block_table,
                                 table_width, page_size, tokens, n_q, n_kv, head_dim, v_dim, scale, window, keep_first,
                                 out_scale, runs, partial, nullptr, status, stream);
}
