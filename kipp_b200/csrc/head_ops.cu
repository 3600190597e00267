// Work on the heads of a projection that the plain per-head norm + rotation kernel does not
// cover, and products that run head by head.
//
// kipp_head_segments: the columns of a projection row are cut into SEGMENTS of heads; each
// segment says where its heads lie, what is done to them and where they go:
//   bias       a float32 vector added first (the projection's bias);
//   norm       division of the head by its root mean square (eps inside the root), times a
//              weight of the head's size; or (norm_all) division of ALL heads of the segment by the
//              root mean square of the whole run of heads x dim columns, times a weight of that size;
//   rotation   of the dims [rot_off, rot_off + rot) of the head: pair (i, i + rot/2) turns by the
//              angle of the step's (cos, sin) table for the token; or (interleaved) pair (2i, 2i + 1);
//   target     a row of an activation buffer (queries), or the token's slot in the key or value
//              pages, where several heads of a segment may share one page row side by side
//              (two score maps of one key head; a latent and a rotated part that form one key).
// A warp takes one (token, head); all arithmetic is float32.  With this one kernel a mixer
// states its layout as data: keys made of parts, biases, rotation of a head's tail.
//
// kipp_head_matmul: out[t, h, :] = W_h a[t, h, :] for every head h, W_h [n, k] row-major, with
// float32 accumulation, all heads in one launch: in bfloat16 on the tensor cores (mma.sync); in
// 32-bit, or where rows do not start on 16-byte boundaries, few tokens by a kernel that reads the
// weights once and more tokens in tiles on the CUDA cores.  (Products with a latent: keys absorbed into queries, values expanded after the
// weighted sum.)
#include "common.cuh"
#include <math.h>

namespace {
constexpr int MAX_SEGMENTS = 4;

struct HeadSegment {
    int src_off, heads, dim, src_stride;     // columns of the projection row: head i at src_off + i * src_stride
    int rot_off, rot;                        // rotated dims of a head (rot 0: none)
    int target;                              // 0 activation rows, 1 key pages, 2 value pages
    int dst_off, dst_stride;                 // activation: head i at dst_off + i * dst_stride of the token's row
    int heads_per_row;                       // pages: this many heads side by side in one page row
    int norm_all;                            // 1: one mean square over all heads of the segment, norm_w [heads * dim]
    int interleaved;                         // 1: the rotation pairs dim 2i with dim 2i + 1
    const float* bias;                       // [heads * dim] or null
    const float* norm_w;                     // [dim] ([heads * dim] with norm_all) or null
    const float* cos_sin;                    // [tokens, rot / 2, 2] or null
    void* dst;                               // activation buffer of the compute type (target 0)
    long long ld_dst;
};

struct SegmentArgs {
    HeadSegment seg[MAX_SEGMENTS];
    int n_segments, total_heads;
    const void* src; long long ld_src;
    void* k_pages; void* v_pages;
    int k_row, v_row, n_kv;                  // elements of a page row, rows (kv heads) per slot
    const int* positions; const int* entry_of_token; const int* block_table;
    int table_width, page_size, tokens, write_cache;
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(128)
head_segments_kernel(const SegmentArgs a, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wg >= (long long)a.tokens * a.total_heads) return;
    const int t = (int)(wg / a.total_heads);
    int hh = (int)(wg % a.total_heads), si = 0;
    while (si + 1 < a.n_segments && hh >= a.seg[si].heads) { hh -= a.seg[si].heads; ++si; }
    const HeadSegment& g = a.seg[si];
    const int D = g.dim;
    const T* src = static_cast<const T*>(a.src) + (size_t)t * a.ld_src + g.src_off + (size_t)hh * g.src_stride;
    const float* bias = g.bias ? g.bias + (size_t)hh * D : nullptr;

    T* dst;
    bool into_cache = false;
    if (g.target == 0) {
        dst = static_cast<T*>(g.dst) + (size_t)t * g.ld_dst + g.dst_off + (size_t)hh * g.dst_stride;
    } else {
        if (!(a.write_cache & 1)) return;
        const int pos = a.positions[t], slot = pos / a.page_size;
        const int page = slot < a.table_width ? a.block_table[(size_t)a.entry_of_token[t] * a.table_width + slot] : -1;
        if (page < 0) {                       // unmapped page: refuse, never write
            if (lane == 0) atomicExch(status, 2);
            return;
        }
        const int row = hh / g.heads_per_row, within = hh % g.heads_per_row;
        const int row_len = g.target == 1 ? a.k_row : a.v_row;
        T* base = static_cast<T*>(g.target == 1 ? a.k_pages : a.v_pages);
        dst = base + (((size_t)page * a.n_kv + row) * a.page_size + pos % a.page_size) * row_len + g.dst_off +
              (size_t)within * D;
        into_cache = true;
    }

    float inv = 1.f;
    const float* norm_w = g.norm_w;
    if (g.norm_w != nullptr && g.norm_all) {
        // every warp of the token sums the whole run of heads in the same order
        const T* all = static_cast<const T*>(a.src) + (size_t)t * a.ld_src + g.src_off;
        const int n = g.heads * D;
        constexpr int VEC = 16 / (int)sizeof(T);
        float ss = 0.f;
        if (g.bias == nullptr && n % VEC == 0 && ((uintptr_t)all & 15) == 0) {
            // 16 bytes per lane and step (the same lanes take the same elements for every head's warp)
            for (int i = VEC * lane; i < n; i += 32 * VEC) {
                const uint4 raw = *reinterpret_cast<const uint4*>(all + i);
                const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const float v = to_f32(e[j]);
                    ss = fmaf(v, v, ss);
                }
            }
        } else {
            for (int i = lane; i < n; i += 32) {
                const float v = to_f32(all[i]) + (g.bias ? g.bias[i] : 0.f);
                ss = fmaf(v, v, ss);
            }
        }
        inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + a.eps);
        norm_w = g.norm_w + (size_t)hh * D;
    } else if (g.norm_w != nullptr) {
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) {
            const float v = to_f32(src[i]) + (bias ? bias[i] : 0.f);
            ss = fmaf(v, v, ss);
        }
        inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + a.eps);
    }
    const int half = g.rot / 2;
    const float2* cs = (g.cos_sin != nullptr && g.rot > 0) ? reinterpret_cast<const float2*>(g.cos_sin) + (size_t)t * half
                                                           : nullptr;
    auto value = [&](int i) {
        float v = to_f32(src[i]) + (bias ? bias[i] : 0.f);
        if (norm_w != nullptr) v = v * inv * norm_w[i];
        return v;
    };
    for (int i = lane; i < D; i += 32) {
        float v = value(i);
        const int r = i - g.rot_off;
        if (cs != nullptr && r >= 0 && r < g.rot) {
            // first of a pair: u cos - v sin; second: v cos + u sin (u the first, v the second)
            const bool low = g.interleaved ? (r & 1) == 0 : r < half;
            const float2 c = cs[g.interleaved ? r >> 1 : (low ? r : r - half)];
            const float other = value(g.interleaved ? (low ? i + 1 : i - 1) : (low ? i + half : i - half));
            v = low ? v * c.x - other * c.y : v * c.x + other * c.y;
        }
        if (into_cache) {
            if (a.write_cache & 2) v = __bfloat162float(__float2bfloat16_rn(v));
            v = cache_value(v);
        }
        dst[i] = from_f32<T>(v);
    }
}

// ---------------------------------------------------------------------------
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__global__ void __launch_bounds__(256)
head_matmul_kernel(T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, int M, int N, int K,
                   long long lda, long long a_head, long long w_head, long long ldc, long long c_head) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z;
    A += (size_t)h * a_head;
    W += (size_t)h * w_head;
    C += (size_t)h * c_head;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i, am = m0 + lrow, wn = n0 + lrow;
            As[lk + i][lrow] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
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
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(size_t)m * ldc + n] = from_f32<T>(acc[i][j]);
        }
    }
}

// Few tokens: the product is bound by reading W once.  A warp takes one output feature of one
// head for up to MT tokens; lanes stride over k (the same order for every token).
constexpr int MT = 8;
template <typename T>
__global__ void __launch_bounds__(256)
head_matvec_kernel(T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, int M, int N, int K,
                   long long lda, long long a_head, long long w_head, long long ldc, long long c_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), h = blockIdx.z, m0 = blockIdx.y * MT;
    if (n >= N) return;
    const T* w = W + (size_t)h * w_head + (size_t)n * K;
    const T* a = A + (size_t)h * a_head + (size_t)m0 * lda;
    const int rows = min(MT, M - m0);
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float wv = to_f32(w[k]);
#pragma unroll
        for (int i = 0; i < MT; ++i)
            if (i < rows) acc[i] = fmaf(to_f32(a[(size_t)i * lda + k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        const float s = warp_sum(acc[i]);
        if (i < rows && lane == 0) C[(size_t)h * c_head + (size_t)(m0 + i) * ldc + n] = from_f32<T>(s);
    }
}

// In bfloat16: the same product on the tensor cores (mma.sync m16n8k16), all heads in one launch.  A block of 4 warps takes 64 tokens x 64 features of one head; K is walked in steps of 32
// through shared memory (16-byte asynchronous copies, zeros beyond M, N and K); a warp owns 16
// tokens x 64 features.  The sum over k runs in the same order for every token.
constexpr int HM = 64, HN = 64, HK = 32, HLD = HK + 8;
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__global__ void __launch_bounds__(128)
head_matmul_mma_kernel(bf16* __restrict__ C, const bf16* __restrict__ A, const bf16* __restrict__ W, int M, int N, int K,
                       long long lda, long long a_head, long long w_head, long long ldc, long long c_head) {
    __shared__ __align__(16) bf16 As[HM * HLD];
    __shared__ __align__(16) bf16 Ws[HN * HLD];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.z;
    A += (size_t)h * a_head;
    W += (size_t)h * w_head;
    C += (size_t)h * c_head;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int m0 = blockIdx.y * HM, n0 = blockIdx.x * HN;
    float acc[HN / 8][4];
#pragma unroll
    for (int j = 0; j < HN / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HK) {
        __syncthreads();                                            // the step before has read its tiles
        // 64 rows x 4 chunks of 8 elements for each operand: 256 chunks, two per thread and operand
        for (int i = tid; i < HM * (HK / 8); i += 128) {
            const int r = i >> 2, c = (i & 3) * 8;
            const bool ka = k0 + c < K;
            const bool oa = ka && m0 + r < M, ow = ka && n0 + r < N;
            cp_async16(smem_address(As + r * HLD + c), oa ? A + (size_t)(m0 + r) * lda + k0 + c : A, oa ? 16 : 0);
            cp_async16(smem_address(Ws + r * HLD + c), ow ? W + (size_t)(n0 + r) * K + k0 + c : W, ow ? 16 : 0);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < HK; ks += 16) {
            const bf16* ar = As + (warp * 16 + gid) * HLD + ks + tig * 2;
            uint32_t a[4];
            a[0] = *reinterpret_cast<const uint32_t*>(ar);
            a[1] = *reinterpret_cast<const uint32_t*>(ar + 8 * HLD);
            a[2] = *reinterpret_cast<const uint32_t*>(ar + 8);
            a[3] = *reinterpret_cast<const uint32_t*>(ar + 8 * HLD + 8);
#pragma unroll
            for (int j = 0; j < HN / 8; ++j) {
                const bf16* wr = Ws + (j * 8 + gid) * HLD + ks + tig * 2;
                mma_bf16_16816(acc[j], a, *reinterpret_cast<const uint32_t*>(wr), *reinterpret_cast<const uint32_t*>(wr + 8));
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp * 16 + gid + 8 * half;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < HN / 8; ++j) {
            const int n = n0 + j * 8 + tig * 2;
            if (n + 1 < N) {
                *reinterpret_cast<__nv_bfloat162*>(C + (size_t)m * ldc + n) = __floats2bfloat162_rn(acc[j][2 * half], acc[j][2 * half + 1]);
            } else if (n < N) {
                C[(size_t)m * ldc + n] = __float2bfloat16_rn(acc[j][2 * half]);
            }
        }
    }
}

// out[h][n][k] = in[h][k][n]: the matrices of every head transposed (at bind time).
template <typename T>
__global__ void transpose_heads_kernel(T* __restrict__ out, const T* __restrict__ in, int rows, int cols) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const size_t base = (size_t)blockIdx.y * rows * cols;
    const int r = (int)(i / cols), c = (int)(i % cols);
    out[base + (size_t)c * rows + r] = in[base + i];
}

template <typename T>
int launch_head_matmul(void* C, const void* A, const void* W, int M, int N, int K, int heads, long long lda,
                       long long a_head, long long w_head, long long ldc, long long c_head, cudaStream_t s) {
    // the tensor-core kernel: bfloat16 at any number of tokens (a decoded token and a prompt's token
    // then sum in the same order), rows of both operands on 16-byte boundaries, results on 4-byte ones
    if (sizeof(T) == 2 && K % 8 == 0 && lda % 8 == 0 && a_head % 8 == 0 && w_head % 8 == 0 && ldc % 2 == 0 &&
        c_head % 2 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0 && ((uintptr_t)C & 3) == 0) {
        const dim3 grid((unsigned)((N + HN - 1) / HN), (unsigned)((M + HM - 1) / HM), (unsigned)heads);
        if (grid.y > 65535) return KIPP_ERR_ARG;
        return kipp_launch(head_matmul_mma_kernel, grid, dim3(128), 0, s, 1, (bf16*)C, (const bf16*)A, (const bf16*)W, M, N, K,
                           lda, a_head, w_head, ldc, c_head);
    }
    if (M <= 2 * MT) {
        const dim3 grid((unsigned)((N + 7) / 8), (unsigned)((M + MT - 1) / MT), (unsigned)heads);
        return kipp_launch(head_matvec_kernel<T>, grid, dim3(256), 0, s, 1, (T*)C, (const T*)A, (const T*)W, M, N, K, lda,
                           a_head, w_head, ldc, c_head);
    }
    const dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), (unsigned)heads);
    if (grid.y > 65535) return KIPP_ERR_ARG;
    return kipp_launch(head_matmul_kernel<T>, grid, dim3(256), 0, s, 1, (T*)C, (const T*)A, (const T*)W, M, N, K, lda,
                       a_head, w_head, ldc, c_head);
}
}  // namespace

// `segments` points at n_segments HeadSegment records (host memory; the layout is the host
// core's HeadSegment, kernels.hpp).  write_cache: bit 0 write keys and values, bit 1 round them to
// bfloat16 first (32-bit cache).
extern "C" int kipp_head_segments(const void* src, long long ld_src, int dtype, const void* segments, int n_segments,
                                  void* k_pages, void* v_pages, int k_row, int v_row, int n_kv, const int* positions,
                                  const int* entry_of_token, const int* block_table, int table_width, int page_size,
                                  int tokens, int write_cache, float eps, int* status, void* stream) {
    if (tokens <= 0 || n_segments <= 0) return 0;
    if (n_segments > MAX_SEGMENTS || segments == nullptr || page_size <= 0) return KIPP_ERR_ARG;
    SegmentArgs a = {};
    const HeadSegment* seg = static_cast<const HeadSegment*>(segments);
    for (int i = 0; i < n_segments; ++i) {
        const HeadSegment& g = seg[i];
        if (g.heads <= 0 || g.dim <= 0 || g.rot < 0 || (g.rot & 1) || g.rot_off < 0 || g.rot_off + g.rot > g.dim ||
            g.target < 0 || g.target > 2 || (g.target == 0 && g.dst == nullptr) || (g.target != 0 && g.heads_per_row <= 0) ||
            (g.rot > 0 && g.cos_sin == nullptr) || (g.norm_all && g.src_stride != g.dim))
            return KIPP_ERR_ARG;
        if (g.target == 1 && (k_pages == nullptr || g.dst_off + g.heads_per_row * g.dim > k_row)) return KIPP_ERR_ARG;
        if (g.target == 2 && (v_pages == nullptr || g.dst_off + g.heads_per_row * g.dim > v_row)) return KIPP_ERR_ARG;
        if (g.target != 0 && (g.heads + g.heads_per_row - 1) / g.heads_per_row > n_kv) return KIPP_ERR_ARG;
        a.seg[i] = g;
        a.total_heads += g.heads;
    }
    a.n_segments = n_segments;
    a.src = src; a.ld_src = ld_src; a.k_pages = k_pages; a.v_pages = v_pages;
    a.k_row = k_row; a.v_row = v_row; a.n_kv = n_kv;
    a.positions = positions; a.entry_of_token = entry_of_token; a.block_table = block_table;
    a.table_width = table_width; a.page_size = page_size; a.tokens = tokens; a.write_cache = write_cache; a.eps = eps;
    const long long warps = (long long)tokens * a.total_heads, blocks = (warps + 3) / 4;
    if (blocks > 0x7fffffffLL) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(head_segments_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, 1, a, status);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(head_segments_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, s, 1, a, status);
    return KIPP_ERR_DTYPE;
}

// C[t, h, 0:N] = W_h A[t, h, 0:K]: row t of head h of A at A + h * a_head + t * lda, W_h at
// W + h * w_head as [N, K], the result at C + h * c_head + t * ldc; all in `dtype`.
extern "C" int kipp_head_matmul(void* C, const void* A, const void* W, int dtype, int M, int N, int K, int heads,
                                long long lda, long long a_head, long long w_head, long long ldc, long long c_head,
                                void* stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return 0;
    if (K <= 0 || heads > 65535) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KIPP_DT_F32) return launch_head_matmul<float>(C, A, W, M, N, K, heads, lda, a_head, w_head, ldc, c_head, s);
    if (dtype == KIPP_DT_BF16) return launch_head_matmul<bf16>(C, A, W, M, N, K, heads, lda, a_head, w_head, ldc, c_head, s);
    return KIPP_ERR_DTYPE;
}

// out[h] = in[h]^T for `heads` row-major matrices of [rows, cols] in `dtype`.
extern "C" int kipp_transpose_heads(void* out, const void* in, int dtype, int heads, int rows, int cols, void* stream) {
    if (heads <= 0 || rows <= 0 || cols <= 0) return 0;
    if (heads > 65535) return KIPP_ERR_ARG;
    const long long n = (long long)rows * cols;
    const dim3 grid((unsigned)((n + 255) / 256), (unsigned)heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KIPP_DT_F32)
        return kipp_launch(transpose_heads_kernel<float>, grid, dim3(256), 0, s, 1, (float*)out, (const float*)in, rows, cols);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(transpose_heads_kernel<bf16>, grid, dim3(256), 0, s, 1, (bf16*)out, (const bf16*)in, rows, cols);
    return KIPP_ERR_DTYPE;
}
