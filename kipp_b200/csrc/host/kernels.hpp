// The kernels as the host core calls them: typed wrappers over the `extern "C"` launchers of
// the kernel libraries, and the choice between kernels where several can do an operation
// (tensor-core or CUDA-core product; tcgen05, mma.sync or CUDA-core attention).  The Python
// package's kernel functions call the same launchers.
//
// No sizes of a model and no property of the device stand here as constants: tile sizes and
// split rules belong to the attention kernels and are kept beside them (AttentionPlanner).
#pragma once
#include <algorithm>
#include <cmath>

#include "runtime.hpp"

namespace kipp {

enum Epilogue : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

// The work lists of the paged attention kernels for one step (device pointers into the
// step's metadata) and what the host needs to choose a kernel.
struct AttentionWork {
    const int* decode_rows = nullptr;      // [n_decode] entries that bring one token
    int n_decode = 0;
    const int* split_keys = nullptr;       // [n_decode] keys per split of each decoded token
    int stream_ctas = 0;                   // > 0: the decoded tokens' key tiles are dealt out in equal runs to
                                           // that many CTAs instead (split_keys is not read)
    const int* prefill_work = nullptr;     // [(entry, first token)] per 64-token tile, entries of > 1 token
    int n_prefill_items = 0;
    const int* all_work = nullptr;         // the same over every entry
    int n_all_items = 0;
    const int* prefill_work128 = nullptr;  // per 128-token tile, entries of > 1 token
    int n_prefill_items128 = 0;
    int longest_portion = 0;               // most tokens an entry of > 1 token brings
    int entries = 0, tokens = 0;
};

// Folding an RMSNorm into the products around it (kipp_gemm_tc_fold, few-token kernel): a residual
// add leaves what the NEXT norm needs (xn = bf16(new residual x norm_w), sums of squares per 32
// features in ssq_out); a store or SwiGLU product whose input lacks the norm's per-token factor
// takes it from such sums (ssq_in).  The layout is the kernel library's kipp_gemm_norm_fold.
struct NormFold {
    const void* norm_w = nullptr;
    int norm_w_dtype = 0;
    void* xn = nullptr;
    long long ldn = 0;
    float* ssq_out = nullptr;
    const float* ssq_in = nullptr;
    int ssq_in_slots = 0;
    float inv_n = 0.f, eps = 0.f;
};

// Where the rows of a fused q/k/v projection go when they skip the stored product
// (kipp_gemm_tc_heads): per-head norm, rotation, queries to q_out, keys and values into the pages.
// The layout is the kernel library's kipp_gemm_head_sink.
struct HeadSink {
    void* q_out = nullptr;
    void* k_pages = nullptr;
    void* v_pages = nullptr;
    const void* q_norm_w = nullptr;
    const void* k_norm_w = nullptr;
    int norm_dtype = 0;
    float eps = 0.f;
    const void* cos_sin = nullptr;
    const int* positions = nullptr;
    const int* entry_of_token = nullptr;
    const int* block_table = nullptr;
    int table_width = 0, page_size = 0, n_q = 0, n_kv = 0, write_cache = 0;
};

struct PagedCacheView {
    void* k_pages = nullptr;               // [pages, kv_heads, page_size, head_dim] of one run's cache
    void* v_pages = nullptr;
    int n_pages = 0;
    const int* block_table = nullptr;      // int32 [entries, table_width] of this step
    int table_width = 0;
    int page_size = 0;
};

// Options of the mixed-head attention kernel beside the mix (the layout is the kernel library's
// MixExtras, attention_mix.cu): a sink per head in the softmax's denominator, several score maps
// per head that share their values (n_q then counts the maps), the combination of two maps into
// one head, values that are the head of their key rows, a gate per head and token.
struct AttentionExtras {
    const float* sink = nullptr;
    int key_maps = 1;
    int values_in_keys = 0;
    int diff = 0;
    float lambda = 0.f, diff_eps = 0.f, diff_scale = 1.f;
    const void* gate = nullptr;
    long long ld_gate = 0;
    int gate_off = 0;
    int chunk = 0;                         // > 0: a query sees the keys j <= p of its own block of `chunk` positions
    float softcap = 0.f;                   // > 0: a scaled score s becomes softcap * tanh(s / softcap)
    bool any() const { return sink || key_maps != 1 || values_in_keys || diff || gate || chunk || softcap > 0.f; }
};

// A run of heads in a projection row and what becomes of them (the layout is the kernel
// library's HeadSegment, head_ops.cu).
struct HeadSegment {
    int src_off = 0, heads = 0, dim = 0, src_stride = 0;
    int rot_off = 0, rot = 0;
    int target = 0;                        // 0 activation rows, 1 key pages, 2 value pages
    int dst_off = 0, dst_stride = 0;
    int heads_per_row = 1;
    int norm_all = 0;                      // 1: one mean square over all heads of the segment, norm_w [heads * dim]
    int interleaved = 0;                   // 1: the rotation pairs dim 2i with dim 2i + 1
    const float* bias = nullptr;
    const float* norm_w = nullptr;
    const float* cos_sin = nullptr;
    void* dst = nullptr;
    long long ld_dst = 0;
};

enum Activation : int { ACT_RELU = 0, ACT_RELU_SQUARED = 1, ACT_GELU_TANH = 2, ACT_SILU = 3 };

class Ops {
public:
    cudaStream_t stream = nullptr;
    int* status = nullptr;                 // int32[4] on the device: what kernels refused or gave up
    Workspace* workspace = nullptr;
    long long launches = 0;                // kernels of this package launched through this object
    bool prefill_tensor_core = true;       // prompt portions on tcgen05 where the sizes allow
    bool mix_tensor_core = true;           // prompt steps of the mixed-head attention on mma.sync where the sizes allow
    bool moe_tensor_core = true;           // the experts' products on the tensor cores where the sizes allow

    static constexpr int DECODE_MAX_SPLITS = 32;
    static constexpr int PREFILL_TC_MIN_TOKENS = 64;   // shorter portions waste a 128-row tile

    void embed_gather(float* out, const void* table, int table_dtype, const int* ids, int tokens, int hidden,
                      int vocab) {
        using Fn = int (*)(float*, const void*, int, const int*, int, int, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_embed_gather");
        run(f(out, table, table_dtype, ids, tokens, hidden, vocab, status, stream), "embed_gather");
    }

    // out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight, float32 arithmetic.
    void rmsnorm(void* out, int out_dtype, const float* x, const void* weight, int weight_dtype, const int* rows,
                 int n_rows, int size, float eps) {
        using Fn = int (*)(void*, int, const float*, const void*, int, const int*, int, int, float, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_rmsnorm");
        run(f(out, out_dtype, x, weight, weight_dtype, rows, n_rows, size, eps, stream), "rmsnorm");
    }

    // out[r] = (x - mean) / sqrt(var + eps) * w + b over each row (bias may be null), float32 arithmetic.
    void layernorm(void* out, int out_dtype, const float* x, const float* w, const float* b, const int* rows,
                   int n_rows, int size, float eps) {
        using Fn = int (*)(void*, int, const float*, const float*, const float*, const int*, int, int, float, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_layernorm");
        run(f(out, out_dtype, x, w, b, rows, n_rows, size, eps, stream), "layernorm");
    }
    // out = act(z) element by element in the compute type (Activation).
    void activation(void* out, long long ld_out, const void* z, long long ld_z, int dtype, int rows, int n, int kind) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_activation");
        run(f(out, ld_out, z, ld_z, dtype, rows, n, kind, stream), "activation");
    }

    static bool gemm_tc_ok(int dtype, const void* a, long long lda, const void* w, long long ldw) {
        return dtype == BF16 && lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0;
    }

    // out = a @ w^T with float32 accumulation; a [M, K] (lda), w [N, K] (ldw), both of `dtype`.
    // EPI_STORE: out[M, N]; EPI_ADD: float32 out[M, N] += product; EPI_SWIGLU: out[M, N/2] =
    // silu(p[:, 0::2]) * p[:, 1::2].  float32 runs on the CUDA cores, bfloat16 on the tensor-core
    // kernel where it takes the operands.
    // Whether a product of these operands can scale its result rows (NormFold::ssq_in): the
    // tensor-core kernels do, at every number of rows.
    static bool gemm_scale_ok(int dtype, const void* a, long long lda, const void* w, long long ldw) {
        return gemm_tc_ok(dtype, a, lda, w, ldw);
    }
    // Whether a residual add of M rows can leave what the next norm needs (NormFold::norm_w), and
    // should: measured on a 36-layer, 2,560-wide model the two launches saved per layer are 3-4 %
    // of a decode step of 1 to 8 tokens, 0.6 % at 32, and at 64 the epilogue's extra work per
    // token costs 0.4 % more than they save.
    static constexpr int EMIT_PAYS_UP_TO = 32;
    static bool gemm_emit_ok(int M) {
        using Fn = int (*)(int);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_fold_ok");
        return M <= EMIT_PAYS_UP_TO && f(M) != 0;
    }

    // x * w rounded to out's type and the rows' sums of squares: the norm with its per-row factor
    // left to the product that follows (see NormFold).
    void rmsnorm_deferred(void* out, int out_dtype, float* ssq, const float* x, const void* w, int w_dtype,
                          const int* rows, int n_rows, int size) {
        using Fn = int (*)(void*, int, float*, const float*, const void*, int, const int*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_rmsnorm_deferred");
        run(f(out, out_dtype, ssq, x, w, w_dtype, rows, n_rows, size, stream), "rmsnorm_deferred");
    }

    // `activation` (an Activation, or -1 for none) is applied to a stored product: inside the
    // tensor-core kernel's epilogue on the float32 sums, else by the element-wise kernel afterwards.
    void gemm(void* out, int out_dtype, long long ldc, const void* a, long long lda, const void* w, long long ldw,
              int dtype, int M, int N, int K, Epilogue epilogue, const NormFold* fold = nullptr, int activation = -1) {
        if (M <= 0 || N <= 0) return;
        if (activation >= 0 && (epilogue != EPI_STORE || out_dtype != dtype))
            fail(KIPP_E_STATE, "only a stored product of the compute type can carry an activation");
        if (fold != nullptr && !(gemm_scale_ok(dtype, a, lda, w, ldw) && (fold->norm_w == nullptr || gemm_emit_ok(M))))
            fail(KIPP_E_STATE, "a product was asked to fold a norm that its kernel cannot fold");   // parts ask first
        if (gemm_tc_ok(dtype, a, lda, w, ldw)) {
            using Fn = int (*)(void*, int, const void*, const void*, int, int, int, long long, long long, long long, int,
                               int, int, int, const NormFold*, int*, void*);
            static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_fold");
            const int code = (int)epilogue | (activation >= 0 ? (activation + 1) << 8 : 0);
            run(f(out, out_dtype, a, w, M, N, K, lda, ldw, ldc, code, 0, 0, 0, fold, status, stream), "gemm_tc", 1,
                profiling ? format("gemm_tc %d x %d", N, K).c_str() : nullptr);
            if (fold != nullptr && fold->ssq_in != nullptr) ++folded_norms;
        } else {
            using Fn = int (*)(void*, int, const void*, const void*, int, int, int, int, int, int, int, int, void*);
            static Fn f = kernel_symbol<Fn>("gemm_simt", "kipp_gemm_simt");
            run(f(out, out_dtype, a, w, dtype, M, N, K, (int)lda, (int)ldw, (int)ldc, (int)epilogue, stream),
                "gemm_simt");
            if (activation >= 0) this->activation(out, ldc, out, ldc, out_dtype, M, N, activation);
        }
    }

    // Whether the fused q/k/v projection of a step can do per-head norm, rotation and the cache
    // write in its own epilogue (projection_to_heads) instead of storing the product.
    static bool projection_to_heads_ok(int dtype, const void* a, long long lda, const void* w, long long ldw, int M,
                                       int head_dim, int rotary_dim) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_heads_ok");
        return gemm_tc_ok(dtype, a, lda, w, ldw) && f(M, head_dim, rotary_dim) != 0;
    }
    // a [M, K] x w [(n_q + 2 n_kv) head_dim, K]^T with what qk_norm_rope_write does to the product
    // in the epilogue (the same bits); `fold` may carry the row factors of a deferred norm, and
    // `cos_sin` is the step's rope_table_by_pair.
    void projection_to_heads(const void* a, long long lda, const void* w, long long ldw, int M, int N, int K,
                             const NormFold* fold, const PagedCacheView& cache, void* q_out, const void* q_norm_w,
                             const void* k_norm_w, int norm_dtype, float eps, const float* cos_sin,
                             const int* positions, const int* entry_of_token, int n_q, int n_kv, bool write_cache) {
        HeadSink sink;
        sink.q_out = q_out; sink.k_pages = cache.k_pages; sink.v_pages = cache.v_pages;
        sink.q_norm_w = q_norm_w; sink.k_norm_w = k_norm_w; sink.norm_dtype = norm_dtype; sink.eps = eps;
        sink.cos_sin = cos_sin; sink.positions = positions; sink.entry_of_token = entry_of_token;
        sink.block_table = cache.block_table; sink.table_width = cache.table_width; sink.page_size = cache.page_size;
        sink.n_q = n_q; sink.n_kv = n_kv; sink.write_cache = write_cache ? 1 : 0;
        using Fn = int (*)(const void*, const void*, int, int, int, long long, long long, const NormFold*,
                           const HeadSink*, int*, void*);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_heads");
        run(f(a, w, M, N, K, lda, ldw, fold, &sink, status, stream), "gemm_tc_heads", 1,
            profiling ? format("gemm_tc %d x %d to heads", N, K).c_str() : nullptr);
        if (fold != nullptr && fold->ssq_in != nullptr) ++folded_norms;
        ++projections_to_heads;
    }

    // float32 [tokens, half, 2]: (cos, sin) of position * inv_freq, made once per step.
    void rope_table(float* out, const int* positions, const float* inv_freq, int tokens, int half) {
        using Fn = int (*)(void*, const int*, const float*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_rope_table");
        run(f(out, positions, inv_freq, tokens, half, stream), "rope_table");
    }
    // The same values as float32 [half, tokens, 2], as projection_to_heads reads them.
    void rope_table_by_pair(float* out, const int* positions, const float* inv_freq, int tokens, int half) {
        using Fn = int (*)(void*, const int*, const float*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_rope_table_by_pair");
        run(f(out, positions, inv_freq, tokens, half, stream), "rope_table");
    }

    // The step's table with cos and sin both multiplied by `magnitude`.
    void rope_table_scaled(float* out, const int* positions, const float* inv_freq, int tokens, int half, bool by_pair,
                           float magnitude) {
        using Fn = int (*)(void*, const int*, const float*, int, int, int, float, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_rope_table_scaled");
        run(f(out, positions, inv_freq, tokens, half, by_pair ? 1 : 0, magnitude, stream), "rope_table");
    }

    // Per-head RMSNorm of q and k, rotation, q to q_out [T, n_q, D], k and v into the pages.
    // write_cache: bit 0 write keys and values, bit 1 round them to bfloat16 first (32-bit cache).
    void qk_norm_rope_write(const void* qkv, int ld_qkv, void* q_out, const PagedCacheView& cache, int dtype,
                            const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps, const float* cos_sin,
                            int rotary_dim, const int* positions, const int* entry_of_token, int tokens, int n_q,
                            int n_kv, int head_dim, int write_cache, int value_dim = 0) {
        using Fn = int (*)(const void*, int, void*, void*, void*, int, const void*, const void*, int, float, const void*,
                           int, const int*, const int*, const int*, int, int, int, int, int, int, int, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("rope_cache", "kipp_qk_norm_rope_write_v");
        run(f(qkv, ld_qkv, q_out, cache.k_pages, cache.v_pages, dtype, q_norm_w, k_norm_w, norm_dtype, eps, cos_sin,
              cos_sin ? rotary_dim : 0, positions, entry_of_token, cache.block_table, cache.table_width,
              cache.page_size, tokens, n_q, n_kv, head_dim, value_dim > 0 ? value_dim : head_dim, write_cache, status,
              stream),
            "qk_norm_rope_write");
    }

    // Attention whose heads' scores are mixed before the softmax (head_mix [n_q, n_q] float32, or
    // null), with a window that keeps the first keep_first positions and value heads of v_dim;
    // the result is scaled by out_scale.  Scores, mix, softmax and weighted sum in float32.
    // Tokens per work item of the tensor-core prompt kernel of attention_mix.
    static int attention_mix_tile() {
        using Fn = int (*)();
        static Fn f = kernel_symbol<Fn>("attention_mix", "kipp_attention_mix_mma_tile");
        return f();
    }
    // Steps of more than this many tokens take the tensor-core kernel where it takes the sizes;
    // shorter ones are cut into runs of keys on the CUDA-core kernel.
    static constexpr int MIX_MMA_MIN_TOKENS = 64;
    // `tiles`: (entry, first token) per attention_mix_tile() tokens over every entry of the step
    // (MixTilePlanner), or null.
    void attention_mix(void* out, const void* q, const PagedCacheView& cache, int dtype, const float* head_mix,
                       const int* positions, const int* entry_of_token, int tokens, int n_q, int n_kv, int head_dim,
                       int v_dim, float scale, int window, int keep_first, float out_scale, const int* tiles = nullptr,
                       int n_tiles = 0, const int* q_start = nullptr, const int* context_len = nullptr,
                       const AttentionExtras* extras = nullptr) {
        using Fn = int (*)(void*, const void*, const void*, const void*, int, const float*, const int*, const int*,
                           const int*, int, int, int, int, int, int, int, float, int, int, float, int, float*, const void*,
                           int*, void*);
        using Fr = int (*)(int, int, int, int);
        using Fs = long long (*)(int, int, int, int);
        using Fo = int (*)(int, int, int, int, int, int);
        using Fm = int (*)(void*, const void*, const void*, const void*, const float*, const int*, int, const int*,
                           const int*, const int*, int, int, int, int, int, int, float, int, int, float, const void*, int*,
                           void*);
        static Fn f = kernel_symbol<Fn>("attention_mix", "kipp_attention_mix_ex");
        static Fr runs_of = kernel_symbol<Fr>("attention_mix", "kipp_attention_mix_runs");
        static Fs scratch_of = kernel_symbol<Fs>("attention_mix", "kipp_attention_mix_scratch_floats");
        static Fo mma_ok = kernel_symbol<Fo>("attention_mix", "kipp_attention_mix_mma_kv_per_block");
        static Fm mma = kernel_symbol<Fm>("attention_mix", "kipp_attention_mix_mma_ex");
        const bool aligned = (((uintptr_t)out | (uintptr_t)q | (uintptr_t)cache.k_pages | (uintptr_t)cache.v_pages) & 15) == 0;
        // (the tensor-core prompt kernel takes every option but values that lie in their key rows)
        const bool in_keys = extras != nullptr && extras->values_in_keys;
        const int maps = extras != nullptr ? extras->key_maps : 1;
        if (dtype == BF16 && mix_tensor_core && !in_keys && tokens > MIX_MMA_MIN_TOKENS && tiles != nullptr && n_tiles > 0 &&
            aligned && (maps == 1 || head_mix == nullptr) &&
            mma_ok(n_q, n_kv, head_dim, v_dim, maps, head_mix != nullptr ? 1 : 0) > 0) {
            run(mma(out, q, cache.k_pages, cache.v_pages, head_mix, tiles, n_tiles, q_start, context_len, cache.block_table,
                    cache.table_width, cache.page_size, n_q, n_kv, head_dim, v_dim, scale, window, keep_first, out_scale,
                    extras, status, stream),
                "attention_mix_mma");
            ++mix_mma_launches;
            return;
        }
        // a step of few tokens is cut into runs of keys (the table's width bounds the context)
        // (a block of positions spans as many key tiles as a window of its size)
        const int chunk = extras != nullptr ? extras->chunk : 0;
        const int runs = runs_of(tokens, chunk > 0 ? chunk : window, chunk > 0 ? 0 : keep_first,
                                 cache.table_width * cache.page_size);
        float* partial = runs > 1 ? workspace->get<float>("attention_mix_runs", (size_t)scratch_of(tokens, runs, n_q, v_dim))
                                  : nullptr;
        // one key row per token that is also its value (a latent), all heads on it: the heads of a
        // token are the rows of a tensor-core tile
        using Fk = int (*)(int, int, int);
        using Fsk = int (*)(void*, const void*, const void*, const int*, const int*, const int*, int, int, int, int, int, int,
                            float, int, float, int, float*, const void*, int*, void*);
        static Fk shared_ok = kernel_symbol<Fk>("attention_mix", "kipp_attention_shared_key_ok");
        static Fsk shared = kernel_symbol<Fsk>("attention_mix", "kipp_attention_shared_key");
        if (dtype == BF16 && mix_tensor_core && extras != nullptr && extras->values_in_keys && extras->key_maps == 1 &&
            !extras->diff && head_mix == nullptr && n_kv == 1 && keep_first == 0 &&
            (((uintptr_t)out | (uintptr_t)q | (uintptr_t)cache.k_pages) & 15) == 0 && shared_ok(n_q, head_dim, v_dim)) {
            run(shared(out, q, cache.k_pages, positions, entry_of_token, cache.block_table, cache.table_width, cache.page_size,
                       tokens, n_q, head_dim, v_dim, scale, window, out_scale, runs, partial, extras, status, stream),
                "attention_shared_key", runs > 1 ? 2 : 1);
            ++shared_key_launches;
            return;
        }
        run(f(out, q, cache.k_pages, cache.v_pages, dtype, head_mix, positions, entry_of_token, cache.block_table,
              cache.table_width, cache.page_size, tokens, n_q, n_kv, head_dim, v_dim, scale, window, keep_first,
              out_scale, runs, partial, extras, status, stream),
            "attention_mix", runs > 1 ? 2 : 1);
    }

    // Bias, per-head norm, rotation of a part of the head and the way to an activation buffer or
    // into the pages for up to four runs of heads of a projection row (head_ops.cu).
    void head_segments(const void* src, long long ld_src, int dtype, const HeadSegment* segments, int n_segments,
                       const PagedCacheView* cache, int k_row, int v_row, int n_kv, const int* positions,
                       const int* entry_of_token, int tokens, int write_cache, float eps) {
        using Fn = int (*)(const void*, long long, int, const void*, int, void*, void*, int, int, int, const int*,
                           const int*, const int*, int, int, int, int, float, int*, void*);
        static Fn f = kernel_symbol<Fn>("head_ops", "kipp_head_segments");
        run(f(src, ld_src, dtype, segments, n_segments, cache ? cache->k_pages : nullptr, cache ? cache->v_pages : nullptr,
              k_row, v_row, n_kv, positions, entry_of_token, cache ? cache->block_table : nullptr,
              cache ? cache->table_width : 0, cache ? cache->page_size : 1, tokens, write_cache, eps, status, stream),
            "head_segments");
    }
    // C[t, h, :] = W_h A[t, h, :] for every head: W_h [N, K] at w + h * w_head, rows of head h at
    // a + h * a_head + t * lda, results at c + h * c_head + t * ldc; one launch for all heads
    // (head_ops.cu chooses between its kernels by the number of tokens, the type and the alignment).
    void head_matmul(void* c, long long ldc, long long c_head, const void* a, long long lda, long long a_head,
                     const void* w, long long w_head, int dtype, int M, int N, int K, int heads) {
        using Fn = int (*)(void*, const void*, const void*, int, int, int, int, int, long long, long long, long long,
                           long long, long long, void*);
        static Fn f = kernel_symbol<Fn>("head_ops", "kipp_head_matmul");
        run(f(c, a, w, dtype, M, N, K, heads, lda, a_head, w_head, ldc, c_head, stream), "head_matmul");
    }
    // out[h] = in[h]^T for `heads` row-major matrices of [rows, cols]
    void transpose_heads(void* out, const void* in, int dtype, int heads, int rows, int cols) {
        using Fn = int (*)(void*, const void*, int, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("head_ops", "kipp_transpose_heads");
        run(f(out, in, dtype, heads, rows, cols, stream), "transpose_heads");
    }

    // Whether the recurrent scan kernels take heads of these sizes.
    static bool recurrent_scan_ok(int dim, int v_dim, bool delta) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_recurrent_scan_ok");
        return f(dim, v_dim, delta ? 1 : 0) != 0;
    }
    // kind: 0 retention, 1 delta rule, 2 gated memory, 3 wkv
    float* recurrent_scratch(int tokens, int heads, int dim, int v_dim, int kind) {
        using Fn = long long (*)(int, int, int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_recurrent_scratch_floats");
        return workspace->get<float>("recurrent_scratch", (size_t)f(tokens, heads, dim, v_dim, kind));
    }
    static bool gated_memory_ok(int dim, int v_dim) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_recurrent_scan_ok");
        return f(dim, v_dim, 2) != 0;
    }
    // float32 values of one request slot of the gated memory's state
    static long long gated_memory_state_floats(int heads, int dim, int v_dim) {
        using Fn = long long (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_gated_memory_state_floats");
        return f(heads, dim, v_dim);
    }
    // The matrix memory with exponential gates held stable by a running maximum (recurrent.cu):
    // m_t = max(f_t + m_{t-1}, i_t), S_t = e^(f_t + m_{t-1} - m_t) S_{t-1} + e^(i_t - m_t) k_t v_t^T, n_t alike,
    // o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6); then root-mean-square division, weight, gate.
    void gated_memory_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int q_off,
                           int k_off, int v_off, int g_off, int i_off, int f_off, const float* i_bias,
                           const float* f_bias, const float* norm_w, float* state, const int* q_start, const int* slots,
                           int entries, int tokens, int heads, int dim, int v_dim, float gate_cap, float q_scale,
                           float eps, float out_scale, int gate) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, int, int, int, const float*,
                           const float*, const float*, float*, const int*, const int*, int, int, int, int, int, float,
                           float, float, float, int, float*, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_gated_memory_scan");
        float* scratch = recurrent_scratch(tokens, heads, dim, v_dim, 2);
        run(f(out, ld_out, proj, ld_proj, dtype, q_off, k_off, v_off, g_off, i_off, f_off, i_bias, f_bias, norm_w, state,
              q_start, slots, entries, tokens, heads, dim, v_dim, gate_cap, q_scale, eps, out_scale, gate, scratch, stream),
            "gated_memory_scan", 3);
    }
    // S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t over each entry's tokens, from the state in
    // its slot and back into it; q and k rotated by the step's table and k scaled; then per-head
    // root-mean-square division, gate (1 silu, 2 sigmoid of the g columns), out_scale.
    void retention_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int q_off,
                        int k_off, int v_off, int g_off, float* state, const float* decay, const float* cos_sin,
                        int rot, const int* q_start, const int* slots, int entries, int tokens, int heads, int dim,
                        int v_dim, float k_scale, float eps, float out_scale, int gate) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, int, float*, const float*,
                           const float*, int, const int*, const int*, int, int, int, int, int, float, float, float, int,
                           float*, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_retention_scan");
        float* scratch = recurrent_scratch(tokens, heads, dim, v_dim, 0);
        run(f(out, ld_out, proj, ld_proj, dtype, q_off, k_off, v_off, g_off, state, decay, cos_sin, rot, q_start, slots,
              entries, tokens, heads, dim, v_dim, k_scale, eps, out_scale, gate, scratch, stream),
            "retention_scan", 3);
    }
    // S_t = diag(w_t) S_{t-1} - (a_t u_t)(u_t^T S_{t-1}) + k_t v_t^T, o_t = S_t^T r_t (see recurrent.cu).
    void delta_rule_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int r_off,
                         int k_off, int v_off, int g_off, int a_off, const void* w_raw, long long ld_w,
                         const float* a_bias, const float* w_bias, const float* norm_w, float* state,
                         const int* q_start, const int* slots, int entries, int tokens, int heads, int dim,
                         float eps, float out_scale, int gate) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, int, int, const void*, long long,
                           const float*, const float*, const float*, float*, const int*, const int*, int, int, int, int,
                           float, float, int, float*, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_delta_rule_scan");
        float* scratch = recurrent_scratch(tokens, heads, dim, dim, 1);
        run(f(out, ld_out, proj, ld_proj, dtype, r_off, k_off, v_off, g_off, a_off, w_raw, ld_w, a_bias, w_bias, norm_w,
              state, q_start, slots, entries, tokens, heads, dim, eps, out_scale, gate, scratch, stream),
            "delta_rule_scan", 3);
    }
    void tanh_rows(void* out, long long ld_out, const void* in, long long ld_in, int dtype, int rows, int cols) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_tanh_rows");
        run(f(out, ld_out, in, ld_in, dtype, rows, cols, stream), "tanh_rows");
    }
    // y = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 per row, N = division by the row's root mean square.
    void polynorm(void* out, long long ld_out, const void* z, long long ld_z, int dtype, const float* coef, int rows,
                  int n, float eps) {
        using Fn = int (*)(void*, long long, const void*, long long, int, const float*, int, int, float, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_polynorm");
        run(f(out, ld_out, z, ld_z, dtype, coef, rows, n, eps, stream), "polynorm");
    }
    void add_f32(float* x, const float* y, long long n) {
        using Fn = int (*)(float*, const float*, long long, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_add_f32");
        run(f(x, y, n, stream), "add_f32");
    }
    // x[t, :] += table[row(t), :] with row = (previous token * mul_prev + token * mul_cur) mod buckets, the
    // table's extra last row at position 0; the token before a step's first one is last_token[slot * stride].
    void hashed_pair_add(float* x, const void* table, int table_dtype, const int* ids, const int* positions,
                         const int* entry_of_token, const int* q_start, const int* slots, const int* last_token,
                         long long stride, int tokens, int hidden, int vocab, long long buckets, long long mul_prev,
                         long long mul_cur) {
        using Fn = int (*)(float*, const void*, int, const int*, const int*, const int*, const int*, const int*, const int*,
                           long long, int, int, int, long long, long long, long long, int*, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_hashed_pair_add");
        run(f(x, table, table_dtype, ids, positions, entry_of_token, q_start, slots, last_token, stride, tokens, hidden,
              vocab, buckets, mul_prev, mul_cur, status, stream),
            "hashed_pair_add");
    }
    // last_token[slots[e] * stride] = the last token entry e brings in this step
    void keep_last_token(int* last_token, long long stride, const int* ids, const int* q_start, const int* slots,
                         int entries) {
        using Fn = int (*)(int*, long long, const int*, const int*, const int*, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_keep_last_token");
        run(f(last_token, stride, ids, q_start, slots, entries, stream), "keep_last_token");
    }
    // x[r, :] += mult * y[r, :] * rsqrt(mean(y[r, :]^2) + eps) * w, all float32 (w keeps its storage type)
    // copy_bf16 (or null): the new x rounded to bfloat16, for the sublayer that reads the stream next
    void rmsnorm_scaled_add(float* x, const float* y, const void* w, int w_dtype, int rows, int size, float eps,
                            float mult, void* copy_bf16 = nullptr) {
        using Fn = int (*)(float*, const float*, const void*, int, int, int, float, float, void*, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_rmsnorm_scaled_add");
        run(f(x, y, w, w_dtype, rows, size, eps, mult, copy_bf16, stream), "rmsnorm_scaled_add");
    }
    // Hyper-connections (elementwise.cu): the residual stream as `streams` copies, `stride` floats apart.
    // y given: x_t <- sum_s mix[s, t] x_s + mult out_w[t] y; h given: h = rmsnorm(sum_s in_w[s] x_s).
    static int hyper_connection_max_streams() {
        using Fn = int (*)();
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_hyper_connection_max_streams");
        return f();
    }
    // clear_y: y is left zeroed for the sublayer that adds its output into it next.
    void hyper_connection(float* x, long long stride, int streams, float* y, bool clear_y, const float* mix, const float* out_w,
                          float mult, const float* in_w, const void* norm_w, int norm_w_dtype, float eps, void* h,
                          int h_dtype, int rows, int size) {
        using Fn = int (*)(float*, long long, int, float*, int, const float*, const float*, float, const float*, const void*,
                           int, float, void*, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_hyper_connection");
        run(f(x, stride, streams, y, clear_y ? 1 : 0, mix, out_w, mult, in_w, norm_w, norm_w_dtype, eps, h, h_dtype, rows, size,
              stream),
            "hyper_connection");
    }
    void sum_streams(float* out, const float* x, long long stride, int streams, long long n) {
        using Fn = int (*)(float*, const float*, long long, int, long long, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_sum_streams");
        run(f(out, x, stride, streams, n, stream), "sum_streams");
    }
    // The gated activation with limits, g sigmoid(alpha g) (u + 1) with g = min(gate + b, limit) and
    // u = clamp(up + b', -limit, limit): `bias` [2 n] float32 interleaved (gate_0, up_0, ...) or null;
    // row_gate [rows] float32 or null: the row is also multiplied by sigmoid of it.
    struct Glu {
        float alpha = 1.f, limit = 0.f;
        const float* bias = nullptr;
        const float* row_gate = nullptr;
    };
    // out[r, i] = glu(proj[r, 2 i], proj[r, 2 i + 1]): the stored product's neighbouring columns
    void glu_limited(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int rows, int n,
                     const Glu& glu) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, int, int, const float*, const float*,
                           int, float, float, const float*, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_glu_limited");
        run(f(out, ld_out, proj, ld_proj, dtype, rows, n, 0, 1, 2, glu.bias, glu.bias ? glu.bias + 1 : nullptr, 2, glu.limit,
              glu.alpha, glu.row_gate, stream),
            "glu_limited");
    }
    // out [M, N / 2] = glu of a [M, K] x w [N, K]^T whose rows are interleaved (gate_0, up_0, gate_1, ...):
    // in the tensor-core product's epilogue where it takes the operands, else a stored product (scratch
    // [M, ld_scratch]) and the element-wise kernel.
    void gemm_glu(void* out, int out_dtype, long long ldc, const void* a, long long lda, const void* w, long long ldw, int dtype,
                  int M, int N, int K, const Glu& glu, const NormFold* fold, void* scratch, long long ld_scratch) {
        if (M <= 0 || N <= 0) return;
        if (gemm_tc_ok(dtype, a, lda, w, ldw) && out_dtype == dtype) {
            using Fn = int (*)(void*, int, const void*, const void*, int, int, int, long long, long long, long long,
                               const NormFold*, const Glu*, int*, void*);
            static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_glu");
            run(f(out, out_dtype, a, w, M, N, K, lda, ldw, ldc, fold, &glu, status, stream), "gemm_tc", 1,
                profiling ? format("gemm_tc %d x %d glu", N, K).c_str() : nullptr);
            if (fold != nullptr && fold->ssq_in != nullptr) ++folded_norms;
            ++glu_epilogues;
            return;
        }
        gemm(scratch, dtype, ld_scratch, a, lda, w, ldw, dtype, M, N, K, EPI_STORE, fold);
        glu_limited(out, ldc, scratch, ld_scratch, dtype, M, N / 2, glu);
    }
    // The grouped product (gemm_grouped) with the gated epilogue: every group's rows interleaved.
    void gemm_grouped_glu(void* out, int out_dtype, long long ldc, const void* a, long long lda, const void* w, int rows, int N,
                          int K, int groups, const Glu& glu, const int* expert_of_tile, const int* n_tiles, int tile_rows) {
        using Fn = int (*)(void*, int, const void*, const void*, int, int, int, long long, long long, int, const int*, const int*,
                           int, const Glu*, int*, void*);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_grouped_glu");
        run(f(out, out_dtype, a, w, rows, N, K, lda, ldc, groups, expert_of_tile, n_tiles, tile_rows, &glu, status, stream),
            "gemm_tc_grouped", 1, profiling ? format("gemm_tc_grouped %d x %d glu", N, K).c_str() : nullptr);
        ++glu_epilogues;
    }
    // out[r] = w . h[r, :] in float32
    void row_dot(float* out, const void* h, long long ldh, int dtype, const float* w, int rows, int size) {
        using Fn = int (*)(float*, const void*, long long, int, const float*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_row_dot");
        run(f(out, h, ldh, dtype, w, rows, size, stream), "row_dot");
    }
    void add_row_bias(float* x, const float* bias, int rows, int size) {
        using Fn = int (*)(float*, const float*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_add_row_bias");
        run(f(x, bias, rows, size, stream), "add_row_bias");
    }
    void softcap_f32(float* x, long long n, float cap) {
        using Fn = int (*)(float*, long long, float, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_softcap_f32");
        run(f(x, n, cap, stream), "softcap_f32");
    }
    void scale_f32(float* x, long long n, float scale) {
        using Fn = int (*)(float*, long long, float, void*);
        static Fn f = kernel_symbol<Fn>("elementwise", "kipp_scale_f32");
        run(f(x, n, scale, stream), "scale_f32");
    }

    // Token shift (recurrent.cu): out[s][t, :] = h[t, :] + (h'[t, :] - h[t, :]) * mu[s, :], h' the row of the token
    // before in the same sequence (the slot's kept row for a portion's first token); then the keep.
    void token_shift_mix(void* out, long long out_stride, const void* h, const float* mu, const float* prev,
                         long long slot_stride, const int* q_start, const int* entry_of_token, const int* slots,
                         int dtype, int tokens, int hidden, int n_mix) {
        using Fn = int (*)(void*, long long, const void*, const float*, const float*, long long, const int*, const int*,
                           const int*, int, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_token_shift_mix");
        run(f(out, out_stride, h, mu, prev, slot_stride, q_start, entry_of_token, slots, dtype, tokens, hidden, n_mix,
              stream),
            "token_shift_mix");
    }
    void token_shift_keep(float* prev, long long slot_stride, const void* h, const int* q_start, const int* slots,
                          int dtype, int entries, int hidden) {
        using Fn = int (*)(float*, long long, const void*, const int*, const int*, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_token_shift_keep");
        run(f(prev, slot_stride, h, q_start, slots, dtype, entries, hidden, stream), "token_shift_keep");
    }
    static bool wkv_ok(int dim) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_recurrent_scan_ok");
        return f(dim, dim, 3) != 0;
    }
    // o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_{t-1} + k_t v_t^T with
    // w = exp(-exp(w_raw + w_bias)) (recurrent.cu); then root-mean-square division, weight, gate.
    void wkv_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int r_off, int k_off,
                  int v_off, int g_off, const void* w_raw, long long ld_w, const float* w_bias, const float* bonus,
                  const float* norm_w, float* state, long long slot_stride, const int* q_start, const int* slots,
                  int entries, int tokens, int heads, int dim, float eps, float out_scale, int gate) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, int, const void*, long long,
                           const float*, const float*, const float*, float*, long long, const int*, const int*, int, int,
                           int, int, float, float, int, float*, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_wkv_scan");
        float* scratch = recurrent_scratch(tokens, heads, dim, dim, 3);
        run(f(out, ld_out, proj, ld_proj, dtype, r_off, k_off, v_off, g_off, w_raw, ld_w, w_bias, bonus, norm_w, state,
              slot_stride, q_start, slots, entries, tokens, heads, dim, eps, out_scale, gate, scratch, stream),
            "wkv_scan", 3);
    }

    // The state space layer (recurrent.cu, kind 4): convolution, dt, the recurrence, gate and grouped norm.
    static bool ssd_ok(int dim, int v_dim) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_recurrent_scan_ok");
        return f(dim, v_dim, 4) != 0;
    }
    static int ssd_max_taps() {
        using Fn = int (*)();
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_ssd_max_taps");
        return f();
    }
    static long long ssd_state_floats(int heads, int groups, int dim, int v_dim, int taps) {
        using Fn = long long (*)(int, int, int, int, int);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_ssd_state_floats");
        return f(heads, groups, dim, v_dim, taps);
    }
    void ssd_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype, int z_off, int xbc_off,
                  int dt_off, const float* conv_w, const float* conv_b, int taps, const float* dt_bias, const float* a_log,
                  const float* d_skip, const float* norm_w, int norm_groups, float* state, long long slot_stride,
                  const int* q_start, const int* entry_of_token, const int* slots, int entries, int tokens, int heads,
                  int groups, int dim, int v_dim, float eps) {
        using Fn = int (*)(void*, long long, const void*, long long, int, int, int, int, const float*, const float*, int,
                           const float*, const float*, const float*, const float*, int, float*, long long, const int*,
                           const int*, const int*, int, int, int, int, int, int, float, float*, float*, void*);
        static Fn f = kernel_symbol<Fn>("recurrent", "kipp_ssd_scan");
        float* scratch = recurrent_scratch(tokens, heads, dim, v_dim, 4);
        float* conv_out = workspace->get<float>("state_space_conv", (size_t)tokens * ((size_t)heads * v_dim + 2 * (size_t)groups * dim));
        run(f(out, ld_out, proj, ld_proj, dtype, z_off, xbc_off, dt_off, conv_w, conv_b, taps, dt_bias, a_log, d_skip, norm_w,
              norm_groups, state, slot_stride, q_start, entry_of_token, slots, entries, tokens, heads, groups, dim, v_dim, eps,
              scratch, conv_out, stream),
            "ssd_scan", taps > 1 ? 5 : 4);
    }

    // Routing by scores (moe.cu): softmax over all `outputs`, the choice by score + correction, weights
    // score / sum of the chosen x weight_scale; outputs from `experts` on are identity experts (negative ids).
    void moe_route_scores(int* expert_of, float* weight_of, const void* h, long long ldh, int dtype, const float* router,
                          const float* correction, int tokens, int hidden, int outputs, int experts, int top,
                          float weight_scale) {
        using Fn = int (*)(int*, float*, const void*, long long, int, const float*, const float*, int, int, int, int, int, float,
                           void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_route_scores");
        run(f(expert_of, weight_of, h, ldh, dtype, router, correction, tokens, hidden, outputs, experts, top, weight_scale,
              stream),
            "moe_route");
    }
    // The combine where pairs with a negative expert id stand for the token's own input h.
    void moe_combine_identity(float* y, const float* rows, const float* weight_of, const int* expert_of, const void* h,
                              long long ldh, int dtype, int tokens, int hidden, int top, const int* place_of_pair = nullptr) {
        using Fn = int (*)(float*, const float*, const float*, const int*, const void*, long long, int, int, int, int,
                           const int*, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_combine_identity");
        run(f(y, rows, weight_of, expert_of, h, ldh, dtype, tokens, hidden, top, place_of_pair, stream), "moe_combine");
    }

    // Routed experts (moe.cu).  route: the `top` largest of z = W_r h + b per token (float32) and the
    // softmax over them; lists: the (token, choice) pairs sorted by expert and cut into tiles, on the
    // device; expert_gemm: one product of every tile; combine: y[t] += sum_k weight x row.
    static int moe_max_tiles(int pairs, int experts) {
        using Fn = int (*)(int, int);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_max_tiles");
        return f(pairs, experts);
    }
    void moe_route(int* expert_of, float* weight_of, const void* h, long long ldh, int dtype, const float* router,
                   const float* bias, int tokens, int hidden, int experts, int top) {
        using Fn = int (*)(int*, float*, const void*, long long, int, const float*, const float*, int, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_route");
        run(f(expert_of, weight_of, h, ldh, dtype, router, bias, tokens, hidden, experts, top, stream), "moe_route");
    }
    void moe_lists(int* sorted_pair, int* tile_info, int* n_tiles, const int* expert_of, int pairs, int experts) {
        using Fn = int (*)(int*, int*, int*, const int*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_lists");
        run(f(sorted_pair, tile_info, n_tiles, expert_of, pairs, experts, stream), "moe_lists");
    }
    void moe_gemm(void* out, int out_dtype, long long ldo, const void* a, long long lda, const void* w, long long w_expert,
                  int dtype, int N, int K, int top, bool gather, bool scatter, int activation, const int* sorted_pair,
                  const int* tile_info, const int* n_tiles, int pairs, int experts) {
        using Fn = int (*)(void*, int, long long, const void*, long long, const void*, long long, int, int, int, int, int,
                           int, int, const int*, const int*, const int*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_gemm");
        run(f(out, out_dtype, ldo, a, lda, w, w_expert, dtype, N, K, top, gather ? 1 : 0, scatter ? 1 : 0, activation,
              sorted_pair, tile_info, n_tiles, pairs, experts, stream),
            "moe_gemm", 1, profiling ? format("moe_gemm %d x %d", N, K).c_str() : nullptr);
    }
    void moe_combine(float* y, const float* rows, const float* weight_of, int tokens, int hidden, int top,
                     const int* place_of_pair = nullptr) {
        using Fn = int (*)(float*, const float*, const float*, int, int, int, const int*, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_combine");
        run(f(y, rows, weight_of, tokens, hidden, top, place_of_pair, stream), "moe_combine");
    }
    // The grouped road of prompt-sized steps: the pairs' rows sorted by expert, every expert's rows
    // padded to whole tiles of the tcgen05 prompt kernel, and one grouped product per projection.
    // rows of a tile: those of the prompt kernel where a step brings many rows per expert, else
    // those of the few-token kernel, which streams an expert's weights once per tile of 16 rows
    static int grouped_tile_rows(int tokens, int pairs, int experts) {
        using Fn = int (*)();
        static Fn many = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_group_rows");
        static Fn few = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_group_rows_few");
        return tokens >= 256 && pairs >= 64LL * experts ? many() : few();
    }
    static bool moe_grouped_ok(int dtype, int hidden, int inter) {
        return dtype == BF16 && hidden % 8 == 0 && inter % 8 == 0;
    }
    static int moe_max_padded_tiles(int pairs, int experts, int tile_rows) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_max_padded_tiles");
        return f(pairs, experts, tile_rows);
    }
    void moe_padded_lists(int* place_of_pair, int* expert_of_tile, int* n_tiles, const int* expert_of, int pairs,
                          int experts, int tile_rows) {
        using Fn = int (*)(int*, int*, int*, const int*, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_padded_lists");
        run(f(place_of_pair, expert_of_tile, n_tiles, expert_of, pairs, experts, tile_rows, stream), "moe_lists");
    }
    void moe_gather_rows(void* dst, const void* src, long long ld_src, const int* place_of_pair, int pairs, int top,
                         int hidden) {
        using Fn = int (*)(void*, const void*, long long, const int*, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("moe", "kipp_moe_gather_rows");
        run(f(dst, src, ld_src, place_of_pair, pairs, top, hidden, stream), "moe_gather_rows");
    }
    // out[r, :] = act(a[r, :] x w[expert_of_tile[r / tile]]^T) for the rows of the tiles in use
    void gemm_grouped(void* out, int out_dtype, long long ldc, const void* a, long long lda, const void* w, int rows, int N,
                      int K, int groups, int activation, const int* expert_of_tile, const int* n_tiles, int tile_rows) {
        using Fn = int (*)(void*, int, const void*, const void*, int, int, int, long long, long long, int, int, const int*,
                           const int*, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("gemm_tc", "kipp_gemm_tc_grouped");
        const int code = (int)EPI_STORE | (activation >= 0 ? (activation + 1) << 8 : 0);
        run(f(out, out_dtype, a, w, rows, N, K, lda, ldc, groups, code, expert_of_tile, n_tiles, tile_rows, status, stream),
            "gemm_tc_grouped", 1, profiling ? format("gemm_tc_grouped %d x %d", N, K).c_str() : nullptr);
    }

    static bool attention_mma_supported(int head_dim, int n_q, int n_kv) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_mma_supported");
        return f(head_dim, n_q, n_kv) != 0;
    }
    static bool attention_decode_supported(int head_dim, int n_q, int n_kv) {
        using Fn = int (*)(int, int, int);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_supported");
        return f(head_dim, n_q, n_kv) != 0;
    }
    static bool attention_tc_supported(int head_dim, int n_q, int n_kv, int page_size) {
        using Fn = int (*)(int, int, int);
        using Fp = int (*)(int);
        static Fn f = kernel_symbol<Fn>("attention_tc", "kipp_attn_prefill_tc_supported");
        static Fp g = kernel_symbol<Fp>("attention_tc", "kipp_attn_prefill_tc_page_ok");
        return f(head_dim, n_q, n_kv) != 0 && g(page_size) != 0;
    }

    // The stream cut of a step's decoded tokens, where the planner asks for it and the kernel takes the step.
    static bool decode_stream_ok(int n_decode) {
        using Fn = int (*)(int, int);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_stream_ok");
        return f(n_decode, DECODE_MAX_SPLITS) != 0;
    }
    static int decode_stream_ctas(const AttentionWork& work) {
        return work.stream_ctas > 0 && decode_stream_ok(work.n_decode) ? work.stream_ctas : 0;
    }

    float* decode_scratch(int n, int n_q, int head_dim) {
        size_t floats = (size_t)n * n_q * DECODE_MAX_SPLITS * (head_dim + 2) + (size_t)n * n_q;
        if (floats < (1u << 20)) floats = 1u << 20;
        return workspace->get<float>("attention_decode_scratch", floats);
    }
    // Causal grouped-query attention of the step's tokens over the paged cache.
    void attention(void* out, const void* q, const PagedCacheView& cache, int dtype, const AttentionWork& work,
                   const int* positions, const int* entry_of_token, const int* q_start, const int* context_len,
                   int n_q, int n_kv, int head_dim, float scale, int window) {
        if (dtype == BF16 && attention_mma_supported(head_dim, n_q, n_kv)) {
            attention_tensor_core(out, q, cache, work, q_start, context_len, n_q, n_kv, head_dim, scale, window);
            return;
        }
        using Fn = int (*)(void*, const void*, const void*, const void*, int, const int*, const int*, const int*, int,
                           int, int, int, int, int, float, int, int*, void*);
        static Fn f = kernel_symbol<Fn>("attention_simt", "kipp_paged_attention_simt");
        run(f(out, q, cache.k_pages, cache.v_pages, dtype, positions, entry_of_token, cache.block_table,
              cache.table_width, cache.page_size, work.tokens, n_q, n_kv, head_dim, scale, window, status, stream),
            "attention_simt");
    }

    // Whether a step can take attention_decode_fused: decoded tokens only, bfloat16, a head size
    // and group the split-K kernel takes, the whole head rotated or none of it.
    static bool attention_decode_fused_ok(const AttentionWork& work, int dtype, int n_q, int n_kv, int head_dim,
                                          int rotary_dim) {
        return dtype == BF16 && work.n_decode > 0 && work.n_decode == work.entries && work.entries == work.tokens &&
               (rotary_dim == 0 || rotary_dim == head_dim) && attention_mma_supported(head_dim, n_q, n_kv) &&
               attention_decode_supported(head_dim, n_q, n_kv);
    }

    // qk_norm_rope_write and attention of a step of decoded tokens in one pair of launches: the
    // attention kernel normalises and rotates the raw queries and the new key itself and writes
    // the new key and value into the pages.
    void attention_decode_fused(void* out, const void* qkv, long long ld_qkv, const PagedCacheView& cache,
                                const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps,
                                const float* cos_sin, bool write_cache, const AttentionWork& work, const int* q_start,
                                const int* context_len, int n_q, int n_kv, int head_dim, float scale, int window) {
        using Fn = int (*)(void*, const void*, long long, void*, void*, const void*, const void*, int, float, const void*,
                           int, const int*, const int*, const int*, int, int, const int*, int, int, int, int, float, int,
                           int, const int*, int, int, float*, int*, void*);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_mma_fused");
        float* scratch = decode_scratch(work.n_decode, n_q, head_dim);
        run(f(out, qkv, ld_qkv, cache.k_pages, cache.v_pages, q_norm_w, k_norm_w, norm_dtype, eps, cos_sin,
              write_cache ? 1 : 0, q_start, context_len, cache.block_table, cache.table_width, cache.page_size,
              work.decode_rows, work.n_decode, n_q, n_kv, head_dim, scale, window, DECODE_MAX_SPLITS, work.split_keys, 1,
              decode_stream_ctas(work), scratch, status, stream),
            "attn_decode_mma_fused", 2);
        ++fused_decode_launches;
        if (decode_stream_ctas(work) > 0) ++stream_decode_launches;
    }

    // The first maximum of each row; long rows are shared among blocks (two launches then).
    void argmax_rows(const float* logits, long long ld, int rows, int n, int* out) {
        using Fn = int (*)(const float*, long long, int, int, int*, void*, long long, void*);
        using Fb = long long (*)(int, int);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_argmax_rows_split");
        static Fb bytes = kernel_symbol<Fb>("sampling", "kipp_argmax_scratch_bytes");
        const long long need = bytes(rows, n);
        void* scratch = need > 0 ? workspace->buffer("argmax_parts", (size_t)need) : nullptr;
        run(f(logits, ld, rows, n, out, scratch, need, stream), "argmax_rows", need > 0 ? 2 : 1);
    }
    void sample_rows(const float* logits, long long ld, int rows, int n, const float* temperature, const int* top_k,
                     const float* top_p, const float* min_p, const double* uniform, int* out) {
        using Fn = int (*)(const float*, long long, int, int, const float*, const int*, const float*, const float*,
                           const double*, int*, void*);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_sample_rows");
        run(f(logits, ld, rows, n, temperature, top_k, top_p, min_p, uniform, out, stream), "sample_rows");
    }
    void apply_penalties(float* logits, long long ld, int rows, int n, const int* recent, int recent_width,
                         const int* recent_count, const float* repetition, const float* presence,
                         const float* frequency, const int* bias_tokens, const float* bias_values, int bias_width,
                         const int* bias_count) {
        using Fn = int (*)(float*, long long, int, int, const int*, int, const int*, const float*, const float*,
                           const float*, const int*, const float*, int, const int*, void*);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_apply_penalties");
        run(f(logits, ld, rows, n, recent, recent_width, recent_count, repetition, presence, frequency, bias_tokens,
              bias_values, bias_width, bias_count, stream),
            "apply_penalties");
    }
    // Between two greedy decode steps on the device: `next` become the step's tokens and row
    // *counter of `ring`, positions and cached lengths move on by one.
    void burst_advance(int* tokens, int* positions, int* context_len, const int* next, int* ring, int* counter, int n,
                       int ring_rows) {
        using Fn = int (*)(int*, int*, int*, const int*, int*, int*, int, int, void*);
        static Fn f = kernel_symbol<Fn>("sampling", "kipp_burst_advance");
        run(f(tokens, positions, context_len, next, ring, counter, n, ring_rows, stream), "burst_advance");
    }
    // The keys per split of every decoded token, chosen on the device for the lengths a
    // burst_advance left, by AttentionPlanner's rule.
    void decode_replan(int* split_keys, const int* context_len, const int* rows, int n, int pairs_per_entry,
                       int resident_ctas, int fixed_tiles, int max_splits, int own_length) {
        using Fn = int (*)(int*, const int*, const int*, int, int, int, int, int, int, void*);
        static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_replan");
        run(f(split_keys, context_len, rows, n, pairs_per_entry, resident_ctas, fixed_tiles, max_splits, own_length,
              stream),
            "attn_decode_replan");
    }
    void convert_rows(void* dst, int dst_dtype, long long dst_pitch, const void* src, int src_dtype,
                      long long src_pitch, long long rows, long long cols) {
        using Fn = int (*)(void*, int, long long, const void*, int, long long, long long, long long, void*);
        static Fn f = kernel_symbol<Fn>("convert", "kipp_convert_rows");
        run(f(dst, dst_dtype, dst_pitch, src, src_dtype, src_pitch, rows, cols, stream), "convert_rows");
    }

private:
    void run(int code, const char* what, int kernels = 1, const char* label = nullptr) {
        kernel_check(code, what);
        launches += kernels;
        if (profiling) mark(label ? label : what);
    }

    void attention_tensor_core(void* out, const void* q, const PagedCacheView& cache, const AttentionWork& work,
                               const int* q_start, const int* context_len, int n_q, int n_kv, int head_dim,
                               float scale, int window) {
        const bool use_decode = work.n_decode > 0 && attention_decode_supported(head_dim, n_q, n_kv);
        const int* tiles = use_decode ? work.prefill_work : work.all_work;
        const int items = use_decode ? work.n_prefill_items : work.n_all_items;
        const bool aligned = (((uintptr_t)out | (uintptr_t)q | (uintptr_t)cache.k_pages | (uintptr_t)cache.v_pages) &
                              15) == 0;
        if (prefill_tensor_core && work.n_prefill_items128 > 0 && work.longest_portion >= PREFILL_TC_MIN_TOKENS &&
            (use_decode || work.n_decode == 0) && aligned &&
            attention_tc_supported(head_dim, n_q, n_kv, cache.page_size)) {
            using Fn = int (*)(void*, const void*, int, const void*, const void*, int, const int*, const int*, const int*,
                               int, int, const int*, int, int, int, int, float, int, int*, void*);
            static Fn f = kernel_symbol<Fn>("attention_tc", "kipp_attn_prefill_tc");
            run(f(out, q, work.tokens, cache.k_pages, cache.v_pages, cache.n_pages, q_start, context_len, cache.block_table,
                  cache.table_width, cache.page_size, work.prefill_work128, work.n_prefill_items128, n_q, n_kv,
                  head_dim, scale, window, status, stream),
                "attn_prefill_tc");
            ++tc_prefill_launches;
        } else if (items > 0) {
            using Fn = int (*)(void*, const void*, const void*, const void*, const int*, const int*, const int*, int, int,
                               const int*, int, int, int, int, float, int, void*);
            static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_prefill_mma");
            run(f(out, q, cache.k_pages, cache.v_pages, q_start, context_len, cache.block_table, cache.table_width,
                  cache.page_size, tiles, items, n_q, n_kv, head_dim, scale, window, stream),
                "attn_prefill_mma");
        }
        if (use_decode) {
            using Fn = int (*)(void*, const void*, const void*, const void*, const int*, const int*, const int*, int, int,
                               const int*, int, int, int, int, float, int, int, const int*, int, int, float*, void*);
            static Fn f = kernel_symbol<Fn>("attention_mma", "kipp_attn_decode_mma");
            float* scratch = decode_scratch(work.n_decode, n_q, head_dim);
            run(f(out, q, cache.k_pages, cache.v_pages, q_start, context_len, cache.block_table, cache.table_width,
                  cache.page_size, work.decode_rows, work.n_decode, n_q, n_kv, head_dim, scale, window,
                  DECODE_MAX_SPLITS, work.split_keys, 1, decode_stream_ctas(work), scratch, stream),
                "attn_decode_mma", 2);
        }
    }

public:
    // Where a step's time goes: while `profiling` is set every launch is followed by an event on
    // the stream; profile_stop() waits for them and gives the time between consecutive events
    // per kernel name in milliseconds (steps run without graphs meanwhile, so gaps between
    // launches are part of the figures: read them as shares).
    bool profiling = false;
    void profile_start() {
        profile_clear();
        profiling = true;
        mark("(start)");
    }
    std::vector<std::pair<std::string, double>> profile_stop() {
        profiling = false;
        std::vector<std::pair<std::string, double>> out;
        if (!marks_.empty()) cuda_check(cudaEventSynchronize(marks_.back().second), "profile events");
        for (size_t i = 1; i < marks_.size(); ++i) {
            float ms = 0.f;
            cuda_check(cudaEventElapsedTime(&ms, marks_[i - 1].second, marks_[i].second), "profile events");
            bool found = false;
            for (auto& kv : out)
                if (kv.first == marks_[i].first) { kv.second += ms; found = true; break; }
            if (!found) out.emplace_back(marks_[i].first, (double)ms);
        }
        profile_clear();
        return out;
    }
    ~Ops() { profile_clear(); }

private:
    std::vector<std::pair<std::string, cudaEvent_t>> marks_;
    void mark(const std::string& what) {
        cudaEvent_t ev = nullptr;
        cuda_check(cudaEventCreate(&ev), "profile event");
        cuda_check(cudaEventRecord(ev, (cudaStream_t)stream), "profile event");
        marks_.emplace_back(what, ev);
    }
    void profile_clear() {
        for (auto& m : marks_) cudaEventDestroy(m.second);
        marks_.clear();
    }

public:
    long long tc_prefill_launches = 0;      // launches of the tcgen05 prompt attention (tests look at it)
    long long fused_decode_launches = 0;
    long long folded_norms = 0;          // norms that ran inside the products around them
    long long stream_decode_launches = 0;   // decode attention dealt out as a stream
    long long projections_to_heads = 0;     // q/k/v projections with norm, rotation and cache write inside
    long long mix_mma_launches = 0;         // launches of the tensor-core kernel of the mixed-head attention
    long long shared_key_launches = 0;      // launches of the tensor-core kernel for one shared key row per token
    long long glu_epilogues = 0;            // gated activations with limits that ran inside a tensor-core product
};

}  // namespace kipp
